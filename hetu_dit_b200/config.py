"""Plain configuration records with the field names the hot path reads.

Shapes follow the reference's hetu_dit/config/config.py (RuntimeConfig :58,
SequenceParallelConfig :102, PipeFusionParallelConfig :145, ParallelConfig
:182, EngineConfig :247, InputConfig :263); only what the denoising path uses
is kept.
"""
from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class RuntimeConfig:
    warmup_steps: int = 1
    dtype: torch.dtype = torch.bfloat16
    adjust_strategy: str = "p2p"  # base | cache | p2p


@dataclass
class SequenceParallelConfig:
    ulysses_degree: int = 1
    ring_degree: int = 1

    @property
    def sp_degree(self) -> int:
        return self.ulysses_degree * self.ring_degree


@dataclass
class PipeFusionParallelConfig:
    pp_degree: int = 1
    num_pipeline_patch: Optional[int] = None
    attn_layer_num_for_pp: Optional[List[int]] = None

    def __post_init__(self):
        if self.num_pipeline_patch is None:
            self.num_pipeline_patch = self.pp_degree  # config.py:159-163
        if self.attn_layer_num_for_pp is not None and len(self.attn_layer_num_for_pp) != self.pp_degree:
            raise ValueError("attn_layer_num_for_pp needs one entry per pipeline stage")


@dataclass
class TensorParallelConfig:
    tp_degree: int = 1


@dataclass
class DataParallelConfig:
    dp_degree: int = 1
    cfg_degree: int = 1


@dataclass
class ParallelConfig:
    sp_config: SequenceParallelConfig = field(default_factory=SequenceParallelConfig)
    pp_config: PipeFusionParallelConfig = field(default_factory=PipeFusionParallelConfig)
    tp_config: TensorParallelConfig = field(default_factory=TensorParallelConfig)
    dp_config: DataParallelConfig = field(default_factory=DataParallelConfig)

    @property
    def world_size(self) -> int:
        return (self.sp_config.sp_degree * self.pp_config.pp_degree * self.tp_config.tp_degree *
                self.dp_config.dp_degree * self.dp_config.cfg_degree)

    # flat views, as the reference's ParallelConfig exposes them (config.py:204-244)
    @property
    def tp_degree(self) -> int:
        return self.tp_config.tp_degree

    @property
    def sp_degree(self) -> int:
        return self.sp_config.sp_degree

    @property
    def ulysses_degree(self) -> int:
        return self.sp_config.ulysses_degree

    @property
    def ring_degree(self) -> int:
        return self.sp_config.ring_degree

    @property
    def pp_degree(self) -> int:
        return self.pp_config.pp_degree

    @property
    def cfg_degree(self) -> int:
        return self.dp_config.cfg_degree

    @property
    def dp_degree(self) -> int:
        return self.dp_config.dp_degree


@dataclass
class InputConfig:
    height: int = 1024
    width: int = 1024
    num_frames: int = 1
    batch_size: int = 1
    prompt: str = ""
    negative_prompt: str = ""
    num_inference_steps: int = 20
    max_sequence_length: int = 256
    seed: int = 42
    output_type: str = "latent"
    task_id: str = ""


@dataclass
class EngineConfig:
    runtime_config: RuntimeConfig = field(default_factory=RuntimeConfig)
    parallel_config: ParallelConfig = field(default_factory=ParallelConfig)
    input_config: InputConfig = field(default_factory=InputConfig)
    # which global ranks run the stages of the current request (set by the scheduler; config.py:253-258)
    encode_stage_rank: Optional[int] = None
    diffusion_stage_ranks: Optional[List[int]] = None

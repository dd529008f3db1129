"""Per-request runtime state of the denoising stage: PipeFusion patch bookkeeping.

Interface of the reference's DiTRuntimeState
(hetu_dit/core/distributed/runtime_state.py:97-707): set_input_parameters,
set_video_input_parameters, set_patched_mode, next_patch and the pp_patches_*
index lists that the KV cache, the patch coordinator and the pipelines read.
All of it is host-side integer arithmetic and must agree with the reference
index for index.
"""
from dataclasses import dataclass
from typing import List, Optional

from ...config import EngineConfig
from . import parallel_state as ps


@dataclass
class ModelGeometry:
    """What the reference reads off the diffusers pipeline object (runtime_state.py:129-170)."""
    num_attention_heads: int
    attention_head_dim: int
    patch_size: int = 2
    in_channels: int = 16
    vae_scale_factor: int = 8            # image models
    vae_scale_factor_spatial: int = 8    # video models
    vae_scale_factor_temporal: int = 4
    kind: str = "image"                  # image | cogvideox | hunyuan_video


def split_patches(latent_height: int, latent_width: int, patch_size: int, num_pipeline_patch: int, sp_world: int,
                  sp_rank: int, strict_last_patch: bool = True):
    """Row bands ("pipeline patches") of the latent and this SP rank's share of each.

    The band height is ceil(H / n) rounded up to a multiple of patch_size * sp_world, which can
    reduce the number of bands. Rank r owns slice r (of sp_world equal slices) of every band.
    Index lists are produced with the reference's own flattening
    (runtime_state.py:386-446: a rank-major list read back band-major), which matters only when
    the last band is shorter than the others.
    """
    if latent_height % sp_world != 0:
        raise ValueError("The height of the input is not divisible by the number of sequence parallel devices")
    quantum = patch_size * sp_world
    band = (latent_height + num_pipeline_patch - 1) // num_pipeline_patch
    band = (band + quantum - 1) // quantum * quantum
    n_band = (latent_height + band - 1) // band
    tail = latent_height - band * (n_band - 1)
    if strict_last_patch and tail % quantum != 0:
        raise ValueError(
            f"The height of the last pipeline patch is {tail}, which is not a multiple of (patch_size * "
            f"num_sp_patches): {patch_size} * {sp_world}. Please try to adjust 'num_pipeline_patches or sp_degree "
            f"argument so that the condition are met ")
    band_heights = [band] * (n_band - 1) + [tail]

    flat = [h // sp_world for _ in range(sp_world) for h in band_heights]
    prefix = [0]
    for h in flat:
        prefix.append(prefix[-1] + h)
    heights, bounds = [], []
    for b in range(n_band):
        lo = b * sp_world
        heights.append(flat[lo + sp_rank])
        window = prefix[lo:lo + sp_world + 1]
        bounds.append(window[sp_rank:sp_rank + 2])
    local_start = [0]
    for h in heights:
        local_start.append(local_start[-1] + h)
    per_row = latent_width // patch_size
    tok_bounds = [[per_row * (s // patch_size), per_row * (e // patch_size)] for s, e in bounds]
    tok_num = [e - s for s, e in tok_bounds]
    tok_local = [0]
    for n in tok_num:
        tok_local.append(tok_local[-1] + n)
    return n_band, heights, local_start, bounds, tok_local, tok_bounds, tok_num


class DiTRuntimeState:
    def __init__(self, geometry: ModelGeometry, config: EngineConfig, is_serving: bool = False, cur_metadata=None,
                 text_encoder_cur_metadata=None):
        self.geometry = geometry
        self.runtime_config = config.runtime_config
        self.parallel_config = config.parallel_config
        self.input_config = config.input_config
        self.is_serving = is_serving
        self.cur_metadata = cur_metadata
        self.text_encoder_cur_metadata = text_encoder_cur_metadata
        self.ready = False
        self.patch_mode = False
        self.pipeline_patch_idx = 0
        self.num_pipeline_patch = config.parallel_config.pp_config.num_pipeline_patch
        self.max_condition_sequence_length: Optional[int] = None
        self.split_text_embed_in_sp = False
        self.p2p_state = "free"
        self.worker_state = {}
        self.pp_patches_height: Optional[List[int]] = None
        self.pp_patches_start_idx_local: Optional[List[int]] = None
        self.pp_patches_start_end_idx_global: Optional[List[List[int]]] = None
        self.pp_patches_token_start_idx_local: Optional[List[int]] = None
        self.pp_patches_token_start_end_idx_global: Optional[List[List[int]]] = None
        self.pp_patches_token_num: Optional[List[int]] = None
        self.backbone_patch_size = geometry.patch_size
        self.backbone_inner_dim = geometry.num_attention_heads * geometry.attention_head_dim
        self.backbone_in_channel = geometry.in_channels
        self.vae_scale_factor = geometry.vae_scale_factor
        self.vae_scale_factor_spatial = geometry.vae_scale_factor_spatial
        self.vae_scale_factor_temporal = geometry.vae_scale_factor_temporal
        self.cogvideox = geometry.kind == "cogvideox"
        self.hunyuan_video = geometry.kind == "hunyuan_video"
        u = config.parallel_config.sp_config.ulysses_degree
        if geometry.num_attention_heads % u != 0 or geometry.num_attention_heads < u:
            raise RuntimeError(
                f"transformer backbone has {geometry.num_attention_heads} heads, which is not divisible by or "
                f"smaller than ulysses_degree {u}.")

    # -- p2p state flag (runtime_state.py:53,67-71) --------------------------------------
    def get_p2p_state(self):
        return self.p2p_state

    def set_p2p_state(self, state: str):
        if state not in ("free", "adjusting", "computing"):
            raise ValueError(state)
        self.p2p_state = state

    # -- request shape -------------------------------------------------------------------
    def set_input_parameters(self, height=None, width=None, batch_size=None, num_inference_steps=None, seed=None,
                             max_condition_sequence_length=None, split_text_embed_in_sp: bool = False):
        ic = self.input_config
        ic.num_inference_steps = num_inference_steps or ic.num_inference_steps
        self.max_condition_sequence_length = max_condition_sequence_length
        self.split_text_embed_in_sp = False  # the reference forces this off (runtime_state.py:188)
        if self.runtime_config.warmup_steps > ic.num_inference_steps:
            self.runtime_config.warmup_steps = ic.num_inference_steps
        if seed is not None:
            ic.seed = seed
        if (not self.ready or (height and ic.height != height) or (width and ic.width != width)
                or (batch_size and ic.batch_size != batch_size)):
            ic.height, ic.width = height or ic.height, width or ic.width
            ic.batch_size = batch_size or ic.batch_size
            self._calc_patches_metadata()
            self._reset_recv_buffer()
        self.ready = True

    def set_video_input_parameters(self, height=None, width=None, num_frames=None, batch_size=None,
                                   num_inference_steps=None, seed=None, split_text_embed_in_sp: bool = False):
        ic = self.input_config
        ic.num_inference_steps = num_inference_steps or ic.num_inference_steps
        if self.runtime_config.warmup_steps > ic.num_inference_steps:
            self.runtime_config.warmup_steps = ic.num_inference_steps
        self.split_text_embed_in_sp = False
        if seed is not None:
            ic.seed = seed
        if (not self.ready or (height and ic.height != height) or (width and ic.width != width)
                or (num_frames and ic.num_frames != num_frames) or (batch_size and ic.batch_size != batch_size)):
            ic.height, ic.width = height or ic.height, width or ic.width
            ic.num_frames = num_frames or ic.num_frames
            ic.batch_size = batch_size or ic.batch_size
            if self.cogvideox:
                self._calc_cogvideox_patches_metadata()
            elif not self.hunyuan_video:  # HunyuanVideo chunks tokens inside the transformer wrapper instead
                self._calc_patches_metadata()
            self._reset_recv_buffer()
        self.ready = True

    def set_patched_mode(self, patch_mode: bool):
        self.patch_mode = patch_mode
        self.pipeline_patch_idx = 0

    def next_patch(self):
        if self.patch_mode:
            self.pipeline_patch_idx += 1
            if self.pipeline_patch_idx == self.num_pipeline_patch:
                self.pipeline_patch_idx = 0
        else:
            self.pipeline_patch_idx = 0

    # -- patch metadata ------------------------------------------------------------------
    def _store(self, res):
        (self.num_pipeline_patch, self.pp_patches_height, self.pp_patches_start_idx_local,
         self.pp_patches_start_end_idx_global, self.pp_patches_token_start_idx_local,
         self.pp_patches_token_start_end_idx_global, self.pp_patches_token_num) = res

    def _calc_patches_metadata(self):
        g = self.vae_scale_factor
        self._store(split_patches(self.input_config.height // g, self.input_config.width // g, self.backbone_patch_size,
                                  self.parallel_config.pp_config.num_pipeline_patch,
                                  ps.get_sequence_parallel_world_size(), ps.get_sequence_parallel_rank()))

    def _calc_cogvideox_patches_metadata(self):
        g = self.vae_scale_factor_spatial
        self._store(split_patches(self.input_config.height // g, self.input_config.width // g, self.backbone_patch_size,
                                  self.parallel_config.pp_config.num_pipeline_patch,
                                  ps.get_sequence_parallel_world_size(), ps.get_sequence_parallel_rank(),
                                  strict_last_patch=False))

    def _reset_recv_buffer(self):
        pp = ps.get_pp_group_or_none()
        if pp is not None:
            pp.reset_buffer()

    def patches_metadata(self):
        return {
            "num_pipeline_patch": self.num_pipeline_patch,
            "pp_patches_height": self.pp_patches_height,
            "pp_patches_start_idx_local": self.pp_patches_start_idx_local,
            "pp_patches_start_end_idx_global": self.pp_patches_start_end_idx_global,
            "pp_patches_token_start_idx_local": self.pp_patches_token_start_idx_local,
            "pp_patches_token_start_end_idx_global": self.pp_patches_token_start_end_idx_global,
            "pp_patches_token_num": self.pp_patches_token_num,
        }


_RUNTIME: Optional[DiTRuntimeState] = None


def runtime_state_is_initialized() -> bool:
    return _RUNTIME is not None


def get_runtime_state() -> DiTRuntimeState:
    assert _RUNTIME is not None, "Runtime state has not been initialized."
    return _RUNTIME


def initialize_runtime_state(geometry: ModelGeometry, engine_config: EngineConfig, is_serving: bool = False,
                             cur_metadata=None, text_encoder_cur_metadata=None) -> DiTRuntimeState:
    global _RUNTIME
    _RUNTIME = DiTRuntimeState(geometry, engine_config, is_serving, cur_metadata, text_encoder_cur_metadata)
    return _RUNTIME


def reset_runtime_state(geometry: Optional[ModelGeometry] = None, engine_config: Optional[EngineConfig] = None,
                        **kw) -> Optional[DiTRuntimeState]:
    """Plan switch (worker.py:587): drop the old state; build a new one when a config is given."""
    global _RUNTIME
    _RUNTIME = None
    if geometry is not None and engine_config is not None:
        return initialize_runtime_state(geometry, engine_config, **kw)
    return None

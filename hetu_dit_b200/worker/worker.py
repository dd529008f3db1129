"""Per-GPU worker: the plan API the executor drives by method name.

Mirrors the reference's hetu_dit/worker/worker.py: init_static_env (:183-332),
init_instance_model (:415), switch_parallel_env (:480-598), hotspa_model (:1571-1993),
execute_diffusion_stage (:1009-1183), get_worker_state (:1527-1563), rpc_find_sources (:2079).

A plan names the global ranks it runs on and its degrees. Switching plans re-binds the groups
(arithmetic only -- there is no communicator pool to look up), drops the stale-KV buffers and the
per-request runtime state, and resets the activation heap. hotspa_model then brings this rank's
transformer blocks to the (pipeline, tensor) ranges of the new plan: blocks or slices already on
the GPU are re-used, missing pieces are pulled from peers' parameter arenas with one strided-copy
launch, the rest comes from the CPU master copy.

The host channel between workers (Ray RPC in the reference) is abstracted as
`exchange(obj) -> [obj of every rank]`; tests and the benchmark pass torch.distributed's
all_gather_object.
"""
import time
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..config import EngineConfig
from ..core.distributed import parallel_state as ps
from ..core.distributed.peer import ParamArena, PeerHeap
from ..core.distributed.runtime_state import (ModelGeometry, get_runtime_state, initialize_runtime_state,
                                              reset_runtime_state, runtime_state_is_initialized)
from ..core.resource_manager.cache_manager import reset_cache_manager
from ..model_executor.cache.transformer_cache import TransformerBlockCache
from ..utils import get_gpu_metadata


class Worker:
    def __init__(self, rank: int, world_size: int, local_rank: Optional[int] = None,
                 exchange: Optional[Callable[[object], List[object]]] = None, heap_bytes: int = 1 << 30,
                 arena_bytes: int = 1 << 30):
        self.rank, self.world_size = rank, world_size
        self.local_rank = rank if local_rank is None else local_rank
        self.exchange = exchange or (lambda obj: [obj])
        self.heap_bytes, self.arena_bytes = heap_bytes, arena_bytes
        self.device = torch.device("cuda", self.local_rank)
        self.heap: Optional[PeerHeap] = None
        self.arena: Optional[ParamArena] = None
        self.engine_config: Optional[EngineConfig] = None
        self.geometry: Optional[ModelGeometry] = None
        self.cpu_full_transformer = None
        self.transformer = None
        self.pipeline = None
        self.cache: Optional[TransformerBlockCache] = None
        self.cur_metadata = None
        self.plan_ranks: List[int] = [rank]
        self.worker_state: Dict[str, object] = {"task": None, "stage": "idle"}

    # ------------------------------------------------------------------ start-up
    def init_static_env(self):
        """Device, peer heap, parameter arena and the (solo) initial plan. Collective over all workers."""
        torch.cuda.set_device(self.device)
        gather = (lambda b: self.exchange(b)) if self.world_size > 1 else None
        self.heap = PeerHeap(self.heap_bytes, self.rank, self.world_size, self.device, gather)
        self.arena = ParamArena(self.arena_bytes, self.rank, self.world_size, self.device, gather)
        ps.init_distributed_environment(self.rank, self.world_size, self.heap)
        self.cache = TransformerBlockCache(device=self.device, allocator=self.arena.alloc, deallocator=self.arena.free)

    def init_instance_model(self, cpu_full_transformer, geometry: ModelGeometry, make_pipeline):
        """cpu_full_transformer: the CPU master copy (source of truth for every slice);
        make_pipeline(transformer) builds the denoising pipeline around the GPU transformer."""
        import copy
        self.cpu_full_transformer = cpu_full_transformer
        self.geometry = geometry
        # GPU twin without blocks: embeddings and heads are small and live on every rank
        blocks = {n: getattr(cpu_full_transformer, n) for n in self.cache.block_list_names()
                  if hasattr(cpu_full_transformer, n)}
        for n in blocks:
            setattr(cpu_full_transformer, n, torch.nn.ModuleList([]))
        twin = copy.deepcopy(cpu_full_transformer).to(self.device)
        for n, b in blocks.items():
            setattr(cpu_full_transformer, n, b)
        self.transformer = twin
        self.pipeline = make_pipeline(twin)
        self.pipeline.stage_sliced = True

    # ------------------------------------------------------------------ plan switch
    def switch_parallel_env(self, engine_config: EngineConfig, ranks: Sequence[int]):
        """Bind the groups of the new plan and drop everything sized for the old one."""
        pc = engine_config.parallel_config
        sp = pc.sp_config
        degrees = dict(tp=pc.tp_config.tp_degree, ulysses=sp.ulysses_degree, ring=sp.ring_degree,
                       pp=pc.pp_config.pp_degree, cfg=pc.dp_config.cfg_degree, dp=pc.dp_config.dp_degree)
        prod = 1
        for v in degrees.values():
            prod *= v
        if prod != len(ranks):
            raise ValueError(f"plan degrees {degrees} need {prod} ranks, got {len(ranks)}")
        self.engine_config = engine_config
        self.plan_ranks = sorted(ranks)
        ps.get_parallel_groups().activate_plan(self.plan_ranks, **degrees)
        self.heap.reset()
        reset_runtime_state()
        reset_cache_manager()
        initialize_runtime_state(self.geometry, engine_config, is_serving=True, cur_metadata=self.cur_metadata)

    def rpc_find_sources(self, pieces) -> List[int]:
        """uids of the pieces this worker's cache can serve; none while it is re-slicing itself."""
        if runtime_state_is_initialized() and get_runtime_state().get_p2p_state() == "adjusting":
            return []
        return self.cache.find_sources(pieces)

    def hotspa_model(self):
        """Migrate parameters to the ranges of the active plan (collective over ALL workers, because any of
        them may be asked to serve pieces). Returns the byte counts by source for the caller's log."""
        rt = get_runtime_state()
        rt.set_p2p_state("adjusting")
        old = self.cur_metadata or {"tensor_parallel": (0.0, 1.0), "pipeline_parallel": (0.0, 0.0)}
        new = get_gpu_metadata(ps.get_pipeline_parallel_rank(), ps.get_pipeline_parallel_world_size(),
                               ps.get_tensor_model_parallel_rank(), ps.get_tensor_model_parallel_world_size())
        strategy = self.engine_config.runtime_config.adjust_strategy
        peer_dirs = None
        if strategy == "p2p" and self.world_size > 1:
            mine = self.cache.directory(ptr_of=self.arena.offset_of)
            everyone = self.exchange(mine)
            peer_dirs = {}
            for r, d in enumerate(everyone):
                if r == self.rank or not d:
                    continue
                fixed = {}
                for idx, entry in d.items():
                    tensors = {name: {k: (self.arena.peer_ptr(r, v[0]),) + tuple(v[1:]) for k, v in kinds.items()}
                               for name, kinds in entry["tensors"].items()}
                    fixed[idx] = {"tp_range": entry["tp_range"], "tensors": tensors}
                peer_dirs[r] = fixed
        if strategy == "base":
            # full reload from the CPU master copy: forget what is cached first
            for idx in list(self.cache.cache):
                self.cache._release(self.cache.cache.pop(idx)[0])
        self.cache.adjust_pipeline(self.transformer, self.cpu_full_transformer, old["pipeline_parallel"],
                                   new["pipeline_parallel"], old["tensor_parallel"], new["tensor_parallel"],
                                   slice_bias=True, peer_directories=peer_dirs)
        if self.world_size > 1:
            # nobody may evict or overwrite a block a peer is still pulling from
            torch.cuda.synchronize(self.device)
            self.exchange(None)
        self.cur_metadata = new
        rt.cur_metadata = new
        if hasattr(self.transformer, "register_cache"):
            self.transformer.register_cache()
        pieces = self.cache._last_p2p_all_pieces
        rt.set_p2p_state("free")
        return {"pieces": len(pieces), "from_peers": sum(1 for p in pieces if p.source_rank >= 0),
                "from_cpu": sum(1 for p in pieces if p.source_rank < 0)}

    # ------------------------------------------------------------------ execution
    def execute_diffusion_stage(self, latents, prompt_embeds, pooled, num_inference_steps: int, height: int = 1024,
                                width: int = 1024):
        rt = get_runtime_state()
        rt.set_p2p_state("computing")
        self.worker_state.update(task="diffusion", stage="diffusion", diffusion_start_time=time.time())
        rt.set_input_parameters(height=height, width=width, batch_size=1, num_inference_steps=num_inference_steps)
        out = self.pipeline.diffusion_stage(latents, prompt_embeds, pooled, num_inference_steps)
        torch.cuda.synchronize(self.device)
        self.heap.check()
        self.worker_state.update(task=None, stage="idle", diffusion=time.time() - self.worker_state["diffusion_start_time"],
                                 diffusion_mem=torch.cuda.max_memory_allocated(self.device))
        rt.set_p2p_state("free")
        return out

    def get_worker_state(self):
        return dict(self.worker_state, rank=self.rank, plan=list(self.plan_ranks), cached_blocks=sorted(self.cache.cache),
                    arena_bytes=self.arena.bytes_in_use() if self.arena else 0)

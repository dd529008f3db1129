"""Per-GPU worker: the plan API the executor drives by method name.

Mirrors the reference's hetu_dit/worker/worker.py with its method names and signatures, because the executor
calls them by name with positional / keyword arguments (executor/gpu_executor.py:176-220):
init_static_env (:183-332), init_instance_model (:415), switch_parallel_env(world_size, ranks, engine_config)
(:480-598), async hotspa_model(engine_config) (:1571-1993), execute_diffusion_stage(encode_stage_results,
engine_config, input_config, model_class, task_id) (:1009-1183), execute_encode_diffusion_stage (:1185-1394),
get_worker_state (:1527-1563), rpc_find_sources (:2079). run_worker_method() is the by-name call.

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

from ..config import EngineConfig, InputConfig
from ..core.distributed import parallel_state as ps
from ..core.distributed.utils import RankGenerator
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
        self.states: Dict[str, object] = {}       # per-request timing / status record (worker.py `self.states`)
        self.encode = self._synthetic_encode      # stand-in for the text encoders, see execute_encode_diffusion_stage

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
    def switch_parallel_env(self, world_size: int, ranks: Sequence[int] = (), engine_config: EngineConfig = None) -> None:
        """Bind the groups of the new plan and drop everything sized for the old one. Same signature and the
        same sequence of set_activate_* calls as the reference (worker/worker.py:480-598); `world_size` is
        the number of ranks of the plan, as the executor passes it."""
        ranks = list(ranks)
        pc = engine_config.parallel_config
        if len(ranks) != pc.tp_degree * pc.sp_degree * pc.pp_degree * pc.cfg_degree * pc.dp_degree:
            raise AssertionError("Product of parallel degrees must equal length of ranks")
        groups = ps.get_parallel_groups()
        groups.set_activate_world_group(len(ranks), ranks, [ranks])
        rank_map = {i: r for i, r in enumerate(sorted(ranks))}
        gen = RankGenerator(tp=pc.tp_degree, sp=pc.sp_degree, pp=pc.pp_degree, cfg=pc.cfg_degree, dp=pc.dp_degree,
                            order="tp-sp-pp-cfg-dp")

        def mapped(axis):
            return [[rank_map[r] for r in g] for g in gen.get_ranks(axis)]

        groups.set_activate_tp_group(degree=len(ranks), ranks=ranks, group_ranks=mapped("tp"))
        groups.set_activate_sp_group(degree=len(ranks), ranks=ranks, group_ranks=mapped("sp"),
                                     ulysses_degree=pc.ulysses_degree, ring_degree=pc.ring_degree)
        groups.set_activate_pp_group(degree=len(ranks), ranks=ranks, group_ranks=mapped("pp"))
        groups.set_activate_cfg_group(degree=len(ranks), ranks=ranks, group_ranks=mapped("cfg"))
        groups.set_activate_dp_group(degree=len(ranks), ranks=ranks, group_ranks=mapped("dp"))
        self.engine_config = engine_config
        self.plan_ranks = sorted(ranks)
        # activation buffers of the old plan: the heap is re-used from its start by the new group
        self.heap.reset()
        reset_runtime_state()
        reset_cache_manager()
        initialize_runtime_state(self.geometry, engine_config, is_serving=True, cur_metadata=self.cur_metadata)
        # Built right away, as the first heap allocation after the reset: a sender addresses the receiver's
        # inbox by its own inbox offset, so every stage must carve it from the same place.
        if pc.pp_degree > 1:
            ps.get_pp_group()
        self._heap_mark = self.heap.mark()
        self._last_request_shape = None

    def rpc_find_sources(self, pieces) -> List[int]:
        """uids of the pieces this worker's cache can serve; none while it is re-slicing itself."""
        if runtime_state_is_initialized() and get_runtime_state().get_p2p_state() == "adjusting":
            return []
        return self.cache.find_sources(pieces)

    async def hotspa_model(self, engine_config: EngineConfig = None):
        """Migrate parameters to the ranges of the active plan (worker/worker.py:1571; collective over ALL
        workers, because any of them may be asked to serve pieces). A coroutine, as in the reference, where the
        executor awaits it on every worker; the work itself is synchronous GPU / host work. Returns the byte
        counts by source for the caller's log."""
        return self._migrate(engine_config or self.engine_config)

    def _migrate(self, engine_config: EngineConfig):
        rt = get_runtime_state()
        rt.set_p2p_state("adjusting")
        old = self.cur_metadata or {"tensor_parallel": (0.0, 1.0), "pipeline_parallel": (0.0, 0.0)}
        new = get_gpu_metadata(ps.get_pipeline_parallel_rank(), ps.get_pipeline_parallel_world_size(),
                               ps.get_tensor_model_parallel_rank(), ps.get_tensor_model_parallel_world_size())
        strategy = engine_config.runtime_config.adjust_strategy
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
        # Peers pull from the addresses in the directories exchanged above while this rank re-slices and evicts:
        # memory released during the switch is parked and only handed back once every rank's pulls are done.
        self.cache.defer_release = self.world_size > 1
        try:
            self.cache.adjust_pipeline_sync(self.transformer, self.cpu_full_transformer, old["pipeline_parallel"],
                                            new["pipeline_parallel"], old["tensor_parallel"],
                                            new["tensor_parallel"], slice_bias=True, peer_directories=peer_dirs)
            if self.world_size > 1:
                torch.cuda.synchronize(self.device)
                self.exchange(None)
        finally:
            self.cache.defer_release = False
            self.cache.flush_released()
        self.cur_metadata = new
        rt.cur_metadata = new
        if hasattr(self.transformer, "register_cache"):
            self.transformer.register_cache()
        pieces = self.cache._last_p2p_all_pieces
        rt.set_p2p_state("free")
        return {"pieces": len(pieces), "from_peers": sum(1 for p in pieces if p.source_rank >= 0),
                "from_cpu": sum(1 for p in pieces if p.source_rank < 0)}

    # ------------------------------------------------------------------ execution
    def _returns_latents(self, engine_config: EngineConfig) -> bool:
        """Which worker hands the latents back (worker.py:1053-1066): the last pipeline stage under PipeFusion,
        else the first of the request's diffusion ranks."""
        if engine_config.parallel_config.pp_degree > 1:
            return ps.is_pipeline_last_stage()
        first = (engine_config.diffusion_stage_ranks or self.plan_ranks)[0]
        return self.rank == first

    def _run_diffusion(self, latents, prompt_embeds, pooled, engine_config, input_config, task_id):
        rt = get_runtime_state()
        rt.set_p2p_state("computing")
        t1 = time.perf_counter()
        self.states.update(running_task=task_id, task_start_time=t1, stage_name="diffusion", diffusion_start_time=t1)
        rt.worker_state = self.states
        rt.set_input_parameters(height=input_config.height, width=input_config.width,
                                batch_size=input_config.batch_size or 1,
                                num_inference_steps=input_config.num_inference_steps)
        # A request shape (resolution, batch, text length) the previous request did not have: the exchange buffers in
        # the peer heap are named by shape, so the heap goes back to where the plan left it (else a long trace of
        # many shapes fills it), the CUDA graphs that hold the old buffers' addresses are dropped, and every
        # pipeline stage forgets its inbox layout (the text-stream message changes size) -- on every rank of the
        # plan, between the same two requests.
        request_shape = (input_config.height, input_config.width, input_config.batch_size or 1, tuple(prompt_embeds.shape))
        if request_shape != getattr(self, "_last_request_shape", None):
            if getattr(self, "_last_request_shape", None) is not None and getattr(self, "_heap_mark", None) is not None:
                self.heap.rewind(self._heap_mark)
                ps.get_parallel_groups().void_captured_graphs()
            pp = ps.get_pp_group_or_none()
            if pp is not None:
                pp.reset_buffer()
            self._last_request_shape = request_shape
        out = self.pipeline.diffusion_stage(latents, prompt_embeds, pooled, input_config.num_inference_steps)
        torch.cuda.synchronize(self.device)
        self.heap.check()
        t2 = time.perf_counter()
        self.states["diffusion"] = t2 - t1
        self.states["diffusion_mem"] = torch.cuda.max_memory_allocated(self.device)
        results = {"before": t1, "after": t2, "inner_results": self.states.copy()}
        self.states = {}
        rt.set_p2p_state("free")
        return results, (out if self._returns_latents(engine_config) else None)

    def _latents_for(self, input_config: InputConfig) -> torch.Tensor:
        """Initial noise of a request: seeded, in the packed-token layout the -shaped pipelines take."""
        g = self.geometry
        h, w = input_config.height // g.vae_scale_factor // g.patch_size, input_config.width // g.vae_scale_factor // g.patch_size
        gen = torch.Generator().manual_seed(int(input_config.seed))
        lat = torch.randn(input_config.batch_size or 1, h * w, g.in_channels * g.patch_size ** 2, generator=gen)
        return lat.to(self.device, self.engine_config.runtime_config.dtype)

    def execute_diffusion_stage(self, encode_stage_results, engine_config: EngineConfig = None,
                                input_config: InputConfig = None, model_class=None, task_id: str = None):
        """The denoising loop of one request on this worker (worker/worker.py:1009-1183): embeddings come from the
        encode stage as {"prompt_embeds", "pooled_prompt_embeds"[, "latents"]}. Returns (timing record, latents
        or None) -- the latents only on the worker that owns the result, as in the reference."""
        engine_config = engine_config or self.engine_config
        input_config = input_config or engine_config.input_config
        latents = encode_stage_results.get("latents")
        if latents is None:
            latents = self._latents_for(input_config)
        dev = self.device
        return self._run_diffusion(latents.to(dev), encode_stage_results["prompt_embeds"].to(dev),
                                   encode_stage_results["pooled_prompt_embeds"].to(dev), engine_config, input_config,
                                   task_id)

    def execute_encode_diffusion_stage(self, engine_config: EngineConfig = None, input_config: InputConfig = None,
                                       model_class=None, task_id: str = None):
        """Encode + denoise on the same worker (worker/worker.py:1185-1394). Text encoders are outside this
        package: `self.encode(input_config)` supplies the embeddings (by default seeded synthetic ones of the
        model's text width, a pure function of the prompt and the requested length)."""
        engine_config = engine_config or self.engine_config
        input_config = input_config or engine_config.input_config
        enc = self.encode(input_config)
        results, latents = self.execute_diffusion_stage(enc, engine_config, input_config, model_class, task_id)
        results["store"] = time.perf_counter()
        return results, latents

    def _synthetic_encode(self, input_config: InputConfig):
        import zlib
        shape = getattr(self.cpu_full_transformer, "shape", None)
        text_dim = shape.text_dim if shape is not None else 4096
        pooled_dim = max(shape.pooled_dim, 1) if shape is not None else 2048
        gen = torch.Generator().manual_seed(zlib.crc32(str(input_config.prompt).encode()) & 0x7fffffff)
        dtype = self.engine_config.runtime_config.dtype
        B = input_config.batch_size or 1
        return {"prompt_embeds": torch.randn(B, input_config.max_sequence_length, text_dim, generator=gen).to(dtype),
                "pooled_prompt_embeds": torch.randn(B, pooled_dim, generator=gen).to(dtype)}

    def get_worker_state(self):
        """The status record the engine polls (worker/worker.py:1527-1563), plus what this implementation knows
        about its plan and its parameter cache."""
        now = time.perf_counter()
        st = self.states
        result = {"rank": self.rank, "running_task": st.get("running_task"), "last_detected_time": now,
                  "task_start_time": st.get("task_start_time"),
                  "memory": torch.cuda.memory_allocated(self.device) if torch.cuda.is_available() else 0,
                  "running_stage": st.get("stage_name"), "estimated_running_time": st.get("estimated_running_time")}
        if result["running_stage"] is not None:
            run = now - st.get(f"{result['running_stage']}_start_time", 0)
            result["stage_running_time"] = run if run else None
        else:
            result["stage_running_time"] = None
        result["task_running_time"] = (now - result["task_start_time"]) if result["task_start_time"] else None
        if result["estimated_running_time"] is not None and result["task_running_time"] is not None:
            left = result["estimated_running_time"] - result["task_running_time"]
            result["estimated_idle_time"] = left if left > 0 else 2
        else:
            result["estimated_idle_time"] = 0
        result.update(plan=list(self.plan_ranks), cached_blocks=sorted(self.cache.cache) if self.cache else [],
                      arena_bytes=self.arena.bytes_in_use() if self.arena else 0)
        return result


def run_worker_method(worker: Worker, method: str, *args, **kwargs):
    """Calls a worker method by name the way the reference's executor does
    (RayGPUExecutorAsync._run_workers_async, executor/gpu_executor.py:176-220): positional and keyword
    arguments are passed through unchanged, coroutine methods are awaited."""
    import asyncio
    import inspect
    out = getattr(worker, method)(*args, **kwargs)
    if inspect.iscoroutine(out):
        out = asyncio.run(out)
    return out

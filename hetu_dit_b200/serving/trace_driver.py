"""Serving-trace driver: a minimal in-process stand-in for the reference's scheduler and engine loop.

The reference replays a request trace against its HTTP server (examples/api_benchmark_example_with_trace.py:80-127):
requests arrive at recorded times, the ILP scheduler (out of scope here) picks a parallel plan per request, the
engine switches the workers to it (worker.switch_parallel_env + worker.hotspa_model, worker/worker.py:480-598,
1571-1993) and runs the diffusion stage. This module keeps exactly the part of that loop that exercises the
denoising hot path: seeded Poisson arrivals, first-in-first-out admission, a fixed table from resolution to
(PipeFusion degree, Ulysses degree), every plan change through the worker plan API -- parameter slices migrate
between GPUs over the peer arena -- and the request executed by Worker.execute_diffusion_stage.

One process per GPU runs the same deterministic loop (SPMD); a request's service time is the maximum over the
ranks, measured on real executions. Arrival times are virtual: the queue is simulated with the measured service
times (start = max(arrival, previous finish)), so no GPU time is spent idling between arrivals. Reported: mean
and 95th-percentile request latency and the share of requests within 5x the single-GPU latency of their
resolution (the deadline rule of the serving-trace configuration; the reference's own deadline estimate is
hetu_dit/utils.py:267-288).
"""
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Sequence, Tuple

import numpy as np
import torch

from ..config import EngineConfig, InputConfig
from ..worker.worker import Worker, run_worker_method

RESOLUTIONS = (512, 768, 1024, 1536)

# resolution -> (PipeFusion degree, Ulysses degree) per node size; 4 pipeline patches wherever pp > 1.
# Chosen from measured service times on B200 (20 steps, CFG batch 2): the smallest images are served fastest by one
# GPU (0.20 s against 0.32 s on two PipeFusion stages), and several of them fit side by side on the node; the
# PipeFusion plan of the configuration (degree 4, 4 patches) is kept for 768 x 768; larger images take Ulysses
# degrees 2 and 4, which leaves room for other requests beside them (degree 8 would take the whole node for a
# request that gains little from it at these sizes).
PLAN_TABLE: Dict[int, Dict[int, Tuple[int, int]]] = {
    8: {512: (1, 1), 768: (4, 1), 1024: (1, 2), 1536: (1, 4)},
    4: {512: (1, 1), 768: (4, 1), 1024: (1, 2), 1536: (1, 4)},
    2: {512: (1, 1), 768: (2, 1), 1024: (1, 2), 1536: (1, 2)},
    1: {512: (1, 1), 768: (1, 1), 1024: (1, 1), 1536: (1, 1)},
}


@dataclass
class Request:
    index: int
    arrival_s: float
    resolution: int
    text_len: int
    steps: int
    seed: int


def make_trace(n_requests: int = 2000, rate_per_s: float = 2.0, seed: int = 0, steps: int = 20,
               resolutions: Sequence[int] = RESOLUTIONS, text_range: Tuple[int, int] = (77, 333)) -> List[Request]:
    """Seeded synthetic trace: Poisson arrivals, resolutions uniform over `resolutions`, text length uniform in
    [text_range[0], text_range[1]]."""
    rng = np.random.default_rng(seed)
    arrivals = np.cumsum(rng.exponential(1.0 / rate_per_s, n_requests))
    res = rng.choice(np.asarray(resolutions), n_requests)
    text = rng.integers(text_range[0], text_range[1] + 1, n_requests)
    return [Request(i, float(arrivals[i]), int(res[i]), int(text[i]), steps, 1000 + i) for i in range(n_requests)]


def engine_config_for(pp: int, ulysses: int, patches: int = 4, warmup_steps: int = 1,
                      dtype: torch.dtype = torch.bfloat16) -> EngineConfig:
    cfg = EngineConfig()
    cfg.parallel_config.pp_config.pp_degree = pp
    cfg.parallel_config.pp_config.num_pipeline_patch = patches if pp > 1 else 1
    cfg.parallel_config.sp_config.ulysses_degree = ulysses
    cfg.runtime_config.warmup_steps = warmup_steps
    cfg.runtime_config.dtype = dtype
    return cfg


def estimate_ddl(t_dict: Dict[int, float]) -> int:
    """The reference's deadline for a request shape (hetu_dit/utils.py:267-288): with t_dict = {GPUs k: latency on
    k GPUs}, k* the largest k whose speed-up over one GPU is at least 0.8 k, the deadline is
    int(round(4 t_k*) * 1.1) + 2 seconds."""
    t1 = t_dict[1]
    best_k = 1
    for k, tk in t_dict.items():
        if (t1 / tk) / k >= 0.8 and k > best_k:
            best_k = k
    return int(round(t_dict[best_k] * 4) * 1.1) + 2


def reference_deadlines(resolutions: Sequence[int], service: Sequence[float], gpus_needed: Sequence[int],
                        single_gpu: Dict[int, float]) -> np.ndarray:
    """Per request, estimate_ddl() over the latencies this run knows for its resolution: one GPU, and the GPUs of
    the plan the table gave it (mean service time of that resolution)."""
    by_res: Dict[int, Dict[int, list]] = {}
    for r, s, k in zip(resolutions, service, gpus_needed):
        by_res.setdefault(r, {}).setdefault(k, []).append(s)
    ddl = {}
    for r, per_k in by_res.items():
        t = {1: single_gpu[r]}
        for k, v in per_k.items():
            if k != 1:
                t[k] = float(np.mean(v))
        ddl[r] = estimate_ddl(t)
    return np.asarray([float(ddl[r]) for r in resolutions])


def summarize(latencies: np.ndarray, deadlines: np.ndarray) -> Dict[str, float]:
    return {"mean_s": float(latencies.mean()), "p50_s": float(np.percentile(latencies, 50)),
            "p95_s": float(np.percentile(latencies, 95)), "max_s": float(latencies.max()),
            "slo_attainment": float((latencies <= deadlines).mean())}


def simulate_fifo(arrivals: Sequence[float], service: Sequence[float]) -> np.ndarray:
    """Latency of every request of a single first-in-first-out server."""
    finish, out = 0.0, []
    for a, s in zip(arrivals, service):
        start = max(a, finish)
        finish = start + s
        out.append(finish - a)
    return np.asarray(out)


def simulate_fifo_gpus(arrivals: Sequence[float], service: Sequence[float], gpus_needed: Sequence[int],
                       total_gpus: int) -> np.ndarray:
    """Latency of every request when a request occupies gpus_needed[i] of the node's GPUs for service[i] seconds
    and requests are admitted first-in-first-out: request i starts once it has arrived, request i - 1 has
    started (no overtaking) and enough GPUs are free; it takes the GPUs that became free first. Requests on
    disjoint GPUs run at the same time, as they do under the reference's engine (one executor per GPU group)."""
    free_at = [0.0] * total_gpus
    prev_start, out = 0.0, []
    for a, s, k in zip(arrivals, service, gpus_needed):
        k = min(max(int(k), 1), total_gpus)
        order = sorted(range(total_gpus), key=lambda g: free_at[g])
        start = max(a, prev_start, free_at[order[k - 1]])
        for g in order[:k]:
            free_at[g] = start + s
        prev_start = start
        out.append(start + s - a)
    return np.asarray(out)


class TraceDriver:
    def __init__(self, worker: Worker, all_reduce_max: Callable[[float], float], text_dim: int, pooled_dim: int):
        """all_reduce_max(x): maximum of x over all worker processes (any host channel)."""
        self.worker = worker
        self.world = worker.world_size
        self.reduce_max = all_reduce_max
        self.text_dim, self.pooled_dim = text_dim, pooled_dim
        self.current_plan = None
        self.stats = {"switches": 0, "switch_s": 0.0, "pieces_from_peers": 0, "pieces_from_cpu": 0}

    def _embeds(self, req: Request):
        dtype = self.worker.engine_config.runtime_config.dtype if self.worker.engine_config else torch.bfloat16
        gen = torch.Generator().manual_seed(req.seed)
        return {"prompt_embeds": torch.randn(2, req.text_len, self.text_dim, generator=gen).to(dtype),
                "pooled_prompt_embeds": torch.randn(2, self.pooled_dim, generator=gen).to(dtype)}

    def _switch(self, ranks: List[int], pp: int, ulysses: int) -> float:
        """Every worker takes part: the plan's ranks bind the plan, the others a solo plan; the migration is
        collective because any worker may be asked to serve slices."""
        key = (tuple(ranks), pp, ulysses)
        if key == self.current_plan:
            return 0.0
        torch.cuda.synchronize(self.worker.device)
        t0 = time.perf_counter()
        w = self.worker
        if w.rank in ranks:
            cfg = engine_config_for(pp, ulysses)
            cfg.diffusion_stage_ranks = list(ranks)
            run_worker_method(w, "switch_parallel_env", len(ranks), list(ranks), cfg)
        else:
            cfg = engine_config_for(1, 1)
            cfg.diffusion_stage_ranks = [w.rank]
            run_worker_method(w, "switch_parallel_env", 1, [w.rank], cfg)
        moved = run_worker_method(w, "hotspa_model", cfg)
        torch.cuda.synchronize(w.device)
        dt = self.reduce_max(time.perf_counter() - t0)
        self.current_plan = key
        self.stats["switches"] += 1
        self.stats["switch_s"] += dt
        self.stats["pieces_from_peers"] += moved["from_peers"]
        self.stats["pieces_from_cpu"] += moved["from_cpu"]
        return dt

    def _execute(self, req: Request, ranks: List[int]) -> float:
        w = self.worker
        torch.cuda.synchronize(w.device)
        t0 = time.perf_counter()
        if w.rank in ranks:
            inp = InputConfig(height=req.resolution, width=req.resolution, num_inference_steps=req.steps,
                              seed=req.seed, max_sequence_length=req.text_len)
            run_worker_method(w, "execute_diffusion_stage", self._embeds(req), w.engine_config, inp, None,
                              task_id=f"req{req.index}")
        torch.cuda.synchronize(w.device)
        return self.reduce_max(time.perf_counter() - t0)

    def single_gpu_latency(self, steps: int, text_len: int = 205) -> Dict[int, float]:
        """Latency of one request per resolution on one GPU (every rank runs its own solo plan at once)."""
        out = {}
        self._switch_solo()
        for res in RESOLUTIONS:
            req = Request(-1, 0.0, res, text_len, steps, 7)
            self._execute(req, [self.worker.rank])          # warm-up: allocator, first-use set-up
            out[res] = self._execute(req, [self.worker.rank])
        return out

    def _switch_solo(self):
        w = self.worker
        cfg = engine_config_for(1, 1)
        cfg.diffusion_stage_ranks = [w.rank]
        run_worker_method(w, "switch_parallel_env", 1, [w.rank], cfg)
        run_worker_method(w, "hotspa_model", cfg)
        self.current_plan = ("solo",)

    def run(self, trace: List[Request], slo_factor: float = 5.0, single_gpu: Dict[int, float] = None):
        table = PLAN_TABLE[self.world]
        single_gpu = single_gpu or self.single_gpu_latency(trace[0].steps)
        service, switch_part, need = [], [], []
        for req in trace:
            pp, u = table[req.resolution]
            ranks = list(range(pp * u))
            sw = self._switch(ranks, pp, u)
            ex = self._execute(req, ranks)
            service.append(sw + ex)
            switch_part.append(sw)
            need.append(pp * u)
        arrivals = [r.arrival_s for r in trace]
        deadlines = np.asarray([slo_factor * single_gpu[r.resolution] for r in trace])
        # requests are executed one at a time here; on the virtual clock those that fit side by side on disjoint
        # GPUs overlap. The one-request-at-a-time figures are kept beside them.
        lat = simulate_fifo_gpus(arrivals, service, need, self.world)
        res = summarize(lat, deadlines)
        res["one_request_at_a_time"] = summarize(simulate_fifo(arrivals, service), deadlines)
        # the same latencies against the reference's own deadline rule
        ref_ddl = reference_deadlines([r.resolution for r in trace], service, need, single_gpu)
        res["slo_attainment_reference_deadline"] = float((lat <= ref_ddl).mean())
        res.update(requests=len(trace), service_mean_s=float(np.mean(service)), switch_share=float(
            np.sum(switch_part) / max(np.sum(service), 1e-9)), single_gpu_latency_s=single_gpu, **self.stats)
        per_res = {}
        for r in RESOLUTIONS:
            idx = [i for i, q in enumerate(trace) if q.resolution == r]
            if idx:
                per_res[r] = {"n": len(idx), "service_mean_s": float(np.mean([service[i] for i in idx])),
                              "plan": f"pp{table[r][0]}xulysses{table[r][1]}"}
        res["per_resolution"] = per_res
        return res

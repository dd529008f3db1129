"""Denoise-step benchmark: Flux.1-dev-shaped DiT, one step over 4096 image + 512 text tokens, bf16.

    python bench.py --gpus N --steps K --warmup W            # this repo's sm_100a path
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path (SDPA, fp32)

N = 1 runs the whole model on one GPU; N > 1 shards the sequence with Ulysses SP degree N (one
process per GPU, launched by torch.distributed.run), so scaling is "strong". One JSON line is
printed by rank 0. `value` is tokens/s of the whole job with inputs resident in HBM; `e2e` is the
same step driven from pinned host buffers with the host<->device copies inside the timed region.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC, UNIT = "denoise_step_tokens_per_s", "tokens/s"

# The benchmark configurations: shape, latent token grid, text tokens, and the sequence-parallel plan per GPU
# count as (ulysses, ring). "flux" is the default (the configuration the headline metric is quoted on).
CONFIGS = {
    "flux": dict(shape="FLUX_DEV", grid=(64, 64), s_txt=512, plans={1: (1, 1), 2: (2, 1), 4: (4, 1), 8: (8, 1)},
                 shard="rows", workload="flux.1-dev-shaped denoise step, 4096 image + 512 text tokens, batch 1, "
                                         "19 double + 38 single blocks, hidden 3072, 24x128 heads"),
    "sd3": dict(shape="SD3_MEDIUM", grid=(64, 64), s_txt=333, plans={1: (1, 1), 2: (2, 1), 4: (4, 1), 8: (8, 1)},
                shard="rows", workload="sd3-medium-shaped denoise step, 4096 image + 333 text tokens, batch 1, "
                                       "24 joint blocks, hidden 1536, 24x64 heads"),
    "cogvideox": dict(shape="COGVIDEOX_5B", grid=(11, 48, 85), s_txt=224,
                      plans={1: (1, 1), 2: (1, 2), 4: (1, 4), 8: (1, 8)}, shard="frame_rows",
                      workload="cogvideox-1.5-5b-shaped denoise step, 44880 video + 224 text tokens, batch 1, "
                               "42 blocks, hidden 3072, 48x64 heads"),
    "hunyuan": dict(shape="HUNYUAN_VIDEO", grid=(33, 45, 80), s_txt=256,
                    plans={1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (4, 2)}, shard="chunk",
                    workload="hunyuanvideo-shaped denoise step, 118800 video + 256 text tokens, batch 1, "
                             "20 double + 40 single blocks, hidden 3072, 24x128 heads"),
}
# Tiny twins (8 heads so that every plan up to 8 ranks divides them) for the parity check that precedes the timing.
TINY = {
    "flux": (("flux-tiny", 2, 2, 1024, 8, 128, 64, 128, 96, True, (16, 56, 56), True), {}, (32, 16), 64),
    "sd3": (("sd3-tiny", 3, 0, 512, 8, 64, 64, 128, 96, False, None, False), {}, (32, 16), 40),
    "cogvideox": (("cogvideox-tiny", 3, 0, 512, 8, 64, 128, 128, 0, True, (16, 24, 24), False),
                  dict(text_first=True, rope_on_text=False, qk_norm_kind="layer", block_kind="cogvideox", temb_dim=128),
                  (3, 16, 8), 40),
    "hunyuan": (("hunyuan-tiny", 2, 2, 1024, 8, 128, 64, 128, 96, True, (16, 56, 56), True),
                dict(text_first=False, rope_on_text=False), (3, 16, 8), 32),
}


def _n_tokens(grid):
    n = 1
    for g in grid:
        n *= g
    return n


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p.get("bf16_tflops_sustained", 1383.9), p.get("hbm_gbs", 6550.7), "measured"
    return 1400.0, 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self._stop, self._thr = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i",
                                      str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thr.join(timeout=6)

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(mhz)}


def _inputs(shape, n_img, s_txt, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return dict(latent=torch.randn(1, n_img, shape.token_in, generator=gen).bfloat16(),
                text=torch.randn(1, s_txt, shape.text_dim, generator=gen).bfloat16(),
                pooled=torch.randn(1, max(shape.pooled_dim, 1), generator=gen).bfloat16(),
                t=torch.tensor([1.0]), g=torch.tensor([3.5]))


def _shard_tokens(kind, grid, rank, world):
    """Which latent tokens a sequence-parallel rank holds: (token_offset, count, token_index or None, band grid).
    "rows": a band of rows of the image; "chunk": a contiguous chunk of the flattened token axis (HunyuanVideo,
    transformer_hunyuan_video.py:226-231 of the reference); "frame_rows": a band of rows of every frame (how the
    reference shards video latents, base_pipeline.py:337-344)."""
    n = _n_tokens(grid)
    if world == 1:
        return 0, n, None, grid
    if kind == "rows":
        rows = grid[0] // world
        return rank * rows * grid[1], rows * grid[1], None, (rows, grid[1])
    if kind == "chunk":
        return rank * (n // world), n // world, None, grid
    T, Hh, W = grid
    rows = Hh // world
    idx = (torch.arange(T)[:, None, None] * Hh * W + (rank * rows + torch.arange(rows))[None, :, None] * W
           + torch.arange(W)[None, None, :]).reshape(-1)
    return 0, idx.numel(), idx, grid


# ------------------------------------------------------------------------------------- CPU arm
_CPU_SAMPLE_STATE = {}


def cpu_step_sample(threads, cfg_name="flux", blocks=(1, 1)):
    """Times the reference's CPU path (fp32, F.scaled_dot_product_attention) on a bounded sample of the workload and
    extrapolates to the whole step. Flux / SD3: `blocks` = (double, single) whole blocks at full sequence length.
    Video configurations: the linear layers of one block on 4096 token rows and the attention of 2 heads for 2048
    query rows against the full key/value length, scaled to all rows, heads and blocks.
    Returns (seconds per whole step, description, number of timed blocks, seconds actually measured). The synthetic
    weights and inputs of a configuration are built once and kept for the following calls."""
    import hetu_dit_b200.model_executor.models.shaped_dit as M
    from oracle import attention as oa
    from oracle import shaped_dit as osd
    torch.set_num_threads(threads)
    cfg = CONFIGS[cfg_name]
    shape = getattr(M, cfg["shape"])
    s_img, s_txt = _n_tokens(cfg["grid"]), cfg["s_txt"]
    gen = torch.Generator().manual_seed(0)
    d = shape.hidden
    if cfg_name in ("cogvideox", "hunyuan"):
        S = s_img + s_txt
        rows, heads, q_rows = 4096, 2, 2048
        x = torch.randn(1, rows, d, generator=gen)
        w1, w2 = torch.randn(4 * d, d, generator=gen) * 0.02, torch.randn(d, 4 * d, generator=gen) * 0.02
        wq = torch.randn(4 * d, d, generator=gen) * 0.02  # q, k, v and output projections together
        q = torch.randn(1, q_rows, heads, shape.head_dim, generator=gen)
        k = torch.randn(1, S, heads, shape.head_dim, generator=gen)
        v = torch.randn(1, S, heads, shape.head_dim, generator=gen)
        with torch.no_grad():
            t0 = time.perf_counter()
            torch.nn.functional.linear(torch.nn.functional.gelu(torch.nn.functional.linear(x, w1), approximate="tanh"), w2)
            torch.nn.functional.linear(x, wq)
            t1 = time.perf_counter()
            oa.sdpa(q, k, v)
            t2 = time.perf_counter()
        per_block = (t1 - t0) * (S / rows) + (t2 - t1) * (S / q_rows) * (shape.heads / heads)
        return per_block * shape.n_blocks, (
            f"{cfg_name}: linear layers of one block on {rows} of {S} rows + attention of {heads} of {shape.heads} heads "
            f"for {q_rows} query rows against all {S} keys (fp32 SDPA path), extrapolated to {shape.n_blocks} blocks"), \
            1, t2 - t0

    def weights(mod, prefix):
        return {prefix + "." + k: torch.randn(v.shape, generator=gen) * (0.02 if v.dim() > 1 else 0.0) + (
            1.0 if (v.dim() == 1 and not k.endswith("bias")) else 0.0) for k, v in mod.state_dict().items()}

    if cfg_name not in _CPU_SAMPLE_STATE:
        with torch.device("meta"):
            jb = M.JointBlock(shape)
            sb = M.SingleBlock(shape) if shape.n_single else None
        sd = {}
        sd.update(weights(jb, "j"))
        if sb is not None:
            sd.update(weights(sb, "s"))
        hidden = torch.randn(1, s_img, d, generator=gen)
        context = torch.randn(1, s_txt, d, generator=gen)
        temb = torch.randn(1, d, generator=gen)
        rope = None
        if shape.rope_axes is not None:
            rope = osd.rope_tables(osd.grid_ids(s_txt, cfg["grid"]), shape.rope_axes)
        _CPU_SAMPLE_STATE[cfg_name] = (sd, sb is not None, hidden, context, temb, rope)
    sd, has_single, hidden, context, temb, rope = _CPU_SAMPLE_STATE[cfg_name]
    order = "front" if shape.text_first else "rear"
    with torch.no_grad():
        t0 = time.perf_counter()
        for _ in range(blocks[0]):
            osd.joint_block(sd, "j", hidden, context, temb, rope, shape.heads, shape.head_dim, order)
        t1 = time.perf_counter()
        x = torch.cat([context, hidden], 1)
        n_single = blocks[1] if has_single else 0
        for _ in range(n_single):
            osd.single_block(sd, "s", x, temb, rope, shape.heads, shape.head_dim)
        t2 = time.perf_counter()
    per_double = (t1 - t0) / max(blocks[0], 1)
    per_single = (t2 - t1) / max(n_single, 1)
    total = per_double * shape.n_double + per_single * shape.n_single
    return total, (f"{blocks[0]} double + {n_single} single block(s) of the {cfg_name}-shaped step at full length "
                   f"({s_img}+{s_txt} tokens, fp32 SDPA path), extrapolated to {shape.n_double}+{shape.n_single} blocks"), \
        blocks[0] + n_single, t2 - t0


def static_config(cfg_name, world, replicated_text):
    """What names the measured workload and how it is laid over the GPUs -- the same object on both arms' lines.
    Figures measured during a run go into the line's `detail`, not here."""
    import hetu_dit_b200.model_executor.models.shaped_dit as M
    cfg = CONFIGS[cfg_name]
    shape = getattr(M, cfg["shape"])
    U, R = cfg["plans"].get(world, (world, 1))
    text_layout = "n/a" if world == 1 else (
        "replicated on every rank (reference layout)" if (replicated_text or shape.block_kind != "mmdit"
                                                         or cfg["s_txt"] % world != 0) else "sharded over the ranks")
    return {"workload": cfg["workload"], "parallelism": f"ulysses{U}xring{R}" if world > 1 else "single",
            "text_stream": text_layout, "l2": "weights and activations exceed the 126 MB L2; no explicit flush"}


def run_reference(args):
    """The reference arm: the oracle's fp32 CPU path (the reference itself cannot be imported here) on all host
    cores. A step is one bounded sample of the workload (one block of each kind at full sequence length for the
    image shapes): exactly `--warmup` untimed and `--steps` timed sample steps. `ms_per_step` is the measured time
    of a sample step; `value` is the whole step's throughput, extrapolated from the samples to all blocks."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    cfg = CONFIGS[args.config]
    for _ in range(max(args.warmup, 0)):
        cpu_step_sample(threads, args.config, (1, 1))
    full, measured = [], []
    desc, n_blocks = "", 0
    for _ in range(max(args.steps, 1)):
        t_full, desc, n_blocks, t_meas = cpu_step_sample(threads, args.config, (1, 1))
        full.append(t_full)
        measured.append(t_meas)
    step_s = sorted(full)[len(full) // 2]
    tokens = _n_tokens(cfg["grid"]) + cfg["s_txt"]
    value = tokens / step_s
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sum(measured) / len(measured) * 1e3,
        "ms_per_step_is": "one bounded sample step; value is for the whole step, extrapolated from the samples",
        "ms_per_whole_step_extrapolated": step_s * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": static_config(args.config, args.gpus, args.replicated_text),
        "host": f"cpu, {threads} threads",
        "extrapolated": True, "blocks_timed_per_sample": n_blocks, "samples": len(full),
        "sample_spread_ms": [min(measured) * 1e3, max(measured) * 1e3],
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------- GPU arm
def _block_hooks(model, s_loc):
    """Forward hooks collecting every block's image / video rows of this rank (B, s_loc, hidden)."""
    outs, handles = [], []
    first = model.shape.text_first

    def double(_m, _i, out):
        outs.append(out[0].detach().float())

    def single(_m, _i, out):
        outs.append((out[:, -s_loc:] if first else out[:, :s_loc]).detach().float())

    for b in model.transformer_blocks:
        handles.append(b.register_forward_hook(double))
    for b in model.single_transformer_blocks:
        handles.append(b.register_forward_hook(single))
    return outs, handles


def parity_check(cfg_name, rank, world, plan, dev, ps, dist):
    """Outside the timed region: one step of a tiny seeded model of the benchmarked family under the benchmarked
    plan, every block's output and the final output of this rank's tokens against the same model run by this rank
    alone on all tokens (solo plan, same kernels). Returns the worst cosine / max |a-b| / max |b| over blocks,
    layouts and ranks; raises when a block misses cosine >= 0.9999 or 2e-2."""
    from hetu_dit_b200.model_executor.models.shaped_dit import DiTShape, ShapedDiT
    targs, tkw, grid, s_txt = TINY[cfg_name]
    shape = DiTShape(*targs, **tkw)
    model = ShapedDiT(shape).to(dev).init_weights(seed=11, std=0.05).bfloat16()
    inp = {k: v.to(dev) for k, v in _inputs(shape, _n_tokens(grid), s_txt, seed=12).items()}
    inp["t"] = torch.tensor([0.7], device=dev)
    pg = ps.get_parallel_groups()

    def run(tok0, n, index, band, hook_rows):
        outs, handles = _block_hooks(model, hook_rows)
        lat = inp["latent"][:, tok0:tok0 + n] if index is None else inp["latent"].index_select(1, index.to(dev))
        with torch.no_grad():
            y = model(lat, inp["text"], inp["pooled"], inp["t"], inp["g"], grid=band, token_offset=tok0,
                      full_grid=grid, token_index=None if index is None else index.to(dev))
        for h in handles:
            h.remove()
        torch.cuda.synchronize()
        return outs + [y.float()]

    pg.activate_plan([rank])
    model.register_cache()
    solo = run(0, _n_tokens(grid), None, grid, _n_tokens(grid))
    worst_cos, worst_rel = 1.0, 0.0
    layouts = []
    if world > 1:
        U, R = plan
        pg.activate_plan(list(range(world)), ulysses=U, ring=R)
        model.register_cache()
        tok0, n, index, band = _shard_tokens(CONFIGS[cfg_name]["shard"], grid, rank, world)
        rows = torch.arange(tok0, tok0 + n, device=dev) if index is None else index.to(dev)
        for shard_text in ((True, False) if shape.block_kind == "mmdit" and s_txt % world == 0 else (False,)):
            model.shard_text = shard_text
            layouts.append("sharded" if shard_text else "replicated")
            got = run(tok0, n, index, band, n)
            for a, b in zip(got, solo):
                b = b.index_select(1, rows)
                cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
                rel = ((a - b).abs().max() / b.abs().max()).item()
                worst_cos, worst_rel = min(worst_cos, cos), max(worst_rel, rel)
            ps.get_world_group().barrier()
        t = torch.tensor([-worst_cos, worst_rel], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst_cos, worst_rel = -t[0].item(), t[1].item()
    else:
        # one GPU: the kernel path against itself has nothing to compare; check the solo run is finite
        assert all(torch.isfinite(x).all().item() for x in solo)
    res = {"cos": worst_cos, "max_rel": worst_rel, "vs": "n1", "model": shape.name, "blocks": shape.n_blocks,
           "text_layouts": layouts, "plan": f"ulysses{plan[0]}xring{plan[1]}"}
    if worst_cos < 0.9999 or worst_rel > 2e-2:
        raise SystemExit(f"parity check failed: {res}")
    return res


def run_gpu(args):
    import torch.distributed as dist
    import hetu_dit_b200.model_executor.models.shaped_dit as M
    from hetu_dit_b200 import _C, kernels
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.peer import PeerHeap

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    cfg = CONFIGS[args.config]
    if world not in cfg["plans"]:
        raise SystemExit(f"config {args.config} has no plan for {world} GPUs")
    U, R = cfg["plans"][world]
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    _C.lib()  # fail loudly if the extension is missing
    heap = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

        def gather(b):
            out = [None] * world
            dist.all_gather_object(out, b)
            return out

        # exchange buffers of the video shapes: (tokens, heads / U, 128) x {q, k, v, out} x two generations
        heap = PeerHeap((1 << 30) if args.config in ("flux", "sd3") else (8 << 30), rank, world, dev, gather)
    ps.init_distributed_environment(rank, world, heap)

    parity = None
    if not args.no_parity_check:
        parity = parity_check(args.config, rank, world, (U, R), dev, ps, dist)
        if heap is not None:
            heap.check()
            heap.reset()
    ps.get_parallel_groups().activate_plan(list(range(world)), ulysses=U, ring=R)

    shape = getattr(M, cfg["shape"])
    grid, S_TXT = cfg["grid"], cfg["s_txt"]
    S_IMG = _n_tokens(grid)
    # build the model directly on the device in bf16 (no fp32 host copy per rank)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = M.ShapedDiT(shape)
    torch.set_default_dtype(torch.float32)
    model.init_weights(seed=0, std=0.02)
    model.register_cache()
    model.shard_text = not args.replicated_text
    host = {k: v.pin_memory() for k, v in _inputs(shape, S_IMG, S_TXT).items()}
    tok0, s_loc, index, band = _shard_tokens(cfg["shard"], grid, rank, world)
    index_dev = None if index is None else index.to(dev)
    resident = {k: v.to(dev) for k, v in host.items()}

    def step(inp):
        lat = inp["latent"][:, tok0:tok0 + s_loc] if index_dev is None else inp["latent"].index_select(1, index_dev)
        return model(lat, inp["text"], inp["pooled"], inp["t"], inp["g"], grid=band, token_offset=tok0,
                     full_grid=grid, token_index=index_dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms / n

    def graphed(inp):
        """The step through the product's own CUDA-graph replay (ShapedDiT.forward_graphed): captured on the first
        call, replayed afterwards."""
        lat = inp["latent"][:, tok0:tok0 + s_loc] if index_dev is None else inp["latent"].index_select(1, index_dev)
        return model.forward_graphed(lat, inp["text"], inp["pooled"], inp["t"], inp["g"], grid=band, token_offset=tok0,
                                     full_grid=grid, token_index=index_dev)

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            step(resident)
        barrier()
        if args.profile_one_step:
            # profiler aid: exactly one eager step between cudaProfilerStart/Stop, so that
            # `ncu --profile-from-start off` lists this step's launches and nothing else
            torch.cuda.cudart().cudaProfilerStart()
            step(resident)
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStop()
        # (1) eager pass: per-launch CUDA events around every attention kernel (for the roofline) and the
        #     count of this library's launches per step
        kernels.reset_counters()
        kernels.enable_attn_timing(True)
        ms_eager = timed(lambda: step(resident), args.steps)
        launches = kernels.launch_count()
        attn_ms = kernels.attn_timing_summary()
        kernels.enable_attn_timing(False)

        # (2) the timed region proper: the same step captured once in a CUDA graph and replayed, which
        #     takes the Python / launch overhead of ~1.5 k kernels per step off the critical path
        use_graph = not args.no_graph
        run_step = (lambda: graphed(resident)) if use_graph else (lambda: step(resident))
        for _ in range(2):
            run_step()
        barrier()
        with ClockSampler(local_rank) as clk:
            ms_step = timed(run_step, args.steps)

        # (3) end to end: pinned host inputs -> device, step, result -> host, every step
        out_host = torch.empty((1, s_loc, shape.token_in), dtype=torch.bfloat16).pin_memory()

        def e2e_step():
            inp = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
            out_host.copy_((graphed if use_graph else step)(inp), non_blocking=True)

        for _ in range(2):
            e2e_step()
        ms_e2e = timed(e2e_step, args.steps)

        # (4) N > 1, double/single-stream shapes: the same step with the text stream replicated on every rank and
        #     handed to the USP operators as joint tensors (the reference's layout), timed the same way
        ms_replicated = None
        if world > 1 and shape.block_kind == "mmdit" and model.shard_text and S_TXT % world == 0:
            model.shard_text = False
            for _ in range(3):
                run_step()
            barrier()
            ms_replicated = timed(run_step, args.steps)
            model.shard_text = True
    status = _C.device_status(local_rank, clear=True)
    if status[0] != 0:
        raise SystemExit(f"device-side wait timed out during the bench: {status}")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    tokens = S_IMG + S_TXT
    peak_tf, peak_hbm, peak_kind = _peaks()
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = out_host.numel() * out_host.element_size()
    # dominant kernel of this repo: the attention kernel; achieved = algorithmic FLOPs of the timed launches
    # (4 * Sq * Skv * heads * head_dim each) over their summed CUDA-event time
    achieved = attn_ms["flops"] / (attn_ms["total_ms"] * 1e-3) / 1e12 if attn_ms["total_ms"] else None
    # DRAM bytes of one launch at this shape, from the committed ncu summary (single-GPU Flux shape only)
    traffic = None
    prof = os.path.join(ROOT, "profiles", "attn_fwd_kernel_flux_shape.txt")
    if os.path.exists(prof) and world == 1 and args.config == "flux":
        with open(prof) as f:
            for ln in f:
                if ln.startswith("dram_bytes_per_launch:"):
                    traffic = int(ln.split(":")[1])
    step_flops = model.flops_per_step(S_IMG, S_TXT)
    line = {
        "metric": METRIC, "value": tokens / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": static_config(args.config, world, args.replicated_text),
        "detail": {"cuda_graph": use_graph, "fused_linear": bool(kernels.FUSED_LINEAR),
                   "ms_per_step_eager_launches": ms_eager,
                   "ms_per_step_replicated_text": ms_replicated,
                   "step_flops": step_flops,
                   "step_tflops_achieved": step_flops / (ms_step * 1e-3) / 1e12 / world},
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clk.summary(),
        "roofline": {"kernel": f"attn_fwd_kernel<{shape.head_dim},bf16>", "bound": "tensor", "achieved": achieved,
                     "peak": peak_tf, "unit": "TFLOP/s", "frac": (achieved / peak_tf) if achieved else None,
                     "traffic": traffic, "peak_source": f"bf16_tflops_sustained, {peak_kind}",
                     "launches_timed": attn_ms["count"],
                     "flops_per_launch": attn_ms["flops"] / max(attn_ms["count"], 1)},
        "parity_check": parity,
    }
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        total_s, desc, _, _ = cpu_step_sample(threads, args.config, (4, 4))
        line["cpu_baseline"] = {"value": tokens / total_s, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": desc, "extrapolated": True}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


S_IMG, S_TXT = 4096, 512  # the Flux shape, used by the single-kernel cases below


def run_kernel_case(args):
    """Small single-kernel cases for profiler captures: `attn:<batch>` runs the attention kernel alone at
    the Flux shape (4608 tokens, 24 x 128 heads), `copy:<MiB>` the strided copy kernel."""
    from hetu_dit_b200 import kernels
    kind, _, arg = args.kernel_case.partition(":")
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    extra = {}
    if kind == "attn":
        B = int(arg or 1)
        q, k, v = (torch.randn(B, S_IMG + S_TXT, 24, 128, device=dev, dtype=torch.bfloat16) for _ in range(3))
        fn = lambda: kernels.attn_fwd([q], [k], [v])
        work = 4.0 * B * (S_IMG + S_TXT) ** 2 * 24 * 128
        unit = "TFLOP/s"
    elif kind == "attn64":
        # the SD3-shaped attention: 4096 image + 154 text tokens (padded to 160 rows of storage), 24 heads of 64,
        # `arg` batch entries (2 = the classifier-free-guidance batch)
        B = int(arg or 2)
        q, k, v = (torch.randn(B, 4096 + 154, 24, 64, device=dev, dtype=torch.bfloat16) for _ in range(3))
        fn = lambda: kernels.attn_fwd([q], [k], [v])
        work = 4.0 * B * (4096 + 154) ** 2 * 24 * 64
        unit = "TFLOP/s"
    elif kind in ("attnheads", "attnheads1"):
        # the shape one rank attends after the Ulysses exchange: `arg` of the 24 heads, all 4608 tokens.
        # "attnheads" lets the wrapper split the KV range (and reports its choice), "attnheads1" forbids it.
        Hl = int(arg or 3)
        q, k, v = (torch.randn(1, S_IMG + S_TXT, Hl, 128, device=dev, dtype=torch.bfloat16) for _ in range(3))
        split = 1 if kind == "attnheads1" else None
        fn = lambda: kernels.attn_fwd([q], [k], [v], kv_split=split)
        extra["kv_split"] = 1 if split == 1 else kernels._pick_kv_split([q], [k], 1, Hl)
        work = 4.0 * (S_IMG + S_TXT) ** 2 * Hl * 128
        unit = "TFLOP/s"
    elif kind == "copy":
        n = int(arg or 512) << 20
        a = torch.empty(n, dtype=torch.uint8, device=dev)
        b = torch.empty(n, dtype=torch.uint8, device=dev)
        fn = lambda: kernels.copy_pieces([(a.data_ptr(), b.data_ptr(), 1, 0, 0, 1, 0, 0, n)], dev)
        work = 2.0 * n / 1e-3 / 1e12 * 1e-3  # bytes moved (read + write) expressed so work/ms/1e9 -> TB/s
        work = 2.0 * n
        unit = "GB/s"
    elif kind == "normrope":
        B = int(arg or 8)
        S = S_IMG + S_TXT
        q, k = (torch.randn(B, S, 24, 128, device=dev, dtype=torch.bfloat16) for _ in range(2))
        w = torch.ones(128, device=dev, dtype=torch.bfloat16)
        ang = torch.rand(S, 64, device=dev) * 6.28
        cos, sin = torch.cos(ang).repeat_interleave(2, -1).contiguous(), torch.sin(ang).repeat_interleave(2, -1).contiguous()
        fn = lambda: kernels.qk_norm_rope([(q, w, True, True), (k, w, True, True)], cos=cos, sin=sin)
        work = 2.0 * 2 * q.numel() * 2  # q and k, read + written once, 2 bytes each
        unit = "GB/s"
    elif kind == "lnmod":
        B = int(arg or 16)
        x = torch.randn(B, S_IMG + S_TXT, 3072, device=dev, dtype=torch.bfloat16)
        mod = torch.randn(B, 2 * 3072, device=dev, dtype=torch.bfloat16)
        sh, sc = mod.chunk(2, dim=-1)
        out = torch.empty_like(x)
        fn = lambda: kernels.ln_modulate(x, sh, sc, out=out)
        work = 2.0 * x.numel() * 2
        unit = "GB/s"
    elif kind == "gate":
        B = int(arg or 16)
        x = torch.randn(B, S_IMG + S_TXT, 3072, device=dev, dtype=torch.bfloat16)
        y = torch.randn_like(x)
        gate = torch.randn(B, 3072, device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(x)
        fn = lambda: kernels.gate_residual(x, gate, y, out=out)
        work = 3.0 * x.numel() * 2
        unit = "GB/s"
    elif kind in ("linear", "linearlib"):
        # linear:<rows>:<n>:<k>:<bias|gelu_tanh|gate_residual>[:<tile_m>x<tile_n>] -- the fused tensor-core kernel;
        # linearlib:... the library GEMM followed by the one-pass tail kernel it replaces
        parts = arg.split(":")
        M, N, K = (int(v) for v in parts[:3])
        epi = parts[3] if len(parts) > 3 else "bias"
        tm, tn = (int(v) for v in parts[4].split("x")) if len(parts) > 4 else (0, 0)
        x = torch.randn(1, M, K, device=dev, dtype=torch.bfloat16)
        lin = torch.nn.Linear(K, N, device=dev, dtype=torch.bfloat16)
        res = torch.randn(1, M, N, device=dev, dtype=torch.bfloat16)
        gate = torch.randn(1, N, device=dev, dtype=torch.bfloat16)
        out = torch.empty(1, M, N, device=dev, dtype=torch.bfloat16)
        if kind == "linear":
            fn = lambda: kernels.linear_fused(x, lin.weight, lin.bias, epi, residual=res, gate=gate, out=out, tile_m=tm,
                                              tile_n=tn)
        elif epi == "gelu_tanh":
            fn = lambda: kernels.gelu_tanh(lin(x), out=out)
        elif epi == "gate_residual":
            fn = lambda: kernels.gate_residual(res, gate, lin(x), out=out)
        else:
            fn = lambda: lin(x)
        work = 2.0 * M * N * K
        unit = "TFLOP/s"
    else:
        raise SystemExit(f"unknown kernel case {args.kernel_case}")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    rate = work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
    print(json.dumps({"kernel_case": args.kernel_case, "ms_per_launch": ms, "rate": rate, "unit": unit, **extra}),
          flush=True)


USP_CASES = {
    # name: (heads, head_dim, image/video tokens, text tokens, joint strategy, {world: (ulysses, ring)})
    "flux": (24, 128, 4096, 512, "front", {2: (2, 1), 4: (4, 1), 8: (8, 1)}),
    "cogvideox": (48, 64, 44880, 224, "front", {2: (1, 2), 4: (1, 4), 8: (1, 8)}),
    "hunyuan": (24, 128, 118800, 256, "rear", {8: (4, 2), 4: (2, 2), 2: (2, 1)}),
}


def run_usp_case(args):
    """Operator-level timing of one USP attention layer at the shape of one of the benchmark configurations under torchrun:
    `usp:<flux|cogvideox|hunyuan>`. Prints ms per layer (max over ranks), TFLOP/s per GPU, and the share of
    the layer that is not attention compute (exchange, barriers, copies)."""
    import torch.distributed as dist
    from hetu_dit_b200 import _C, kernels
    from hetu_dit_b200.core import parallel as P
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.peer import PeerHeap
    name = args.kernel_case.split(":")[1]
    H, D, s_img, s_txt, strategy, plans = USP_CASES[name]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device(f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}")
    torch.cuda.set_device(dev)
    U, R = plans[world]
    dist.init_process_group("nccl", device_id=dev)

    def gather(b):
        out = [None] * world
        dist.all_gather_object(out, b)
        return out

    s_loc = s_img // world
    kv_bytes = 2 * s_img * H * D * 2 // max(U, 1)
    heap = PeerHeap(max(1 << 30, 6 * kv_bytes), rank, world, dev, gather)
    ps.init_distributed_environment(rank, world, heap)
    ps.initialize_model_parallel(sequence_parallel_degree=world, ulysses_degree=U, ring_degree=R)
    torch.manual_seed(rank)
    q, k, v = (torch.randn(1, s_loc, H, D, device=dev, dtype=torch.bfloat16) for _ in range(3))
    jq, jk, jv = (torch.randn(1, s_txt, H, D, device=dev, dtype=torch.bfloat16) for _ in range(3))
    layer = P.hetuDiTJointLongContextAttention()

    def op():
        return layer(None, q, k, v, joint_tensor_query=jq, joint_tensor_key=jk, joint_tensor_value=jv,
                     joint_strategy=strategy)

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    for _ in range(3):
        op()
    ms_layer = timed(op, args.steps)
    # compute only: the same attention work on local copies, no exchange
    Hl = H // U
    s_q = s_img // R + s_txt
    qg = torch.randn(1, s_q, Hl, D, device=dev, dtype=torch.bfloat16)
    kg = torch.randn(1, s_img + s_txt, Hl, D, device=dev, dtype=torch.bfloat16)
    vg = torch.randn_like(kg)
    for _ in range(3):
        kernels.attn_fwd([qg], [kg], [vg])
    ms_compute = timed(lambda: kernels.attn_fwd([qg], [kg], [vg]), args.steps)
    heap.check()
    if rank == 0:
        flops = 4.0 * s_q * (s_img + s_txt) * Hl * D
        print(json.dumps({"usp_case": name, "n_gpus": world, "ulysses": U, "ring": R, "ms_per_layer": ms_layer,
                          "ms_attention_only": ms_compute, "tflops_per_gpu": flops / (ms_layer * 1e-3) / 1e12,
                          "exposed_non_compute_frac": max(0.0, 1 - ms_compute / ms_layer)}), flush=True)
    dist.destroy_process_group()


def run_trace(args):
    """The serving-trace configuration on N GPUs: SD3-medium-shaped model, seeded Poisson arrivals at 2
    requests/s, four resolutions, text length 77..333, 20 steps per request, PipeFusion with 4 patches and one
    warm-up step, the plan (PipeFusion degree x Ulysses degree) taken from a fixed table per resolution and every
    change of plan made through the worker plan API with parameter-slice migration. Prints mean / p95 request
    latency and the share of requests within 5x their single-GPU latency. `--trace-requests` shortens the
    2000-request trace (the line says so)."""
    import torch.distributed as dist
    import hetu_dit_b200.model_executor.models.shaped_dit as M
    from hetu_dit_b200 import _C, kernels
    from hetu_dit_b200.core.distributed.runtime_state import ModelGeometry
    from hetu_dit_b200.model_executor.pipelines.pipeline_sd3_shaped import SD3ShapedPipeline
    from hetu_dit_b200.serving.trace_driver import TraceDriver, make_trace
    from hetu_dit_b200.worker.worker import Worker

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    _C.lib()
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def exchange(obj):
        if world == 1:
            return [obj]
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    def reduce_max(x):
        if world == 1:
            return float(x)
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    shape = M.SD3_MEDIUM
    # the CPU master copy every slice is cut from: built on the GPU (seeded), then moved to host memory
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = M.ShapedDiT(shape)
    torch.set_default_dtype(torch.float32)
    model.init_weights(seed=0, std=0.02)
    cpu_master = model.cpu()
    del model
    torch.cuda.empty_cache()
    worker = Worker(rank, world, local_rank=local_rank, exchange=exchange, heap_bytes=1 << 30, arena_bytes=6 << 30)
    worker.init_static_env()
    worker.init_instance_model(cpu_master, ModelGeometry(shape.heads, shape.head_dim),
                               lambda t: SD3ShapedPipeline(t, guidance_scale=5.0))
    driver = TraceDriver(worker, reduce_max, shape.text_dim, shape.pooled_dim)
    n_req = args.trace_requests
    trace = make_trace(2000, rate_per_s=2.0, seed=0, steps=20)[:n_req]
    kernels.reset_counters()
    t0 = time.perf_counter()
    with ClockSampler(local_rank) as clk:
        res = driver.run(trace)
    wall = time.perf_counter() - t0
    status = _C.device_status(local_rank, clear=True)
    if status[0] != 0:
        raise SystemExit(f"device-side wait timed out during the trace: {status}")
    if rank == 0:
        line = {"metric": "trace_request_latency_p95", "value": res["p95_s"], "unit": "s", "n_gpus": world,
                "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic",
                "config": {"workload": "SD3-medium-shaped serving trace: Poisson arrivals 2 req/s (seed 0), 20 steps, "
                                       "resolutions 512/768/1024/1536 squared, text 77..333 tokens, CFG batch 2, "
                                       "PipeFusion 4 patches, 1 warm-up step, FIFO admission (a request occupies "
                                       "pp x sp GPUs; requests on disjoint GPUs overlap), plan per resolution "
                                       "from a fixed table, plan switches through the worker API",
                           "requests": n_req, "requests_in_full_trace": 2000,
                           "arrivals": "virtual clock; service times measured on the GPUs one request at a time "
                                       "(max over ranks)",
                           "slo": "latency <= 5 x single-GPU latency of the same resolution"},
                "trace": res, "wall_s": wall, "gpu_launches": kernels.launch_count(), "clocks": clk.summary()}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="flux", choices=sorted(CONFIGS) + ["trace"],
                    help="which benchmark configuration to run (default: the Flux.1-dev-shaped step); `trace` is "
                         "the serving trace of the SD3-medium-shaped model")
    ap.add_argument("--trace-requests", type=int, default=200,
                    help="--config trace: how many of the 2000 requests of the trace to run")
    ap.add_argument("--no-parity-check", action="store_true",
                    help="skip the tiny-model parity check that precedes the timed region")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a captured CUDA graph")
    ap.add_argument("--replicated-text", action="store_true",
                    help="N > 1: keep the whole text stream on every rank (the reference's layout) instead of "
                         "sharding it with the image tokens")
    ap.add_argument("--profile-one-step", action="store_true",
                    help="wrap one extra eager step in cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--kernel-case", default="",
                    help="one kernel instead of the step: attn:<batch>, attn64:<batch>, attnheads:<heads> (attnheads1: no KV split), "
                         "copy:<MiB>, normrope:<batch>, lnmod:<batch>, gate:<batch>, "
                         "linear:<rows>:<n>:<k>:<tail>[:<tile_m>x<tile_n>], linearlib:<rows>:<n>:<k>:<tail>, "
                         "usp:<flux|cogvideox|hunyuan>")
    args = ap.parse_args()
    if args.kernel_case.startswith("usp:"):
        run_usp_case(args)
    elif args.kernel_case:
        run_kernel_case(args)
    elif args.config == "trace":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the serving trace has no CPU arm: the reference's "
                              "scheduler and HTTP engine are outside the denoising hot path"}), flush=True)
        else:
            run_trace(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()

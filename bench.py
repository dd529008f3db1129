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

S_IMG, S_TXT, GRID = 4096, 512, (64, 64)
METRIC, UNIT = "denoise_step_tokens_per_s", "tokens/s"


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


def _inputs(shape, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return dict(latent=torch.randn(1, S_IMG, shape.token_in, generator=gen).bfloat16(),
                text=torch.randn(1, S_TXT, shape.text_dim, generator=gen).bfloat16(),
                pooled=torch.randn(1, shape.pooled_dim, generator=gen).bfloat16(),
                t=torch.tensor([1.0]), g=torch.tensor([3.5]))


# ------------------------------------------------------------------------------------- CPU arm
def cpu_step_sample(threads, blocks=(1, 1)):
    """Times the reference's CPU path on a bounded sample of the workload: `blocks` = (double, single)
    blocks of the Flux-shaped model at full sequence length, fp32, F.scaled_dot_product_attention.
    Returns (seconds for a whole 19+38-block step, extrapolated; description)."""
    from hetu_dit_b200.model_executor.models.shaped_dit import FLUX_DEV, JointBlock, SingleBlock, rope_tables
    from oracle import shaped_dit as osd
    torch.set_num_threads(threads)
    shape = FLUX_DEV
    gen = torch.Generator().manual_seed(0)
    d = shape.hidden

    def weights(mod, prefix):
        return {prefix + "." + k: torch.randn(v.shape, generator=gen) * (0.02 if v.dim() > 1 else 0.0) + (
            1.0 if (v.dim() == 1 and not k.endswith("bias")) else 0.0) for k, v in mod.state_dict().items()}

    with torch.device("meta"):
        jb, sb = JointBlock(shape), SingleBlock(shape)
    sd = {}
    sd.update(weights(jb, "j"))
    sd.update(weights(sb, "s"))
    hidden = torch.randn(1, S_IMG, d, generator=gen)
    context = torch.randn(1, S_TXT, d, generator=gen)
    temb = torch.randn(1, d, generator=gen)
    ids = torch.zeros(S_TXT + S_IMG, 3)
    yy, xx = torch.meshgrid(torch.arange(GRID[0]), torch.arange(GRID[1]), indexing="ij")
    ids[S_TXT:, 1], ids[S_TXT:, 2] = yy.flatten(), xx.flatten()
    rope = rope_tables(ids, shape.rope_axes)
    with torch.no_grad():
        t0 = time.perf_counter()
        for _ in range(blocks[0]):
            osd.joint_block(sd, "j", hidden, context, temb, rope, shape.heads, shape.head_dim, "front")
        t1 = time.perf_counter()
        x = torch.cat([context, hidden], 1)
        for _ in range(blocks[1]):
            osd.single_block(sd, "s", x, temb, rope, shape.heads, shape.head_dim)
        t2 = time.perf_counter()
    per_double = (t1 - t0) / max(blocks[0], 1)
    per_single = (t2 - t1) / max(blocks[1], 1)
    total = per_double * shape.n_double + per_single * shape.n_single
    return total, (f"{blocks[0]} double + {blocks[1]} single block(s) of the Flux-shaped step at full length "
                   f"({S_IMG}+{S_TXT} tokens, fp32 SDPA path), extrapolated to 19+38 blocks")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    for _ in range(max(args.warmup, 0) and 1):
        cpu_step_sample(threads, (1, 0))
    times = []
    desc = ""
    for _ in range(max(1, min(args.steps, 3))):
        t, desc = cpu_step_sample(threads, (1, 1))
        times.append(t)
    times.sort()
    step_s = times[len(times) // 2]
    value = (S_IMG + S_TXT) / step_s
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "flux.1-dev-shaped denoise step, 4096 image + 512 text tokens, batch 1",
                   "parallelism": "cpu"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------- GPU arm
def run_gpu(args):
    import torch.distributed as dist
    from hetu_dit_b200 import _C, kernels
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.peer import PeerHeap
    from hetu_dit_b200.model_executor.models.shaped_dit import FLUX_DEV, ShapedDiT

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
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

        heap = PeerHeap(1 << 30, rank, world, dev, gather)
    ps.init_distributed_environment(rank, world, heap)
    ps.initialize_model_parallel(sequence_parallel_degree=world, ulysses_degree=world, ring_degree=1)

    shape = FLUX_DEV
    # build the 11.9 B-parameter model directly on the device in bf16 (no 48 GB fp32 host copy per rank)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = ShapedDiT(shape)
    torch.set_default_dtype(torch.float32)
    model.init_weights(seed=0, std=0.02)
    model.register_cache()
    model.shard_text = not args.replicated_text
    host = {k: v.pin_memory() for k, v in _inputs(shape).items()}
    s_loc = S_IMG // world
    rows_loc = GRID[0] // world
    tok0 = rank * s_loc

    def shard(latent):
        return latent[:, tok0:tok0 + s_loc]

    resident = {k: v.to(dev) for k, v in host.items()}

    def step(inp):
        return model(shard(inp["latent"]), inp["text"], inp["pooled"], inp["t"], inp["g"], grid=(rows_loc, GRID[1]),
                     token_offset=tok0, full_grid=GRID)

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
        graph, out_static = None, None
        if not args.no_graph:
            try:
                side = torch.cuda.Stream(device=dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    step(resident)
                torch.cuda.current_stream(dev).wait_stream(side)
                barrier()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    out_static = step(resident)
                barrier()
            except Exception as e:  # capture is an optimisation; the eager path stays valid
                print(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); timing eager launches",
                      file=sys.stderr)
                graph = None
        run_step = graph.replay if graph is not None else (lambda: step(resident))
        for _ in range(2):
            run_step()
        with ClockSampler(local_rank) as clk:
            ms_step = timed(run_step, args.steps)

        # (3) end to end: pinned host inputs -> device, step, result -> host, every step
        out_host = torch.empty((1, s_loc, shape.token_in), dtype=torch.bfloat16).pin_memory()

        def e2e_step():
            if graph is not None:
                for k, v in host.items():
                    resident[k].copy_(v, non_blocking=True)
                graph.replay()
                out_host.copy_(out_static, non_blocking=True)
            else:
                inp = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
                out_host.copy_(step(inp), non_blocking=True)

        for _ in range(2):
            e2e_step()
        ms_e2e = timed(e2e_step, args.steps)
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
    # dominant kernel of this repo: the attention kernel (one launch per block, 57 per step)
    heads_loc = shape.heads // world
    s_q_gathered = tokens  # replicated text queries are attended once per head slice, not once per rank
    attn_flops = 4.0 * s_q_gathered * tokens * heads_loc * shape.head_dim
    achieved = attn_flops / (attn_ms["mean_ms"] * 1e-3) / 1e12 if attn_ms["mean_ms"] else None
    # DRAM bytes of one launch at this shape, from the committed ncu summary (single-GPU shape only)
    traffic = None
    prof = os.path.join(ROOT, "profiles", "attn_fwd_kernel_flux_shape.txt")
    if os.path.exists(prof) and world == 1:
        with open(prof) as f:
            for ln in f:
                if ln.startswith("dram_bytes_per_launch:"):
                    traffic = int(ln.split(":")[1])
    line = {
        "metric": METRIC, "value": tokens / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "flux.1-dev-shaped denoise step, 4096 image + 512 text tokens, batch 1, "
                               "19 double + 38 single blocks, hidden 3072, 24x128 heads",
                   "parallelism": f"ulysses{world}" if world > 1 else "single",
                   "text_stream": "n/a" if world == 1 else ("replicated on every rank (reference layout)"
                                                            if args.replicated_text else "sharded over the ranks"),
                   "l2": "weights (23.8 GB) and activations exceed the 126 MB L2; no explicit flush",
                   "cuda_graph": graph is not None, "ms_per_step_eager_launches": ms_eager,
                   "step_flops": model.flops_per_step(S_IMG, S_TXT),
                   "step_tflops_achieved": model.flops_per_step(S_IMG, S_TXT) / (ms_step * 1e-3) / 1e12 / world},
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clk.summary(),
        "roofline": {"kernel": "attn_fwd_kernel<128,bf16>", "bound": "tensor", "achieved": achieved, "peak": peak_tf,
                     "unit": "TFLOP/s", "frac": (achieved / peak_tf) if achieved else None, "traffic": traffic,
                     "peak_source": f"bf16_tflops_sustained, {peak_kind}", "launches_timed": attn_ms["count"],
                     "flops_per_launch": attn_flops},
    }
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        total_s, desc = cpu_step_sample(threads, (1, 1))
        line["cpu_baseline"] = {"value": tokens / total_s, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": desc}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    """Operator-level timing of one USP attention layer at a BASELINE config's shape under torchrun:
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a captured CUDA graph")
    ap.add_argument("--replicated-text", action="store_true",
                    help="N > 1: keep the whole text stream on every rank (the reference's layout) instead of "
                         "sharding it with the image tokens")
    ap.add_argument("--profile-one-step", action="store_true",
                    help="wrap one extra eager step in cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--kernel-case", default="",
                    help="one kernel instead of the step: attn:<batch>, attnheads:<heads> (attnheads1: no KV split), "
                         "copy:<MiB>, normrope:<batch>, lnmod:<batch>, gate:<batch>, usp:<flux|cogvideox|hunyuan>")
    args = ap.parse_args()
    if args.kernel_case.startswith("usp:"):
        run_usp_case(args)
    elif args.kernel_case:
        run_kernel_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()

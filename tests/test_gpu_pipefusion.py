"""PipeFusion denoising of a tiny SD3-shaped model against the CPU oracle: one GPU (patches + stale K/V on a
single stage) and two GPUs through the worker plan API (stage hand-off, plan switch, slice migration)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny():
    from hetu_dit_b200.model_executor.models.shaped_dit import DiTShape, ShapedDiT
    shape = DiTShape("sd3-tiny", 4, 0, 256, 4, 64, 64, 128, 96, False, None, False)
    model = ShapedDiT(shape).init_weights(seed=11, std=0.05).bfloat16()
    gen = torch.Generator().manual_seed(12)
    lat = torch.randn(1, 32 * 16, 64, generator=gen).bfloat16()       # 256 x 128 image -> 32 x 16 latent rows / cols... tokens
    prompt = torch.randn(2, 19, 128, generator=gen).bfloat16()
    pooled = torch.randn(2, 96, generator=gen).bfloat16()
    return shape, model, lat, prompt, pooled


def test_single_stage_patches_with_stale_kv():
    from hetu_dit_b200 import _C
    from hetu_dit_b200.config import EngineConfig
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.runtime_state import ModelGeometry, initialize_runtime_state, reset_runtime_state
    from hetu_dit_b200.core.resource_manager.cache_manager import reset_cache_manager
    from hetu_dit_b200.model_executor.pipelines.pipeline_sd3_shaped import SD3ShapedPipeline
    from oracle import attention as oa
    from oracle import pipefusion as opf
    shape, model, lat, prompt, pooled = _tiny()
    dev = torch.device("cuda:0")
    ps.destroy_model_parallel()
    reset_cache_manager()
    cfg = EngineConfig()
    cfg.parallel_config.pp_config.num_pipeline_patch = 4
    cfg.runtime_config.warmup_steps = 1
    rt = initialize_runtime_state(ModelGeometry(4, 64), cfg)
    rt.set_input_parameters(height=512, width=256, batch_size=1, num_inference_steps=4)  # 64 x 32 latent -> 32 x 16 tokens
    assert rt.pp_patches_token_num == [128] * 4
    gpu_model = model.to(dev)
    gpu_model.register_cache()
    pipe = SD3ShapedPipeline(gpu_model, guidance_scale=4.0, grid=(32, 16))
    got = pipe.diffusion_stage(lat.to(dev), prompt.to(dev), pooled.to(dev), 4)
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0
    sd = {k: v.float().cpu() for k, v in gpu_model.state_dict().items()}
    want = opf.denoise(sd, shape, lat, prompt, pooled, 4, 4.0, [128] * 4, 1, (32, 16))
    cos, rel = oa.cosine_and_max_rel(got.cpu(), want)
    _close(cos, rel)
    # the stale K/V matters: the result is closer to the patched oracle than to the un-patched one
    full = opf.denoise(sd, shape, lat, prompt, pooled, 4, 4.0, [512], 1, (32, 16))
    g = got.cpu().float()
    assert (g - want).abs().mean() < (g - full).abs().mean()
    reset_runtime_state()
    reset_cache_manager()


def _tiny_flux():
    from hetu_dit_b200.model_executor.models.shaped_dit import DiTShape, ShapedDiT
    shape = DiTShape("flux-tiny", 2, 3, 256, 4, 64, 64, 128, 96, True, (16, 24, 24), True)
    model = ShapedDiT(shape).init_weights(seed=21, std=0.05).bfloat16()
    gen = torch.Generator().manual_seed(22)
    lat = torch.randn(1, 32 * 16, 64, generator=gen).bfloat16()
    prompt = torch.randn(1, 24, 128, generator=gen).bfloat16()
    pooled = torch.randn(1, 96, generator=gen).bfloat16()
    return shape, model, lat, prompt, pooled


def test_flux_single_stage_patches_with_stale_kv():
    """Flux-shaped PipeFusion on one stage: rotary rows per patch, stale K/V in double and single blocks."""
    from hetu_dit_b200 import _C
    from hetu_dit_b200.config import EngineConfig
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.runtime_state import ModelGeometry, initialize_runtime_state, reset_runtime_state
    from hetu_dit_b200.core.resource_manager.cache_manager import reset_cache_manager
    from hetu_dit_b200.model_executor.pipelines.pipeline_flux_shaped import FluxShapedPipeline
    from oracle import attention as oa
    from oracle import pipefusion as opf
    shape, model, lat, prompt, pooled = _tiny_flux()
    dev = torch.device("cuda:0")
    ps.destroy_model_parallel()
    reset_cache_manager()
    cfg = EngineConfig()
    cfg.parallel_config.pp_config.num_pipeline_patch = 4
    cfg.runtime_config.warmup_steps = 1
    rt = initialize_runtime_state(ModelGeometry(4, 64), cfg)
    rt.set_input_parameters(height=512, width=256, batch_size=1, num_inference_steps=4)
    assert rt.pp_patches_token_num == [128] * 4
    gpu_model = model.to(dev)
    gpu_model.register_cache()
    pipe = FluxShapedPipeline(gpu_model, guidance_scale=3.5, grid=(32, 16))
    got = pipe.diffusion_stage(lat.to(dev), prompt.to(dev), pooled.to(dev), 4)
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0
    sd = {k: v.float().cpu() for k, v in gpu_model.state_dict().items()}
    want = opf.denoise_flux(sd, shape, lat, prompt, pooled, 4, 3.5, [128] * 4, 1, (32, 16))
    cos, rel = oa.cosine_and_max_rel(got.cpu(), want)
    _close(cos, rel)
    full = opf.denoise_flux(sd, shape, lat, prompt, pooled, 4, 3.5, [512], 1, (32, 16))
    g = got.cpu().float()
    assert (g - want).abs().mean() < (g - full).abs().mean()
    reset_runtime_state()
    reset_cache_manager()


# Final latents after 4 to 8 denoising steps with guidance against the fp32 oracle: cosine and max |a - b| / max |b|.
# The per-step bound (0.9999, 2e-2) is held by the model-level tests; several 16-bit steps compound, measured here
# 0.99990 to 0.999995 and 0.006 to 0.015.
COS_MIN, MAX_REL = 0.9998, 2e-2


def _close(cos, rel, tag=""):
    print(f"parity {tag}: cosine {cos:.6f} max_rel {rel:.4f}")
    assert cos >= COS_MIN and rel <= MAX_REL, (tag, cos, rel)


def call(worker, method, *args, **kwargs):
    """By-name call with the reference's positional / keyword arguments, as its executor makes it."""
    from hetu_dit_b200.worker.worker import run_worker_method
    return run_worker_method(worker, method, *args, **kwargs)


def diffuse(worker, cfg, lat, prompt, pooled, steps, both=False):
    """execute_diffusion_stage(encode_stage_results, engine_config, input_config, model_class, task_id): returns
    the latents on the worker that owns the result. Under sequence parallelism without PipeFusion the reference
    returns them on the first diffusion rank only; `both` asks every rank in turn so that each can check."""
    from hetu_dit_b200.config import InputConfig
    enc = {"prompt_embeds": prompt, "pooled_prompt_embeds": pooled, "latents": lat}
    inp = InputConfig(height=512, width=256, num_inference_steps=steps)
    if both:
        cfg.diffusion_stage_ranks = [worker.rank]
    results, latents = call(worker, "execute_diffusion_stage", enc, cfg, inp, None, task_id="t0")
    assert results["after"] >= results["before"] and results["inner_results"]["running_task"] == "t0"
    return latents


def _flux_worker_case(rank, world, port, errq):
    """Two PipeFusion stages of the Flux-shaped model through the worker plan API: stage 0 holds the double
    blocks, stage 1 the single blocks, which re-use the text stream that arrives with patch 0."""
    import traceback
    try:
        import os
        import torch.distributed as dist
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from hetu_dit_b200.config import EngineConfig
        from hetu_dit_b200.core.distributed.runtime_state import ModelGeometry
        from hetu_dit_b200.model_executor.pipelines.pipeline_flux_shaped import FluxShapedPipeline
        from hetu_dit_b200.worker.worker import Worker
        from oracle import attention as oa
        from oracle import pipefusion as opf

        def exchange(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out

        shape, model, lat, prompt, pooled = _tiny_flux()
        sd = {k: v.float() for k, v in model.state_dict().items()}
        w = Worker(rank, world, exchange=exchange, heap_bytes=128 << 20, arena_bytes=64 << 20)
        w.init_static_env()
        w.init_instance_model(model, ModelGeometry(4, 64), lambda t: FluxShapedPipeline(t, guidance_scale=3.5, grid=(32, 16)))
        dev = w.device
        cfg = EngineConfig()
        cfg.parallel_config.pp_config.pp_degree = 2
        cfg.parallel_config.pp_config.num_pipeline_patch = 4
        cfg.runtime_config.warmup_steps = 1
        call(w, "switch_parallel_env", 2, [0, 1], cfg)
        call(w, "hotspa_model", cfg)
        assert sorted(w.cache.cache) == ([0, 1] if rank == 0 else [2, 3, 4])
        out = diffuse(w, cfg, lat, prompt, pooled, 4)
        if rank == 1:
            want = opf.denoise_flux(sd, shape, lat, prompt, pooled, 4, 3.5, [128] * 4, 1, (32, 16), stage_starts=(0, 2))
            cos, rel = oa.cosine_and_max_rel(out.cpu(), want)
            _close(cos, rel, "flux pp2")
        else:
            assert out is None
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def test_flux_two_stage_pipeline_two_gpus():
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    try:
        mp.spawn(_flux_worker_case, args=(2, 29813, errq), nprocs=2, join=True)
    except Exception:
        msgs = []
        while not errq.empty():
            msgs.append(errq.get())
        pytest.fail("\n".join(msgs) or "worker failed")


def _worker_case(rank, world, port, errq):
    import traceback
    try:
        import os
        import torch.distributed as dist
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from hetu_dit_b200.config import EngineConfig
        from hetu_dit_b200.core.distributed.runtime_state import ModelGeometry
        from hetu_dit_b200.model_executor.pipelines.pipeline_sd3_shaped import SD3ShapedPipeline
        from hetu_dit_b200.worker.worker import Worker
        from oracle import attention as oa
        from oracle import pipefusion as opf

        def exchange(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out

        shape, model, lat, prompt, pooled = _tiny()
        sd = {k: v.float() for k, v in model.state_dict().items()}
        w = Worker(rank, world, exchange=exchange, heap_bytes=128 << 20, arena_bytes=64 << 20)
        w.init_static_env()
        w.init_instance_model(model, ModelGeometry(4, 64), lambda t: SD3ShapedPipeline(t, guidance_scale=4.0, grid=(32, 16)))
        dev = w.device

        # plan A: PipeFusion over both GPUs, 4 patches, 1 warm-up step; all weights come from the CPU master
        cfg = EngineConfig()
        cfg.parallel_config.pp_config.pp_degree = 2
        cfg.parallel_config.pp_config.num_pipeline_patch = 4
        cfg.runtime_config.warmup_steps = 1
        call(w, "switch_parallel_env", 2, [0, 1], cfg)
        stats = call(w, "hotspa_model", cfg)
        assert stats["from_peers"] == 0 and sorted(w.cache.cache) == ([0, 1] if rank == 0 else [2, 3])
        out = diffuse(w, cfg, lat, prompt, pooled, 4)
        want = opf.denoise(sd, shape, lat, prompt, pooled, 4, 4.0, [128] * 4, 1, (32, 16))
        if rank == 1:
            cos, rel = oa.cosine_and_max_rel(out.cpu(), want)
            _close(cos, rel, "pp2")
        else:
            assert out is None
        # Eight steps: steps 2..5 of the patch pipeline are captured per patch and replayed from CUDA graphs. The
        # result must be the eager one bit for bit (same kernels, same order), twice in a row (the second request
        # captures anew over the same inbox and stale-KV buffers), and match the oracle.
        want8 = opf.denoise(sd, shape, lat, prompt, pooled, 8, 4.0, [128] * 4, 1, (32, 16))
        outs8 = []
        for graph in (False, True, True):
            w.pipeline.use_cuda_graph = graph
            outs8.append(diffuse(w, cfg, lat, prompt, pooled, 8))
        w.pipeline.use_cuda_graph = True
        if rank == 1:
            cos, rel = oa.cosine_and_max_rel(outs8[0].cpu(), want8)
            _close(cos, rel, "pp2 eight steps")
            assert torch.equal(outs8[0], outs8[1]) and torch.equal(outs8[1], outs8[2]), "graph replay differs from eager"

        # plan B: two independent single-GPU plans; each rank pulls the blocks it lacks from its peer
        cfg1 = EngineConfig()
        cfg1.parallel_config.pp_config.num_pipeline_patch = 4
        cfg1.runtime_config.warmup_steps = 1
        call(w, "switch_parallel_env", 1, [rank], engine_config=cfg1)
        stats = call(w, "hotspa_model", engine_config=cfg1)
        assert stats["from_peers"] > 0 and stats["from_cpu"] == 0, stats
        assert sorted(w.cache.cache) == [0, 1, 2, 3]
        for i, blk in enumerate(w.transformer.transformer_blocks):
            ref = model.transformer_blocks[i].state_dict()
            for k, v in blk.state_dict().items():
                assert torch.equal(v.cpu(), ref[k]), (i, k)
        out = diffuse(w, cfg1, lat, prompt, pooled, 4)
        cos, rel = oa.cosine_and_max_rel(out.cpu(), want)
        _close(cos, rel, "solo")
        state = call(w, "get_worker_state")
        assert state["running_task"] is None and state["running_stage"] is None and state["rank"] == rank

        # plan C: Ulysses degree 2 over both GPUs, 4 patches of which every rank holds one half; nothing to
        # migrate (both ranks hold all blocks). The whole latents come back on both ranks (end-of-denoise
        # gather). The oracle models the order in which the reference keeps the stale K/V under Ulysses.
        cfg2 = EngineConfig()
        cfg2.parallel_config.sp_config.ulysses_degree = 2
        cfg2.parallel_config.pp_config.num_pipeline_patch = 4
        cfg2.runtime_config.warmup_steps = 1
        call(w, "switch_parallel_env", 2, [0, 1], cfg2)
        stats = call(w, "hotspa_model", cfg2)
        assert stats["from_peers"] == 0 and stats["from_cpu"] == 0, stats
        from hetu_dit_b200.core.distributed.runtime_state import get_runtime_state
        out = diffuse(w, cfg2, lat, prompt, pooled, 4, both=True)
        assert get_runtime_state().pp_patches_token_num == [64] * 4
        want_sp = opf.denoise(sd, shape, lat, prompt, pooled, 4, 4.0, [128] * 4, 1, (32, 16), ulysses=2)
        cos, rel = oa.cosine_and_max_rel(out.cpu(), want_sp)
        _close(cos, rel, "ulysses2")
        # and without patches the sequence-parallel result is the plain one
        cfg3 = EngineConfig()
        cfg3.parallel_config.sp_config.ulysses_degree = 2
        call(w, "switch_parallel_env", 2, [0, 1], cfg3)
        call(w, "hotspa_model", cfg3)
        out = diffuse(w, cfg3, lat, prompt, pooled, 2, both=True)
        want_full = opf.denoise(sd, shape, lat, prompt, pooled, 2, 4.0, [512], 0, (32, 16))
        cos, rel = oa.cosine_and_max_rel(out.cpu(), want_full)
        _close(cos, rel, "ulysses2 unpatched")

        # plans D and E: a tensor-parallel re-slice in which each rank pulls from the slice its peer is replacing
        # at the same time. D (2 pipeline stages, at most 2 cached blocks) leaves blocks 0-1 whole on rank 0 and
        # 2-3 whole on rank 1. E (tensor parallel 2) makes rank 0 cut its blocks down to the first half of the
        # rows / columns -- releasing the whole tensors -- while rank 1 pulls the second half of those very
        # tensors, and vice versa. The released memory must not be re-used before the peer's pull has run.
        w.cache.max_num_cached_blocks = 2
        cfg4 = EngineConfig()
        cfg4.parallel_config.pp_config.pp_degree = 2
        call(w, "switch_parallel_env", 2, [0, 1], cfg4)
        call(w, "hotspa_model", cfg4)
        assert sorted(w.cache.cache) == ([0, 1] if rank == 0 else [2, 3])
        w.cache.max_num_cached_blocks = 1 << 30
        cfg5 = EngineConfig()
        cfg5.parallel_config.tp_config.tp_degree = 2
        call(w, "switch_parallel_env", 2, [0, 1], cfg5)
        stats = call(w, "hotspa_model", cfg5)
        assert stats["from_peers"] > 0 and stats["from_cpu"] == 0, stats
        tp = (0.0, 0.5) if rank == 0 else (0.5, 1.0)
        for i, blk in enumerate(w.transformer.transformer_blocks):
            assert w.cache.cache[i][1] == tp
            for name, sub in blk.named_modules():
                if not isinstance(sub, torch.nn.Linear):
                    continue
                ref = dict(model.transformer_blocks[i].named_modules())[name]
                kind = w.cache.choose_tp_split_type(name)
                if kind is None:
                    assert torch.equal(sub.weight.cpu(), ref.weight), (i, name)
                    continue
                dim = 0 if kind == "row" else 1
                lo, hi = w.cache.range_to_indices(tp, ref.weight.shape[dim])
                want_w = ref.weight[lo:hi] if dim == 0 else ref.weight[:, lo:hi]
                assert torch.equal(sub.weight.cpu(), want_w), (i, name, kind)
                if kind == "row" and ref.bias is not None:
                    assert torch.equal(sub.bias.cpu(), ref.bias[lo:hi]), (i, name, "bias")
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def test_worker_plan_switch_and_migration_two_gpus():
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    try:
        mp.spawn(_worker_case, args=(2, 29811, errq), nprocs=2, join=True)
    except Exception:
        msgs = []
        while not errq.empty():
            msgs.append(errq.get())
        pytest.fail("\n".join(msgs) or "worker failed")


def _pp_sp_case(rank, world, port, errq):
    """PipeFusion (2 stages, 4 patches, 1 warm-up step) combined with Ulysses degree 2 on four GPUs through the
    worker plan API -- the combination the serving trace uses -- then a switch to Ulysses 4 without PipeFusion."""
    import traceback
    try:
        import os
        import torch.distributed as dist
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from hetu_dit_b200.config import EngineConfig
        from hetu_dit_b200.core.distributed import parallel_state as ps
        from hetu_dit_b200.core.distributed.runtime_state import ModelGeometry
        from hetu_dit_b200.model_executor.pipelines.pipeline_sd3_shaped import SD3ShapedPipeline
        from hetu_dit_b200.worker.worker import Worker
        from oracle import attention as oa
        from oracle import pipefusion as opf

        def exchange(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out

        shape, model, lat, prompt, pooled = _tiny()
        sd = {k: v.float() for k, v in model.state_dict().items()}
        w = Worker(rank, world, exchange=exchange, heap_bytes=128 << 20, arena_bytes=64 << 20)
        w.init_static_env()
        w.init_instance_model(model, ModelGeometry(4, 64), lambda t: SD3ShapedPipeline(t, guidance_scale=4.0))
        cfg = EngineConfig()
        cfg.parallel_config.pp_config.pp_degree = 2
        cfg.parallel_config.pp_config.num_pipeline_patch = 4
        cfg.parallel_config.sp_config.ulysses_degree = 2
        cfg.runtime_config.warmup_steps = 1
        call(w, "switch_parallel_env", 4, [0, 1, 2, 3], cfg)
        call(w, "hotspa_model", cfg)
        # rank order is tp-sp-pp: ranks 0, 1 are stage 0 (the two Ulysses ranks), ranks 2, 3 stage 1
        assert ps.get_pipeline_parallel_rank() == rank // 2 and ps.get_ulysses_parallel_rank() == rank % 2
        assert sorted(w.cache.cache) == ([0, 1] if rank < 2 else [2, 3])
        out = diffuse(w, cfg, lat, prompt, pooled, 4)
        want = opf.denoise(sd, shape, lat, prompt, pooled, 4, 4.0, [128] * 4, 1, (32, 16), ulysses=2)
        if rank >= 2:
            cos, rel = oa.cosine_and_max_rel(out.cpu(), want)
            _close(cos, rel, "pp2 x ulysses2")
        else:
            assert out is None
        cfg2 = EngineConfig()
        cfg2.parallel_config.sp_config.ulysses_degree = 4
        call(w, "switch_parallel_env", 4, [0, 1, 2, 3], cfg2)
        stats = call(w, "hotspa_model", cfg2)
        assert stats["from_cpu"] == 0 and sorted(w.cache.cache) == [0, 1, 2, 3], stats
        out = diffuse(w, cfg2, lat, prompt, pooled, 2, both=True)
        want_full = opf.denoise(sd, shape, lat, prompt, pooled, 2, 4.0, [512], 0, (32, 16))
        cos, rel = oa.cosine_and_max_rel(out.cpu(), want_full)
        _close(cos, rel, "ulysses4")
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def test_worker_pipefusion_with_sequence_parallelism_four_gpus():
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    try:
        mp.spawn(_pp_sp_case, args=(4, 29815, errq), nprocs=4, join=True)
    except Exception:
        msgs = []
        while not errq.empty():
            msgs.append(errq.get())
        pytest.fail("\n".join(msgs) or "worker failed")

"""Worker body of the multi-GPU parity tests: one process per GPU, ranks exchange IPC handles over gloo."""
import json
import os
import sys
import traceback

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

COS_MIN, MAX_REL = 0.9999, 2e-2


def _setup(rank, world, port, heap_bytes=256 << 20):
    import torch.distributed as dist
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.peer import PeerHeap
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)

    def gather(b):
        out = [None] * world
        dist.all_gather_object(out, b)
        return out

    heap = PeerHeap(heap_bytes, rank, world, dev, gather)
    ps.init_distributed_environment(rank, world, heap)
    return dist, ps, heap, dev


def _close(got, want, what):
    from oracle import attention as oa
    cos, rel = oa.cosine_and_max_rel(got.float().cpu(), want)
    assert cos >= COS_MIN and rel <= MAX_REL, f"{what}: cosine {cos} max_rel {rel}"


def usp_case(rank, world, port, fixture, errq):
    """Runs one tests/golden/usp_*.npz case with the product operators and compares with the recorded outputs."""
    try:
        dist, ps, heap, dev = _setup(rank, world, port)
        from hetu_dit_b200.core import parallel as P
        from hetu_dit_b200.core.distributed.runtime_state import ModelGeometry, initialize_runtime_state, reset_runtime_state
        from hetu_dit_b200.core.resource_manager.cache_manager import get_cache_manager
        from hetu_dit_b200.config import EngineConfig
        with np.load(fixture) as f:
            d = {k: f[k] for k in f.files}
        spec = json.loads(str(d.pop("spec")))
        assert spec["world"] == world
        t = {k: torch.from_numpy(v) for k, v in d.items()}
        U, R, S = spec["ulysses"], spec["ring"], spec["s_loc"]
        ps.initialize_model_parallel(sequence_parallel_degree=U * R, ulysses_degree=U, ring_degree=R)
        bf = torch.bfloat16

        def loc(x, n):
            return x[:, rank * n:(rank + 1) * n].to(dev, bf).contiguous()

        layer = getattr(P, spec["cls"])()
        kw = {}
        if spec["joint_strategy"] != "none":
            kw = dict(joint_tensor_query=t["jq"].to(dev, bf), joint_tensor_key=t["jk"].to(dev, bf),
                      joint_tensor_value=t["jv"].to(dev, bf), joint_strategy=spec["joint_strategy"])
        if not spec["kv_cache"]:
            for _ in range(2):  # twice: buffers and flags are re-used across layers
                out = layer(None, loc(t["q"], S), loc(t["k"], S), loc(t["v"], S), **kw)
            heap.check()
            _close(out, t[f"out_rank{rank}"], f"rank {rank}")
        else:
            cfg = EngineConfig()
            cfg.parallel_config.sp_config.ulysses_degree, cfg.parallel_config.sp_config.ring_degree = U, R
            cfg.parallel_config.pp_config.num_pipeline_patch = 2
            rt = initialize_runtime_state(ModelGeometry(spec["heads"], spec["head_dim"]), cfg)
            tok = S // 2
            rt.num_pipeline_patch = 2
            rt.pp_patches_token_num = [tok, tok]
            rt.pp_patches_token_start_idx_local = [0, tok, 2 * tok]
            attn_obj = object()
            get_cache_manager().register_cache_entry(attn_obj, "attn", "sequence_parallel_attn_cache")
            rt.set_patched_mode(False)
            out0 = layer(attn_obj, loc(t["q"], S), loc(t["k"], S), loc(t["v"], S), **kw)
            heap.check()
            _close(out0, t[f"out_warmup_rank{rank}"], f"warm-up rank {rank}")
            rt.set_patched_mode(True)
            rt.pipeline_patch_idx = 1
            out1 = layer(attn_obj, loc(t["fresh_q"], tok), loc(t["fresh_k"], tok), loc(t["fresh_v"], tok), **kw)
            heap.check()
            _close(out1, t[f"out_patch1_rank{rank}"], f"patch rank {rank}")
            reset_runtime_state()
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def model_sp_case(rank, world, port, kind, ulysses, errq):
    """One denoise step of a tiny Flux- / SD3-shaped model under sequence parallelism: every rank's band of the
    output against the CPU oracle of the whole model, with the text stream sharded and with the reference's
    replicated text layout."""
    try:
        dist, ps, heap, dev = _setup(rank, world, port)
        from hetu_dit_b200 import _C
        from hetu_dit_b200.model_executor.models.shaped_dit import DiTShape, ShapedDiT
        from oracle import attention as oa
        from oracle import shaped_dit as osd
        ps.initialize_model_parallel(sequence_parallel_degree=world, ulysses_degree=ulysses, ring_degree=world // ulysses)
        if kind == "flux":
            shape = DiTShape("flux-tiny", 2, 3, 512, 4, 128, 64, 256, 96, True, (16, 56, 56), True)
        else:
            shape = DiTShape("sd3-tiny", 3, 0, 256, 4, 64, 64, 256, 128, False, None, False)
        model = ShapedDiT(shape).init_weights(seed=3, std=0.05).bfloat16()
        gh, gw, s_txt = 24, 12, 32
        gen = torch.Generator().manual_seed(21)
        lat = torch.randn(1, gh * gw, shape.token_in, generator=gen).bfloat16()
        txt = torch.randn(1, s_txt, shape.text_dim, generator=gen).bfloat16()
        pooled = torch.randn(1, shape.pooled_dim, generator=gen).bfloat16()
        t, g = torch.tensor([0.7]), torch.tensor([3.5])
        sd = {k: v.float() for k, v in model.state_dict().items()}
        want = osd.denoise_step(sd, shape, lat, txt, pooled, t, g, grid=(gh, gw))
        model = model.to(dev)
        model.register_cache()
        rows = gh // world
        s_loc = rows * gw
        tok0 = rank * s_loc
        outs = {}
        # text stream sharded / replicated (the reference's layout); adaLN vectors computed by every rank / shared
        # out over the ranks (each computes every world-th block's and stores them to its peers)
        for shard_text, shard_mod in ((True, False), (False, False), (True, True), (True, True)):
            model.shard_text = shard_text
            model.shard_modulation_from = 2 if shard_mod else 0
            with torch.no_grad():
                got = model(lat[:, tok0:tok0 + s_loc].to(dev), txt.to(dev), pooled.to(dev), t.to(dev), g.to(dev),
                            grid=(rows, gw), token_offset=tok0, full_grid=(gh, gw))
            torch.cuda.synchronize()
            heap.check()
            assert _C.device_status(rank, clear=True)[0] == 0
            cos, rel = oa.cosine_and_max_rel(got.float().cpu(), want[:, tok0:tok0 + s_loc])
            assert cos >= 0.9999 and rel <= 2e-2, f"rank {rank} shard_text={shard_text}: cosine {cos} max_rel {rel}"
            if (shard_text, shard_mod) in outs:  # the second round re-uses the gathered buffer and the flags
                assert torch.equal(outs[(shard_text, shard_mod)], got), "second sharded-modulation step differs"
            outs[(shard_text, shard_mod)] = got
            ps.get_world_group().barrier()
        # the same vectors, whoever computed them: bit-identical step
        assert torch.equal(outs[(True, False)], outs[(True, True)]), "sharded adaLN vectors changed the result"
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def all_gather_case(rank, world, port, errq):
    """Group all_gather over peer stores: concatenation along a dim and separate tensors, bit-exact, repeated
    with fresh data so that the alternating gathered buffers are exercised."""
    try:
        dist, ps, heap, dev = _setup(rank, world, port)
        ps.initialize_model_parallel(sequence_parallel_degree=world, ulysses_degree=world)
        g = ps.get_sp_group()
        for rnd in range(4):
            gen = torch.Generator().manual_seed(100 + rnd)
            parts = [torch.randn(2, 16, 24, 32, generator=gen).bfloat16() for _ in range(world)]
            mine = parts[rank].to(dev)
            got = g.all_gather(mine, dim=0)
            assert torch.equal(got.cpu(), torch.cat(parts, 0)), f"dim 0 round {rnd}"
            got = g.all_gather(mine, dim=-2)
            assert torch.equal(got.cpu(), torch.cat(parts, 2)), f"dim -2 round {rnd}"
            lst = g.all_gather(mine.transpose(1, 2), separate_tensors=True)
            assert len(lst) == world and all(torch.equal(a.cpu(), b.transpose(1, 2)) for a, b in zip(lst, parts))
            ints = g.all_gather(torch.full((3,), rank * 10 + rnd, dtype=torch.int64, device=dev))
            assert ints.cpu().tolist() == [r * 10 + rnd for r in range(world) for _ in range(3)]
        heap.check()
        solo = ps.get_tp_group()
        x = torch.ones(3, device=dev)
        assert solo.all_gather(x) is x          # single-rank group: the input itself, as in the reference
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def pipefusion_case(rank, world, port, errq):
    """Ring of stages passes patches around twice; payloads must arrive bit-exact and in FIFO order."""
    try:
        dist, ps, heap, dev = _setup(rank, world, port)
        ps.initialize_model_parallel(pipeline_parallel_degree=world)
        pp = ps.get_pp_group()
        pp.set_config(torch.bfloat16)
        gen = torch.Generator().manual_seed(77)
        shapes = [(2, 96, 1536), (2, 96, 1536), (2, 64, 1536), (2, 333, 1536)]
        names = [("latent", 0), ("latent", 1), ("latent", 2), ("encoder_hidden_states", 0)]
        payload = [[torch.randn(s, generator=gen).bfloat16() for s in shapes] for _ in range(3)]  # 3 rounds
        prev_idx = (rank - 1) % world
        for rnd in range(3):
            for (name, idx), src in zip(names, payload[rnd]):
                # every stage sends its own variant so a misrouted message is detected
                pp.pipeline_isend((src + rank).to(dev), name=name, segment_idx=idx)
            for (name, idx) in names:
                pp.add_pipeline_recv_task(idx, name)
            for (name, idx), src in zip(names, payload[rnd]):
                pp.recv_next()
                got = pp.get_pipeline_recv_data(idx=idx, name=name)
                heap.check()
                assert torch.equal(got.cpu(), src + prev_idx), f"rank {rank} round {rnd} {name}[{idx}]"
            ps.get_world_group().barrier()
        heap.check()
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def barrier_timeout_case(rank, world, port, errq):
    """A rank that never joins a barrier: the others' bounded wait runs out and reports the silent peer."""
    try:
        dist, ps, heap, dev = _setup(rank, world, port)
        from hetu_dit_b200 import _C
        ps.initialize_model_parallel(sequence_parallel_degree=world, ulysses_degree=world)
        g = ps.get_world_group()
        g.barrier()
        heap.check()
        if rank != world - 1:
            g.barrier(max_spins=20000)  # the last rank stays away (host-side failure)
            try:
                heap.check()
                raise AssertionError("expected a peer timeout")
            except _C.HditError as e:
                assert e.code == _C.HDIT_ERR_PEER_TIMEOUT and f"detail={world - 1}" in str(e), str(e)
            # the context is still usable afterwards
            x = torch.ones(8, device=dev) * 2
            assert x.sum().item() == 16
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise


def handoff_case(rank, world, port, errq):
    """Stage hand-off of latents to a "decode" rank over the peer heap: bit-exact, repeated (the slot is re-used),
    surviving a plan switch (heap reset) in between, several shapes and dtypes."""
    try:
        dist, ps, heap, dev = _setup(rank, world, port)
        from hetu_dit_b200.core.distributed.handoff import StageHandoff
        ho = StageHandoff(heap, slot_bytes=4 << 20)
        ps.initialize_model_parallel(sequence_parallel_degree=world, ulysses_degree=world)
        decode = world - 1
        shapes = [((1, 16, 64, 64), torch.bfloat16), ((2, 16, 24, 40), torch.float16), ((1, 16, 5, 12, 20), torch.float32)]
        for rnd, (shape, dtype) in enumerate(shapes):
            gen = torch.Generator().manual_seed(500 + rnd)
            want = torch.randn(shape, generator=gen).to(dtype)
            if rank == 0:
                ho.send(decode, want.to(dev))
            if rank == decode:
                got = ho.recv(0)
                assert got.dtype == dtype and tuple(got.shape) == shape and torch.equal(got.cpu(), want), rnd
            heap.check()
            dist.barrier()
            heap.reset()                       # a plan switch drops the activation buffers, not the slots
            heap.alloc((1024,), torch.uint8, name="after_reset")
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(f"rank {rank}:\n{traceback.format_exc()}")
        raise

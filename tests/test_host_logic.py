"""CPU tests of the host-side mirror: bookkeeping against the reference-generated fixtures, library exports,
argument checking, and the multi-rank protocol logic on `gloo` ranks."""
import ctypes
import json
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def book(golden_dir):
    with open(os.path.join(golden_dir, "bookkeeping.json")) as f:
        return json.load(f)


def test_library_exports_every_declared_symbol():
    """The C-ABI library loads without a GPU and exports everything include/hdit.h declares."""
    from hetu_dit_b200 import _C
    lib = ctypes.CDLL(_C.LIB_PATH)
    with open(os.path.join(ROOT, "include", "hdit.h")) as f:
        header = f.read()
    names = re.findall(r"HDIT_API\s+[\w\s\*]+?\b(hdit_\w+)\s*\(", header)
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} is declared but not exported"
    assert _C.lib().hdit_version() >= 100


def test_ctypes_structs_match_header_layout(tmp_path):
    """The ctypes mirrors have the size (and a few probed field offsets) the C compiler gives include/hdit.h."""
    import subprocess
    from hetu_dit_b200 import _C
    src = tmp_path / "sizes.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "hdit.h"\n'
        'int main(void) { printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(hdit_seg), sizeof(hdit_copy_piece), '
        'sizeof(hdit_attn_args), sizeof(hdit_norm_rope_tensor), sizeof(hdit_norm_rope_args), '
        'offsetof(hdit_attn_args, n_out_dst), offsetof(hdit_attn_args, q_dst_row0), '
        'offsetof(hdit_norm_rope_tensor, dst), sizeof(hdit_gemm_args), offsetof(hdit_gemm_args, stream)); '
        'return 0; }\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    want = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    got = [ctypes.sizeof(_C.Seg), ctypes.sizeof(_C.CopyPiece), ctypes.sizeof(_C.AttnArgs),
           ctypes.sizeof(_C.NormRopeTensor), ctypes.sizeof(_C.NormRopeArgs), _C.AttnArgs.n_out_dst.offset,
           _C.AttnArgs.q_dst_row0.offset, _C.NormRopeTensor.dst.offset, ctypes.sizeof(_C.GemmArgs),
           _C.GemmArgs.stream.offset]
    assert got == want


def test_no_cpu_path():
    from hetu_dit_b200 import kernels
    q = torch.zeros(1, 8, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        kernels.attn_fwd([q], [q], [q])


def test_argument_checks_without_gpu():
    """Bad arguments are rejected on the host before any CUDA call."""
    from hetu_dit_b200 import _C
    a = _C.AttnArgs()
    a.dtype, a.head_dim, a.batch, a.heads, a.n_q_seg, a.n_kv_seg = _C.HDIT_BF16, 96, 1, 1, 1, 1
    assert _C.lib().hdit_attn_fwd(ctypes.byref(a)) == _C.HDIT_ERR_SHAPE
    g = _C.GemmArgs()
    g.dtype, g.m, g.n, g.k = _C.HDIT_BF16, 16, 12, 64  # n not a multiple of 8
    g.a = g.w = g.out = 256
    g.lda = g.ldw = 64
    g.ldo = 16
    assert _C.lib().hdit_linear_fused(ctypes.byref(g)) == _C.HDIT_ERR_SHAPE
    g.n, g.epilogue = 16, 7
    assert _C.lib().hdit_linear_fused(ctypes.byref(g)) == _C.HDIT_ERR_BAD_ARG
    # gated residual over batch entries of fewer than 32 rows: a warp's rows would span more than two entries
    g.epilogue, g.m, g.rows_per_batch = _C.GEMM_BIAS_GATE_RESIDUAL, 64, 16
    g.residual = g.gate = 256
    g.ldr = g.gate_batch_stride = 16
    assert _C.lib().hdit_linear_fused(ctypes.byref(g)) == _C.HDIT_ERR_SHAPE
    a.head_dim, a.n_kv_seg = 64, 11
    assert _C.lib().hdit_attn_fwd(ctypes.byref(a)) == _C.HDIT_ERR_SHAPE
    assert b"n_kv_seg" in _C.lib().hdit_last_error()
    assert _C.lib().hdit_attn_fwd(None) == _C.HDIT_ERR_BAD_ARG
    assert _C.lib().hdit_copy_pieces(None, 3, None) == _C.HDIT_ERR_BAD_ARG
    assert _C.lib().hdit_kv_scatter(None, None, None, 1, 1, 0, 1, 2, 2, 2, None) == _C.HDIT_ERR_BAD_ARG


def test_patch_metadata_matches_reference(book):
    from hetu_dit_b200.core.distributed.runtime_state import split_patches
    keys = ("num_pipeline_patch", "pp_patches_height", "pp_patches_start_idx_local", "pp_patches_start_end_idx_global",
            "pp_patches_token_start_idx_local", "pp_patches_token_start_end_idx_global", "pp_patches_token_num")
    for c in book["patches_metadata"]:
        args = (c["height"] // c["vae"], c["width"] // c["vae"], c["patch"], c["num_pipeline_patch"], c["sp_world"],
                c["sp_rank"])
        strict = c["variant"] == "image"
        if "error" in c:
            with pytest.raises(ValueError):
                split_patches(*args, strict_last_patch=strict)
        else:
            assert dict(zip(keys, split_patches(*args, strict_last_patch=strict))) == c["result"], c


def test_runtime_state_object(book):
    from hetu_dit_b200.config import EngineConfig
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.runtime_state import ModelGeometry, initialize_runtime_state, reset_runtime_state
    ps.destroy_model_parallel()
    cfg = EngineConfig()
    cfg.parallel_config.pp_config.num_pipeline_patch = 4
    rt = initialize_runtime_state(ModelGeometry(24, 64), cfg)
    rt.set_input_parameters(height=1024, width=1024, batch_size=1, num_inference_steps=20)
    want = next(c for c in book["patches_metadata"] if c["variant"] == "image" and c["height"] == 1024 and
                c["width"] == 1024 and c["num_pipeline_patch"] == 4 and c["sp_world"] == 1)
    assert rt.patches_metadata() == want["result"]
    rt.set_patched_mode(True)
    seen = []
    for _ in range(6):
        seen.append(rt.pipeline_patch_idx)
        rt.next_patch()
    assert seen == [0, 1, 2, 3, 0, 1]
    rt.set_patched_mode(False)
    rt.next_patch()
    assert rt.pipeline_patch_idx == 0
    with pytest.raises(RuntimeError):
        bad = EngineConfig()
        bad.parallel_config.sp_config.ulysses_degree = 5
        initialize_runtime_state(ModelGeometry(24, 64), bad)
    reset_runtime_state()


def test_rank_generator_matches_reference(book):
    from hetu_dit_b200.core.distributed.utils import RankGenerator, generate_masked_orthogonal_rank_groups
    for c in book["rank_generator"]:
        g = RankGenerator(c["tp"], c["sp"], c["pp"], c["cfg"], c["dp"], "tp-sp-pp-cfg-dp", rank_offset=c["rank_offset"])
        for tok, groups in c["groups"].items():
            assert g.get_ranks(tok) == groups
    for c in book["masked_orthogonal"]:
        assert generate_masked_orthogonal_rank_groups(c["world"], c["sizes"], c["mask"]) == c["groups"]
    with pytest.raises(RuntimeError):
        RankGenerator(2, 1, 1, 1, 1, "sp-pp")


def test_seq_parallel_groups_match_reference(book):
    from hetu_dit_b200.core.distributed.parallel_state import set_seq_parallel_pg
    for c in book["seq_parallel_groups"]:
        for rank, groups in c["per_rank"].items():
            u, r = set_seq_parallel_pg(c["ulysses"], c["ring"], int(rank), len(c["ranks"]), c["ranks"],
                                       use_ulysses_low=c["use_ulysses_low"])
            assert u.ranks == groups["ulysses"] and r.ranks == groups["ring"], c


def test_comm_pool_enumeration_matches_reference(book):
    from hetu_dit_b200.core.distributed.parallel_state import ParallelGroups
    pg = ParallelGroups(0, 1)
    for c in book["rank_combinations"]:
        assert pg._generate_rank_combinations(c["world"], c["base"]) == c["result"]
    for c in book["group_partitions"]:
        assert pg._generate_group_ranks(c["ranks"]) == c["result"]


def test_plan_activation_on_rank_subset():
    """A U2 x R2 plan placed on ranks {1, 3, 4, 6} of an 8-rank node, seen from every member."""
    from hetu_dit_b200.core.distributed import parallel_state as ps
    members = [1, 3, 4, 6]
    for me in members:
        pg = ps.ParallelGroups(me, 8)
        pg.activate_plan(members, ulysses=2, ring=2)
        sp = pg.group("sp")
        assert sp.ranks == members and sp.rank_in_group == members.index(me)
        i = members.index(me)
        assert sp.ulysses_group.ranks == ([1, 3] if i < 2 else [4, 6])
        assert sp.ring_group.ranks == ([1, 4] if i % 2 == 0 else [3, 6])
        assert ps.PROCESS_GROUP.ULYSSES_PG is sp.ulysses_group and ps.PROCESS_GROUP.RING_PG is sp.ring_group
        assert pg.group("pp").ranks == [me] and pg.group("tp").world_size == 1
    pg = ps.ParallelGroups(5, 8)
    pg.activate_plan(range(8), ulysses=2, pp=4)  # tp-sp-pp order: sp pairs are consecutive, pp stride 2
    assert pg.group("sp").ranks == [4, 5] and pg.group("pp").ranks == [1, 3, 5, 7]
    with pytest.raises(ValueError):
        pg.activate_plan(range(8), ulysses=3)
    with pytest.raises(ValueError):
        pg.activate_plan([0, 1], ulysses=2)  # rank 5 is not a member
    ps.destroy_model_parallel()


def test_cache_manager_contract():
    from hetu_dit_b200.core.resource_manager.cache_manager import CacheManager
    cm = CacheManager()
    with pytest.raises(ValueError):
        cm.register_cache_entry(object(), "mlp")
    with pytest.raises(ValueError):
        cm.register_cache_entry(object(), "attn", "other")
    layer = object()
    cm.register_cache_entry(layer, "attn")
    k, v = torch.zeros(1, 4, 8), torch.ones(1, 4, 8)
    # no runtime state -> nothing cached, the fresh tensors come back (no GPU needed)
    from hetu_dit_b200.core.distributed.runtime_state import reset_runtime_state
    reset_runtime_state()
    rk, rv = cm.update_and_get_kv_cache([k, v], layer)
    assert rk is k and rv is v
    cm._reset_cache()
    assert cm.cache == {}


def test_operator_argument_errors():
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.parallel import hetuDiTJointLongContextAttention, hetuDiTLongContextAttention
    from hetu_dit_b200.core.parallel.ring import ring_flash_attn_func
    ps.destroy_model_parallel()
    with pytest.raises(RuntimeError):
        hetuDiTLongContextAttention(ring_impl_type="zigzag", use_kv_cache=True)
    op = hetuDiTJointLongContextAttention()
    q = torch.zeros(1, 8, 2, 64)
    with pytest.raises(ValueError):
        op(None, q, q, q, joint_tensor_query=q, joint_tensor_key=q, joint_tensor_value=q, joint_strategy="middle")
    with pytest.raises(ValueError):
        op(None, q, q, q, joint_tensor_query=None, joint_tensor_key=q, joint_tensor_value=q, joint_strategy="rear")
    with pytest.raises(ValueError):
        ring_flash_attn_func(q, q, q, joint_strategy="rear")
    with pytest.raises(AssertionError):
        ring_flash_attn_func(q, q, q, alibi_slopes=torch.zeros(2))
    # the Ulysses-only operator (ulysses/attn_layer.py:69-83 of the reference): same two ValueErrors
    from hetu_dit_b200.core.parallel import hetuDiTUlyssesAttention
    uly = hetuDiTUlyssesAttention(use_fa=False, use_kv_cache=False)
    for bad in ("none", "middle"):
        with pytest.raises(ValueError):
            uly(None, q, q, q, joint_tensor_query=q, joint_tensor_key=q, joint_tensor_value=q, joint_strategy=bad)
    with pytest.raises(ValueError):
        hetuDiTUlyssesAttention(scatter_idx=1, gather_idx=2)


def _gloo_worker(rank, world, port, errq):
    import traceback
    try:
        import torch.distributed as dist
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from hetu_dit_b200.core.distributed import parallel_state as ps
        from hetu_dit_b200.core.distributed.runtime_state import split_patches
        # every rank derives the same plan from the same inputs, with no collective on the data path
        ps.init_distributed_environment(rank, world, None)
        ps.initialize_model_parallel(sequence_parallel_degree=world, ulysses_degree=world)
        mine = (ps.get_sp_group().ranks, ps.get_ulysses_parallel_rank(), ps.get_sequence_parallel_world_size())
        seen = [None] * world
        dist.all_gather_object(seen, mine)
        assert all(s[0] == list(range(world)) and s[2] == world for s in seen)
        assert sorted(s[1] for s in seen) == list(range(world))
        # SP ranks own disjoint token ranges of every patch that tile the image
        meta = split_patches(128, 128, 2, 4, world, rank)
        allm = [None] * world
        dist.all_gather_object(allm, meta[5])
        covered = sorted(tuple(r) for m in allm for r in m)
        assert covered[0][0] == 0 and covered[-1][1] == 4096
        assert all(covered[i][1] == covered[i + 1][0] for i in range(len(covered) - 1))
        # a multi-rank group without a peer heap cannot move data and says so
        with pytest.raises(RuntimeError):
            ps.get_sp_group().barrier()
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put(traceback.format_exc())
        raise


def test_two_rank_host_protocol_on_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    try:
        mp.spawn(_gloo_worker, args=(2, 29641, errq), nprocs=2, join=True)
    except Exception:
        msgs = []
        while not errq.empty():
            msgs.append(errq.get())
        pytest.fail("\n".join(msgs) or "gloo worker failed")


def test_oracle_warmup_cache_order_under_ulysses():
    """Rank-major, patch-minor order of the stale K/V a warm-up step leaves under Ulysses (the oracle's model of
    cache_manager.py:170-184 of the reference); degree 1 is the identity."""
    from oracle.pipefusion import warmup_cache_order
    assert warmup_cache_order([4, 4], 1).tolist() == list(range(8))
    assert warmup_cache_order([4, 4], 2).tolist() == [0, 1, 4, 5, 2, 3, 6, 7]
    assert warmup_cache_order([4, 4, 2], 2).tolist() == [0, 1, 4, 5, 8, 2, 3, 6, 7, 9]


def test_oracle_flux_pipefusion_is_consistent_with_the_plain_step():
    """The Flux-shaped PipeFusion oracle: one un-patched step is the plain model step + one Euler update; with as
    many warm-up steps as steps the patches never matter; stale K/V makes the patched result differ, a little."""
    import torch
    from hetu_dit_b200.model_executor.models.shaped_dit import DiTShape, ShapedDiT
    from oracle import pipefusion as opf
    from oracle import shaped_dit as osd
    shape = DiTShape("flux-tiny", 1, 2, 128, 2, 64, 64, 64, 32, True, (16, 24, 24), True)
    sd = {k: v.float() for k, v in ShapedDiT(shape).init_weights(seed=5, std=0.05).state_dict().items()}
    gen = torch.Generator().manual_seed(9)
    lat = torch.randn(1, 8 * 4, 64, generator=gen)
    txt = torch.randn(1, 6, 64, generator=gen)
    pooled = torch.randn(1, 32, generator=gen)
    sig = opf.flow_match_sigmas(1)
    one = opf.denoise_flux(sd, shape, lat, txt, pooled, 1, 3.5, [32], 0, (8, 4))
    step = osd.denoise_step(sd, shape, lat, txt, pooled, sig[:1], torch.tensor([3.5]), grid=(8, 4))
    assert torch.allclose(one, lat + (sig[1] - sig[0]) * step, atol=1e-5)
    full = opf.denoise_flux(sd, shape, lat, txt, pooled, 3, 3.5, [32], 0, (8, 4))
    warm = opf.denoise_flux(sd, shape, lat, txt, pooled, 3, 3.5, [16, 16], 3, (8, 4))
    assert torch.equal(full, warm)
    patched = opf.denoise_flux(sd, shape, lat, txt, pooled, 3, 3.5, [16, 16], 1, (8, 4))
    staged = opf.denoise_flux(sd, shape, lat, txt, pooled, 3, 3.5, [16, 16], 1, (8, 4), stage_starts=(0, 2))
    diff = (patched - full).abs().max().item()
    assert 0 < diff < 0.5 * full.abs().max().item()
    assert 0 < (staged - patched).abs().max().item() < diff * 10


def test_kv_split_choice_follows_the_wave_model():
    """The wrapper's split-KV choice is pure host arithmetic: split when the grid leaves most SMs idle or
    spills a little over a wave, never for grids that fill the GPU or for short KV ranges -- and not where the
    library's own interleaved mode (one query tile per CTA, no merge pass) is cheaper still."""
    from hetu_dit_b200.kernels import _interleave_cost, _pick_kv_split

    class T:
        def __init__(self, s, d):
            self.shape = (1, s, 1, d)

    def pick(batch, heads, d, s):
        return _pick_kv_split([T(s, d)], [T(s, d)], batch, heads)

    def pick_no_il(batch, heads, d, s):
        return _pick_kv_split([T(s, d)], [T(s, d)], batch, heads, kv_interleave=1)

    # with the interleaved mode forbidden: the split-KV wave model alone
    assert pick_no_il(1, 3, 128, 4608) == 2     # Ulysses 8 of 24 heads: 54 CTAs on 148 SMs
    assert pick_no_il(1, 6, 128, 4608) == 1     # 108 CTAs: two half-length waves cost what one wave costs
    assert pick_no_il(1, 24, 128, 4608) == 1    # the single-GPU grid
    assert pick_no_il(1, 3, 128, 17776) == 2    # 210 CTAs = 1.4 waves -> 3 half-length waves
    assert pick_no_il(1, 6, 128, 17776) == 1
    assert pick_no_il(2, 3, 128, 377) == 1      # 3 KV blocks: nothing to split
    assert _pick_kv_split([T(512, 128), T(4096, 128)], [T(4608, 128)], 1, 3, kv_interleave=1) == 2
    # left to the library: 54 CTAs become 108 interleaved ones (measured 48 us against 59 us for the split)
    assert pick(1, 3, 128, 4608) == 1
    assert pick(1, 24, 128, 4608) == 1
    assert pick(1, 6, 128, 17776) == 1
    # the interleaved cost model in wave units: 12 heads (216 pairs = 2 waves) pay off, 6 and 24 heads do not
    paired = lambda heads, blocks=36: -(-18 * heads // 148) * (blocks + 6.0)
    assert _interleave_cost(36, 36, 1, 12) < paired(12) and _interleave_cost(36, 36, 1, 3) < paired(3)
    assert _interleave_cost(36, 36, 1, 6) > paired(6) and _interleave_cost(36, 36, 1, 24) > paired(24)


@pytest.mark.parametrize("sp,n_patch,height", [(2, 4, 64), (4, 2, 64), (2, 3, 48), (1, 4, 64)])
def test_pipeline_sp_split_and_gather_round_trip(monkeypatch, sp, n_patch, height):
    """Every SP rank takes its slice of every pipeline patch; the end-of-denoise gather re-interleaves them patch
    by patch (pipeline_stable_diffusion_3.py:1449-1465 of the reference). Together they are the identity whenever
    all patches have the same height. (With a shorter last patch the reference's own index lists pair the ranks'
    slices inconsistently -- the golden bookkeeping fixtures pin that -- and its gather, like this one, is then
    not the inverse of the split; the slices still cover every row once, which the last assertion of the split
    loop checks for all cases.)"""
    import types
    import torch
    from hetu_dit_b200.core.distributed.runtime_state import split_patches
    from hetu_dit_b200.model_executor.pipelines import pipeline_sd3_shaped as mod
    width = 32
    tokens = (height // 2) * (width // 2)
    latents = torch.arange(tokens * 3, dtype=torch.float32).view(1, tokens, 3)
    metas = [split_patches(height, width, 2, n_patch, sp, r) for r in range(sp)]
    pipe = mod.SD3ShapedPipeline.__new__(mod.SD3ShapedPipeline)
    locals_ = []
    for r in range(sp):
        n, _, _, _, tok_local, tok_bounds, tok_num = metas[r]
        rt = types.SimpleNamespace(num_pipeline_patch=n, pp_patches_token_start_idx_local=tok_local,
                                   pp_patches_token_start_end_idx_global=tok_bounds, pp_patches_token_num=tok_num)
        monkeypatch.setattr(mod, "get_runtime_state", lambda rt=rt: rt)
        locals_.append(pipe._sp_local(latents))
        assert locals_[-1].shape[1] == sum(tok_num)
    assert sum(x.shape[1] for x in locals_) == tokens
    group = types.SimpleNamespace(all_gather=lambda x, separate_tensors=False: list(locals_))
    monkeypatch.setattr(mod.ps, "get_sp_group", lambda: group)
    for r in range(sp):
        n, _, _, _, tok_local, tok_bounds, tok_num = metas[r]
        rt = types.SimpleNamespace(num_pipeline_patch=n, pp_patches_token_start_idx_local=tok_local,
                                   pp_patches_token_start_end_idx_global=tok_bounds, pp_patches_token_num=tok_num)
        monkeypatch.setattr(mod, "get_runtime_state", lambda rt=rt: rt)
        assert torch.equal(pipe._sp_gather(locals_[r]), latents)


def test_flux_pipeline_stage_split_and_first_token(monkeypatch):
    """Blocks are numbered double first, then single; a stage takes a contiguous range of that numbering. The
    first token of a call selects its rotary rows: the patch's global start in patch mode."""
    import types
    from hetu_dit_b200.model_executor.pipelines import pipeline_flux_shaped as mod
    pipe = mod.FluxShapedPipeline.__new__(mod.FluxShapedPipeline)
    pipe.stage_sliced = False
    pipe.model = types.SimpleNamespace(transformer_blocks=[f"d{i}" for i in range(3)],
                                       single_transformer_blocks=[f"s{i}" for i in range(5)])
    rt = types.SimpleNamespace(parallel_config=types.SimpleNamespace(pp_config=types.SimpleNamespace(
        attn_layer_num_for_pp=None)), patch_mode=False, pipeline_patch_idx=0,
        pp_patches_token_start_end_idx_global=[[0, 64], [128, 192]])
    monkeypatch.setattr(mod, "get_runtime_state", lambda: rt)
    got = []
    for world in (1, 2, 4):
        monkeypatch.setattr(mod.ps, "get_pipeline_parallel_world_size", lambda world=world: world)
        stages = []
        for r in range(world):
            monkeypatch.setattr(mod.ps, "get_pipeline_parallel_rank", lambda r=r: r)
            stages.append(pipe._stage_blocks())
        got.append(stages)
        assert sum((d for d, _ in stages), []) == pipe.model.transformer_blocks
        assert sum((s for _, s in stages), []) == pipe.model.single_transformer_blocks
    assert got[1] == [(["d0", "d1", "d2"], ["s0"]), ([], ["s1", "s2", "s3", "s4"])]
    assert got[2] == [(["d0", "d1"], []), (["d2"], ["s0"]), ([], ["s1", "s2"]), ([], ["s3", "s4"])]
    rt.parallel_config.pp_config.attn_layer_num_for_pp = [2, 6]
    monkeypatch.setattr(mod.ps, "get_pipeline_parallel_world_size", lambda: 2)
    monkeypatch.setattr(mod.ps, "get_pipeline_parallel_rank", lambda: 0)
    assert pipe._stage_blocks() == (["d0", "d1"], [])
    pipe.stage_sliced = True                      # the worker's block cache already placed this stage's blocks
    assert pipe._stage_blocks() == (pipe.model.transformer_blocks, pipe.model.single_transformer_blocks)

    # rotary rows: the whole table with the first token's row, or -- a whole-image step under sequence
    # parallelism with several patches -- a local table of the text rows followed by this rank's rows
    tab = torch.arange(10 + 640, dtype=torch.float32)[:, None].repeat(1, 4)
    pipe.model._rope = lambda s_txt, grid, device: (tab, -tab)
    pipe.grid = (20, 32)
    monkeypatch.setattr(mod.ps, "get_sequence_parallel_world_size", lambda: 1)
    assert pipe._rope_and_first_token(10, "cpu")[1] == 0
    rt.patch_mode, rt.pipeline_patch_idx = True, 1
    assert pipe._rope_and_first_token(10, "cpu")[1] == 128
    rt.patch_mode = False
    monkeypatch.setattr(mod.ps, "get_sequence_parallel_world_size", lambda: 2)
    (cos, sin), first = pipe._rope_and_first_token(10, torch.device("cpu"))
    rows = list(range(10)) + list(range(10, 74)) + list(range(138, 202))
    assert first == 0 and cos[:, 0].tolist() == [float(r) for r in rows] and torch.equal(sin, -cos)
    rt.pp_patches_token_start_end_idx_global = [[256, 512]]
    assert pipe._rope_and_first_token(10, "cpu")[1] == 256


def test_worker_plan_api_signatures_match_the_reference():
    """The executor calls worker methods by name with positional / keyword arguments
    (executor/gpu_executor.py:176-220 of the reference), so the parameter lists are part of the boundary:
    switch_parallel_env (worker/worker.py:480-482), hotspa_model (:1571, a coroutine), execute_diffusion_stage
    (:1009-1016), execute_encode_diffusion_stage (:1185-1191), get_worker_state (:1527)."""
    import inspect
    from hetu_dit_b200.worker.worker import Worker, run_worker_method

    def params(fn):
        return [p for p in inspect.signature(fn).parameters if p != "self"]

    # the parameter lists as they stand in the reference's source (read out of worker/worker.py by
    # tests/golden/make_golden.py)
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bookkeeping.json")) as f:
        want = json.load(f)["worker_signatures"]
    assert sorted(want) == ["execute_diffusion_stage", "execute_encode_diffusion_stage", "get_worker_state",
                            "hotspa_model", "switch_parallel_env"]
    for name, sig in want.items():
        fn = getattr(Worker, name)
        assert params(fn) == sig["params"], name
        assert inspect.iscoroutinefunction(fn) == sig["coroutine"], name
    for name in ("init_static_env", "init_instance_model", "rpc_find_sources"):
        assert callable(getattr(Worker, name))

    class Stub:
        def sync(self, a, b=2):
            return a + b

        async def coro(self, engine_config=None):
            return ("awaited", engine_config)

    assert run_worker_method(Stub(), "sync", 1, b=5) == 6
    assert run_worker_method(Stub(), "coro", engine_config="cfg") == ("awaited", "cfg")


def test_set_activate_groups_with_the_reference_call_forms():
    """ParallelGroups.set_activate_*(degree, ranks, group_ranks) as worker.py:493-556 of the reference calls
    them, for a plan on ranks {1, 3, 4, 6} of 8 with ulysses 2 x pp 2: same groups as activate_plan."""
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.utils import RankGenerator
    ranks = [1, 3, 4, 6]
    for me in ranks:
        a = ps.ParallelGroups(me, 8, None)
        a.activate_plan(ranks, ulysses=2, pp=2)
        b = ps.ParallelGroups(me, 8, None)
        rank_map = {i: r for i, r in enumerate(sorted(ranks))}
        gen = RankGenerator(tp=1, sp=2, pp=2, cfg=1, dp=1, order="tp-sp-pp-cfg-dp")
        mapped = lambda axis: [[rank_map[r] for r in g] for g in gen.get_ranks(axis)]
        b.set_activate_world_group(len(ranks), ranks, [ranks])
        b.set_activate_tp_group(degree=4, ranks=ranks, group_ranks=mapped("tp"))
        b.set_activate_sp_group(degree=4, ranks=ranks, group_ranks=mapped("sp"), ulysses_degree=2, ring_degree=1)
        b.set_activate_pp_group(degree=4, ranks=ranks, group_ranks=mapped("pp"))
        b.set_activate_cfg_group(degree=4, ranks=ranks, group_ranks=mapped("cfg"))
        b.set_activate_dp_group(degree=4, ranks=ranks, group_ranks=mapped("dp"))
        for axis in ("world", "tp", "sp", "pp", "cfg", "dp"):
            assert a.group(axis).ranks == b.group(axis).ranks, (me, axis)
        assert a.group("sp").ulysses_group.ranks == b.group("sp").ulysses_group.ranks
    ps.destroy_model_parallel()


# ----------------------------------------------------------------------------- PipeFusion schedule order
def _pipefusion_cases():
    import json
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "pipefusion_order.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("case", _pipefusion_cases(),
                         ids=lambda c: f"{c['pipeline']}pp{c['stages']}s{c['stage']}m{c['num_pipeline_patch']}n{c['steps']}w{c['warmup']}")
def test_pipefusion_schedule_order_matches_reference(case, monkeypatch):
    """Every stage's order of receives, receive-queue operations, forwards (patch index, step, text source),
    scheduler steps and sends through the warm-up and the patch pipeline is the one the reference's
    _sync_pipeline / _init_async_pipeline / _async_pipeline produce, for its SD3 pipeline
    (model_executor/pipelines/pipeline_stable_diffusion_3.py:1352-1678) and its Flux pipeline
    (pipelines/pipeline_flux.py:428-760), run with recording stand-ins by tests/golden/make_golden.py."""
    import types
    from hetu_dit_b200.model_executor.pipelines import pipeline_flux_shaped
    from hetu_dit_b200.model_executor.pipelines import pipeline_sd3_shaped as mod
    stages, stage, n_patch = case["stages"], case["stage"], case["num_pipeline_patch"]
    events, tokens = [], 4

    class Group:
        def pipeline_recv(self, idx=-1, name="latent"):
            events.append(["recv", name or "latent", idx])
            return torch.zeros(1, tokens * n_patch, 8)

        def pipeline_send(self, tensor, name="latent", segment_idx=-1):
            events.append(["send", name, segment_idx])

        pipeline_isend = pipeline_send

        def add_pipeline_recv_task(self, idx=-1, name="latent"):
            events.append(["add_recv_task", name or "latent", idx])

        def recv_next(self):
            events.append(["recv_next"])

        def get_pipeline_recv_data(self, idx=-1, name="latent"):
            events.append(["get", name, idx])
            return torch.zeros(1, tokens, 8)

    class State:
        ready = False
        num_pipeline_patch = n_patch
        pp_patches_token_num = [tokens] * n_patch
        runtime_config = types.SimpleNamespace(warmup_steps=case["warmup"])
        pipeline_patch_idx = 0

        def set_patched_mode(self, patch_mode):
            events.append(["patched_mode", bool(patch_mode)])
            self.pipeline_patch_idx = 0

        def next_patch(self):
            self.pipeline_patch_idx = (self.pipeline_patch_idx + 1) % n_patch

    state, group = State(), Group()
    fake_ps = types.SimpleNamespace(
        get_pp_group=lambda: group, is_pipeline_first_stage=lambda: stage == 0,
        is_pipeline_last_stage=lambda: stage == stages - 1, get_pipeline_parallel_world_size=lambda: stages,
        get_sequence_parallel_world_size=lambda: 1)
    monkeypatch.setattr(mod, "ps", fake_ps)
    monkeypatch.setattr(mod, "get_runtime_state", lambda: state)
    monkeypatch.setattr(mod, "flow_match_sigmas", lambda n, device=None: torch.arange(n + 1, dtype=torch.float32))
    prompt = torch.zeros(2, 3, 8)

    cls = pipeline_flux_shaped.FluxShapedPipeline if case["pipeline"] == "flux" else mod.SD3ShapedPipeline
    pipe = object.__new__(cls)

    def backbone(latents, encoder_hidden_states, pooled, t, guide=True):
        assert guide == (stage != stages - 1)  # the last stage leaves guidance to the fused step
        events.append(["forward", state.pipeline_patch_idx, int(t),
                       "prompt" if encoder_hidden_states is prompt else "received"])
        return latents, torch.zeros(2, 3, 8)

    def guided_step(noise_pred, last_latents, i, send_as=None, **_):
        events.append(["step", int(i)])
        if send_as is not None:
            events.append(["send", send_as[0], send_as[1]])
        return noise_pred

    pipe._backbone_forward = backbone
    pipe._guided_step = guided_step
    out = pipe.diffusion_stage(torch.zeros(1, tokens * n_patch, 8), prompt, None, case["steps"])
    assert (out is not None) == (stage == stages - 1)
    assert events[-1] == ["patched_mode", False]  # the entry point leaves the runtime state unpatched
    assert events[:-1] == case["events"]


# ----------------------------------------------------------------------------- position rows per rank
def _pos_cases():
    import json
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "pos_embed_rows.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("case", _pos_cases(),
                         ids=lambda c: f"{c['height']}x{c['width']}m{c['num_pipeline_patch']}sp{c['sp_world']}r{c['sp_rank']}")
def test_position_rows_match_reference_patch_embed(case, monkeypatch):
    """The rows of the position table a rank adds to its tokens -- whole-image mode and every patch of patch
    mode -- are the rows the reference's patch-embedding wrapper slices
    (model_executor/diffusion_executor/layers/embeddings.py:90-112), run on a table of row numbers by
    tests/golden/make_golden.py."""
    import types
    from hetu_dit_b200.model_executor.pipelines import pipeline_sd3_shaped as mod
    cell = case["vae"] * case["patch"]
    gh, gw = case["height"] // cell, case["width"] // cell
    state = types.SimpleNamespace(pp_patches_token_start_end_idx_global=[tuple(b) for b in case["bounds"]],
                                  patch_mode=False, pipeline_patch_idx=0)
    monkeypatch.setattr(mod, "get_runtime_state", lambda: state)
    monkeypatch.setattr(mod, "ps", types.SimpleNamespace(get_sequence_parallel_world_size=lambda: case["sp_world"]))
    pipe = object.__new__(mod.SD3ShapedPipeline)
    pipe.grid = (gh, gw)
    pipe.model = types.SimpleNamespace(
        _sincos_pos=lambda h, w, device, dtype: torch.arange(h * w, dtype=torch.float32).reshape(1, h * w, 1))

    def rows(n):
        return pipe._positions(n, "cpu", torch.float32)[0, :, 0].long().tolist()

    def flat(runs):
        return [i for s, e in runs for i in range(s, e)]

    n_local = sum(e - s for s, e in case["bounds"])
    assert rows(n_local) == flat(case["whole_image_rows"])
    state.patch_mode = True
    for p, runs in enumerate(case["patch_rows"]):
        state.pipeline_patch_idx = p
        assert rows(case["bounds"][p][1] - case["bounds"][p][0]) == flat(runs)
    with pytest.raises(ValueError):
        pipe._positions(n_local + 1, "cpu", torch.float32)


def test_trace_admission_on_disjoint_gpus():
    """The serving trace's virtual clock: one request at a time against requests that occupy part of the node
    and overlap on disjoint GPUs; first-in-first-out start order in both."""
    from hetu_dit_b200.serving.trace_driver import simulate_fifo, simulate_fifo_gpus
    arrivals, service = [0.0, 0.1, 0.2, 0.3], [1.0, 1.0, 1.0, 1.0]
    np.testing.assert_allclose(simulate_fifo(arrivals, service), [1.0, 1.9, 2.8, 3.7])
    # every request takes the whole node: the same as one server
    np.testing.assert_allclose(simulate_fifo_gpus(arrivals, service, [4, 4, 4, 4], 4), [1.0, 1.9, 2.8, 3.7])
    # half the node each: two at a time
    np.testing.assert_allclose(simulate_fifo_gpus(arrivals, service, [2, 2, 2, 2], 4), [1.0, 1.0, 1.8, 1.8])
    # a whole-node request in the middle holds back the small ones behind it (no overtaking)
    np.testing.assert_allclose(simulate_fifo_gpus(arrivals, service, [1, 4, 1, 1], 4), [1.0, 1.9, 2.8, 2.7])


def test_stage_block_split_matches_reference():
    """Which double / single blocks a pipeline stage holds: stage_block_range + the Flux pipeline's slicing against
    the reference's _split_transformer_blocks (models/transformers/base_transformer.py:65-146), recorded by
    tests/golden/make_golden.py for SD3-, Flux-, CogVideoX- and HunyuanVideo-sized block lists."""
    import json
    from hetu_dit_b200.model_executor.pipelines.pipeline_sd3_shaped import stage_block_range
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "stage_split.json")) as f:
        cases = json.load(f)
    assert len(cases) >= 60
    for c in cases:
        nd, ns = c["n_double"], c["n_single"]
        lo, hi = stage_block_range(nd + ns, c["stage"], c["stages"], c["attn_layer_num_for_pp"])
        double = list(range(min(lo, nd), min(hi, nd)))
        single = list(range(max(lo - nd, 0), max(hi - nd, 0)))
        assert double == c["double"] and single == c["single"], c
        # after_flags: the stage holds the last block of that list
        want_flags = {"transformer_blocks": bool(double) and double[-1] == nd - 1}
        if ns:
            want_flags["single_transformer_blocks"] = bool(single) and single[-1] == ns - 1
        assert want_flags == c["after_flags"], c


def test_scheduler_step_matches_reference_wrapper():
    """The flow-matching Euler step of the pipelines against the reference's scheduler wrapper
    (schedulers/scheduling_flow_match_euler_discrete.py:22-129, recorded by tests/golden/make_golden.py): the same
    16-bit result bit for bit (the wrapper rounds prediction * sigma to the prediction's type and forms
    (sample - (sample - product)) / sigma in fp32; so do the pipelines and the fused kernel), and the step index
    advances once per step -- after the last patch in patch mode -- which the pipelines get by indexing with the step
    counter of their own loop."""
    import json
    from hetu_dit_b200.model_executor.pipelines import pipeline_sd3_shaped as mod
    with np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "scheduler_step.npz")) as f:
        calls = json.loads(str(f["calls"]))
        data = {k: f[k] for k in f.files if k != "calls"}
    pipe = object.__new__(mod.SD3ShapedPipeline)
    pipe.sigmas = torch.from_numpy(data["sigmas"])
    assert len(calls) >= 20
    for c in calls:
        dtype = torch.bfloat16 if c["dtype"] == "bf16" else torch.float16
        mo = torch.from_numpy(data[c["key"] + "/model_output"]).to(dtype)
        x = torch.from_numpy(data[c["key"] + "/sample"]).to(dtype)
        want = torch.from_numpy(data[c["key"] + "/prev_sample"]).to(dtype)
        got = pipe._scheduler_step(mo, x, c["step_index"])
        assert got.dtype == dtype and torch.equal(got, want), c
        # one advance per step: every call outside patch mode, the last patch only inside it
        assert c["advanced"] == (1 if (not c["patch_mode"] or c["patch"] == c["patches"] - 1) else 0)


def test_trace_deadline_rule_matches_reference():
    """estimate_ddl of the serving-trace driver against the reference's (hetu_dit/utils.py:267-288, recorded in
    bookkeeping.json), and the per-request deadlines the driver derives from it."""
    import json
    from hetu_dit_b200.serving.trace_driver import estimate_ddl, reference_deadlines
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bookkeeping.json")) as f:
        cases = json.load(f)["estimate_ddl"]
    assert len(cases) >= 9
    for c in cases:
        assert estimate_ddl({int(k): v for k, v in c["t"].items()}) == c["ddl"], c
    single = {512: 0.144, 1536: 1.28}
    ddl = reference_deadlines([512, 1536, 512, 1536], [0.2, 0.6, 0.3, 0.58], [1, 4, 1, 4], single)
    assert ddl.tolist() == [float(estimate_ddl({1: 0.144})), float(estimate_ddl({1: 1.28, 4: 0.59}))] * 2


def test_operator_coordinator_and_cache_surface_matches_reference():
    """Parameter names, their order and their literal defaults of the USP operators, the pipeline group
    coordinator and the stale-KV cache manager, as written in the reference's source (read out by
    tests/golden/make_golden.py): a caller written against the reference binds the same arguments here. Parameters
    this repository adds come after the reference's and have defaults."""
    import inspect
    import json
    from hetu_dit_b200.core import parallel as P
    from hetu_dit_b200.core.distributed.group_coordinator import PipelineGroupCoordinator
    from hetu_dit_b200.core.resource_manager.cache_manager import CacheManager
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bookkeeping.json")) as f:
        want = json.load(f)["api_surface"]
    assert len(want) == 23
    from hetu_dit_b200.core.distributed.peer import PeerGroup
    from hetu_dit_b200.core.distributed.runtime_state import DiTRuntimeState
    from hetu_dit_b200.core.parallel.ring.ring_flash_attn import ring_flash_attn_func
    from hetu_dit_b200.model_executor.cache.base_cache import BaseBlockCache
    owners = {"PipelineGroupCoordinator": PipelineGroupCoordinator, "CacheManager": CacheManager,
              "GroupCoordinator": PeerGroup,          # the groups the getters return here
              "DiTRuntimeState": DiTRuntimeState, "BaseBlockCache": BaseBlockCache}
    for key, sig in want.items():
        if "." in key:
            cls_name, meth = key.split(".")
            fn = getattr(owners.get(cls_name) or getattr(P, cls_name), meth)
        else:
            fn = {"ring_flash_attn_func": ring_flash_attn_func}[key]
        assert inspect.iscoroutinefunction(fn) == sig["coroutine"], key
        params = [p for p in inspect.signature(fn).parameters.values() if p.name != "self"]
        positional = [p for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)]
        names = [p.name for p in positional]
        assert names[:len(sig["params"])] == sig["params"], (key, names)
        for p in positional[len(sig["params"]):]:
            assert p.default is not p.empty, (key, p.name)          # additions never become required
        by_name = {p.name: p for p in positional}
        for name, default in sig["defaults"].items():
            got = by_name[name].default
            got = list(got) if isinstance(got, tuple) else got
            assert got == default, (key, name, got, default)


def _stage_forward_cases():
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "stage_forward.npz"))
    import json
    calls = json.loads(str(z["calls"]))
    groups = {}
    for c in calls:
        groups.setdefault((c["model"], c["stages"]), []).append(c)
    return z, groups


@pytest.mark.parametrize("model,stages", [(m, s) for m in ("sd3", "flux") for s in (1, 2, 3, 4)])
def test_stage_forward_matches_reference_transformer_wrappers(model, stages, monkeypatch):
    """The stage forward of the two pipelines (_transformer) against forward() of the reference's SD3 and Flux
    transformer wrappers (transformer_sd3.py:43-198, transformer_flux.py:45-217), which tests/golden/make_golden.py
    ran on stand-in embedders, blocks and output layers: which stage embeds, which blocks a stage runs and in what
    order, text rows joined in front of the image rows for the single blocks and split off again, the SD3 wrapper's
    re-use of every block's text input of patch 0 for the later patches, output norm and projection on the last
    stage only, and what a stage hands on. The stand-in arithmetic below repeats the generator's."""
    import types
    import torch.nn.functional as F
    from hetu_dit_b200.model_executor.pipelines import pipeline_flux_shaped as fmod
    from hetu_dit_b200.model_executor.pipelines import pipeline_sd3_shaped as smod
    z, groups = _stage_forward_cases()
    calls = groups[(model, stages)]
    d = 8
    n_double, n_single = calls[0]["n_double"], calls[0]["n_single"]

    def double(i):
        def f(hidden, text, temb, rope, tok0=0):
            h = hidden * 1.5 + text.mean(1, keepdim=True) + temb[:, None] + (i + 1)
            c = text * 0.5 + hidden.mean(1, keepdim=True) * 0.25 - (i + 1)
            return h, c
        return f

    def single(j):
        def f(x, temb, rope, s_txt, tok0=0):
            rows = torch.arange(x.shape[1], dtype=x.dtype)[None, :, None]
            return x * 1.25 + rows * 0.01 * (j + 1) + temb[:, None]
        return f

    ones = lambda e: torch.ones(e.shape[0], d, dtype=torch.float64)
    m = types.SimpleNamespace(
        time_embed=lambda e: 0.125 * ones(e), guidance_embed=lambda e: 0.0625 * ones(e),
        pooled_embed=lambda p: p.sum(-1, keepdim=True).expand(-1, d),
        x_embedder=lambda h: h * 2.0 + 1.0, context_embedder=lambda c: c * 3.0 - 1.0,
        transformer_blocks=[double(i) for i in range(n_double)],
        single_transformer_blocks=[single(j) for j in range(n_single)],
        norm_out=types.SimpleNamespace(linear=lambda x: torch.cat([0.1 * x, 0.2 * x], dim=-1)),    # (scale, shift)
        proj_out=lambda h: h * 7.0)
    cls = smod.SD3ShapedPipeline if model == "sd3" else fmod.FluxShapedPipeline
    pipe = cls.__new__(cls)
    pipe.model, pipe.stage_sliced, pipe.guidance_scale = m, False, 3.5
    pipe.shape = types.SimpleNamespace(hidden=d, out_norm_scale_first=True)
    pipe._positions = lambda n, device, dtype: 0.0
    pipe._rope_and_first_token = lambda s_txt, device: (None, 0)
    rt = types.SimpleNamespace(parallel_config=types.SimpleNamespace(pp_config=types.SimpleNamespace(
        attn_layer_num_for_pp=None)), patch_mode=False, pipeline_patch_idx=0)
    for mod in (smod, fmod):
        monkeypatch.setattr(mod, "get_runtime_state", lambda: rt)
    monkeypatch.setattr(fmod.kernels, "ln_modulate", lambda h, shift, scale: F.layer_norm(
        h, (d,), eps=1e-6) * (1 + scale[:, None]) + shift[:, None])
    monkeypatch.setattr(smod.ps, "get_pipeline_parallel_world_size", lambda: stages)
    caches = [dict() for _ in range(stages)]
    pooled = torch.from_numpy(z[f"{model}/pp{stages}/pooled"])
    assert len(calls) == 4 * stages
    for c in calls:
        stage = c["stage"]
        monkeypatch.setattr(smod.ps, "get_pipeline_parallel_rank", lambda stage=stage: stage)
        monkeypatch.setattr(smod.ps, "is_pipeline_first_stage", lambda stage=stage: stage == 0)
        monkeypatch.setattr(smod.ps, "is_pipeline_last_stage", lambda stage=stage: stage == stages - 1)
        rt.patch_mode, rt.pipeline_patch_idx = c["mode"] == "patch", c["patch"] or 0
        pipe.encoder_hidden_states_cache = caches[stage]            # one wrapper per stage in the reference
        h_in, c_in = torch.from_numpy(z[c["key"] + "/in_h"]), torch.from_numpy(z[c["key"] + "/in_c"])
        h, text = pipe._transformer(h_in, c_in, pooled, torch.full((2,), 0.5, dtype=torch.float64))
        want = torch.from_numpy(z[c["key"] + "/out_h"])
        assert h.shape == want.shape and torch.allclose(h, want, rtol=1e-12, atol=1e-12), c
        if c["text_out"]:
            want_c = torch.from_numpy(z[c["key"] + "/out_c"])
            assert torch.allclose(text, want_c, rtol=1e-12, atol=1e-12), c


def test_worker_state_record_matches_reference(book, monkeypatch):
    """get_worker_state against the reference's method (worker/worker.py:1527-1563) run on stand-in workers with a
    fixed clock (tests/golden/make_golden.py): every key of the reference's record with the same value; this
    repository's extra keys come on top."""
    from hetu_dit_b200.worker import worker as wmod
    cases = book["worker_state"]
    assert len(cases) == 6
    for c in cases:
        w = wmod.Worker.__new__(wmod.Worker)
        w.rank, w.states, w.device = c["rank"], dict(c["states"]), torch.device("cpu")
        w.plan_ranks, w.cache, w.arena = [c["rank"]], None, None
        monkeypatch.setattr(wmod.time, "perf_counter", lambda now=c["now"]: now)
        got = w.get_worker_state()
        for key, want in c["result"].items():
            assert got[key] == want and type(got[key]) is type(want), (key, got[key], want, c["states"])
        assert {"plan", "cached_blocks", "arena_bytes"} <= set(got)


def test_adjust_pipeline_coroutine_takes_the_reference_argument_forms():
    """BaseBlockCache.adjust_pipeline (base_cache.py:243-282 of the reference): a coroutine that takes the model as
    (transformer, cpu_full_transformer), (text_encoder, cpu_full_text_encoder) or (model, cpu_full_model), by keyword
    or position, and raises TypeError without any of them."""
    import asyncio
    from hetu_dit_b200.model_executor.cache.base_cache import BaseBlockCache

    class Recorder(BaseBlockCache):
        def __init__(self):
            self.calls = []

        def adjust_pipeline_sync(self, *args, **kwargs):
            self.calls.append((args, kwargs))
            return args[0]

    c = Recorder()
    gpu, cpu = object(), object()
    ranges = dict(old_pp_range=(0, 0), new_pp_range=(0.0, 0.5), old_tp_range=(0.0, 1.0), new_tp_range=(0.0, 0.5))
    assert asyncio.run(c.adjust_pipeline(transformer=gpu, cpu_full_transformer=cpu, slice_bias=True, **ranges)) is gpu
    assert asyncio.run(c.adjust_pipeline(text_encoder=gpu, cpu_full_text_encoder=cpu, **ranges)) is gpu
    assert asyncio.run(c.adjust_pipeline(model=gpu, cpu_full_model=cpu, **ranges)) is gpu
    assert asyncio.run(c.adjust_pipeline(gpu, cpu, (0, 0), (0.0, 0.5), (0.0, 1.0), (0.0, 0.5),
                                         peer_directories={1: {}})) is gpu
    labels = [kw["component_name"] for _, kw in c.calls]
    assert labels == ["Transformer", "TextEncoder", None, "Transformer"]
    for args, kw in c.calls:
        assert args == (gpu, cpu, (0, 0), (0.0, 0.5), (0.0, 1.0), (0.0, 0.5)) and kw["slice_bias"] is True
    assert c.calls[3][1]["peer_directories"] == {1: {}} and c.calls[0][1]["peer_directories"] is None
    with pytest.raises(TypeError):
        asyncio.run(c.adjust_pipeline(transformer=gpu, **ranges))

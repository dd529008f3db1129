"""Block- and model-level GPU parity of the -shaped DiT against the CPU oracle."""
import pytest
import torch

from oracle import attention as oa
from oracle import shaped_dit as osd

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(shape, s_img, s_txt, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(1, s_img, shape.token_in, generator=gen).bfloat16(),
            torch.randn(1, s_txt, shape.text_dim, generator=gen).bfloat16(),
            torch.randn(1, max(shape.pooled_dim, 1), generator=gen).bfloat16(), torch.tensor([0.5]), torch.tensor([3.5]))


TINY = {
    # kind: (shape arguments, grid)
    "flux": (("flux-tiny", 2, 3, 512, 4, 128, 64, 256, 96, True, (16, 56, 56), True), {}, (20, 12)),
    "sd3": (("sd3-tiny", 3, 0, 256, 4, 64, 64, 256, 128, False, None, False), {}, (20, 12)),
    "cogvideox": (("cogvideox-tiny", 3, 0, 256, 4, 64, 128, 256, 0, True, (16, 24, 24), False),
                  dict(text_first=True, rope_on_text=False, qk_norm_kind="layer", block_kind="cogvideox", temb_dim=128),
                  (3, 10, 8)),
    "hunyuan": (("hunyuan-tiny", 2, 3, 512, 4, 128, 64, 256, 96, True, (16, 56, 56), True),
                dict(text_first=False, rope_on_text=False), (3, 10, 8)),
}


def tiny_shape(kind):
    from hetu_dit_b200.model_executor.models.shaped_dit import DiTShape
    args, kw, grid = TINY[kind]
    return DiTShape(*args, **kw), grid


def per_element_rel(got, want, floor=1e-2):
    """Per-element |a - b| / |b| over the elements whose magnitude is at least `floor` * max |b|: (largest,
    99.9th percentile). With 16-bit storage an element at 1 % of the block's largest value carries an absolute
    error that is a visible fraction of itself, so the largest ratio is reported and only loosely bounded; the
    percentile is the figure to read."""
    got, want = got.float(), want.float()
    big = want.abs() >= floor * want.abs().max()
    r = ((got - want).abs()[big] / want.abs()[big]).flatten()
    return r.max().item(), torch.quantile(r[:4_000_000], 0.999).item()


def hook_block_outputs(model, s_txt):
    """Forward hooks that collect every block's image / video stream output (B, S_img, hidden)."""
    outs, handles = [], []
    first = model.shape.text_first

    def double(_m, _inp, out):
        outs.append(out[0].detach().float().cpu())

    def single(_m, _inp, out):
        outs.append((out[:, s_txt:] if first else out[:, :out.shape[1] - s_txt]).detach().float().cpu())

    for b in model.transformer_blocks:
        handles.append(b.register_forward_hook(double))
    for b in model.single_transformer_blocks:
        handles.append(b.register_forward_hook(single))
    return outs, handles


@pytest.fixture
def fused_linear(request, monkeypatch):
    """Runs the test with the blocks' linear layers + tails as separate kernels (False) or fused (True)."""
    from hetu_dit_b200 import kernels
    monkeypatch.setattr(kernels, "FUSED_LINEAR", bool(request.param))
    monkeypatch.setattr(kernels, "FUSED_LINEAR_MIN_ROWS", 0)
    monkeypatch.setattr(kernels, "FUSED_LINEAR_MAX_ROWS", 1 << 40)
    return bool(request.param)


@pytest.mark.parametrize("fused_linear", [False, True], indirect=True, ids=["unfused", "fused_linear"])
@pytest.mark.parametrize("kind", ["flux", "sd3", "cogvideox", "hunyuan"])
def test_tiny_model_step(kind, fused_linear):
    """One step of a tiny model of each shape: every block's output and the final output against the fp32
    oracle, cosine >= 0.9999 and max |a-b| / max |b| <= 2e-2 per block; the per-element relative error over the
    elements above 1 % of the block's largest magnitude is bounded too."""
    from hetu_dit_b200 import _C
    from hetu_dit_b200.model_executor.models.shaped_dit import ShapedDiT
    shape, grid = tiny_shape(kind)
    n_tok = 1
    for g in grid:
        n_tok *= g
    model = ShapedDiT(shape).to(DEV).init_weights(seed=3, std=0.05).bfloat16()
    lat, txt, pooled, t, g = _inputs(shape, n_tok, 33)
    outs, handles = hook_block_outputs(model, 33)
    with torch.no_grad():
        got = model(lat.to(DEV), txt.to(DEV), pooled.to(DEV), t.to(DEV), g.to(DEV), grid=grid)
        torch.cuda.synchronize()
        assert _C.device_status(0, clear=True)[0] == 0
        sd = {k: v.float().cpu() for k, v in model.state_dict().items()}
        want_blocks = []
        want = osd.denoise_step(sd, shape, lat, txt, pooled, t, g, grid=grid, block_outputs=want_blocks)
    for h in handles:
        h.remove()
    assert len(outs) == len(want_blocks) == shape.n_blocks
    for i, (a, b) in enumerate(list(zip(outs, want_blocks)) + [(got.cpu(), want)]):
        cos, rel = oa.cosine_and_max_rel(a, b)
        elem_max, elem_p999 = per_element_rel(a, b)
        print(f"{kind} block {i}: cosine {cos:.6f} max_rel {rel:.4f} per-element rel max {elem_max:.3f} "
              f"p99.9 {elem_p999:.4f}")
        assert cos >= 0.9999 and rel <= 2e-2, (kind, i, cos, rel)
        assert elem_max <= 1.5 and elem_p999 <= 0.5, (kind, i, elem_max, elem_p999)


def test_joint_block_output_tolerance():
    """One Flux-shaped double block at hidden 3072: per-block cosine >= 0.9999, max relative error <= 2e-2."""
    from hetu_dit_b200.model_executor.models.shaped_dit import FLUX_DEV, JointBlock, rope_tables
    torch.manual_seed(0)
    blk = JointBlock(FLUX_DEV).to(DEV)
    gen = torch.Generator(device=DEV).manual_seed(5)
    with torch.no_grad():
        for n, p in blk.named_parameters():
            if p.dim() > 1:
                p.copy_(torch.randn(p.shape, generator=gen, device=DEV) * 0.02)
            elif n.endswith("bias"):
                p.zero_()
    blk = blk.bfloat16()
    S_txt, gh, gw = 64, 16, 24
    g2 = torch.Generator().manual_seed(6)
    hidden = torch.randn(1, gh * gw, 3072, generator=g2).bfloat16()
    context = torch.randn(1, S_txt, 3072, generator=g2).bfloat16()
    temb = torch.randn(1, 3072, generator=g2).bfloat16()
    ids = torch.zeros(S_txt + gh * gw, 3)
    yy, xx = torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij")
    ids[S_txt:, 1], ids[S_txt:, 2] = yy.flatten(), xx.flatten()
    rope = rope_tables(ids, FLUX_DEV.rope_axes)
    with torch.no_grad():
        h, c = blk(hidden.to(DEV), context.to(DEV), temb.to(DEV), (rope[0].to(DEV), rope[1].to(DEV)))
        torch.cuda.synchronize()
        sd = {"b." + k: v.float().cpu() for k, v in blk.state_dict().items()}
        wh, wc = osd.joint_block(sd, "b", hidden.float(), context.float(), temb.float(), rope, 24, 128, "front")
    for got, want in ((h, wh), (c, wc)):
        cos, rel = oa.cosine_and_max_rel(got.cpu(), want)
        assert cos >= 0.9999 and rel <= 2e-2, (cos, rel)


def _seed_block(blk, seed):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    with torch.no_grad():
        for n, p in blk.named_parameters():
            if p.dim() > 1:
                p.copy_(torch.randn(p.shape, generator=gen, device=DEV) * 0.02)
            elif n.endswith("bias"):
                p.zero_()
    return blk.bfloat16()


def test_single_block_output_tolerance():
    """One Flux-shaped single block at hidden 3072: per-block cosine >= 0.9999, max relative error <= 2e-2."""
    from hetu_dit_b200.model_executor.models.shaped_dit import FLUX_DEV, SingleBlock, rope_tables
    blk = _seed_block(SingleBlock(FLUX_DEV).to(DEV), 7)
    S_txt, gh, gw = 64, 16, 24
    g2 = torch.Generator().manual_seed(8)
    x = torch.randn(1, S_txt + gh * gw, 3072, generator=g2).bfloat16()
    temb = torch.randn(1, 3072, generator=g2).bfloat16()
    rope = rope_tables(osd.grid_ids(S_txt, (gh, gw)), FLUX_DEV.rope_axes)
    with torch.no_grad():
        got = blk(x.to(DEV), temb.to(DEV), (rope[0].to(DEV), rope[1].to(DEV)), S_txt)
        torch.cuda.synchronize()
        sd = {"b." + k: v.float().cpu() for k, v in blk.state_dict().items()}
        want = osd.single_block(sd, "b", x.float(), temb.float(), rope, 24, 128)
    cos, rel = oa.cosine_and_max_rel(got.cpu(), want)
    assert cos >= 0.9999 and rel <= 2e-2, (cos, rel)
    elem_max, elem_p999 = per_element_rel(got.cpu(), want)
    assert elem_max <= 1.5 and elem_p999 <= 0.5, (elem_max, elem_p999)


def test_full_size_flux_block_row_subset():
    """One Flux-shaped double block at the benchmark's size (hidden 3072, 4096 image + 512 text tokens): the
    block's image-stream output on 256 rows spread over the sequence against the fp32 oracle of the same rows.
    Attention rows are independent given K and V, so the oracle computes K / V for all tokens but queries, the
    output projection and the MLP only for the chosen rows."""
    import torch.nn.functional as F
    from hetu_dit_b200.model_executor.models.shaped_dit import FLUX_DEV, JointBlock, rope_tables
    blk = _seed_block(JointBlock(FLUX_DEV).to(DEV), 9)
    S_txt, gh, gw, d, H, D = 512, 64, 64, 3072, 24, 128
    g2 = torch.Generator().manual_seed(10)
    hidden = torch.randn(1, gh * gw, d, generator=g2).bfloat16()
    context = torch.randn(1, S_txt, d, generator=g2).bfloat16()
    temb = torch.randn(1, d, generator=g2).bfloat16()
    rope = rope_tables(osd.grid_ids(S_txt, (gh, gw)), FLUX_DEV.rope_axes)
    with torch.no_grad():
        h, _ = blk(hidden.to(DEV), context.to(DEV), temb.to(DEV), (rope[0].to(DEV), rope[1].to(DEV)))
        torch.cuda.synchronize()
        sd = {"b." + k: v.float().cpu() for k, v in blk.state_dict().items()}
        rows = torch.arange(0, gh * gw, 16)[:256]
        hf, cf, tf = hidden.float(), context.float(), temb.float()
        mod = osd._lin(sd, "b.norm1.linear", F.silu(tf)).chunk(6, dim=-1)
        cmod = osd._lin(sd, "b.norm1_context.linear", F.silu(tf)).chunk(6, dim=-1)
        hn = osd._mod(F.layer_norm(hf, (d,), eps=1e-6), mod[0], mod[1])
        cn = osd._mod(F.layer_norm(cf, (d,), eps=1e-6), cmod[0], cmod[1])
        a = "b.attn.module"
        k = osd._qk(sd, a, osd._lin(sd, a + ".to_k", hn), H, D, "norm_k", rope, S_txt)
        v = osd._heads(osd._lin(sd, a + ".to_v", hn), H, D)
        tk = osd._qk(sd, a, osd._lin(sd, a + ".add_k_proj", cn), H, D, "norm_added_k", rope, 0)
        tv = osd._heads(osd._lin(sd, a + ".add_v_proj", cn), H, D)
        q_all = osd._qk(sd, a, osd._lin(sd, a + ".to_q", hn), H, D, "norm_q", rope, S_txt)
        o = oa.sdpa(q_all[:, rows], torch.cat([tk, k], 1), torch.cat([tv, v], 1)).reshape(1, len(rows), d)
        img = osd._lin(sd, a + ".to_out.0", o)
        hr = hf[:, rows] + mod[2][:, None] * img
        hr = hr + mod[5][:, None] * osd._ff(sd, "b.ff", osd._mod(F.layer_norm(hr, (d,), eps=1e-6), mod[3], mod[4]))
    cos, rel = oa.cosine_and_max_rel(h[:, rows.to(DEV)].cpu(), hr)
    assert cos >= 0.9999 and rel <= 2e-2, (cos, rel)


def test_graph_replay_matches_eager_bit_for_bit():
    """ShapedDiT.forward_graphed: the captured step replayed twice with fresh inputs equals the eager step bit
    for bit, and a second shape gets its own graph."""
    from hetu_dit_b200 import _C
    from hetu_dit_b200.model_executor.models.shaped_dit import ShapedDiT
    shape, grid = tiny_shape("flux")
    model = ShapedDiT(shape).to(DEV).init_weights(seed=5, std=0.05).bfloat16()
    with torch.no_grad():
        for seed in (0, 1, 2):
            lat, txt, pooled, t, g = (x.to(DEV) for x in _inputs(shape, grid[0] * grid[1], 33, seed=seed))
            eager = model(lat, txt, pooled, t, g, grid=grid).clone()
            got = model.forward_graphed(lat, txt, pooled, t, g, grid=grid)
            torch.cuda.synchronize()
            assert torch.equal(got, eager), seed
        for seed in (3, 4):
            lat, txt, pooled, t, g = (x.to(DEV) for x in _inputs(shape, 10 * 12, 20, seed=seed))
            assert torch.equal(model.forward_graphed(lat, txt, pooled, t, g, grid=(10, 12)),
                               model(lat, txt, pooled, t, g, grid=(10, 12)))
    cache = model.__dict__["_step_graphs"]
    # per shape: the first call runs eagerly (and is the warm-up), the second captures, every later one replays
    assert cache.captures == 2 and cache.replays == 3
    assert _C.device_status(0, clear=True)[0] == 0


def test_pipeline_whole_image_steps_replay_from_a_graph():
    """The SD3-shaped pipeline without pipeline patches replays its stage forward from a CUDA graph: same latents
    as with the graph switched off, bit for bit, over several steps and two requests."""
    from hetu_dit_b200.config import EngineConfig
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.runtime_state import ModelGeometry, initialize_runtime_state, reset_runtime_state
    from hetu_dit_b200.core.resource_manager.cache_manager import reset_cache_manager
    from hetu_dit_b200.model_executor.models.shaped_dit import DiTShape, ShapedDiT
    from hetu_dit_b200.model_executor.pipelines.pipeline_sd3_shaped import SD3ShapedPipeline
    ps.destroy_model_parallel()
    reset_cache_manager()
    shape = DiTShape("sd3-tiny", 3, 0, 256, 4, 64, 64, 128, 96, False, None, False)
    model = ShapedDiT(shape).to(DEV).init_weights(seed=11, std=0.05).bfloat16()
    rt = initialize_runtime_state(ModelGeometry(4, 64), EngineConfig())
    rt.set_input_parameters(height=512, width=256, batch_size=1, num_inference_steps=3)
    pipe = SD3ShapedPipeline(model, guidance_scale=4.0)
    outs = {}
    for use_graph in (False, True):
        pipe.use_cuda_graph = use_graph
        for req in range(2):
            gen = torch.Generator().manual_seed(40 + req)
            lat = torch.randn(1, 32 * 16, 64, generator=gen).bfloat16().to(DEV)
            prompt = torch.randn(2, 19, 128, generator=gen).bfloat16().to(DEV)
            pooled = torch.randn(2, 96, generator=gen).bfloat16().to(DEV)
            outs[(use_graph, req)] = pipe.diffusion_stage(lat, prompt, pooled, 3).clone()
    torch.cuda.synchronize()
    for req in range(2):
        assert torch.equal(outs[(True, req)], outs[(False, req)]), req
    assert pipe._graphs.captures == 1 and pipe._graphs.replays == 5
    reset_runtime_state()
    reset_cache_manager()

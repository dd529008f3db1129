"""GPU parity of the tcgen05 attention kernel (through the C ABI) against the CPU oracle.

Acceptance for 16-bit activations: cosine similarity >= 0.9999 and
max |got - want| / max |want| <= 2e-2 per output block.
"""
import pytest
import torch

from oracle import attention as oa

pytestmark = pytest.mark.gpu

COS_MIN = 0.9999
MAX_REL = 2e-2
LSE_ATOL = 2e-3


def _mk(shape, dtype, gen, transposed=False):
    B, S, H, D = shape
    if transposed:
        return torch.randn(B, H, S, D, generator=gen, dtype=torch.float32).to(dtype).transpose(1, 2)
    return torch.randn(B, S, H, D, generator=gen, dtype=torch.float32).to(dtype)


def _check(out, lse, qs, ks, vs, scale=None):
    q, k, v = (torch.cat(x, 1) for x in (qs, ks, vs))
    want, want_lse = oa.attention_with_lse(q, k, v, scale)
    cos, rel = oa.cosine_and_max_rel(out.cpu(), want)
    assert cos >= COS_MIN and rel <= MAX_REL, (cos, rel)
    if lse is not None:
        assert (lse.cpu() - want_lse).abs().max().item() <= LSE_ATOL


def _run(qs, ks, vs, **kw):
    from hetu_dit_b200 import _C, kernels
    dev = torch.device("cuda:0")
    out, lse = kernels.attn_fwd([t.to(dev) for t in qs], [t.to(dev) for t in ks], [t.to(dev) for t in vs],
                                return_lse=True, **kw)
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0
    return out, lse


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("sq,skv", [(1, 1), (63, 65), (64, 64), (65, 127), (127, 129), (128, 128), (129, 63),
                                    (300, 500), (256, 1024), (513, 257)])
def test_single_segment(D, sq, skv):
    gen = torch.Generator().manual_seed(sq * 1000 + skv + D)
    q, k, v = _mk((2, sq, 3, D), torch.bfloat16, gen), _mk((2, skv, 3, D), torch.bfloat16, gen), _mk(
        (2, skv, 3, D), torch.bfloat16, gen)
    out, lse = _run([q], [k], [v])
    _check(out, lse, [q], [k], [v])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [64, 128])
def test_joint_segments(D, dtype):
    """[image; text] ("rear") and [text; image] ("front") without a concatenated copy."""
    gen = torch.Generator().manual_seed(7 + D)
    img = [_mk((1, 333, 4, D), dtype, gen) for _ in range(3)]
    txt = [_mk((1, 77, 4, D), dtype, gen) for _ in range(3)]
    for order in ((img, txt), (txt, img)):
        qs, ks, vs = [order[0][0], order[1][0]], [order[0][1], order[1][1]], [order[0][2], order[1][2]]
        out, lse = _run(qs, ks, vs)
        _check(out, lse, qs, ks, vs)


def test_transposed_layout_and_scale():
    gen = torch.Generator().manual_seed(11)
    q, k, v = (_mk((2, 200, 4, 128), torch.bfloat16, gen, transposed=True) for _ in range(3))
    out, lse = _run([q], [k], [v], softmax_scale=0.05)
    _check(out, lse, [q], [k], [v], scale=0.05)


def test_many_kv_segments():
    gen = torch.Generator().manual_seed(12)
    q = _mk((1, 150, 2, 64), torch.bfloat16, gen)
    lens = [5, 128, 129, 1, 64, 200, 33, 17, 256, 90]
    ks = [_mk((1, n, 2, 64), torch.bfloat16, gen) for n in lens]
    vs = [_mk((1, n, 2, 64), torch.bfloat16, gen) for n in lens]
    out, lse = _run([q], ks, vs)
    _check(out, lse, [q], ks, vs)


def test_large_score_range():
    """Scores far apart exercise the lazy running-max rescale of O in TMEM."""
    gen = torch.Generator().manual_seed(13)
    q = _mk((1, 128, 1, 64), torch.bfloat16, gen) * 4
    k = _mk((1, 1024, 1, 64), torch.bfloat16, gen)
    k[:, 512:] *= 6  # later blocks carry much larger scores
    v = _mk((1, 1024, 1, 64), torch.bfloat16, gen)
    out, lse = _run([q], [k], [v])
    _check(out, lse, [q], [k], [v])


@pytest.mark.parametrize("D", [64, 128])
def test_partial_and_merge_modes(D):
    """Ring-style accumulation: PARTIAL_FIRST, PARTIAL_MERGE, MERGE_FINAL over KV blocks == one shot."""
    from hetu_dit_b200 import _C, kernels
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(14 + D)
    q = _mk((2, 190, 3, D), torch.bfloat16, gen).to(dev)
    blocks = [(_mk((2, n, 3, D), torch.bfloat16, gen).to(dev), _mk((2, n, 3, D), torch.bfloat16, gen).to(dev))
              for n in (200, 77, 300)]
    acc = torch.empty(2, 190, 3, D, dtype=torch.float32, device=dev)
    acc_lse = torch.empty(2, 3, 190, dtype=torch.float32, device=dev)
    kernels.attn_fwd([q], [blocks[0][0]], [blocks[0][1]], mode=_C.ATTN_PARTIAL_FIRST, acc_out=acc, acc_lse=acc_lse)
    kernels.attn_fwd([q], [blocks[1][0]], [blocks[1][1]], mode=_C.ATTN_PARTIAL_MERGE, acc_out=acc, acc_lse=acc_lse)
    out, lse = kernels.attn_fwd([q], [blocks[2][0]], [blocks[2][1]], mode=_C.ATTN_MERGE_FINAL, acc_out=acc,
                                acc_lse=acc_lse, return_lse=True)
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0
    _check(out, lse, [q.cpu()], [b[0].cpu() for b in blocks], [b[1].cpu() for b in blocks])


@pytest.mark.parametrize("name,H,D,s_img,s_txt,order", [
    ("sd3-medium", 24, 64, 4096, 333, "rear"),
    ("flux.1-dev", 24, 128, 4096, 512, "front"),
])
def test_baseline_image_shapes(name, H, D, s_img, s_txt, order):
    gen = torch.Generator().manual_seed(15)
    img = [_mk((1, s_img, H, D), torch.bfloat16, gen) for _ in range(3)]
    txt = [_mk((1, s_txt, H, D), torch.bfloat16, gen) for _ in range(3)]
    a, b = (img, txt) if order == "rear" else (txt, img)
    qs, ks, vs = [a[0], b[0]], [a[1], b[1]], [a[2], b[2]]
    out, lse = _run(qs, ks, vs)
    # the CPU oracle on every head would take minutes; check 4 heads fully
    hs = [0, 7, 13, H - 1]
    _check(out[:, :, hs], lse[:, hs], [t[:, :, hs] for t in qs], [t[:, :, hs] for t in ks], [t[:, :, hs] for t in vs])


@pytest.mark.parametrize("name,H,D,s_vid,s_txt", [
    ("cogvideox-1.5-5b", 48, 64, 44880, 224),
    ("hunyuanvideo u4", 6, 128, 118800, 256),
])
def test_video_shapes_properties(name, H, D, s_vid, s_txt):
    """Full-size video sequences: the oracle checks a slice of rows; size-independent
    properties cover the rest (softmax rows sum to one; block merge equals one shot)."""
    from hetu_dit_b200 import _C, kernels
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(16)
    Hs = 2  # two heads of the full-length sequence keep the test to a few seconds
    q = _mk((1, 640, Hs, D), torch.bfloat16, gen).to(dev)
    k = _mk((1, s_vid, Hs, D), torch.bfloat16, gen).to(dev)
    v = _mk((1, s_vid, Hs, D), torch.bfloat16, gen).to(dev)
    tk = _mk((1, s_txt, Hs, D), torch.bfloat16, gen).to(dev)
    tv = _mk((1, s_txt, Hs, D), torch.bfloat16, gen).to(dev)
    out, lse = kernels.attn_fwd([q], [tk, k], [tv, v], return_lse=True)
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0
    _check(out[:, :128], lse[:, :, :128], [q[:, :128].cpu()], [tk.cpu(), k.cpu()], [tv.cpu(), v.cpu()])
    # V = 1 -> every output element is 1 (rows of P sum to one)
    ones_v, ones_t = torch.ones_like(v), torch.ones_like(tv)
    o1 = kernels.attn_fwd([q], [tk, k], [ones_t, ones_v])
    assert (o1.float() - 1).abs().max().item() <= 1e-2
    # two halves merged by log-sum-exp == one shot
    half = s_vid // 2
    acc = torch.empty(1, 640, Hs, D, dtype=torch.float32, device=dev)
    acc_lse = torch.empty(1, Hs, 640, dtype=torch.float32, device=dev)
    kernels.attn_fwd([q], [tk, k[:, :half]], [tv, v[:, :half]], mode=_C.ATTN_PARTIAL_FIRST, acc_out=acc, acc_lse=acc_lse)
    o2, lse2 = kernels.attn_fwd([q], [k[:, half:]], [v[:, half:]], mode=_C.ATTN_MERGE_FINAL, acc_out=acc,
                                acc_lse=acc_lse, return_lse=True)
    torch.cuda.synchronize()
    cos, rel = oa.cosine_and_max_rel(o2, out)
    assert cos >= COS_MIN and rel <= MAX_REL
    assert (lse2 - lse).abs().max().item() <= LSE_ATOL


@pytest.mark.parametrize("D,dtype", [(64, torch.bfloat16), (128, torch.bfloat16), (128, torch.float16)])
@pytest.mark.parametrize("n_split", [2, 3, 16])
def test_split_kv_matches_single_launch(D, dtype, n_split):
    """KV range split over several CTAs per query tile pair + log-sum-exp combine == one launch == oracle.
    Ragged joint segments put a block boundary inside every split; n_split 16 exceeds what 11 KV blocks
    allow, so the library uses fewer."""
    gen = torch.Generator().manual_seed(40 + D + n_split)
    qs = [_mk((2, 300, 3, D), dtype, gen), _mk((2, 77, 3, D), dtype, gen)]
    lens = [77, 640, 333, 129]
    ks = [_mk((2, n, 3, D), dtype, gen) for n in lens]
    vs = [_mk((2, n, 3, D), dtype, gen) for n in lens]
    out, lse = _run(qs, ks, vs, kv_split=n_split)
    _check(out, lse, qs, ks, vs)
    ref, ref_lse = _run(qs, ks, vs, kv_split=1)
    cos, rel = oa.cosine_and_max_rel(out.float().cpu(), ref.float().cpu())
    # both round to 16 bits independently: an element may differ by one unit in the last place
    assert cos >= COS_MIN and rel <= MAX_REL, (cos, rel)
    assert (lse - ref_lse).abs().max().item() <= 1e-4


def test_split_kv_auto_small_grid():
    """The shape one rank sees after the Ulysses exchange at degree 8 of a 24-head model: 3 heads of the whole
    sequence. Left alone, the library fills the GPU by itself (interleaved mode, or a KV split when that mode is
    forbidden); strided output (heads of a wider buffer) is honoured either way."""
    from hetu_dit_b200 import kernels
    gen = torch.Generator().manual_seed(77)
    q, k, v = (_mk((1, 2400, 3, 128), torch.bfloat16, gen) for _ in range(3))
    assert kernels._pick_kv_split([q], [k], 1, 3, kv_interleave=1) > 1
    for interleave in (0, 1):
        wide = torch.zeros(1, 2400, 6, 128, dtype=torch.bfloat16, device="cuda:0")
        out, lse = _run([q], [k], [v], out=wide[:, :, 3:], kv_interleave=interleave)
        _check(out, lse, [q], [k], [v])
        assert wide[:, :, :3].abs().max().item() == 0


def test_split_kv_argument_errors():
    from hetu_dit_b200 import _C, kernels
    dev = torch.device("cuda:0")
    q = torch.zeros(1, 256, 2, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(_C.HditError) as e:
        kernels.attn_fwd([q], [q], [q], kv_split=17)
    assert e.value.code == _C.HDIT_ERR_BAD_ARG


def test_argument_errors():
    from hetu_dit_b200 import _C, kernels
    dev = torch.device("cuda:0")
    q = torch.zeros(1, 8, 2, 96, dtype=torch.bfloat16, device=dev)
    with pytest.raises(_C.HditError) as e:
        kernels.attn_fwd([q], [q], [q])
    assert e.value.code == _C.HDIT_ERR_SHAPE
    q = torch.zeros(1, 8, 2, 64, dtype=torch.bfloat16, device=dev)
    empty = torch.zeros(1, 0, 2, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(_C.HditError):
        kernels.attn_fwd([q], [empty], [empty])
    with pytest.raises(TypeError):
        kernels.attn_fwd([q.float()], [q.float()], [q.float()])


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("sq,lens", [(1, (1,)), (128, (128, 128)), (129, (643,)), (300, (1500, 20)), (77, (200,)),
                                     (260, (5, 128, 129, 1, 64))])
def test_interleaved_kv_mode_matches_oracle(D, sq, lens):
    """One query tile per CTA, even / odd KV blocks on its two halves, merged in shared memory: odd and even
    block counts, a single block (half 1 idle), ragged tails, several segments."""
    gen = torch.Generator().manual_seed(sq + sum(lens) + D)
    q = _mk((2, sq, 3, D), torch.bfloat16, gen)
    ks = [_mk((2, n, 3, D), torch.bfloat16, gen) for n in lens]
    vs = [_mk((2, n, 3, D), torch.bfloat16, gen) for n in lens]
    out, lse = _run([q], ks, vs, kv_split=1, kv_interleave=2)
    _check(out, lse, [q], ks, vs)


def test_interleaved_kv_mode_partial_and_merge():
    """The interleaved mode under the ring's PARTIAL_FIRST -> MERGE_FINAL sequence equals one shot."""
    from hetu_dit_b200 import _C, kernels
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(31)
    q = _mk((1, 300, 2, 128), torch.bfloat16, gen).to(dev)
    k1, v1, k2, v2 = (_mk((1, n, 2, 128), torch.bfloat16, gen).to(dev) for n in (700, 700, 400, 400))
    acc = torch.empty(1, 300, 2, 128, device=dev)
    acc_lse = torch.empty(1, 2, 300, device=dev)
    kernels.attn_fwd([q], [k1], [v1], mode=_C.ATTN_PARTIAL_FIRST, acc_out=acc, acc_lse=acc_lse, kv_interleave=2)
    out, lse = kernels.attn_fwd([q], [k2], [v2], mode=_C.ATTN_MERGE_FINAL, acc_out=acc, acc_lse=acc_lse,
                                return_lse=True, kv_interleave=2)
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0
    _check(out, lse, [q.cpu()], [k1.cpu(), k2.cpu()], [v1.cpu(), v2.cpu()])


@pytest.mark.parametrize("kv_split,kv_interleave", [(1, 1), (1, 2), (2, 1)])
def test_result_scatter_from_the_epilogue(kv_split, kv_interleave):
    """The attention epilogue (or the split-KV merge pass) stores each result row into the buffer of the rank
    that owns it: joint rows to every destination, image rows of owner u to destination u -- bit-identical to
    the plain call followed by the copy, for the paired, the interleaved and the split-KV launch."""
    from hetu_dit_b200 import _C, kernels
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(41)
    B, H, D, U, S, J = 2, 2, 128, 4, 96, 100
    jq, iq = _mk((B, J, H, D), torch.bfloat16, gen).to(dev), _mk((B, U * S, H, D), torch.bfloat16, gen).to(dev)
    k, v = _mk((B, 900, H, D), torch.bfloat16, gen).to(dev), _mk((B, 900, H, D), torch.bfloat16, gen).to(dev)
    plain = kernels.attn_fwd([jq, iq], [k], [v], kv_split=kv_split, kv_interleave=kv_interleave)
    # destinations are wider than the slice written (2 * H heads), as the peers' gathered output buffers are
    bufs = [torch.zeros(B, J + S, 2 * H, D, device=dev, dtype=torch.bfloat16) for _ in range(U)]
    dst = kernels.RawDst([x[:, :, H:].data_ptr() for x in bufs], bufs[0].stride()[:3])
    kernels.attn_fwd([jq, iq], [k], [v], kv_split=kv_split, kv_interleave=kv_interleave, out_dsts=dst,
                     q_rows_per_dst=[0, S], q_dst_row0=[0, J])
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0
    for u in range(U):
        assert torch.equal(bufs[u][:, :J, H:], plain[:, :J])
        assert torch.equal(bufs[u][:, J:, H:], plain[:, J + u * S:J + (u + 1) * S])
        assert bufs[u][:, :, :H].abs().max().item() == 0
    _check(plain, None, [jq.cpu(), iq.cpu()], [k.cpu()], [v.cpu()])


@pytest.mark.parametrize("strategy", ["none", "rear", "front"])
def test_ulysses_only_operator_on_one_rank(strategy):
    """hetuDiTUlyssesAttention (the reference's core/parallel/ulysses/attn_layer.py:12-155) with an Ulysses group of
    one rank: the text rows join the image rows behind ("rear") or in front ("front") in Q, K and V, no exchange."""
    from hetu_dit_b200 import _C
    from hetu_dit_b200.core.parallel import hetuDiTUlyssesAttention
    gen = torch.Generator().manual_seed(31)
    dev = torch.device("cuda:0")
    q, k, v = (_mk((1, 200, 4, 64), torch.bfloat16, gen) for _ in range(3))
    jq, jk, jv = (_mk((1, 24, 4, 64), torch.bfloat16, gen) for _ in range(3))
    layer = hetuDiTUlyssesAttention(use_fa=False, use_kv_cache=False)
    kw = {}
    if strategy != "none":
        kw = dict(joint_tensor_query=jq.to(dev), joint_tensor_key=jk.to(dev), joint_tensor_value=jv.to(dev),
                  joint_strategy=strategy)
    out = layer(None, q.to(dev), k.to(dev), v.to(dev), **kw)
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0

    def join(x, j):
        return x if strategy == "none" else torch.cat([x, j] if strategy == "rear" else [j, x], dim=1)

    want, _ = oa.attention_with_lse(join(q, jq), join(k, jk), join(v, jv), None)
    cos, rel = oa.cosine_and_max_rel(out.cpu(), want)
    assert out.shape == want.shape and cos >= COS_MIN and rel <= MAX_REL, (cos, rel)
    with pytest.raises(ValueError):
        layer(None, q.to(dev), k.to(dev), v.to(dev), joint_tensor_query=jq.to(dev), joint_tensor_key=jk.to(dev),
              joint_tensor_value=jv.to(dev), joint_strategy="none")

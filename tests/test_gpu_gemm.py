"""GPU parity of the fused linear layer (C ABI: hdit_linear_fused) against an fp32 torch restatement of what the
reference runs unfused: torch.nn.Linear (one rounding to 16 bits), then the eager GELU or gated residual
(layers/feedforward.py:73-78 and the residual additions around layers/attention_processor.py:207-449).

Tolerance for 16-bit activations: cosine >= 0.9999 and max|a - b| / max|b| <= 2e-2 per case."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _want(x, w, b, epilogue, residual=None, gate=None):
    y = F.linear(x.float(), w.float(), b.float() if b is not None else None).to(x.dtype).float()
    if epilogue == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    elif epilogue == "gate_residual":
        y = residual.float() + gate.float()[:, None, :] * y
    return y.to(x.dtype)


def _check(got, want):
    g, w = got.float().flatten(), want.float().flatten()
    assert torch.isfinite(g).all()
    cos = F.cosine_similarity(g, w, dim=0).item()
    rel = ((g - w).abs().max() / w.abs().max().clamp_min(1e-6)).item()
    assert cos >= 0.9999 and rel <= 2e-2, (cos, rel)


def _inputs(B, S, K, N, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(B, S, K, generator=gen).to(dtype).to(DEV)
    w = (torch.randn(N, K, generator=gen) / K ** 0.5).to(dtype).to(DEV)
    b = torch.randn(N, generator=gen).to(dtype).to(DEV)
    res = torch.randn(B, S, N, generator=gen).to(dtype).to(DEV)
    gate = torch.randn(B, N, generator=gen).to(dtype).to(DEV)
    return x, w, b, res, gate


# (tile_m, tile_n, cta_pair): 0 = the library chooses; cta_pair 2 = two CTAs share a 256 x 256 tile
TILES = [(0, 0, 0), (128, 128, 1), (128, 256, 1), (256, 256, 1), (0, 0, 2)]


@pytest.mark.parametrize("epilogue", ["bias", "gelu_tanh", "gate_residual"])
@pytest.mark.parametrize("tile", TILES, ids=lambda t: f"tile{t[0]}x{t[1]}pair{t[2]}")
@pytest.mark.parametrize("B,S,K,N", [(1, 128, 64, 256), (1, 300, 200, 264), (2, 333, 1024, 1160), (1, 576, 3072, 3072)])
def test_linear_fused_matches_unfused_chain(B, S, K, N, tile, epilogue):
    from hetu_dit_b200 import kernels
    x, w, b, res, gate = _inputs(B, S, K, N, torch.bfloat16, B * 1000 + S + K + N)
    got = kernels.linear_fused(x, w, b, epilogue=epilogue, residual=res, gate=gate, tile_m=tile[0], tile_n=tile[1],
                               cta_pair=tile[2])
    torch.cuda.synchronize()
    _check(got, _want(x, w, b, epilogue, res, gate))


def test_linear_fused_many_tiles_per_cta_and_long_k():
    """Few persistent CTAs walk many tiles: both accumulators and every ring stage are re-used many times."""
    from hetu_dit_b200 import kernels
    x, w, b, res, gate = _inputs(1, 1100, 4160, 1544, torch.bfloat16, 7)
    for tile_m, tile_n, pair in TILES[1:]:
        for ctas in (2, 3, 7):
            got = kernels.linear_fused(x, w, b, epilogue="gate_residual", residual=res, gate=gate, tile_m=tile_m,
                                       tile_n=tile_n, max_ctas=ctas, cta_pair=pair)
            torch.cuda.synchronize()
            _check(got, _want(x, w, b, "gate_residual", res, gate))


def test_linear_fused_fp16_no_bias_strided_and_in_place():
    from hetu_dit_b200 import kernels
    x, w, b, res, gate = _inputs(2, 200, 512, 384, torch.float16, 11)
    for pair in (1, 2):
        got = kernels.linear_fused(x, w, None, epilogue="bias", cta_pair=pair)
        _check(got, _want(x, w, None, "bias"))
    # the result lands in a column block of a wider buffer; rows of x are a column block too
    wide_in = torch.zeros(2, 200, 512 + 64, dtype=torch.float16, device=DEV)
    wide_in[..., 64:] = x
    wide_out = torch.full((2, 200, 1024), 7.0, dtype=torch.float16, device=DEV)
    kernels.linear_fused(wide_in[..., 64:], w, b, epilogue="gelu_tanh", out=wide_out[..., 128:128 + 384])
    torch.cuda.synchronize()
    _check(wide_out[..., 128:128 + 384], _want(x, w, b, "gelu_tanh"))
    assert (wide_out[..., :128] == 7.0).all() and (wide_out[..., 128 + 384:] == 7.0).all()
    # out aliases the residual
    want = _want(x, w, b, "gate_residual", res, gate)
    kernels.linear_fused(x, w, b, epilogue="gate_residual", residual=res, gate=gate, out=res)
    torch.cuda.synchronize()
    _check(res, want)


def test_linear_fused_two_dim_and_argument_errors():
    from hetu_dit_b200 import _C, kernels
    x, w, b, _, _ = _inputs(1, 130, 128, 136, torch.bfloat16, 13)
    got = kernels.linear_fused(x[0], w, b)
    torch.cuda.synchronize()
    _check(got, _want(x, w, b, "bias")[0])
    with pytest.raises(_C.HditError):
        kernels.linear_fused(x[..., :60], w[:, :60].contiguous(), b)  # k not a multiple of 8
    with pytest.raises(_C.HditError):
        kernels.linear_fused(x, w, b, tile_n=64)
    with pytest.raises(_C.HditError):
        kernels.linear_fused(x, w, b, tile_n=128, cta_pair=2)
    with pytest.raises(ValueError):
        kernels.linear_fused(x, w[:, :64], b)


def test_linear_fused_flux_mlp_shapes():
    """The shapes of one Flux single block at full size: (4608, 3072) x (12288, 3072)^T with GELU, then
    (4608, 15360) x (3072, 15360)^T with the gated residual; checked on a row subset."""
    from hetu_dit_b200 import kernels
    gen = torch.Generator(device=DEV).manual_seed(5)
    d = 3072
    x = torch.randn(1, 4608, d, device=DEV, generator=gen).to(torch.bfloat16)
    w1 = (torch.randn(4 * d, d, device=DEV, generator=gen) / d ** 0.5).to(torch.bfloat16)
    b1 = torch.randn(4 * d, device=DEV, generator=gen).to(torch.bfloat16)
    w2 = (torch.randn(d, 5 * d, device=DEV, generator=gen) / (5 * d) ** 0.5).to(torch.bfloat16)
    b2 = torch.randn(d, device=DEV, generator=gen).to(torch.bfloat16)
    gate = torch.randn(1, d, device=DEV, generator=gen).to(torch.bfloat16)
    buf = torch.randn(1, 4608, 5 * d, device=DEV, generator=gen).to(torch.bfloat16)
    rows = torch.arange(0, 4608, 37, device=DEV)
    for pair in (1, 2):
        buf[..., d:].zero_()
        kernels.linear_fused(x, w1, b1, epilogue="gelu_tanh", out=buf[..., d:], cta_pair=pair)
        out = kernels.linear_fused(buf, w2, b2, epilogue="gate_residual", residual=x, gate=gate, cta_pair=pair)
        torch.cuda.synchronize()
        _check(buf[:, rows, d:], _want(x[:, rows], w1, b1, "gelu_tanh"))
        _check(out[:, rows], _want(buf[:, rows], w2, b2, "gate_residual", x[:, rows], gate))

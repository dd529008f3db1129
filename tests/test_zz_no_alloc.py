"""The allocation-free two-pass attention entry point against the ordinary one.

hdit_attn_fwd_split_static serves hosts that cannot allocate device memory around a call (all HBM owned
by their own pool, or no tolerance for the device-wide synchronisation an allocation implies): its fp32
partial result sits in a static device array of the library. Here it is driven through the C ABI with
caller-owned inputs and outputs only, twice in a row on different data (the array is shared and keeps
the previous call's contents), and must agree with hdit_attn_fwd within the activation tolerance of the
other attention tests (cosine >= 0.9999, max |a-b| / max |b| <= 2e-2; log-sum-exp within 2e-3).
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(_C, qs, ks, vs, out, lse):
    B, _, H, D = qs[0].shape
    a = _C.AttnArgs()
    a.dtype, a.mode, a.batch, a.heads, a.head_dim = _C.HDIT_BF16, _C.ATTN_FINAL, B, H, D
    a.n_q_seg, a.n_kv_seg, a.softmax_scale = len(qs), len(ks), 0.0

    def fill(seg, t):
        seg.ptr, seg.len = t.data_ptr(), t.shape[1]
        seg.stride_b, seg.stride_s, seg.stride_h = t.stride(0), t.stride(1), t.stride(2)

    for i, t in enumerate(qs):
        fill(a.q[i], t)
    for i, (k, v) in enumerate(zip(ks, vs)):
        fill(a.k[i], k)
        fill(a.v[i], v)
    a.out, a.lse = out.data_ptr(), lse.data_ptr()
    a.out_stride_b, a.out_stride_s, a.out_stride_h = out.stride(0), out.stride(1), out.stride(2)
    a.stream = torch.cuda.current_stream().cuda_stream
    return a


def test_split_static_matches_plain_entry_point_twice():
    from hetu_dit_b200 import _C
    from oracle import attention as oa
    lib = _C.lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    for call, (B, H, D, sq, lens, split) in enumerate([(2, 3, 128, 300, (257, 64, 190), 1),
                                                       (1, 4, 64, 515, (100, 333, 40, 129), 2)]):
        gen = torch.Generator(device=dev).manual_seed(100 + call)

        def mk(n):
            return torch.randn(B, n, H, D, generator=gen, device=dev, dtype=torch.float32).bfloat16()

        q = mk(sq)
        ks, vs = [mk(n) for n in lens], [mk(n) for n in lens]
        out_ref = torch.empty(B, sq, H, D, dtype=torch.bfloat16, device=dev)
        lse_ref = torch.empty(B, H, sq, dtype=torch.float32, device=dev)
        out_new = torch.full_like(out_ref, float("nan"))
        lse_new = torch.full_like(lse_ref, float("nan"))
        _C.check(lib.hdit_attn_fwd(ctypes.byref(_args(_C, [q], ks, vs, out_ref, lse_ref))))
        _C.check(lib.hdit_attn_fwd_split_static(ctypes.byref(_args(_C, [q], ks, vs, out_new, lse_new)), split))
        torch.cuda.synchronize()
        assert _C.device_status(0, clear=True)[0] == 0
        cos, rel = oa.cosine_and_max_rel(out_new, out_ref)
        assert cos >= 0.9999 and rel <= 2e-2, (call, cos, rel)
        assert (lse_new - lse_ref).abs().max().item() <= 2e-3
        # and against the CPU oracle of the whole (unsplit) attention
        want, want_lse = oa.attention_with_lse(q.cpu(), torch.cat([t.cpu() for t in ks], 1),
                                               torch.cat([t.cpu() for t in vs], 1))
        cos, rel = oa.cosine_and_max_rel(out_new.cpu(), want)
        assert cos >= 0.9999 and rel <= 2e-2, ("oracle", call, cos, rel)
        assert (lse_new.cpu() - want_lse).abs().max().item() <= 2e-3


@pytest.mark.parametrize("B,sq,H,D", [(1, 4096, 16, 128), (1, 2048, 64, 64)])
def test_split_static_at_its_documented_limit(B, sq, H, D):
    """Exactly the largest problems the static array holds: 8 Mi accumulator elements (4096 x 16 x 128) and
    128 Ki log-sum-exp entries (2048 x 64 at head_dim 64, which is also 8 Mi accumulator elements). Checked
    against the ordinary entry point everywhere and against the CPU oracle on a subset of heads and rows."""
    from hetu_dit_b200 import _C
    from oracle import attention as oa
    lib = _C.lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    assert B * sq * H * D == 8 << 20 and B * H * sq <= 128 << 10
    gen = torch.Generator(device=dev).manual_seed(7 + D)

    def mk(n):
        return torch.randn(B, n, H, D, generator=gen, device=dev, dtype=torch.float32).bfloat16()

    q = mk(sq)
    lens = (300, 129)
    ks, vs = [mk(n) for n in lens], [mk(n) for n in lens]
    out_ref = torch.empty(B, sq, H, D, dtype=torch.bfloat16, device=dev)
    lse_ref = torch.empty(B, H, sq, dtype=torch.float32, device=dev)
    out_new = torch.full_like(out_ref, float("nan"))
    lse_new = torch.full_like(lse_ref, float("nan"))
    _C.check(lib.hdit_attn_fwd(ctypes.byref(_args(_C, [q], ks, vs, out_ref, lse_ref))))
    _C.check(lib.hdit_attn_fwd_split_static(ctypes.byref(_args(_C, [q], ks, vs, out_new, lse_new)), 1))
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0
    cos, rel = oa.cosine_and_max_rel(out_new, out_ref)
    assert cos >= 0.9999 and rel <= 2e-2, (cos, rel)
    assert (lse_new - lse_ref).abs().max().item() <= 2e-3
    hs, rows = [0, H - 1], slice(sq - 257, sq)   # the last rows and heads sit at the end of the static array
    want, want_lse = oa.attention_with_lse(q[:, rows][:, :, hs].cpu(), torch.cat([t[:, :, hs].cpu() for t in ks], 1),
                                           torch.cat([t[:, :, hs].cpu() for t in vs], 1))
    cos, rel = oa.cosine_and_max_rel(out_new[:, rows][:, :, hs].cpu(), want)
    assert cos >= 0.9999 and rel <= 2e-2, ("oracle", cos, rel)
    assert (lse_new[:, hs][:, :, rows].cpu() - want_lse).abs().max().item() <= 2e-3


def test_split_static_rejects_oversize_and_bad_split():
    from hetu_dit_b200 import _C
    lib = _C.lib()
    dev = torch.device("cuda:0")
    q = torch.zeros(1, 4096, 24, 128, dtype=torch.bfloat16, device=dev)  # 12.6 M accumulator elements > 8 Mi
    k = torch.zeros(1, 128, 24, 128, dtype=torch.bfloat16, device=dev)
    out = torch.empty_like(q)
    lse = torch.empty(1, 24, 4096, dtype=torch.float32, device=dev)
    a = _args(_C, [q], [k, k], [k, k], out, lse)
    assert lib.hdit_attn_fwd_split_static(ctypes.byref(a), 1) == _C.HDIT_ERR_TOO_LARGE
    assert b"static scratch too small" in lib.hdit_last_error()
    small = torch.zeros(1, 64, 2, 64, dtype=torch.bfloat16, device=dev)
    a = _args(_C, [small], [small, small], [small, small], torch.empty_like(small),
              torch.empty(1, 2, 64, dtype=torch.float32, device=dev))
    assert lib.hdit_attn_fwd_split_static(ctypes.byref(a), 0) == _C.HDIT_ERR_BAD_ARG
    assert lib.hdit_attn_fwd_split_static(ctypes.byref(a), 2) == _C.HDIT_ERR_BAD_ARG

"""Tensor-level entry points over the C ABI (torch is used for device memory and streams only)."""
import ctypes

import torch

from . import _C

_DTYPE_CODE = {torch.bfloat16: _C.HDIT_BF16, torch.float16: _C.HDIT_FP16}


def _stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _fill_seg(seg, t):
    if t.dim() != 4:
        raise ValueError(f"expected a (B, S, H, D) tensor, got shape {tuple(t.shape)}")
    if t.stride(3) != 1 and t.shape[3] != 1:
        raise ValueError("the head dimension must be contiguous")
    seg.ptr = t.data_ptr()
    seg.len = t.shape[1]
    seg.stride_b = t.stride(0)
    seg.stride_s = t.stride(1)
    seg.stride_h = t.stride(2)


def attn_fwd(
    q_segs,
    k_segs,
    v_segs,
    *,
    softmax_scale=None,
    out=None,
    return_lse=False,
    mode=_C.ATTN_FINAL,
    acc_out=None,
    acc_lse=None,
):
    """softmax(Q K^T * scale) V over segment lists, (B, S, H, D) layout.

    q_segs / k_segs / v_segs are lists of tensors that are logically concatenated
    along S (no copy is made). Returns `out` of shape (B, sum Sq, H, D) in the input
    dtype (and the (B, H, Sq) fp32 log-sum-exp when return_lse is set). In the
    PARTIAL modes nothing is returned; the fp32 running result lives in acc_out /
    acc_lse, which a later MERGE call combines with its own block by log-sum-exp.
    """
    q0 = q_segs[0]
    if not q0.is_cuda:
        raise RuntimeError("hetu_dit_b200 kernels need CUDA tensors; there is no CPU path")
    if q0.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported dtype {q0.dtype}")
    if len(k_segs) != len(v_segs):
        raise ValueError("k and v segment lists differ in length")
    B, _, H, D = q0.shape
    sq = sum(int(t.shape[1]) for t in q_segs)
    a = _C.AttnArgs()
    a.dtype = _DTYPE_CODE[q0.dtype]
    a.mode = mode
    a.batch, a.heads, a.head_dim = B, H, D
    a.n_q_seg, a.n_kv_seg = len(q_segs), len(k_segs)
    a.softmax_scale = float(softmax_scale) if softmax_scale is not None else 0.0
    if len(q_segs) > _C.HDIT_MAX_Q_SEG or len(k_segs) > _C.HDIT_MAX_KV_SEG:
        raise ValueError("too many segments")
    for i, t in enumerate(q_segs):
        _fill_seg(a.q[i], t)
    for i, (k, v) in enumerate(zip(k_segs, v_segs)):
        _fill_seg(a.k[i], k)
        _fill_seg(a.v[i], v)
    writes_out = mode in (_C.ATTN_FINAL, _C.ATTN_MERGE_FINAL)
    lse = None
    if writes_out:
        if out is None:
            out = torch.empty((B, sq, H, D), dtype=q0.dtype, device=q0.device)
        a.out = out.data_ptr()
        a.out_stride_b, a.out_stride_s, a.out_stride_h = out.stride(0), out.stride(1), out.stride(2)
        if return_lse:
            lse = torch.empty((B, H, sq), dtype=torch.float32, device=q0.device)
            a.lse = lse.data_ptr()
    if mode != _C.ATTN_FINAL:
        if acc_out is None or acc_lse is None:
            raise ValueError("acc_out and acc_lse are required for partial / merge modes")
        if acc_out.dtype != torch.float32 or acc_lse.dtype != torch.float32:
            raise TypeError("acc_out / acc_lse must be fp32")
        if tuple(acc_out.shape) != (B, sq, H, D) or not acc_out.is_contiguous():
            raise ValueError("acc_out must be contiguous (B, Sq, H, D)")
        if tuple(acc_lse.shape) != (B, H, sq) or not acc_lse.is_contiguous():
            raise ValueError("acc_lse must be contiguous (B, H, Sq)")
        a.acc_out = acc_out.data_ptr()
        a.acc_lse = acc_lse.data_ptr()
    a.stream = _stream_ptr(q0.device)
    with torch.cuda.device(q0.device):
        _C.check(_C.lib().hdit_attn_fwd(ctypes.byref(a)))
    if not writes_out:
        return None
    return (out, lse) if return_lse else out

"""Tensor-level entry points over the C ABI (torch is used for device memory and streams only)."""
import ctypes
import os

import torch

from . import _C

_DTYPE_CODE = {torch.bfloat16: _C.HDIT_BF16, torch.float16: _C.HDIT_FP16}

# Launch accounting for benchmarks: how many kernels of this library were enqueued, and
# (optionally) CUDA-event pairs around every attention launch on its own stream.
_launches = 0
_attn_timing = False
_attn_events = []


def reset_counters():
    global _launches
    _launches = 0
    _attn_events.clear()


def launch_count() -> int:
    return _launches


def enable_attn_timing(on: bool):
    global _attn_timing
    _attn_timing = bool(on)


def attn_timing_summary():
    """Mean device time of the attention launches recorded since reset_counters() (synchronises)."""
    torch.cuda.synchronize()
    ms = [a.elapsed_time(b) for a, b, _ in _attn_events]
    return {"count": len(ms), "mean_ms": (sum(ms) / len(ms)) if ms else None, "min_ms": min(ms) if ms else None,
            "total_ms": sum(ms), "flops": float(sum(f for _, _, f in _attn_events))}


def _count(n=1):
    global _launches
    _launches += n


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
    kv_split=None,
    kv_interleave=0,
    out_dsts=None,
    q_rows_per_dst=None,
    q_dst_row0=None,
    wait_flags=None,
):
    """softmax(Q K^T * scale) V over segment lists, (B, S, H, D) layout.

    q_segs / k_segs / v_segs are lists of tensors that are logically concatenated
    along S (no copy is made). Returns `out` of shape (B, sum Sq, H, D) in the input
    dtype (and the (B, H, Sq) fp32 log-sum-exp when return_lse is set). In the
    PARTIAL modes nothing is returned; the fp32 running result lives in acc_out /
    acc_lse, which a later MERGE call combines with its own block by log-sum-exp.

    kv_split (FINAL mode only): number of CTAs that share one query tile pair, each over its own
    range of KV blocks, merged by a second small kernel. None picks it from the grid size: a head-
    and sequence-sharded call can have fewer tile pairs than the GPU has SMs.
    kv_interleave: 0 lets the library decide, 1 forbids, 2 forces the mode in which a CTA owns one query tile
    and its two halves take the even and odd KV blocks (merged in shared memory; for small grids).

    out_dsts (a RawDst: device addresses + (b, s, h) element strides): scatter the result rows over these
    buffers instead of returning one tensor -- row r of query segment s goes to destination
    r // q_rows_per_dst[s] at row q_dst_row0[s] + r % q_rows_per_dst[s], or to every destination at row
    q_dst_row0[s] + r when q_rows_per_dst[s] is 0. With the Ulysses peers' output buffers as destinations this
    is the reverse all-to-all done by the attention epilogue. Returns None (or the lse) in that case.

    wait_flags (a FlagWait): flags in this rank's memory that the peers' exchange kernels bump; the kernel's
    loader waits for them before its first load (the barrier after the head exchange, folded into attention).
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
    a.kv_interleave = int(kv_interleave)
    if writes_out and out_dsts is not None:
        a.n_out_dst = len(out_dsts)
        for i, ptr in enumerate(out_dsts.ptrs):
            a.out_dst[i] = ptr
        a.out_stride_b, a.out_stride_s, a.out_stride_h = out_dsts.strides
        for i in range(len(q_segs)):
            a.q_rows_per_dst[i] = int(q_rows_per_dst[i])
            a.q_dst_row0[i] = int(q_dst_row0[i])
        if return_lse:
            lse = torch.empty((B, H, sq), dtype=torch.float32, device=q0.device)
            a.lse = lse.data_ptr()
    elif writes_out:
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
    if wait_flags is not None:
        a.n_wait = len(wait_flags.slots)
        for i, ptr in enumerate(wait_flags.slots):
            a.wait_slots[i] = ptr
        a.wait_epoch = wait_flags.epoch_ptr
        a.wait_spins = int(wait_flags.max_spins)
    a.stream = _stream_ptr(q0.device)
    n_split = 1
    if mode == _C.ATTN_FINAL:
        n_split = _pick_kv_split(q_segs, k_segs, B, H, kv_interleave) if kv_split is None else int(kv_split)
    with torch.cuda.device(q0.device):
        if n_split > 1:
            part_out = torch.empty((n_split, B, sq, H, D), dtype=torch.float32, device=q0.device)
            part_lse = torch.empty((n_split, B, H, sq), dtype=torch.float32, device=q0.device)
            call = lambda: _C.lib().hdit_attn_fwd_splitkv(ctypes.byref(a), n_split, part_out.data_ptr(),
                                                          part_lse.data_ptr())
        else:
            call = lambda: _C.lib().hdit_attn_fwd(ctypes.byref(a))
        if _attn_timing:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _C.check(call())
            e1.record()
            skv = sum(int(t.shape[1]) for t in k_segs)
            _attn_events.append((e0, e1, 4.0 * B * sq * skv * H * D))
        else:
            _C.check(call())
    _count(2 if n_split > 1 else 1)
    if not writes_out:
        return None
    if out_dsts is not None:
        return lse
    return (out, lse) if return_lse else out


_SM_COUNT = 148


def _interleave_cost(q_tiles, kv_blocks, batch, heads):
    """Cost (in KV blocks of one paired CTA) of running one query tile per CTA with the KV blocks interleaved
    over its two halves; the constants are the library's own (csrc/attn_sm100.cu)."""
    ctas_il = q_tiles * heads * batch
    return -(-ctas_il // _SM_COUNT) * ((kv_blocks + 1) // 2 * 1.12 + 6.0)


def _pick_kv_split(q_segs, k_segs, batch, heads, kv_interleave=0):
    """How many ways to split the KV range. One CTA per SM runs a pair of 128-row query tiles over all KV
    blocks, so the launch takes ceil(ctas / SMs) waves; splitting the KV range s ways makes waves of 1/s the
    length and pays a fixed cost per CTA plus the merge pass. Costs are in units of one KV block of one CTA
    (about 2 us at head_dim 128), fitted to timings of 3..12 heads at 4.6k and 17.8k tokens; a split must
    promise 10 % to be taken."""
    q_tiles = sum((int(t.shape[1]) + 127) // 128 for t in q_segs)
    ctas = (q_tiles + 1) // 2 * heads * batch
    kv_blocks = sum((int(t.shape[1]) + 127) // 128 for t in k_segs)
    if ctas <= 0:
        return 1
    if kv_interleave == 2:
        return 1
    sq = sum(int(t.shape[1]) for t in q_segs)
    part_bytes = batch * sq * heads * int(q_segs[0].shape[3]) * 4

    def cost(s):
        waves = -(-ctas * s // _SM_COUNT)
        c = waves * (kv_blocks / s + 6.0)
        return c if s == 1 else c + 5.0 + part_bytes * s / 1e7

    best, best_cost = 1, cost(1) * 0.9
    if kv_interleave == 0 and kv_blocks >= 2:
        # without a split the library itself may interleave; a split has to beat that too
        best_cost = min(best_cost, _interleave_cost(q_tiles, kv_blocks, batch, heads) * 0.95)
    for s in (2, 3, 4):
        if kv_blocks // s >= 4 and cost(s) < best_cost:
            best, best_cost = s, cost(s)
    return best


def copy_pieces(pieces, device):
    """Moves a list of (src_ptr, dst_ptr, n_outer, src_outer_pitch, dst_outer_pitch, rows, src_pitch,
    dst_pitch, row_bytes) boxes (all byte units) on `device`'s current stream."""
    n = len(pieces)
    if n == 0:
        return
    arr = (_C.CopyPiece * n)()
    for i, pc in enumerate(pieces):
        (arr[i].src, arr[i].dst, arr[i].n_outer, arr[i].src_outer_pitch, arr[i].dst_outer_pitch, arr[i].rows,
         arr[i].src_pitch, arr[i].dst_pitch, arr[i].row_bytes) = pc
    with torch.cuda.device(device):
        _C.check(_C.lib().hdit_copy_pieces(arr, n, _stream_ptr(device)))
    _count((n + 39) // 40)


def copy_2d(dst, src):
    """dst[...] = src[...] for two same-shape views whose last dim is contiguous and whose leading dims
    collapse to at most (outer, rows); used for patch hand-off and slice copies."""
    if dst.shape != src.shape or dst.dtype != src.dtype:
        raise ValueError("shape / dtype mismatch")
    if dst.numel() == 0:
        return
    es = src.element_size()
    pieces = [(s.data_ptr(), d.data_ptr(), o, sop * es, dop * es, r, sp * es, dp * es, rb * es)
              for (s, d, o, sop, dop, r, sp, dp, rb) in _collapse(src, dst)]
    copy_pieces(pieces, src.device if src.is_cuda else dst.device)


def _collapse(src, dst):
    """Splits a same-shape (src, dst) view pair into 3-level boxes (element units)."""
    shape = list(src.shape)
    ss, ds = list(src.stride()), list(dst.stride())
    # drop size-1 dims, merge dims that are contiguous in both tensors
    dims = [(n, a, b) for n, a, b in zip(shape, ss, ds) if n != 1]
    if not dims:
        return [(src, dst, 1, 0, 0, 1, 0, 0, 1)]
    merged = [dims[-1]]
    for n, a, b in reversed(dims[:-1]):
        n0, a0, b0 = merged[0]
        if a == a0 * n0 and b == b0 * n0:
            merged[0] = (n * n0, a0, b0)
        else:
            merged.insert(0, (n, a, b))
    if merged[-1][1] != 1 or merged[-1][2] != 1:
        raise ValueError("innermost dimension must be contiguous in both tensors")
    row = merged[-1][0]
    lead = merged[:-1]
    if len(lead) == 0:
        return [(src, dst, 1, 0, 0, 1, 0, 0, row)]
    if len(lead) == 1:
        return [(src, dst, 1, 0, 0, lead[0][0], lead[0][1], lead[0][2], row)]
    if len(lead) == 2:
        return [(src, dst, lead[0][0], lead[0][1], lead[0][2], lead[1][0], lead[1][1], lead[1][2], row)]
    # more than two leading levels: peel the outermost
    out = []
    for i in range(shape[0]):
        out.extend(_collapse(src[i], dst[i]))
    return out


def kv_scatter(kv_cache, new_k, new_v, token_start):
    """kv_cache: (B, S, 2*R) stale buffer in the [K || V] layout; new_k / new_v: (B, n, R)-shaped views
    (any trailing dims, rows contiguous). Writes rows [token_start, token_start + n)."""
    B, S = kv_cache.shape[0], kv_cache.shape[1]
    nk = new_k.reshape(B, new_k.shape[1], -1) if new_k.dim() != 3 else new_k
    nv = new_v.reshape(B, new_v.shape[1], -1) if new_v.dim() != 3 else new_v
    n, R = nk.shape[1], nk.shape[2]
    if kv_cache.shape[2] != 2 * R or not kv_cache.is_contiguous():
        raise ValueError("kv_cache must be contiguous (B, S, 2*row)")
    if nk.stride(2) != 1 or nv.stride(2) != 1 or nk.stride() != nv.stride():
        raise ValueError("new_k / new_v rows must be contiguous and share strides")
    es = kv_cache.element_size()
    with torch.cuda.device(kv_cache.device):
        _C.check(_C.lib().hdit_kv_scatter(kv_cache.data_ptr(), nk.data_ptr(), nv.data_ptr(), B, S, int(token_start), n,
                                          R * es, nk.stride(1) * es, nk.stride(0) * es, _stream_ptr(kv_cache.device)))
    _count()


class FlagSignal:
    """Where an exchange kernel publishes "my rows have landed": for every peer the address (in that peer's
    memory) of the flag this rank bumps (None at this rank's own index), this rank's index, and the device
    addresses of this rank's epoch counter and ticket word."""

    def __init__(self, slots, me, epoch_ptr, ticket_ptr):
        self.slots, self.me, self.epoch_ptr, self.ticket_ptr = list(slots), int(me), int(epoch_ptr), int(ticket_ptr)


class FlagWait:
    """The matching wait: the flags in this rank's memory that the peers bump (None at this rank's own index)
    and the device address of the epoch they must reach."""

    def __init__(self, slots, epoch_ptr, max_spins=20_000_000):
        self.slots, self.epoch_ptr, self.max_spins = list(slots), int(epoch_ptr), int(max_spins)


class RawDst:
    """Destinations given as raw device addresses (e.g. mapped peer memory) plus (b, s, h) strides in elements."""

    def __init__(self, ptrs, strides):
        self.ptrs, self.strides = list(ptrs), tuple(int(x) for x in strides)

    def __len__(self):
        return len(self.ptrs)


def qk_norm_rope(tensors, *, eps=1e-6, cos=None, sin=None, rope_seq_start=0, rope_row0=0, dsts=None,
                 dst_seq_offset=0, range2=None, signal=None):
    """Fused RMSNorm + RoPE (+ head scatter) over up to three (B, S, H, D) tensors.

    tensors: list of (x, norm_weight or None, do_norm, do_rope[, norm_bias]). do_norm: False / 0 = none,
    True / 1 = RMSNorm, 2 = LayerNorm over the head dimension (weight and bias optional). dsts: None for
    in-place, or a list (one entry per tensor) of lists of destination tensors (B, S_dst, H/n_dst, D); all
    tensors share n_dst.

    range2 = (start, [(norm_weight, do_rope[, norm_bias]) per tensor], rope_row0): rows [start, S) take these norm
    weights and rotary rows instead (the norm kind stays the tensor's). signal (a FlagSignal): the kernel's last
    CTA tells the peers that this rank's rows have landed (see FlagWait / attn_fwd's wait_flags).
    """
    x0 = tensors[0][0]
    B, S, H, D = x0.shape
    a = _C.NormRopeArgs()
    a.dtype = _DTYPE_CODE[x0.dtype]
    a.batch, a.seq, a.heads, a.head_dim = B, S, H, D
    a.n_tensors = len(tensors)
    a.eps = eps
    if cos is not None:
        if cos.dtype != torch.float32 or sin.dtype != torch.float32 or not cos.is_contiguous() or not sin.is_contiguous():
            raise TypeError("cos / sin must be contiguous fp32 (rows, D) tables")
        a.cos, a.sin, a.rope_rows = cos.data_ptr(), sin.data_ptr(), cos.shape[0]
    a.rope_seq_start, a.rope_row0 = int(rope_seq_start), int(rope_row0)
    n_dst = 1 if dsts is None else len(dsts[0])
    a.n_dst = n_dst
    for i, (x, w, do_norm, do_rope, *rest) in enumerate(tensors):
        bias = rest[0] if rest else None
        if tuple(x.shape) != (B, S, H, D) or x.stride(3) != 1:
            raise ValueError("all tensors must be (B, S, H, D) with contiguous D")
        t = a.t[i]
        t.x = x.data_ptr()
        t.x_stride_b, t.x_stride_s, t.x_stride_h = x.stride(0), x.stride(1), x.stride(2)
        t.norm_weight = w.data_ptr() if w is not None else None
        t.norm_bias = bias.data_ptr() if bias is not None else None
        t.do_norm, t.do_rope = int(do_norm), int(bool(do_rope))
        outs = [x] if dsts is None else dsts[i]
        if isinstance(outs, RawDst):
            for j, ptr in enumerate(outs.ptrs):
                t.dst[j] = ptr
            t.dst_stride_b, t.dst_stride_s, t.dst_stride_h = outs.strides
        else:
            for j, o in enumerate(outs):
                t.dst[j] = o.data_ptr()
            o0 = outs[0]
            t.dst_stride_b, t.dst_stride_s, t.dst_stride_h = o0.stride(0), o0.stride(1), o0.stride(2)
        t.dst_seq_offset = int(dst_seq_offset)
    if range2 is not None:
        start, per_tensor, row0_2 = range2
        a.range2_start = int(start)
        a.range2_rope_row0 = int(row0_2)
        for i, ent in enumerate(per_tensor):
            w, do_rope, *rest = ent
            a.range2_norm_weight[i] = w.data_ptr() if w is not None else None
            a.range2_norm_bias[i] = rest[0].data_ptr() if rest and rest[0] is not None else None
            a.range2_do_rope[i] = int(bool(do_rope))
    if signal is not None:
        a.n_signal, a.signal_me = len(signal.slots), signal.me
        for i, ptr in enumerate(signal.slots):
            a.signal_slots[i] = ptr
        a.epoch_counter, a.ticket = signal.epoch_ptr, signal.ticket_ptr
    a.stream = _stream_ptr(x0.device)
    with torch.cuda.device(x0.device):
        _C.check(_C.lib().hdit_qk_norm_rope(ctypes.byref(a)))
    _count()


def _require_cuda(t):
    if not t.is_cuda:
        raise RuntimeError("hetu_dit_b200 kernels need CUDA tensors; there is no CPU path")


def _even_rows(x):
    return x.stride(2) == 1 and (x.shape[0] == 1 or x.stride(0) == x.shape[1] * x.stride(1))


def _rows_view(x):
    """(B, S, Dm) tensor -> (rows, dim, rows_per_batch, row_stride); rows must be evenly strided."""
    B, S, Dm = x.shape
    if not _even_rows(x):
        raise ValueError("expected a (B, S, Dm) tensor with contiguous last dim and evenly strided rows")
    return B * S, Dm, S, x.stride(1)


def ln_modulate(x, shift, scale, eps=1e-6, out=None):
    """LayerNorm(x) * (1 + scale[:, None]) + shift[:, None] for x (B, S, Dm), shift / scale (B, Dm) views."""
    _require_cuda(x)
    if out is None:
        out = torch.empty(tuple(x.shape), dtype=x.dtype, device=x.device)
    if x.shape[0] > 1 and not (_even_rows(x) and _even_rows(out)):  # e.g. a token slice of a batch: one launch per batch element
        for b in range(x.shape[0]):
            ln_modulate(x[b:b + 1], shift[b:b + 1], scale[b:b + 1], eps, out[b:b + 1])
        return out
    rows, dim, rpb, xs = _rows_view(x)
    if shift.stride(-1) != 1 or scale.stride(-1) != 1 or shift.stride(0) != scale.stride(0):
        raise ValueError("shift / scale must be (B, Dm) views with contiguous last dim and equal batch stride")
    with torch.cuda.device(x.device):
        _C.check(_C.lib().hdit_ln_modulate(_DTYPE_CODE[x.dtype], x.data_ptr(), shift.data_ptr(), scale.data_ptr(),
                                           out.data_ptr(), rows, dim, rpb, xs, out.stride(1), shift.stride(0), eps,
                                           _stream_ptr(x.device)))
    _count()
    return out


def gate_residual(x, gate, y, out=None):
    """x + gate[:, None] * y for x, y (B, S, Dm) and gate a (B, Dm) view."""
    _require_cuda(x)
    if x.shape != y.shape:
        raise ValueError("x and y differ in shape")
    if out is None:
        out = torch.empty(tuple(x.shape), dtype=x.dtype, device=x.device)
    if x.shape[0] > 1 and not (_even_rows(x) and _even_rows(y) and _even_rows(out)):
        for b in range(x.shape[0]):
            gate_residual(x[b:b + 1], gate[b:b + 1], y[b:b + 1], out[b:b + 1])
        return out
    rows, dim, rpb, xs = _rows_view(x)
    _, _, _, ys = _rows_view(y)
    with torch.cuda.device(x.device):
        _C.check(_C.lib().hdit_gate_residual(_DTYPE_CODE[x.dtype], x.data_ptr(), gate.data_ptr(), y.data_ptr(),
                                             out.data_ptr(), rows, dim, rpb, xs, ys, out.stride(1), gate.stride(0),
                                             _stream_ptr(x.device)))
    _count()
    return out


def gelu_tanh(x, out=None):
    """tanh-approximated GELU over the last dim of a (B, S, Dm) tensor with evenly strided rows; `out` may be
    `x` itself or a column block of a wider buffer with the same (B, S)."""
    _require_cuda(x)
    rows, dim, _, xs = _rows_view(x)
    if out is None:
        out = torch.empty(tuple(x.shape), dtype=x.dtype, device=x.device)
    rows_o, dim_o, _, os_ = _rows_view(out)
    if (rows_o, dim_o) != (rows, dim):
        raise ValueError("out differs from x in shape")
    with torch.cuda.device(x.device):
        _C.check(_C.lib().hdit_gelu_tanh(_DTYPE_CODE[x.dtype], x.data_ptr(), out.data_ptr(), rows, dim, xs, os_,
                                         _stream_ptr(x.device)))
    _count()
    return out


def linear_fused(x, weight, bias=None, epilogue="bias", residual=None, gate=None, out=None, tile_n=0, max_ctas=0,
                 tile_m=0, cta_pair=0):
    """epilogue(x @ weight.T + bias) in one tensor-core kernel (csrc/gemm_sm100.cu). x (B, S, K) or (rows, K) with
    evenly strided rows, weight (N, K) as torch.nn.Linear stores it. epilogue: "bias" (a plain linear layer),
    "gelu_tanh", or "gate_residual" = residual + gate[:, None, :] * linear(x) with gate (B, N) and residual of the
    output's shape. `out` may be a column block of a wider buffer, or `residual` itself."""
    _require_cuda(x)
    if x.dim() == 2:
        res3 = residual.unsqueeze(0) if residual is not None else None
        out3 = out.unsqueeze(0) if out is not None else None
        return linear_fused(x.unsqueeze(0), weight, bias, epilogue, res3, gate, out3, tile_n, max_ctas, tile_m, cta_pair)[0]
    rows, k, _, xs = _rows_view(x)
    n = weight.shape[0]
    if weight.dim() != 2 or weight.shape[1] != k or weight.stride(1) != 1 or weight.dtype != x.dtype:
        raise ValueError("weight must be (N, K), K-contiguous, of x's dtype")
    if out is None:
        out = torch.empty(tuple(x.shape[:-1]) + (n,), dtype=x.dtype, device=x.device)
    rows_o, n_o, _, os_ = _rows_view(out)
    if (rows_o, n_o) != (rows, n):
        raise ValueError("out does not match (rows, N)")
    a = _C.GemmArgs()
    a.dtype = _DTYPE_CODE[x.dtype]
    a.epilogue = {"bias": _C.GEMM_BIAS, "gelu_tanh": _C.GEMM_BIAS_GELU_TANH,
                  "gate_residual": _C.GEMM_BIAS_GATE_RESIDUAL}[epilogue]
    a.m, a.n, a.k = rows, n, k
    a.a, a.lda = x.data_ptr(), xs
    a.w, a.ldw = weight.data_ptr(), weight.stride(0)
    if bias is not None:
        if bias.numel() != n or not bias.is_contiguous() or bias.dtype != x.dtype:
            raise ValueError("bias must be N contiguous elements of x's dtype")
        a.bias = bias.data_ptr()
    a.out, a.ldo = out.data_ptr(), os_
    if epilogue == "gate_residual":
        rows_r, n_r, _, rs = _rows_view(residual)
        if (rows_r, n_r) != (rows, n):
            raise ValueError("residual does not match (rows, N)")
        if gate.dim() != 2 or gate.shape[1] != n or gate.stride(1) != 1 or rows % gate.shape[0] != 0:
            raise ValueError("gate must be (B, N) with rows a multiple of B")
        a.residual, a.ldr = residual.data_ptr(), rs
        a.gate, a.gate_batch_stride = gate.data_ptr(), gate.stride(0)
        a.rows_per_batch = rows // gate.shape[0]
    a.tile_n, a.max_ctas, a.tile_m, a.cta_pair = tile_n, max_ctas, tile_m, cta_pair
    with torch.cuda.device(x.device):
        a.stream = _stream_ptr(x.device)
        _C.check(_C.lib().hdit_linear_fused(ctypes.byref(a)))
    _count()
    return out


# Whether linear_tail() may run the fused tensor-core kernel (csrc/gemm_sm100.cu) instead of the library GEMM
# followed by the one-pass tail kernel, and for which tails. Measured inside the whole step (same box, alternating
# runs): fusing the GELU wins (Flux-shaped 68.3-68.8 against 68.9-69.3 ms, SD3-shaped 11.77 against 11.99 ms per
# step); fusing the gated residuals as well loses (69.5 against 68.1-69.1 ms, 12.32 against 12.00 ms) although alone
# it ties the pair of kernels it replaces -- without multicast loads the kernel moves more operand bytes from L2 per
# flop than the library's, and under the power cap that costs clock. So only the GELU is fused by default.
# HDIT_FUSED_LINEAR=0 turns the fused kernel off, HDIT_FUSED_LINEAR_TAILS=gelu_tanh,gate_residual fuses both tails.
FUSED_LINEAR = os.environ.get("HDIT_FUSED_LINEAR", "1") == "1"
FUSED_LINEAR_TAILS = set(os.environ.get("HDIT_FUSED_LINEAR_TAILS", "gelu_tanh").split(","))
# The fused kernel is used from this row count on. Below, the library's split-K GEMMs fill the GPU better than
# whole output tiles do (measured at 576 to 2304 rows: the fused kernel takes 1.2x to 2x the library GEMM + tail
# kernel).
FUSED_LINEAR_MIN_ROWS = int(os.environ.get("HDIT_FUSED_LINEAR_MIN_ROWS", "4096"))
FUSED_LINEAR_MAX_ROWS = int(os.environ.get("HDIT_FUSED_LINEAR_MAX_ROWS", str(1 << 40)))


def linear_tail(linear, x, epilogue, residual=None, gate=None, out=None):
    """A torch.nn.Linear followed by its elementwise tail ("gelu_tanh", or "gate_residual" = residual +
    gate[:, None] * linear(x)), as one kernel when FUSED_LINEAR is set and the layouts allow it (rows evenly
    strided across the batch), else as the library GEMM plus hdit_gelu_tanh / hdit_gate_residual."""
    fusable = (FUSED_LINEAR and epilogue in FUSED_LINEAR_TAILS and x.is_cuda and x.dim() == 3 and _even_rows(x) and not torch.is_grad_enabled()
               and FUSED_LINEAR_MIN_ROWS <= x.shape[0] * x.shape[1] <= FUSED_LINEAR_MAX_ROWS
               and (out is None or _even_rows(out)) and (residual is None or _even_rows(residual))
               and (gate is None or (gate.stride(-1) == 1 and (x.shape[0] == 1 or x.shape[1] >= 32))))
    if fusable:
        return linear_fused(x, linear.weight, linear.bias, epilogue, residual=residual, gate=gate, out=out)
    y = linear(x)
    if epilogue == "gelu_tanh":
        return gelu_tanh(y, out=y if out is None else out)
    if epilogue == "gate_residual":
        return gate_residual(residual, gate, y, out=out)
    raise ValueError(epilogue)


def cfg_euler_step(noise_pred, sample, sigmas, step_index, guidance_scale, cfg=True, out=None, out_peer_ptr=None):
    """sample + (sigmas[i + 1] - sigmas[i]) * guided(noise_pred) in one pass. noise_pred is (2 * B, ...) =
    [unconditional; conditional] when cfg is set (guided = uncond + scale * (cond - uncond)), else (B, ...) taken as
    it is; sample and the result are (B, ...), contiguous, 16-bit. sigmas: fp32 device tensor. out_peer_ptr: raw
    device address (e.g. the next pipeline stage's inbox slot) that receives a second copy of the result."""
    _require_cuda(sample)
    if not (noise_pred.is_contiguous() and sample.is_contiguous()):
        raise ValueError("noise_pred and sample must be contiguous")
    n = sample.numel()
    if noise_pred.numel() != (2 * n if cfg else n):
        raise ValueError("noise_pred does not match sample")
    if sigmas.dtype != torch.float32 or not sigmas.is_cuda or not 0 <= step_index < sigmas.numel() - 1:
        raise ValueError("sigmas must be a float32 device tensor with step_index + 1 in range")
    if out is None:
        out = torch.empty_like(sample)
    es = noise_pred.element_size()
    uncond = noise_pred.data_ptr()
    cond = uncond + n * es if cfg else None
    with torch.cuda.device(sample.device):
        _C.check(_C.lib().hdit_cfg_euler_step(_DTYPE_CODE[sample.dtype], uncond, cond, sample.data_ptr(), out.data_ptr(),
                                              out_peer_ptr, n, float(guidance_scale), sigmas.data_ptr(), int(step_index),
                                              _stream_ptr(sample.device)))
    _count()
    return out

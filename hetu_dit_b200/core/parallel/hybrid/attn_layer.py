"""USP long-context attention: Ulysses head<->sequence exchange around ring attention.

Interface of the reference's hetu_dit/core/parallel/hybrid/attn_layer.py:
hetuDiTLongContextAttention (:17-139), hetuDiTJointLongContextAttention
(:142-274), hetuDiTFluxLongContextAttention (:277-395); same constructor
arguments, same forward keyword arguments, same output row order.

Data movement differs from the reference by design. Its four NCCL all-to-alls
per layer (yunchang SeqAllToAll4D) become peer stores: one kernel writes the
head slice every Ulysses peer needs straight into that peer's gathered buffer
in the node's peer heap (Q, K and V in one launch), a flag barrier orders it
against the consumers, the tcgen05 attention kernel runs on the gathered
tensors (joint text K/V as an extra segment, never concatenated), and the
context rows are stored back into their owners' output buffers the same way.
"""
import os
from typing import Optional

import torch
from torch import Tensor

from .... import kernels
from ...distributed import parallel_state as ps
from ...distributed.peer import PeerGroup
from .utils import RING_IMPL_DICT

_SUPPORTED_JOINT = ["none", "front", "rear"]


class _UlyssesExchange:
    """The two all-to-alls of one attention call over the peer heap."""

    def __init__(self, group: PeerGroup):
        self.group = group
        self.heap = group.heap
        if group.world_size > 1 and self.heap is None:
            raise RuntimeError("Ulysses attention across ranks needs the peer heap")

    def gather_heads(self, tensors, tags):
        """SeqAllToAll4D(scatter_idx=2, gather_idx=1) for several (B, S_loc, H, D) tensors at once:
        rank r ends up with (B, U*S_loc, H/U, D) holding head slice r of every rank's tokens, in
        group-rank order. Tensors with different S_loc go in separate launches."""
        g, U, me = self.group, self.group.world_size, self.group.rank_in_group
        outs = []
        by_len = {}
        for t, tag in zip(tensors, tags):
            B, S, H, D = t.shape
            if H % U != 0:
                raise RuntimeError(f"{H} heads are not divisible by the Ulysses degree {U}")
            buf, off = self.heap.alloc((B, U * S, H // U, D), t.dtype, name=f"usp_{tag}_{(B, S, H, D)}_{t.dtype}")
            outs.append(buf)
            ptrs = [self.heap.peer_ptr(r, off) for r in g.ranks]
            by_len.setdefault(S, []).append((t, kernels.RawDst(ptrs, buf.stride()[:3])))
        for S, items in by_len.items():
            for i in range(0, len(items), 3):
                chunk = items[i:i + 3]
                kernels.qk_norm_rope([(t, None, False, False) for t, _ in chunk], dsts=[d for _, d in chunk],
                                     dst_seq_offset=me * S)
        g.barrier()
        return outs

    def gather_heads_fused(self, query, key, value, prologue, fold_barrier: bool = False):
        """gather_heads for Q, K and V with the per-head RMSNorm and the rotary embedding of Q and K applied on
        the way: the kernel that normalises and rotates a row stores each head slice straight into the peer
        that attends it, so the projections' output is read once and nothing is written locally.

        prologue: [(row_lo, row_hi, q_norm_weight, k_norm_weight, eps, (cos, sin) or None, rope_row0)], row
        ranges that tile [0, S_loc). One or two ranges (text rows and image rows differ in norm weights and rotary
        rows) go out in ONE launch; more than two fall back to one launch per range.

        fold_barrier: instead of the flag barrier kernel after the exchange, the exchange kernel's last CTA
        signals the peers and the consumer (the attention kernel's loader) waits for the peers' signals: returns
        (q, k, v, FlagWait) -- the caller must hand the FlagWait to the attention call that reads q, k, v, and
        nothing else may read them before."""
        g, U, me = self.group, self.group.world_size, self.group.rank_in_group
        B, S, H, D = query.shape
        if H % U != 0:
            raise RuntimeError(f"{H} heads are not divisible by the Ulysses degree {U}")
        if sorted((lo, hi) for lo, hi, *_ in prologue) != [(lo, hi) for lo, hi, *_ in prologue] or \
                prologue[0][0] != 0 or prologue[-1][1] != S or \
                any(a[1] != b[0] for a, b in zip(prologue, prologue[1:])):
            raise ValueError("prologue row ranges must tile [0, S_loc) in order")
        outs, dsts = [], []
        for t, tag in zip((query, key, value), ("q", "k", "v")):
            if tuple(t.shape) != (B, S, H, D):
                raise ValueError("query, key and value must share one (B, S, H, D) shape")
            buf, off = self.heap.alloc((B, U * S, H // U, D), t.dtype, name=f"usp_{tag}_{(B, S, H, D)}_{t.dtype}")
            outs.append(buf)
            dsts.append(kernels.RawDst([self.heap.peer_ptr(r, off) for r in g.ranks], buf.stride()[:3]))
        signal = wait = None
        if fold_barrier:
            signal, wait = self.heap.folded_barrier(g.ranks)
        ranges = [r for r in prologue if r[1] > r[0]]
        same = len(ranges) == 2 and ranges[0][4] == ranges[1][4] and \
            (ranges[0][5] is None or ranges[1][5] is None or ranges[0][5][0] is ranges[1][5][0]) and \
            (ranges[0][2] is None) == (ranges[1][2] is None)
        if len(ranges) == 1 or same:
            lo, hi, wq, wk, eps, rope, row0 = ranges[0]
            table = rope if rope is not None else (ranges[1][5] if same else None)
            cos, sin = table if table is not None else (None, None)
            range2 = None
            if same:
                lo2, _, wq2, wk2, _, rope2, row0_2 = ranges[1]
                range2 = (lo2, [(wq2, rope2 is not None), (wk2, rope2 is not None), (None, False)], row0_2)
            kernels.qk_norm_rope([(query, wq, wq is not None, rope is not None),
                                  (key, wk, wk is not None, rope is not None),
                                  (value, None, False, False)],
                                 eps=eps, cos=cos, sin=sin, rope_seq_start=0, rope_row0=row0, dsts=dsts,
                                 dst_seq_offset=me * S, range2=range2, signal=signal)
        else:
            for i, (lo, hi, wq, wk, eps, rope, row0) in enumerate(ranges):
                cos, sin = rope if rope is not None else (None, None)
                kernels.qk_norm_rope([(query[:, lo:hi], wq, wq is not None, rope is not None),
                                      (key[:, lo:hi], wk, wk is not None, rope is not None),
                                      (value[:, lo:hi], None, False, False)],
                                     eps=eps, cos=cos, sin=sin, rope_seq_start=0, rope_row0=row0, dsts=dsts,
                                     dst_seq_offset=me * S + lo, signal=signal if i == len(ranges) - 1 else None)
        if fold_barrier:
            return outs + [wait]
        g.barrier()
        return outs

    def scatter_plan(self, B: int, S_tot: int, Hl: int, D: int, dtype, tag: str, joint_len: int = 0,
                     joint_front: bool = True):
        """SeqAllToAll4D(scatter_idx=1, gather_idx=2), (B, U*S_loc, H/U, D) -> (B, S_loc, H, D), as a store plan
        for the attention epilogue instead of a pass of its own: returns (out, scatter) where `out` is this
        rank's (B, joint_len + S_loc, H, D) result buffer in the peer heap and `scatter` tells the attention
        kernel where each of its result rows goes -- the image rows of source rank p into p's buffer, the rows
        of the replicated joint (text) queries, computed once per head slice, into every peer's buffer; both at
        this rank's head slice. The caller runs attention with it and then calls finish().

        Two buffers are used alternately: a peer writes this rank's buffer for layer L+1 only after the barrier
        that follows layer L+1's head exchange, which this rank enters after it has enqueued (on the same stream)
        everything that reads layer L's result; alternating adds one more layer of slack for a caller that keeps
        the returned view a little longer."""
        g, U, me = self.group, self.group.world_size, self.group.rank_in_group
        S = (S_tot - joint_len) // U
        rows = S + joint_len
        # sized for the joint length rounded up to 512 rows, so that requests whose text lengths differ share
        # the buffer instead of growing the heap by one per length
        cap = S + -(-joint_len // 512) * 512
        name = f"usp_{tag}_{(B, cap, Hl * U, D)}_{dtype}_{g.ranks}"
        buf, off = self.heap.alloc((B, cap, Hl * U, D), dtype, name=f"{name}_{self.heap.flip(name)}")
        out = buf[:, :rows]
        es = out.element_size()
        ptrs = [self.heap.peer_ptr(r, off) + me * Hl * D * es for r in g.ranks]
        scatter = dict(dsts=kernels.RawDst(ptrs, out.stride()[:3]),
                       q=(S, joint_len if joint_front else 0),       # (rows per destination, first destination row)
                       joint=(0, 0 if joint_front else S))           # 0 rows per destination = to every destination
        return out, scatter

    def finish(self):
        """Orders the peers' result stores against this rank's readers (and this rank's stores against theirs)."""
        self.group.barrier()

    def scatter_sequence(self, ctx: Tensor, tag: str, joint_len: int = 0, joint_front: bool = True) -> Tensor:
        """The same exchange for a context tensor that already exists (one copy launch): used when the
        attention call cannot scatter by itself."""
        g, U = self.group, self.group.world_size
        B, S_tot, Hl, D = ctx.shape
        S = (S_tot - joint_len) // U
        out, plan = self.scatter_plan(B, S_tot, Hl, D, ctx.dtype, tag, joint_len, joint_front)
        es = ctx.element_size()
        img0_src = joint_len if joint_front else 0      # first image row in ctx
        img0_dst = plan["q"][1]
        jnt_src = 0 if joint_front else U * S
        jnt_dst = plan["joint"][1]
        pieces = []
        for p, base in enumerate(plan["dsts"].ptrs):
            src = ctx[:, img0_src + p * S:img0_src + (p + 1) * S]
            pieces.append((src.data_ptr(), base + img0_dst * out.stride(1) * es, B, ctx.stride(0) * es,
                           out.stride(0) * es, S, ctx.stride(1) * es, out.stride(1) * es, Hl * D * es))
            if joint_len:
                jsrc = ctx[:, jnt_src:jnt_src + joint_len]
                pieces.append((jsrc.data_ptr(), base + jnt_dst * out.stride(1) * es, B, ctx.stride(0) * es,
                               out.stride(0) * es, joint_len, ctx.stride(1) * es, out.stride(1) * es, Hl * D * es))
        kernels.copy_pieces(pieces, ctx.device)
        g.barrier()
        return out


class hetuDiTLongContextAttention(torch.nn.Module):
    ring_impl_type_supported_kv_cache = ["basic"]
    # Fold the barrier between the head exchange and attention into those two kernels (signal from the exchange
    # kernel's last CTA, wait in the attention kernel's loader) instead of a one-warp barrier kernel. Off: measured
    # on the Flux-shaped step at Ulysses 2 it costs 43.6 ms against 39.9 ms per step -- while it waits, the
    # attention grid holds every SM, which starves the GEMMs the blocks run beside attention on a second stream;
    # the one-warp kernel waits for free. It pays where nothing runs beside attention.
    fold_exchange_barrier = os.environ.get("HDIT_FOLD_EXCHANGE_BARRIER", "0") == "1"

    def __init__(self, scatter_idx: int = 2, gather_idx: int = 1, ring_impl_type: str = "basic",
                 use_pack_qkv: bool = False, use_kv_cache: bool = False) -> None:
        super().__init__()
        if scatter_idx != 2 or gather_idx != 1:
            raise ValueError("only the (B, S, H, D) layout with scatter_idx=2, gather_idx=1 is supported")
        self.scatter_idx, self.gather_idx = scatter_idx, gather_idx
        self.ring_impl_type = ring_impl_type
        self.use_pack_qkv = use_pack_qkv
        self.use_kv_cache = use_kv_cache
        if use_kv_cache and ring_impl_type not in self.ring_impl_type_supported_kv_cache:
            raise RuntimeError(f"ring_impl_type: {ring_impl_type} do not support SP kv cache.")
        if ring_impl_type not in RING_IMPL_DICT:
            raise RuntimeError(f"ring_impl_type: {ring_impl_type} is not available")
        self.ring_attn_fn = RING_IMPL_DICT[ring_impl_type]
        self.ring_pg: Optional[PeerGroup] = None
        self.ulysses_pg: Optional[PeerGroup] = None

    # -- shared body -----------------------------------------------------------------------------
    def _bind_groups(self):
        # groups are re-read on every call so a plan switch takes effect without re-creating
        # the operator (hybrid/attn_layer.py:88-90)
        self.use_kv_cache = ps.get_sequence_parallel_world_size() > 1
        self.ring_pg = ps.PROCESS_GROUP.RING_PG
        self.ulysses_pg = ps.PROCESS_GROUP.ULYSSES_PG

    def _kv_hook_runs(self, attn) -> bool:
        """Whether the stale-KV update will launch work on the gathered K / V before attention does."""
        if attn is None or not self.use_kv_cache:
            return False
        from ...distributed.runtime_state import get_runtime_state, runtime_state_is_initialized
        return runtime_state_is_initialized() and get_runtime_state().num_pipeline_patch > 1

    def _run(self, attn, query, key, value, joint_k, joint_v, joint_strategy, dropout_p, softmax_scale, causal,
             window_size, alibi_slopes, deterministic, return_attn_probs, joint_q=None, qk_prologue=None):
        """joint_q stays its own query segment. The reference concatenates it into every rank's query before
        the all-to-all, so each Ulysses rank attends U identical copies of the text queries; here the
        replicated rows are attended once per head slice and their context rows are sent to all peers."""
        U = 1 if self.ulysses_pg is None else self.ulysses_pg.world_size
        wait_flags = None
        if U > 1:
            r = self.ulysses_pg.rank_in_group
            if joint_k is not None:
                hpr = joint_k.shape[-2] // U
                joint_k = joint_k[..., hpr * r:hpr * (r + 1), :]
                joint_v = joint_v[..., hpr * r:hpr * (r + 1), :]
                if joint_q is not None:
                    joint_q = joint_q[..., hpr * r:hpr * (r + 1), :]
            xchg = _UlyssesExchange(self.ulysses_pg)
            if qk_prologue is not None:
                # The barrier after the exchange can fold into the kernels on either side of it when attention is
                # the first (and only) reader of the gathered tensors: no ring pull and no stale-KV update.
                fold = self.fold_exchange_barrier and (self.ring_pg is None or self.ring_pg.world_size == 1) and \
                    not self._kv_hook_runs(attn)
                res = xchg.gather_heads_fused(query, key, value, qk_prologue, fold_barrier=fold)
                query, key, value = res[:3]
                wait_flags = res[3] if fold else None
            else:
                query, key, value = xchg.gather_heads([query, key, value], ["q", "k", "v"])
        elif qk_prologue is not None:
            for lo, hi, wq, wk, eps, rope, row0 in qk_prologue:
                cos, sin = rope if rope is not None else (None, None)
                if hi > lo and (wq is not None or rope is not None):
                    kernels.qk_norm_rope([(query[:, lo:hi], wq, wq is not None, rope is not None),
                                          (key[:, lo:hi], wk, wk is not None, rope is not None)],
                                         eps=eps, cos=cos, sin=sin, rope_seq_start=0, rope_row0=row0)
        scatter = out_buf = None
        if U > 1:
            # the reverse all-to-all is done by the attention epilogue: every result row is stored straight into
            # the buffer of the rank that owns it
            B, S_g, Hl, D = query.shape
            joint_len = 0 if joint_q is None else joint_q.shape[1]
            out_buf, scatter = xchg.scatter_plan(B, S_g + joint_len, Hl, D, query.dtype, "o", joint_len,
                                                 joint_strategy == "front")
        out = self.ring_attn_fn(query, key, value, dropout_p=dropout_p, softmax_scale=softmax_scale, causal=causal,
                                window_size=window_size, alibi_slopes=alibi_slopes, deterministic=deterministic,
                                return_attn_probs=return_attn_probs, group=self.ring_pg,
                                attn_layer=attn if self.use_kv_cache else None, joint_tensor_key=joint_k,
                                joint_tensor_value=joint_v, joint_strategy=joint_strategy, joint_tensor_query=joint_q,
                                out_scatter=scatter, wait_flags=wait_flags)
        if U > 1:
            xchg.finish()
            return out_buf
        return out[0] if isinstance(out, tuple) else out

    @torch.compiler.disable
    def forward(self, attn, query: Tensor, key: Tensor, value: Tensor, *, joint_tensor_query=None,
                joint_tensor_key=None, joint_tensor_value=None, dropout_p=0.0, softmax_scale=None, causal=False,
                window_size=(-1, -1), alibi_slopes=None, deterministic=False, return_attn_probs=False,
                joint_strategy="none", qk_prologue=None) -> Tensor:
        """3 x (B, S/P, H, D) -> (B, S/P, H, D).

        qk_prologue (not in the reference's signature): per-head RMSNorm and rotary embedding of query and key
        that the caller has *not* applied yet, as row ranges [(row_lo, row_hi, q_norm_weight, k_norm_weight,
        eps, (cos, sin) or None, rope_row0)] tiling the local rows. Under Ulysses they are applied by the kernel
        that performs the head exchange (one pass over the projections' output instead of two); without
        Ulysses they are applied in place before the ring."""
        self._bind_groups()
        return self._run(attn, query, key, value, None, None, "none", dropout_p, softmax_scale, causal, window_size,
                         alibi_slopes, deterministic, return_attn_probs, qk_prologue=qk_prologue)


class hetuDiTJointLongContextAttention(hetuDiTLongContextAttention):
    @torch.compiler.disable
    def forward(self, attn, query: Tensor, key: Tensor, value: Tensor, *, joint_tensor_query, joint_tensor_key,
                joint_tensor_value, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                alibi_slopes=None, deterministic=False, return_attn_probs=False, joint_strategy="rear"):
        """Joint text+image attention; output rows are [local; joint] ("rear") or [joint; local] ("front")."""
        self._bind_groups()
        if joint_strategy not in _SUPPORTED_JOINT:
            raise ValueError(
                f"joint_strategy: {joint_strategy} not supprted. supported joint strategy: {_SUPPORTED_JOINT}")
        elif joint_strategy != "none" and joint_tensor_query is None:
            raise ValueError("joint_tensor_query must not be None when joint_strategy is not None")
        return self._run(attn, query, key, value, joint_tensor_key, joint_tensor_value, joint_strategy, dropout_p,
                         softmax_scale, causal, window_size, alibi_slopes, deterministic, return_attn_probs,
                         joint_q=joint_tensor_query if joint_strategy != "none" else None)


class hetuDiTFluxLongContextAttention(hetuDiTLongContextAttention):
    @torch.compiler.disable
    def forward(self, attn, query: Tensor, key: Tensor, value: Tensor, *, joint_tensor_query, joint_tensor_key,
                joint_tensor_value, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                alibi_slopes=None, deterministic=False, return_attn_probs=False, joint_strategy="front"):
        """Flux: text tokens always lead (hybrid/attn_layer.py:327)."""
        self._bind_groups()
        return self._run(attn, query, key, value, joint_tensor_key, joint_tensor_value, "front", dropout_p,
                         softmax_scale, causal, window_size, alibi_slopes, deterministic, return_attn_probs,
                         joint_q=joint_tensor_query)


# names used by the xDiT lineage of this operator
xFuserLongContextAttention = hetuDiTLongContextAttention
xFuserJointLongContextAttention = hetuDiTJointLongContextAttention
xFuserFluxLongContextAttention = hetuDiTFluxLongContextAttention

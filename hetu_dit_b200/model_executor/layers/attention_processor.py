"""Attention processors of the -shaped DiT blocks.

They play the role of the reference's hetuDiTJointAttnProcessor2_0 (SD3,
hetu_dit/model_executor/diffusion_executor/layers/attention_processor.py:632-793)
and hetuDiTFluxAttnProcessor2_0 (:797-987): QKV (+ added QKV) projections,
per-head QK-RMSNorm, rotary embedding, PipeFusion stale-KV update, then either
the single-GPU attention kernel or the USP operator, and the split back into
image and text streams.

What is fused here and eager in the reference: norm + RoPE run as one in-place
kernel over Q and K (the reference round-trips fp32 copies, :68-120); text and
image parts are never concatenated -- they are passed to the attention kernel
as segments; the stale-KV buffer is updated by one scatter kernel.
"""
import torch

from ... import kernels
from ...core.distributed import parallel_state as ps
from ...core.parallel import (hetuDiTFluxLongContextAttention, hetuDiTJointLongContextAttention,
                              hetuDiTLongContextAttention)
from ...core.resource_manager.cache_manager import get_cache_manager


def _heads(x, attn):
    B, S, _ = x.shape
    return x.view(B, S, attn.heads, attn.head_dim)


def _norm_rope(attn, q, k, wq, wk, rope, row0):
    """In-place QK-RMSNorm and RoPE over (B, S, H, D) views; `row0` is the table row of token 0."""
    do_norm = wq is not None
    if not do_norm and rope is None:
        return
    cos, sin = rope if rope is not None else (None, None)
    kernels.qk_norm_rope([(q, wq.weight if do_norm else None, do_norm, rope is not None),
                          (k, wk.weight if do_norm else None, do_norm, rope is not None)],
                         eps=wq.eps if do_norm else 1e-6, cos=cos, sin=sin, rope_seq_start=0, rope_row0=row0)


def _prologue_range(lo, hi, wq, wk, rope, row0):
    """One row range of the operator's qk_prologue: norm weights (or None), eps, rotary tables, first table row."""
    do_norm = wq is not None
    return (lo, hi, wq.weight if do_norm else None, wk.weight if do_norm else None, wq.eps if do_norm else 1e-6,
            rope, row0)


def _project_into(buf, row0, x, linear):
    """buf[:, row0:row0 + S] = linear(x) without a temporary when the rows are one contiguous block."""
    B, S, _ = x.shape
    if B == 1 and not torch.is_grad_enabled():
        torch.addmm(linear.bias, x[0], linear.weight.t(), out=buf[0, row0:row0 + S])
    else:
        buf[:, row0:row0 + S] = linear(x)


class _PlainOperator:
    """Lazily built hetuDiTLongContextAttention (no joint tensors), rebuilt when the SP degree changes."""

    def __init__(self):
        self.op, self.world = None, 0

    def get(self):
        world = ps.get_sequence_parallel_world_size()
        if self.op is None or self.world != world:
            self.op, self.world = hetuDiTLongContextAttention(use_kv_cache=True), world
        return self.op


class JointAttnProcessor:
    """Double-stream (text + image) attention. joint_strategy "rear" = [image; text] (SD3 order,
    attention_processor.py:742-744), "front" = [text; image] (Flux order, :895-897).

    The reference keeps the whole text stream on every sequence-parallel rank and hands it to the USP
    operator as joint tensors. When the caller passes `text_offset` the text stream is sharded like the
    image stream instead (encoder_hidden_states holds rows [text_offset, text_offset + S_txt) of `text_len`
    text tokens): local text and image rows then form one sequence shard and go through the operator
    without joint tensors. Attention is invariant to the order of keys, and every query row comes back to
    the rank that sent it, so the result is the same while the text projections and MLPs are computed
    once instead of once per rank."""

    def __init__(self):
        self.hybrid_seq_parallel_attn = None
        self._hybrid_world = 0
        self._plain = _PlainOperator()

    def _sharded_text(self, attn, hidden_states, encoder_hidden_states, rope, text_total, token_offset, text_offset):
        B, S_img, _ = hidden_states.shape
        S_txt = encoder_hidden_states.shape[1]
        front = rope is not None
        t0, i0 = (0, S_txt) if front else (S_img, 0)
        bufs = []
        for img_p, txt_p in ((attn.to_q, attn.add_q_proj), (attn.to_k, attn.add_k_proj), (attn.to_v, attn.add_v_proj)):
            buf = torch.empty((B, S_txt + S_img, attn.heads * attn.head_dim), dtype=hidden_states.dtype,
                              device=hidden_states.device)
            _project_into(buf, i0, hidden_states, img_p)
            _project_into(buf, t0, encoder_hidden_states, txt_p)
            bufs.append(_heads(buf, attn))
        q, k, v = bufs
        # QK-norm and RoPE ride on the head exchange (or run in place when the plan has no Ulysses exchange)
        ranges = [_prologue_range(i0, i0 + S_img, attn.norm_q, attn.norm_k, rope, text_total + token_offset),
                  _prologue_range(t0, t0 + S_txt, attn.norm_added_q, attn.norm_added_k, rope, text_offset)]
        out = self._plain.get()(attn, q, k, v, dropout_p=0.0, causal=False, qk_prologue=sorted(ranges))
        out = out.reshape(B, S_txt + S_img, attn.heads * attn.head_dim)
        return attn.to_out[0](out[:, i0:i0 + S_img]), attn.to_add_out(out[:, t0:t0 + S_txt])

    def _operator(self, strategy):
        world = ps.get_sequence_parallel_world_size()
        if self.hybrid_seq_parallel_attn is None or self._hybrid_world != world:
            cls = hetuDiTFluxLongContextAttention if strategy == "front" else hetuDiTJointLongContextAttention
            self.hybrid_seq_parallel_attn = cls(use_kv_cache=True)
            self._hybrid_world = world
        return self.hybrid_seq_parallel_attn

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, image_rotary_emb=None, text_len=None,
                 token_offset: int = 0, text_offset=None):
        strategy = "front" if image_rotary_emb is not None else "rear"
        B, S_img, _ = hidden_states.shape
        S_txt = encoder_hidden_states.shape[1]
        if text_offset is not None and ps.get_sequence_parallel_world_size() > 1:
            return self._sharded_text(attn, hidden_states, encoder_hidden_states, image_rotary_emb,
                                      int(text_len or S_txt), token_offset, text_offset)
        q, k, v = (_heads(p(hidden_states), attn) for p in (attn.to_q, attn.to_k, attn.to_v))
        tq, tk, tv = (_heads(p(encoder_hidden_states), attn) for p in (attn.add_q_proj, attn.add_k_proj, attn.add_v_proj))
        _norm_rope(attn, q, k, attn.norm_q, attn.norm_k, image_rotary_emb, S_txt + token_offset)
        _norm_rope(attn, tq, tk, attn.norm_added_q, attn.norm_added_k, image_rotary_emb, 0)

        if ps.get_sequence_parallel_world_size() > 1:
            out = self._operator(strategy)(attn, q, k, v, dropout_p=0.0, causal=False, joint_tensor_query=tq,
                                           joint_tensor_key=tk, joint_tensor_value=tv, joint_strategy=strategy)
        else:
            k, v = get_cache_manager().update_and_get_kv_cache(new_kv=[k, v], layer=attn, slice_dim=1,
                                                               layer_type="attn") if _cached(attn) else (k, v)
            if strategy == "rear":
                out = kernels.attn_fwd([q, tq], [k, tk], [v, tv])
            else:
                out = kernels.attn_fwd([tq, q], [tk, k], [tv, v])
        out = out.reshape(B, out.shape[1], attn.heads * attn.head_dim)
        if strategy == "rear":
            img, txt = out[:, :S_img], out[:, S_img:]
        else:
            txt, img = out[:, :S_txt], out[:, S_txt:]
        return attn.to_out[0](img), attn.to_add_out(txt)


class SingleAttnProcessor:
    """Single-stream attention over the [text; image] sequence (Flux single blocks,
    attention_processor.py:898-901 for the text/image split under SP)."""

    def __init__(self):
        self.hybrid_seq_parallel_attn = None
        self._hybrid_world = 0
        self._plain = _PlainOperator()

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, image_rotary_emb=None, text_len=None,
                 token_offset: int = 0, out=None, text_offset=None, text_total=None):
        """out: optional (B, S, H*D)-shaped view (any row stride) the single-GPU path writes into, e.g. the left
        part of the buffer the block's output projection reads, which saves a concatenation.

        text_offset / text_total: the first `text_len` rows are rows [text_offset, text_offset + text_len) of
        a text stream of text_total tokens that is sharded over the sequence-parallel ranks (see
        JointAttnProcessor); None = the whole text stream is present on every rank, as in the reference."""
        B, S, _ = hidden_states.shape
        q, k, v = (_heads(p(hidden_states), attn) for p in (attn.to_q, attn.to_k, attn.to_v))
        out4 = None if out is None else out.view(B, S, attn.heads, attn.head_dim)
        S_txt = int(text_len or 0)
        if text_offset is not None and ps.get_sequence_parallel_world_size() > 1:
            ranges = [_prologue_range(0, S_txt, attn.norm_q, attn.norm_k, image_rotary_emb, text_offset),
                      _prologue_range(S_txt, S, attn.norm_q, attn.norm_k, image_rotary_emb,
                                      int(text_total) + token_offset)]
            ctx = self._plain.get()(attn, q, k, v, dropout_p=0.0, causal=False, qk_prologue=ranges)
            return ctx.reshape(B, S, attn.heads * attn.head_dim)
        if token_offset == 0:
            _norm_rope(attn, q, k, attn.norm_q, attn.norm_k, image_rotary_emb, 0)
        else:
            _norm_rope(attn, q[:, :S_txt], k[:, :S_txt], attn.norm_q, attn.norm_k, image_rotary_emb, 0)
            _norm_rope(attn, q[:, S_txt:], k[:, S_txt:], attn.norm_q, attn.norm_k, image_rotary_emb, S_txt + token_offset)
        if ps.get_sequence_parallel_world_size() > 1:
            world = ps.get_sequence_parallel_world_size()
            if self.hybrid_seq_parallel_attn is None or self._hybrid_world != world:
                self.hybrid_seq_parallel_attn = hetuDiTFluxLongContextAttention(use_kv_cache=True)
                self._hybrid_world = world
            out = self.hybrid_seq_parallel_attn(attn, q[:, S_txt:], k[:, S_txt:], v[:, S_txt:], dropout_p=0.0,
                                                causal=False, joint_tensor_query=q[:, :S_txt],
                                                joint_tensor_key=k[:, :S_txt], joint_tensor_value=v[:, :S_txt],
                                                joint_strategy="front")
        elif _cached(attn) and S_txt:
            ki, vi = get_cache_manager().update_and_get_kv_cache(new_kv=[k[:, S_txt:], v[:, S_txt:]], layer=attn,
                                                                 slice_dim=1, layer_type="attn")
            out = kernels.attn_fwd([q], [k[:, :S_txt], ki], [v[:, :S_txt], vi], out=out4)
        else:
            out = kernels.attn_fwd([q], [k], [v], out=out4)
        return out.reshape(B, out.shape[1], attn.heads * attn.head_dim) if out4 is None else None


def _cached(attn) -> bool:
    return ("attn", attn) in get_cache_manager().cache


# names of the reference's processors that these stand in for
hetuDiTJointAttnProcessor2_0 = JointAttnProcessor
hetuDiTFluxAttnProcessor2_0 = JointAttnProcessor
hetuDiTFluxSingleAttnProcessor2_0 = SingleAttnProcessor

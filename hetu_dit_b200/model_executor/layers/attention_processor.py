"""Attention processors of the -shaped DiT blocks.

They play the role of the reference's hetuDiTJointAttnProcessor2_0 (SD3,
hetu_dit/model_executor/diffusion_executor/layers/attention_processor.py:632-793),
hetuDiTFluxAttnProcessor2_0 (:797-987), hetuDiTCogVideoXAttnProcessor2_0 (:991-1158) and
hetuDiTHunyuanVideoAttnProcessor2_0 (:1346-1531): QKV (+ added QKV) projections,
per-head QK norm, rotary embedding (on every row for Flux, on the video rows only
for CogVideoX and HunyuanVideo), PipeFusion stale-KV update, then either the
single-GPU attention kernel or the USP operator, and the split back into image
and text streams. Token order: [image; text] ("rear") for SD3 and HunyuanVideo,
[text; image] ("front") for Flux and CogVideoX.

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


def _norm_entry(x, w, rope):
    """One tensor of a qk_norm_rope call: (x, weight, norm code, rotate?, bias)."""
    if w is None:
        return (x, None, 0, rope is not None, None)
    return (x, w.weight, w.kind, rope is not None, getattr(w, "bias", None))


def _norm_rope(attn, q, k, wq, wk, rope, row0, rope_seq_start=0):
    """In-place QK norm and RoPE over (B, S, H, D) views; rows below `rope_seq_start` are normalised but not
    rotated, row `rope_seq_start` takes table row `row0`."""
    if wq is None and rope is None:
        return
    if q.shape[1] == 0:
        return
    cos, sin = rope if rope is not None else (None, None)
    kernels.qk_norm_rope([_norm_entry(q, wq, rope), _norm_entry(k, wk, rope)], eps=wq.eps if wq is not None else 1e-6,
                         cos=cos, sin=sin, rope_seq_start=rope_seq_start, rope_row0=row0)


def _prologue_range(lo, hi, wq, wk, rope, row0):
    """One row range of the operator's qk_prologue: norm weights (or None), eps, rotary tables, first table row."""
    do_norm = wq is not None
    if do_norm and wq.kind != 1:
        raise NotImplementedError("the fused head-exchange prologue applies RMSNorm only")
    return (lo, hi, wq.weight if do_norm else None, wk.weight if do_norm else None, wq.eps if do_norm else 1e-6,
            rope, row0)


def _project_into(buf, row0, x, linear):
    """buf[:, row0:row0 + S] = linear(x) without a temporary when the rows are one contiguous block."""
    B, S, _ = x.shape
    if B == 1 and not torch.is_grad_enabled():
        torch.addmm(linear.bias, x[0], linear.weight.t(), out=buf[0, row0:row0 + S])
    else:
        buf[:, row0:row0 + S] = linear(x)


def _out_proj(linear, x, tail):
    """Output projection; tail = (residual, gate) folds the block's gated residual addition into it."""
    if tail is None:
        return linear(x)
    return kernels.linear_tail(linear, x, "gate_residual", residual=tail[0], gate=tail[1])


class _Operators:
    """Lazily built USP operators of one attention layer, rebuilt when the SP degree changes (the reference
    re-creates them in worker.py:1848-1983 on a plan switch)."""

    def __init__(self):
        self._ops, self._world = {}, 0

    def get(self, cls):
        world = ps.get_sequence_parallel_world_size()
        if self._world != world:
            self._ops, self._world = {}, world
        if cls not in self._ops:
            self._ops[cls] = cls(use_kv_cache=True)
        return self._ops[cls]


class JointAttnProcessor:
    """Double-stream (text + image) attention. joint_strategy "rear" = [image; text] (SD3 order,
    attention_processor.py:742-744; HunyuanVideo :1441-1443), "front" = [text; image] (Flux order, :895-897);
    the owning Attention module's `text_first` selects it, its `rope_on_text` says whether the rotary table
    has rows for the text tokens (Flux) or covers the image / video tokens only (HunyuanVideo :1410-1434).

    The reference keeps the whole text stream on every sequence-parallel rank and hands it to the USP
    operator as joint tensors. When the caller passes `text_offset` the text stream is sharded like the
    image stream instead (encoder_hidden_states holds rows [text_offset, text_offset + S_txt) of `text_len`
    text tokens): local text and image rows then form one sequence shard and go through the operator
    without joint tensors. Attention is invariant to the order of keys, and every query row comes back to
    the rank that sent it, so the result is the same while the text projections and MLPs are computed
    once instead of once per rank."""

    def __init__(self):
        self._ops = _Operators()

    @property
    def hybrid_seq_parallel_attn(self):
        ops = list(self._ops._ops.values())
        return ops[0] if ops else None

    def _sharded_text(self, attn, hidden_states, encoder_hidden_states, rope, text_total, token_offset, text_offset,
                      tails=(None, None)):
        B, S_img, _ = hidden_states.shape
        S_txt = encoder_hidden_states.shape[1]
        t0, i0 = (0, S_txt) if attn.text_first else (S_img, 0)
        bufs = []
        for img_p, txt_p in ((attn.to_q, attn.add_q_proj), (attn.to_k, attn.add_k_proj), (attn.to_v, attn.add_v_proj)):
            buf = torch.empty((B, S_txt + S_img, attn.heads * attn.head_dim), dtype=hidden_states.dtype,
                              device=hidden_states.device)
            _project_into(buf, i0, hidden_states, img_p)
            _project_into(buf, t0, encoder_hidden_states, txt_p)
            bufs.append(_heads(buf, attn))
        q, k, v = bufs
        # QK-norm and RoPE ride on the head exchange (or run in place when the plan has no Ulysses exchange)
        text_rows = text_total if attn.rope_on_text else 0
        ranges = [_prologue_range(i0, i0 + S_img, attn.norm_q, attn.norm_k, rope, text_rows + token_offset),
                  _prologue_range(t0, t0 + S_txt, attn.norm_added_q, attn.norm_added_k,
                                  rope if attn.rope_on_text else None, text_offset)]
        out = self._ops.get(hetuDiTLongContextAttention)(_cache_key(attn), q, k, v, dropout_p=0.0, causal=False,
                                                         qk_prologue=sorted(ranges, key=lambda r: r[0]))
        out = out.reshape(B, S_txt + S_img, attn.heads * attn.head_dim)
        return (_out_proj(attn.to_out[0], out[:, i0:i0 + S_img], tails[0]),
                _out_proj(attn.to_add_out, out[:, t0:t0 + S_txt], tails[1]))

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, image_rotary_emb=None, text_len=None,
                 token_offset: int = 0, text_offset=None, tails=(None, None)):
        """tails = ((residual, gate) | None for the image stream, the same for the text stream): the stream's
        result is residual + gate[:, None] * projected attention output instead of the projected output."""
        strategy = "front" if attn.text_first else "rear"
        B, S_img, _ = hidden_states.shape
        S_txt = encoder_hidden_states.shape[1]
        if text_offset is not None and ps.get_sequence_parallel_world_size() > 1:
            return self._sharded_text(attn, hidden_states, encoder_hidden_states, image_rotary_emb,
                                      int(text_len or S_txt), token_offset, text_offset, tails)
        q, k, v = (_heads(p(hidden_states), attn) for p in (attn.to_q, attn.to_k, attn.to_v))
        tq, tk, tv = (_heads(p(encoder_hidden_states), attn) for p in (attn.add_q_proj, attn.add_k_proj, attn.add_v_proj))
        text_rows = S_txt if attn.rope_on_text else 0
        _norm_rope(attn, q, k, attn.norm_q, attn.norm_k, image_rotary_emb, text_rows + token_offset)
        _norm_rope(attn, tq, tk, attn.norm_added_q, attn.norm_added_k,
                   image_rotary_emb if attn.rope_on_text else None, 0)

        if ps.get_sequence_parallel_world_size() > 1:
            cls = hetuDiTFluxLongContextAttention if strategy == "front" else hetuDiTJointLongContextAttention
            out = self._ops.get(cls)(_cache_key(attn), q, k, v, dropout_p=0.0, causal=False, joint_tensor_query=tq,
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
        return _out_proj(attn.to_out[0], img, tails[0]), _out_proj(attn.to_add_out, txt, tails[1])


class SingleAttnProcessor:
    """Single-stream attention over the [text; image] (Flux) or [image; text] (HunyuanVideo) sequence; the
    text / image split under SP follows attention_processor.py:898-901 and :1464-1468."""

    def __init__(self):
        self._ops = _Operators()

    @property
    def hybrid_seq_parallel_attn(self):
        ops = list(self._ops._ops.values())
        return ops[0] if ops else None

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, image_rotary_emb=None, text_len=None,
                 token_offset: int = 0, out=None, text_offset=None, text_total=None):
        """out: optional (B, S, H*D)-shaped view (any row stride) the single-GPU path writes into, e.g. the left
        part of the buffer the block's output projection reads, which saves a concatenation.

        text_len: how many of the rows are text rows (the first ones when the layer's `text_first` is set, the
        last ones otherwise). text_offset / text_total: those rows are rows [text_offset, text_offset + text_len)
        of a text stream of text_total tokens that is sharded over the sequence-parallel ranks (see
        JointAttnProcessor); None = the whole text stream is present on every rank, as in the reference."""
        B, S, _ = hidden_states.shape
        q, k, v = (_heads(p(hidden_states), attn) for p in (attn.to_q, attn.to_k, attn.to_v))
        out4 = None if out is None else out.view(B, S, attn.heads, attn.head_dim)
        S_txt = int(text_len or 0)
        front = attn.text_first
        t_lo, t_hi = (0, S_txt) if front else (S - S_txt, S)
        i_lo, i_hi = (S_txt, S) if front else (0, S - S_txt)
        rope = image_rotary_emb
        rope_txt = rope if attn.rope_on_text else None
        sp = ps.get_sequence_parallel_world_size()
        if text_offset is not None and sp > 1:
            text_rows = int(text_total) if attn.rope_on_text else 0
            ranges = [_prologue_range(t_lo, t_hi, attn.norm_q, attn.norm_k, rope_txt, text_offset),
                      _prologue_range(i_lo, i_hi, attn.norm_q, attn.norm_k, rope, text_rows + token_offset)]
            ctx = self._ops.get(hetuDiTLongContextAttention)(_cache_key(attn), q, k, v, dropout_p=0.0, causal=False,
                                                             qk_prologue=sorted(ranges, key=lambda r: r[0]))
            return ctx.reshape(B, S, attn.heads * attn.head_dim)
        text_rows = S_txt if attn.rope_on_text else 0
        if front and attn.rope_on_text and token_offset == 0:
            _norm_rope(attn, q, k, attn.norm_q, attn.norm_k, rope, 0)
        elif front and not attn.rope_on_text:
            _norm_rope(attn, q, k, attn.norm_q, attn.norm_k, rope, token_offset, rope_seq_start=S_txt)
        else:
            _norm_rope(attn, q[:, t_lo:t_hi], k[:, t_lo:t_hi], attn.norm_q, attn.norm_k, rope_txt, 0)
            _norm_rope(attn, q[:, i_lo:i_hi], k[:, i_lo:i_hi], attn.norm_q, attn.norm_k, rope, text_rows + token_offset)
        if sp > 1:
            strategy = "front" if front else "rear"
            cls = hetuDiTFluxLongContextAttention if front else hetuDiTJointLongContextAttention
            out = self._ops.get(cls)(_cache_key(attn), q[:, i_lo:i_hi], k[:, i_lo:i_hi], v[:, i_lo:i_hi], dropout_p=0.0,
                                     causal=False, joint_tensor_query=q[:, t_lo:t_hi], joint_tensor_key=k[:, t_lo:t_hi],
                                     joint_tensor_value=v[:, t_lo:t_hi], joint_strategy=strategy)
        elif _cached(attn) and S_txt:
            ki, vi = get_cache_manager().update_and_get_kv_cache(new_kv=[k[:, i_lo:i_hi], v[:, i_lo:i_hi]], layer=attn,
                                                                 slice_dim=1, layer_type="attn")
            out = kernels.attn_fwd([q], [k[:, t_lo:t_hi], ki], [v[:, t_lo:t_hi], vi], out=out4)
        else:
            out = kernels.attn_fwd([q], [k], [v], out=out4)
        return out.reshape(B, out.shape[1], attn.heads * attn.head_dim) if out4 is None else None


class CogVideoXAttnProcessor:
    """Attention of the CogVideoX block (attention_processor.py:991-1158): one set of Q/K/V projections over the
    [text; video] rows, QK norm on every row, rotary embedding on the video rows only (:1075-1082). Under
    sequence parallelism the text rows are replicated on every rank and travel as joint tensors with the
    "front" strategy (:1117-1133); the reference passes attn=None there, so this model never uses the stale-KV
    cache."""

    def __init__(self):
        self._ops = _Operators()

    @property
    def hybrid_seq_parallel_attn(self):
        ops = list(self._ops._ops.values())
        return ops[0] if ops else None

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, image_rotary_emb=None, text_len=None,
                 token_offset: int = 0, **_):
        B, S, _ = hidden_states.shape
        T = int(text_len or 0)
        q, k, v = (_heads(p(hidden_states), attn) for p in (attn.to_q, attn.to_k, attn.to_v))
        _norm_rope(attn, q, k, attn.norm_q, attn.norm_k, image_rotary_emb, token_offset, rope_seq_start=T)
        if ps.get_sequence_parallel_world_size() > 1:
            out = self._ops.get(hetuDiTJointLongContextAttention)(
                None, q[:, T:], k[:, T:], v[:, T:], dropout_p=0.0, causal=False, joint_tensor_query=q[:, :T],
                joint_tensor_key=k[:, :T], joint_tensor_value=v[:, :T], joint_strategy="front")
        else:
            out = kernels.attn_fwd([q], [k], [v])
        return out.reshape(B, S, attn.heads * attn.head_dim)


def _cached(attn) -> bool:
    return ("attn", attn) in get_cache_manager().cache


def _cache_key(attn):
    """What the processors hand to the USP operators as the layer that owns a stale-KV buffer: the layer itself
    for the image models, None for the video models (the reference passes attn=None there,
    attention_processor.py:1117, 1496, so they never touch the KV cache)."""
    return attn if getattr(attn, "stale_kv", True) else None


# names of the reference's processors that these stand in for
hetuDiTJointAttnProcessor2_0 = JointAttnProcessor
hetuDiTFluxAttnProcessor2_0 = JointAttnProcessor
hetuDiTFluxSingleAttnProcessor2_0 = SingleAttnProcessor
hetuDiTCogVideoXAttnProcessor2_0 = CogVideoXAttnProcessor
hetuDiTHunyuanVideoAttnProcessor2_0 = JointAttnProcessor

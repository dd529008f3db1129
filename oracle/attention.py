"""CPU oracle: USP (Ulysses x ring) joint attention of the Hetu-DiT denoising hot path.

TEST INFRASTRUCTURE ONLY. Nothing under hetu_dit_b200/ may import this module.

The arithmetic is fp32 torch on the CPU. `sdpa` is the reference's own
non-flash branch (F.scaled_dot_product_attention, e.g.
hetu_dit/model_executor/diffusion_executor/layers/attention_processor.py:772-783).
The sequence-parallel operators are restated for a list of simulated ranks in
one process; each function cites the reference lines it follows.

Third-party pieces that are absent from the reference tree are restated from
their published behaviour and the reference's call sites:
  yunchang==0.3.5 (setup.py:28): SeqAllToAll4D, RingComm, update_out_and_lse;
  flash_attn (README.md:42 pins 2.6.3): _flash_attn_forward returning (out, lse);
  diffusers RMSNorm (setup.py:25): x * rsqrt(mean(x^2) + eps) * weight.

Parity pins: tests/golden/usp_*.npz were produced by running the reference's
own hybrid/attn_layer.py, ring/ring_flash_attn.py and cache_manager.py source
files on CPU `gloo` ranks with those three third-party pieces stubbed
(tests/golden/make_golden.py); tests/test_oracle_golden.py checks this
restatement against them. apply_rotary_emb is pinned against the lifted
reference function the same way.
"""
import math

import torch
import torch.nn.functional as F


def sdpa(q, k, v, scale=None):
    """(B, S, H, D) in, (B, Sq, H, D) fp32 out; exact softmax attention, no mask, no dropout."""
    q, k, v = (t.float().transpose(1, 2) for t in (q, k, v))
    out = F.scaled_dot_product_attention(q, k, v, dropout_p=0.0, is_causal=False, scale=scale)
    return out.transpose(1, 2).contiguous()


def attention_with_lse(q, k, v, scale=None):
    """What one flash-attention call returns at ring_flash_attn.py:76-87: (out (B,Sq,H,D), lse (B,H,Sq)), fp32."""
    q, k, v = (t.float() for t in (q, k, v))
    if scale is None:
        scale = q.shape[-1] ** -0.5
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    return torch.einsum("bhqk,bkhd->bqhd", p, v), lse


def update_out_and_lse(out, lse, block_out, block_lse):
    """Log-sum-exp combine of two partial attention results (call site ring_flash_attn.py:88).

    out: (B, Sq, H, D) fp32 or None; lse: (B, H, Sq) fp32 or None.
    """
    if out is None:
        return block_out.float(), block_lse.float()
    new_lse = torch.logaddexp(lse, block_lse)
    w_old = torch.exp(lse - new_lse).transpose(1, 2).unsqueeze(-1)
    w_new = torch.exp(block_lse - new_lse).transpose(1, 2).unsqueeze(-1)
    return out * w_old + block_out.float() * w_new, new_lse


def seq_all_to_all_4d(xs, scatter_idx, gather_idx):
    """SeqAllToAll4D over a simulated group: xs[r] is rank r's tensor.

    scatter 2 / gather 1: (B, S/U, H, D) -> (B, S, H/U, D): rank r keeps head
    slice r of every rank's tokens, concatenated along S in group-rank order.
    scatter 1 / gather 2 is the inverse. Call sites hybrid/attn_layer.py:102-110,134-136.
    """
    U = len(xs)
    if U == 1:
        return [xs[0]]
    out = []
    for r in range(U):
        parts = [torch.chunk(xs[src], U, dim=scatter_idx)[r] for src in range(U)]
        out.append(torch.cat(parts, dim=gather_idx).contiguous())
    return out


def ring_attention(qs, ks, vs, scale=None, joint_ks=None, joint_vs=None, joint_strategy="none"):
    """ring_flash_attn_forward (ring/ring_flash_attn.py:9-97) for a simulated ring.

    qs/ks/vs: per-ring-rank (B, S_loc, H, D). joint_ks/joint_vs: per-rank joint
    K/V, appended at the last step ("rear") or prepended at step 0 ("front").
    Rank r sees block (r - step) mod R at `step` (send to r+1, receive from r-1).
    Returns per-rank (out fp32, lse (B, H, Sq)).
    """
    if joint_strategy not in ("none", "front", "rear"):
        raise ValueError(f"joint_strategy: {joint_strategy} not supprted.")
    if joint_strategy != "none" and (joint_ks is None or joint_vs is None):
        raise ValueError("joint_tensor_key & joint_tensor_value must not be None when joint_strategy is not None")
    R = len(qs)
    results = []
    for r in range(R):
        out, lse = None, None
        for step in range(R):
            src = (r - step) % R
            k, v = ks[src], vs[src]
            if joint_strategy == "rear" and step + 1 == R:
                k = torch.cat([k, joint_ks[r]], dim=1)
                v = torch.cat([v, joint_vs[r]], dim=1)
            elif joint_strategy == "front" and step == 0:
                k = torch.cat([joint_ks[r], k], dim=1)
                v = torch.cat([joint_vs[r], v], dim=1)
            b_out, b_lse = attention_with_lse(qs[r], k, v, scale)
            out, lse = update_out_and_lse(out, lse, b_out, b_lse)
        results.append((out, lse))
    return results


def usp_attention(qs, ks, vs, ulysses, ring, scale=None, joint_qs=None, joint_ks=None, joint_vs=None,
                  joint_strategy="none"):
    """hetuDiT{,Joint,Flux}LongContextAttention.forward (hybrid/attn_layer.py:45-139,144-274,279-395)
    for U x R simulated ranks.

    qs/ks/vs: per-SP-rank (B, S_loc, H, D), SP rank = ring_idx * U + ulysses_idx
    (Ulysses groups are consecutive ranks, ring groups have stride U:
    parallel_state.py:679-712). joint_*: per-rank (B, S_t, H, D), replicated.
    Returns the per-rank outputs in the input dtype: rows follow the query
    concat order ([local; joint] for "rear", [joint; local] for "front").
    """
    P = ulysses * ring
    assert len(qs) == P
    dtype = qs[0].dtype
    if joint_strategy not in ("none", "front", "rear"):
        raise ValueError(f"joint_strategy: {joint_strategy} not supprted.")
    if joint_strategy != "none" and joint_qs is None:
        raise ValueError("joint_tensor_query must not be None when joint_strategy is not None")
    if joint_strategy == "rear":
        qs = [torch.cat([q, jq], dim=1) for q, jq in zip(qs, joint_qs)]
    elif joint_strategy == "front":
        qs = [torch.cat([jq, q], dim=1) for q, jq in zip(qs, joint_qs)]
    outs = [None] * P
    # Ulysses all-to-all inside every Ulysses group
    q_l, k_l, v_l, jk_l, jv_l = [None] * P, [None] * P, [None] * P, [None] * P, [None] * P
    for g in range(ring):
        members = [g * ulysses + u for u in range(ulysses)]
        for name, src, dst in (("q", qs, q_l), ("k", ks, k_l), ("v", vs, v_l)):
            res = seq_all_to_all_4d([src[m] for m in members], 2, 1)
            for u, m in enumerate(members):
                dst[m] = res[u]
        if joint_strategy != "none":
            for u, m in enumerate(members):
                hpr = joint_ks[m].shape[-2] // ulysses
                jk_l[m] = joint_ks[m][..., hpr * u:hpr * (u + 1), :]
                jv_l[m] = joint_vs[m][..., hpr * u:hpr * (u + 1), :]
    # ring attention inside every ring group
    ctx = [None] * P
    for u in range(ulysses):
        members = [g * ulysses + u for g in range(ring)]
        res = ring_attention([q_l[m] for m in members], [k_l[m] for m in members], [v_l[m] for m in members], scale,
                             [jk_l[m] for m in members] if joint_strategy != "none" else None,
                             [jv_l[m] for m in members] if joint_strategy != "none" else None, joint_strategy)
        for i, m in enumerate(members):
            ctx[m] = res[i][0].to(dtype)  # ring_flash_attn.py:95
    # reverse all-to-all
    for g in range(ring):
        members = [g * ulysses + u for u in range(ulysses)]
        res = seq_all_to_all_4d([ctx[m] for m in members], 1, 2)
        for u, m in enumerate(members):
            outs[m] = res[u]
    return outs


def apply_rotary_emb(x, cos, sin):
    """attention_processor.py:68-120 with use_real=True, use_real_unbind_dim=-1 (Flux / CogVideoX / HunyuanVideo).

    x: (B, H, S, D); cos, sin: (S, D). Pairs (2i, 2i+1) rotate together; math in fp32, cast back (:111).
    """
    xr = x.reshape(*x.shape[:-1], -1, 2)
    x_real, x_imag = xr[..., 0], xr[..., 1]
    rotated = torch.stack([-x_imag, x_real], dim=-1).flatten(3)
    return (x.float() * cos[None, None].float() + rotated.float() * sin[None, None].float()).to(x.dtype)


def rms_norm(x, weight, eps=1e-6):
    """Per-head RMSNorm over the last dim as the reference's attn.norm_q / norm_k modules compute it
    (call sites attention_processor.py:859-862): variance in fp32; the normalised value is cast to the
    weight's dtype before the multiply when the weight is half precision."""
    dtype = x.dtype
    var = x.float().pow(2).mean(-1, keepdim=True)
    y = x.float() * torch.rsqrt(var + eps)
    if weight is not None:
        if weight.dtype in (torch.float16, torch.bfloat16):
            y = y.to(weight.dtype)
        y = y * weight
    return y.to(dtype)


def kv_cache_update(cache, new_kv, patch_mode, num_pipeline_patch, patch_idx, tok_start_local, slice_dim=1,
                    ulysses_world=1, sequence_parallel=False):
    """CacheManager._naive_cache_update / _sequence_parallel_cache_update (cache_manager.py:117-206).

    Returns the tensor attention reads: the fresh K‖V when not in patch mode, otherwise the stale buffer
    with this patch's token range overwritten.
    """
    if num_pipeline_patch == 1 or not patch_mode:
        return new_kv
    scale = ulysses_world if sequence_parallel else 1
    s, e = scale * tok_start_local[patch_idx], scale * tok_start_local[patch_idx + 1]
    idx = [slice(None)] * cache.dim()
    idx[slice_dim] = slice(s, e)
    cache[tuple(idx)] = new_kv
    return cache


def cosine_and_max_rel(a, b):
    """The two acceptance figures for bf16 activations: cosine similarity and max |a-b| / max |b|."""
    a = a.float().flatten()
    b = b.float().flatten()
    cos = F.cosine_similarity(a, b, dim=0).item()
    denom = b.abs().max().item()
    rel = (a - b).abs().max().item() / (denom if denom > 0 else 1.0)
    return cos, rel


LOG2E = math.log2(math.e)

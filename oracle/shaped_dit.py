"""CPU oracle: one denoising step of the SD3- / Flux- / CogVideoX- / HunyuanVideo-shaped DiT in plain fp32 torch.

TEST INFRASTRUCTURE ONLY. Nothing under hetu_dit_b200/ may import this module.

It consumes the state_dict of hetu_dit_b200.model_executor.models.shaped_dit.
ShapedDiT and recomputes the step with F.linear, F.layer_norm, oracle.attention.
rms_norm / apply_rotary_emb and F.scaled_dot_product_attention -- the path the
reference's processors take without flash-attn or a GPU
(hetu_dit/model_executor/diffusion_executor/layers/attention_processor.py:
759-783 for the joint blocks, :969-979 for the Flux blocks; selection in
hetu_dit/envs.py:81-104). Token order follows the reference: [image; text] for
the SD3 shape (:742-744) and the HunyuanVideo shape (:1441-1443), [text; image]
for the Flux shape (:895-897) and the CogVideoX shape (:1042); the video shapes
rotate the video rows only (:1075-1082, :1410-1434).
Also the timed CPU baseline of bench.py.

Parity unpinned for the block wiring (adaLN order, residuals, MLP): it restates diffusers' MMDiT / Flux
blocks from the architecture description, and diffusers is not installed to record fixtures from. Pinned:
joint_attention / single_attention / cogvideox_attention against the __call__ of the reference's five
attention processors run on a stand-in Attention module (tests/golden/attn_processors.npz: row order of
text and image / video rows, which rows are rotated, RMSNorm or LayerNorm QK norm), and underneath them
attention, RMSNorm + rotary embedding (fixtures recorded from the reference's own code).
"""
import math

import torch
import torch.nn.functional as F

from . import attention as oa


def _lin(sd, prefix, x):
    return F.linear(x, sd[prefix + ".weight"].float(), sd[prefix + ".bias"].float())


def _timestep_embedding(t, dim=256, max_period=10000.0):
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def _mlp_embed(sd, prefix, x):
    return _lin(sd, prefix + ".linear_2", F.silu(_lin(sd, prefix + ".linear_1", x)))


def _mod(x, shift, scale):
    return x * (1 + scale[:, None]) + shift[:, None]


def _ff(sd, prefix, x):
    return _lin(sd, prefix + ".module.net.2", F.gelu(_lin(sd, prefix + ".module.net.0.proj", x), approximate="tanh"))


def _heads(x, H, D):
    return x.view(x.shape[0], x.shape[1], H, D)


def _qk(sd, prefix, x, H, D, norm_name, rope, row0, eps=1e-6):
    """projection -> heads -> QK norm -> RoPE; x (B, S, H*D) -> (B, S, H, D). The norm is an RMSNorm, or a
    LayerNorm over the head dimension when the layer has a norm bias (the CogVideoX shape)."""
    y = _heads(x, H, D)
    w = sd.get(prefix + "." + norm_name + ".weight")
    b = sd.get(prefix + "." + norm_name + ".bias")
    if w is not None and b is not None:
        y = F.layer_norm(y, (D,), w.float(), b.float(), eps)
    elif w is not None:
        y = oa.rms_norm(y, w.float(), eps)
    if rope is not None and y.shape[1] > 0:
        cos, sin = rope
        S = y.shape[1]
        y = oa.apply_rotary_emb(y.transpose(1, 2), cos[row0:row0 + S], sin[row0:row0 + S]).transpose(1, 2)
    return y


def joint_attention(sd, a, h, c, rope, H, D, order, kv_hook=None, row0=None, rope_on_text=True):
    """Joint attention of a double-stream block on the modulated streams h (image / video) and c (text), before the
    output projections: (image rows, text rows), each (B, S, H*D). What the reference's processors return:
    hetuDiTJointAttnProcessor2_0 (attention_processor.py:657-794; order "rear", no QK norm, no rotary table),
    hetuDiTFluxAttnProcessor2_0 with encoder_hidden_states (:824-988; order "front", rotary rows for text and image),
    hetuDiTHunyuanVideoAttnProcessor2_0 with add_q_proj (:1373-1534; order "rear", rotary rows for the video only)."""
    d = h.shape[-1]
    S_txt, S_img = c.shape[1], h.shape[1]
    r0 = (S_txt if rope_on_text else 0) if row0 is None else row0
    q = _qk(sd, a, _lin(sd, a + ".to_q", h), H, D, "norm_q", rope, r0)
    k = _qk(sd, a, _lin(sd, a + ".to_k", h), H, D, "norm_k", rope, r0)
    v = _heads(_lin(sd, a + ".to_v", h), H, D)
    if kv_hook is not None:
        k, v = kv_hook(k, v)
    rope_txt = rope if rope_on_text else None
    tq = _qk(sd, a, _lin(sd, a + ".add_q_proj", c), H, D, "norm_added_q", rope_txt, 0)
    tk = _qk(sd, a, _lin(sd, a + ".add_k_proj", c), H, D, "norm_added_k", rope_txt, 0)
    tv = _heads(_lin(sd, a + ".add_v_proj", c), H, D)
    if order == "rear":
        o = oa.sdpa(torch.cat([q, tq], 1), torch.cat([k, tk], 1), torch.cat([v, tv], 1))
        img, txt = o[:, :S_img], o[:, S_img:]
    else:
        o = oa.sdpa(torch.cat([tq, q], 1), torch.cat([tk, k], 1), torch.cat([tv, v], 1))
        txt, img = o[:, :S_txt], o[:, S_txt:]
    return img.reshape(img.shape[0], S_img, d), txt.reshape(txt.shape[0], S_txt, d)


def joint_block(sd, p, hidden, context, temb, rope, H, D, order, kv_hook=None, row0=None, rope_on_text=True):
    """kv_hook(k_img, v_img) -> (k_all, v_all): PipeFusion's stale-KV cache for the image tokens
    (attention_processor.py:702-707); row0: rotary table row of the first image token; rope_on_text: the
    table has rows for the text tokens (Flux) -- otherwise only the image / video rows are rotated."""
    d = hidden.shape[-1]
    mod = _lin(sd, p + ".norm1.linear", F.silu(temb)).chunk(6, dim=-1)
    cmod = _lin(sd, p + ".norm1_context.linear", F.silu(temb)).chunk(6, dim=-1)
    h = _mod(F.layer_norm(hidden, (d,), eps=1e-6), mod[0], mod[1])
    c = _mod(F.layer_norm(context, (d,), eps=1e-6), cmod[0], cmod[1])
    a = p + ".attn.module"
    img, txt = joint_attention(sd, a, h, c, rope, H, D, order, kv_hook, row0, rope_on_text)
    img = _lin(sd, a + ".to_out.0", img)
    txt = _lin(sd, a + ".to_add_out", txt)
    hidden = hidden + mod[2][:, None] * img
    hidden = hidden + mod[5][:, None] * _ff(sd, p + ".ff", _mod(F.layer_norm(hidden, (d,), eps=1e-6), mod[3], mod[4]))
    context = context + cmod[2][:, None] * txt
    context = context + cmod[5][:, None] * _ff(sd, p + ".ff_context",
                                               _mod(F.layer_norm(context, (d,), eps=1e-6), cmod[3], cmod[4]))
    return hidden, context


def single_attention(sd, a, h, rope, H, D, text_len=None, row0=None, kv_hook=None, text_first=True, rope_on_text=True):
    """Attention of a single-stream block over the modulated joint rows h, before the output projection, (B, S, H*D):
    hetuDiTFluxAttnProcessor2_0 without encoder_hidden_states (attention_processor.py:824-988; [text; image], rotary
    rows for all) and hetuDiTHunyuanVideoAttnProcessor2_0 without add_q_proj (:1373-1534; [video; text], rotary rows
    for the video only). text_len / row0 / kv_hook as in single_block()."""
    d = h.shape[-1]
    if not (text_first and rope_on_text):
        assert kv_hook is None and text_len is not None
        S = h.shape[1]
        t_lo, t_hi = (0, text_len) if text_first else (S - text_len, S)
        i_lo, i_hi = (text_len, S) if text_first else (0, S - text_len)
        ql, kl = _lin(sd, a + ".to_q", h), _lin(sd, a + ".to_k", h)
        rope_txt = rope if rope_on_text else None
        r0 = (text_len if rope_on_text else 0) if row0 is None else row0
        parts_q = {t_lo: _qk(sd, a, ql[:, t_lo:t_hi], H, D, "norm_q", rope_txt, 0),
                   i_lo: _qk(sd, a, ql[:, i_lo:i_hi], H, D, "norm_q", rope, r0)}
        parts_k = {t_lo: _qk(sd, a, kl[:, t_lo:t_hi], H, D, "norm_k", rope_txt, 0),
                   i_lo: _qk(sd, a, kl[:, i_lo:i_hi], H, D, "norm_k", rope, r0)}
        q = torch.cat([parts_q[i] for i in sorted(parts_q)], dim=1)
        k = torch.cat([parts_k[i] for i in sorted(parts_k)], dim=1)
        v = _heads(_lin(sd, a + ".to_v", h), H, D)
        return oa.sdpa(q, k, v).reshape(h.shape[0], h.shape[1], d)
    if text_len is None:
        q = _qk(sd, a, _lin(sd, a + ".to_q", h), H, D, "norm_q", rope, 0)
        k = _qk(sd, a, _lin(sd, a + ".to_k", h), H, D, "norm_k", rope, 0)
    else:
        r0 = text_len if row0 is None else row0
        ql, kl = _lin(sd, a + ".to_q", h), _lin(sd, a + ".to_k", h)
        q = torch.cat([_qk(sd, a, ql[:, :text_len], H, D, "norm_q", rope, 0),
                       _qk(sd, a, ql[:, text_len:], H, D, "norm_q", rope, r0)], dim=1)
        k = torch.cat([_qk(sd, a, kl[:, :text_len], H, D, "norm_k", rope, 0),
                       _qk(sd, a, kl[:, text_len:], H, D, "norm_k", rope, r0)], dim=1)
    v = _heads(_lin(sd, a + ".to_v", h), H, D)
    if kv_hook is not None:
        ki, vi = kv_hook(k[:, text_len:], v[:, text_len:])
        k, v = torch.cat([k[:, :text_len], ki], dim=1), torch.cat([v[:, :text_len], vi], dim=1)
    return oa.sdpa(q, k, v).reshape(h.shape[0], h.shape[1], d)


def single_block(sd, p, x, temb, rope, H, D, text_len=None, row0=None, kv_hook=None, text_first=True,
                 rope_on_text=True):
    """x = [text; image] rows. text_len / row0: the first text_len rows take rotary rows [0, text_len), the
    rest rows [row0, ...) (a patch of the image); kv_hook(k_img, v_img) -> (k_all, v_all) is PipeFusion's
    stale-KV cache of the image tokens (attention_processor.py:898-917 of the reference).
    text_first=False: x = [image; text] (HunyuanVideo single blocks, :1464-1468); rope_on_text=False: only the
    image / video rows are rotated, from table row `row0` (default 0)."""
    d = x.shape[-1]
    shift, scale, gate = _lin(sd, p + ".norm.linear", F.silu(temb)).chunk(3, dim=-1)
    h = _mod(F.layer_norm(x, (d,), eps=1e-6), shift, scale)
    mlp = F.gelu(_lin(sd, p + ".proj_mlp", h), approximate="tanh")
    o = single_attention(sd, p + ".attn.module", h, rope, H, D, text_len, row0, kv_hook, text_first, rope_on_text)
    return x + gate[:, None] * _lin(sd, p + ".proj_out", torch.cat([o, mlp], dim=-1))


def cogvideox_attention(sd, a, x, S_txt, rope, H, D, row0=0):
    """Attention of a CogVideoX block over the modulated rows x = [text; video], before the output projection,
    (B, S, H*D): LayerNorm QK norm, rotary rows for the video only -- what hetuDiTCogVideoXAttnProcessor2_0 returns
    (attention_processor.py:1022-1160)."""
    d = x.shape[-1]
    ql, kl = _lin(sd, a + ".to_q", x), _lin(sd, a + ".to_k", x)
    q = torch.cat([_qk(sd, a, ql[:, :S_txt], H, D, "norm_q", None, 0),
                   _qk(sd, a, ql[:, S_txt:], H, D, "norm_q", rope, row0)], dim=1)
    k = torch.cat([_qk(sd, a, kl[:, :S_txt], H, D, "norm_k", None, 0),
                   _qk(sd, a, kl[:, S_txt:], H, D, "norm_k", rope, row0)], dim=1)
    v = _heads(_lin(sd, a + ".to_v", x), H, D)
    return oa.sdpa(q, k, v).reshape(x.shape[0], x.shape[1], d)


def cogvideox_block(sd, p, hidden, context, temb, rope, H, D, row0=0):
    """CogVideoX-shaped block: shared attention / MLP weights over [text; video], own adaLN vectors per stream,
    rotary embedding on the video rows only (attention_processor.py:1042-1082 of the reference)."""
    d = hidden.shape[-1]
    S_txt = context.shape[1]
    m1 = _lin(sd, p + ".norm1.linear", F.silu(temb)).chunk(6, dim=-1)
    m2 = _lin(sd, p + ".norm2.linear", F.silu(temb)).chunk(6, dim=-1)
    x = torch.cat([_mod(F.layer_norm(context, (d,), eps=1e-6), m1[3], m1[4]),
                   _mod(F.layer_norm(hidden, (d,), eps=1e-6), m1[0], m1[1])], dim=1)
    a = p + ".attn1.module"
    o = _lin(sd, a + ".to_out.0", cogvideox_attention(sd, a, x, S_txt, rope, H, D, row0))
    hidden = hidden + m1[2][:, None] * o[:, S_txt:]
    context = context + m1[5][:, None] * o[:, :S_txt]
    x = torch.cat([_mod(F.layer_norm(context, (d,), eps=1e-6), m2[3], m2[4]),
                   _mod(F.layer_norm(hidden, (d,), eps=1e-6), m2[0], m2[1])], dim=1)
    f = _ff(sd, p + ".ff", x)
    hidden = hidden + m2[2][:, None] * f[:, S_txt:]
    context = context + m2[5][:, None] * f[:, :S_txt]
    return hidden, context


def rope_tables(ids, axes, theta=10000.0):
    cos, sin = [], []
    for i, dim in enumerate(axes):
        freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
        ang = ids[:, i].double()[:, None] * freqs[None]
        cos.append(torch.cos(ang).repeat_interleave(2, dim=-1))
        sin.append(torch.sin(ang).repeat_interleave(2, dim=-1))
    return torch.cat(cos, -1).float(), torch.cat(sin, -1).float()


def sincos_pos(grid_h, grid_w, d):
    yy, xx = torch.meshgrid(torch.arange(grid_h, dtype=torch.float32), torch.arange(grid_w, dtype=torch.float32),
                            indexing="ij")
    omega = 1.0 / (10000 ** (torch.arange(d // 4, dtype=torch.float32) / (d // 4)))
    parts = []
    for g in (yy, xx):
        a = g.flatten()[:, None] * omega[None]
        parts += [torch.sin(a), torch.cos(a)]
    return torch.cat(parts, dim=-1)[None]


def grid_ids(text_rows, grid):
    """Position ids (text_rows + tokens, 3): zero rows for the text, then (frame, row, col) per latent token."""
    g3 = tuple(grid) if len(grid) == 3 else (1,) + tuple(grid)
    n = g3[0] * g3[1] * g3[2]
    ids = torch.zeros(text_rows + n, 3)
    tt, yy, xx = torch.meshgrid(*(torch.arange(g) for g in g3), indexing="ij")
    ids[text_rows:, 0] = tt.flatten()
    ids[text_rows:, 1] = yy.flatten()
    ids[text_rows:, 2] = xx.flatten()
    return ids


def denoise_step(sd, shape, latent_tokens, text_embeds, pooled, timestep, guidance=None, grid=None, max_blocks=None,
                 block_outputs=None):
    """One full step in fp32. `shape` is the DiTShape record; `sd` maps parameter names to tensors; `grid` is
    (rows, cols) or (frames, rows, cols). block_outputs: optional list that receives every block's image /
    video stream output (B, S_img, hidden), in order."""
    sd = {k: v.float() for k, v in sd.items()}
    x, txt = latent_tokens.float(), text_embeds.float()
    B, S_img, _ = x.shape
    S_txt = txt.shape[1]
    if grid is None:
        side = int(math.isqrt(S_img))
        grid = (side, S_img // side)
    H, D, d = shape.heads, shape.head_dim, shape.hidden
    temb = _mlp_embed(sd, "time_embed", _timestep_embedding(timestep * 1000.0))
    if shape.pooled_dim:
        temb = temb + _mlp_embed(sd, "pooled_embed", pooled.float())
    if shape.guidance_embed:
        g = guidance if guidance is not None else torch.ones_like(timestep)
        temb = temb + _mlp_embed(sd, "guidance_embed", _timestep_embedding(g * 1000.0))
    hidden = _lin(sd, "x_embedder", x)
    context = _lin(sd, "context_embedder", txt)
    rope = None
    order = "front" if shape.text_first else "rear"
    if shape.rope_axes is not None:
        rope = rope_tables(grid_ids(S_txt if shape.rope_on_text else 0, grid), shape.rope_axes)
    else:
        hidden = hidden + sincos_pos(grid[0], grid[1], d)
    n = 0
    for i in range(shape.n_double):
        if max_blocks is not None and n >= max_blocks:
            break
        if shape.block_kind == "cogvideox":
            hidden, context = cogvideox_block(sd, f"transformer_blocks.{i}", hidden, context, temb, rope, H, D)
        else:
            hidden, context = joint_block(sd, f"transformer_blocks.{i}", hidden, context, temb, rope, H, D, order,
                                          rope_on_text=shape.rope_on_text)
        if block_outputs is not None:
            block_outputs.append(hidden)
        n += 1
    if shape.block_kind == "cogvideox":
        hidden = F.layer_norm(hidden, (d,), sd["norm_final.weight"], sd["norm_final.bias"], 1e-5)
    if shape.n_single:
        xs = torch.cat([context, hidden] if shape.text_first else [hidden, context], dim=1)
        for i in range(shape.n_single):
            if max_blocks is not None and n >= max_blocks:
                break
            if shape.text_first and shape.rope_on_text:
                xs = single_block(sd, f"single_transformer_blocks.{i}", xs, temb, rope, H, D)
            else:
                xs = single_block(sd, f"single_transformer_blocks.{i}", xs, temb, rope, H, D, text_len=S_txt,
                                  text_first=shape.text_first, rope_on_text=shape.rope_on_text)
            if block_outputs is not None:
                block_outputs.append(xs[:, S_txt:] if shape.text_first else xs[:, :S_img])
            n += 1
        hidden = xs[:, S_txt:] if shape.text_first else xs[:, :S_img]
    # the output norm's projection splits into (scale, shift) in diffusers' AdaLayerNormContinuous (SD3, Flux,
    # HunyuanVideo) and into (shift, scale) in its AdaLayerNorm with chunk_dim=1 (CogVideoX)
    first, second = _lin(sd, "norm_out.linear", F.silu(temb)).chunk(2, dim=-1)
    scale, shift = (first, second) if shape.out_norm_scale_first else (second, first)
    hidden = _mod(F.layer_norm(hidden, (d,), eps=1e-6), shift, scale)
    return _lin(sd, "proj_out", hidden)

"""SD3-medium-, Flux.1-dev-, CogVideoX-1.5-5B- and HunyuanVideo-shaped DiT denoisers with seeded random weights.

The reference takes its block definitions from diffusers (absent here) and wraps
them (hetu_dit/model_executor/diffusion_executor/models/transformers/
transformer_sd3.py:29-198, transformer_flux.py:30-221,
cogvideox_transformer_3d.py:30-175, transformer_hunyuan_video.py:56-345). These
classes restate the architectures from their published shapes -- joint
(double-stream) blocks with adaLN-Zero modulation, optional single-stream blocks,
per-head QK RMSNorm, 3-axis rotary embedding (Flux: over text and image rows;
HunyuanVideo: video rows only, text rows last), and the CogVideoX block (one set
of attention / MLP weights over [text; video] rows, separate adaLN vectors per
stream, LayerNorm over the head dimension of Q and K, rotary embedding on the
video rows only) -- so that one denoising step has the reference model's tensor
shapes, token order, FLOPs and memory traffic. Module names follow
the reference's wrapped layout (`attn.module.to_q`, `ff.module.net.0.proj`,
...) because parameter-slice migration addresses Linear layers by those names
(hetu_dit/model_executor/cache/transformer_cache.py:113-154).

GEMMs, LayerNorm and GELU run through torch (cuBLAS / ATen); QK-norm, RoPE,
the K/V cache and attention run through this package's kernels.
"""
import math
import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import kernels
from ...core.distributed import parallel_state as ps
from ..layers.attention_processor import CogVideoXAttnProcessor, JointAttnProcessor, SingleAttnProcessor


@dataclass
class DiTShape:
    name: str
    n_double: int
    n_single: int
    hidden: int
    heads: int
    head_dim: int
    token_in: int          # features of one latent token after patchify
    text_dim: int
    pooled_dim: int
    qk_norm: bool
    rope_axes: Optional[Tuple[int, int, int]]
    guidance_embed: bool
    latent_channels: int = 16
    patch: int = 2
    text_first: Optional[bool] = None    # token order [text; image] ("front"); None: True when there is a rotary table
    rope_on_text: bool = True            # the rotary table has (zero-angle) rows for the text tokens (Flux)
    qk_norm_kind: str = "rms"            # "rms" or "layer" (LayerNorm with weight and bias over head_dim)
    block_kind: str = "mmdit"            # "mmdit": double (+ single) stream blocks; "cogvideox": n_double CogVideoX blocks
    temb_dim: Optional[int] = None       # width of the timestep embedding; None = hidden
    stale_kv: bool = True                # attention layers keep a PipeFusion stale-KV buffer (image models); the
                                         # reference's video processors pass attn=None and never do
    out_norm_scale_first: bool = True    # the output norm's projection splits into (scale, shift), as diffusers'
                                         # AdaLayerNormContinuous does (SD3, Flux, HunyuanVideo); False: (shift,
                                         # scale), as its AdaLayerNorm with chunk_dim=1 does (CogVideoX)

    def __post_init__(self):
        if self.text_first is None:
            self.text_first = self.rope_axes is not None
        if self.temb_dim is None:
            self.temb_dim = self.hidden

    @property
    def n_blocks(self):
        return self.n_double + self.n_single

    @property
    def joint_strategy(self):
        return "front" if self.text_first else "rear"


SD3_MEDIUM = DiTShape("sd3-medium", 24, 0, 1536, 24, 64, 64, 4096, 2048, False, None, False)
FLUX_DEV = DiTShape("flux.1-dev", 19, 38, 3072, 24, 128, 64, 4096, 768, True, (16, 56, 56), True)
# 42 blocks, 48 x 64 heads, patch 2x2x2 over a 16-channel latent (128 features per token), text front, rotary
# embedding on the video rows only, no pooled text vector, 512-wide timestep embedding
COGVIDEOX_5B = DiTShape("cogvideox-1.5-5b", 42, 0, 3072, 48, 64, 128, 4096, 0, True, (16, 24, 24), False,
                        text_first=True, rope_on_text=False, qk_norm_kind="layer", block_kind="cogvideox", temb_dim=512,
                        stale_kv=False, out_norm_scale_first=False)
# 20 double + 40 single blocks, 24 x 128 heads, patch 1x2x2 (64 features per token), text rear
HUNYUAN_VIDEO = DiTShape("hunyuanvideo", 20, 40, 3072, 24, 128, 64, 4096, 768, True, (16, 56, 56), True,
                         text_first=False, rope_on_text=False, stale_kv=False)


def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


class _MLPEmbed(nn.Module):
    def __init__(self, in_dim, hidden):
        super().__init__()
        self.linear_1 = nn.Linear(in_dim, hidden)
        self.linear_2 = nn.Linear(hidden, hidden)

    def forward(self, x):
        return self.linear_2(F.silu(self.linear_1(x)))


class _Wrapped(nn.Module):
    """The reference wraps diffusers layers as `<wrapper>.module`; names in the block cache depend on it."""

    def __init__(self, module: nn.Module):
        super().__init__()
        self.module = module

    def forward(self, *a, **kw):
        return self.module(*a, **kw)


class _GELUProj(nn.Module):
    def __init__(self, d_in, d_out):
        super().__init__()
        self.proj = nn.Linear(d_in, d_out)

    def forward(self, x):
        return kernels.linear_tail(self.proj, x, "gelu_tanh")


class FeedForward(nn.Module):
    def __init__(self, dim, mult=4):
        super().__init__()
        self.net = nn.ModuleList([_GELUProj(dim, dim * mult), nn.Identity(), nn.Linear(dim * mult, dim)])

    def forward(self, x, residual=None, gate=None):
        """residual / gate given: returns residual + gate[:, None] * mlp(x) (the gated residual addition that
        follows the MLP in an adaLN-Zero block rides on the second linear layer)."""
        x = self.net[1](self.net[0](x))
        if residual is None:
            return self.net[2](x)
        return kernels.linear_tail(self.net[2], x, "gate_residual", residual=residual, gate=gate)


class RMSNormWeight(nn.Module):
    """Holds the per-head RMSNorm weight; the normalisation itself is fused into the QK kernel."""
    kind = 1  # do_norm code of the kernel

    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps


class LayerNormWeight(nn.Module):
    """Weight and bias of a LayerNorm over the head dimension (the QK norm of the CogVideoX shape)."""
    kind = 2

    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))
        self.eps = eps


class Attention(nn.Module):
    def __init__(self, shape: DiTShape, joint: bool, out_proj: bool = True):
        super().__init__()
        d = shape.hidden
        self.heads, self.head_dim = shape.heads, shape.head_dim
        self.text_first, self.rope_on_text = bool(shape.text_first), bool(shape.rope_on_text)
        self.stale_kv = bool(shape.stale_kv)
        norm_cls = LayerNormWeight if shape.qk_norm_kind == "layer" else RMSNormWeight
        self.to_q, self.to_k, self.to_v = nn.Linear(d, d), nn.Linear(d, d), nn.Linear(d, d)
        self.norm_q = norm_cls(shape.head_dim) if shape.qk_norm else None
        self.norm_k = norm_cls(shape.head_dim) if shape.qk_norm else None
        self.to_out = nn.ModuleList([nn.Linear(d, d), nn.Identity()]) if out_proj else None
        if joint:
            self.add_q_proj, self.add_k_proj, self.add_v_proj = nn.Linear(d, d), nn.Linear(d, d), nn.Linear(d, d)
            self.norm_added_q = norm_cls(shape.head_dim) if shape.qk_norm else None
            self.norm_added_k = norm_cls(shape.head_dim) if shape.qk_norm else None
            self.to_add_out = nn.Linear(d, d)
        if shape.block_kind == "cogvideox":
            self.processor = CogVideoXAttnProcessor()
        else:
            self.processor = JointAttnProcessor() if joint else SingleAttnProcessor()

    def forward(self, hidden_states, encoder_hidden_states=None, image_rotary_emb=None, text_len=None,
                token_offset=0, **kw):
        return self.processor(self, hidden_states, encoder_hidden_states=encoder_hidden_states,
                              image_rotary_emb=image_rotary_emb, text_len=text_len, token_offset=token_offset, **kw)


_BRANCH_STREAMS = {}
# Run a double block's text-stream tail beside the image-stream tail on one GPU too (under sequence parallelism it
# always does): HDIT_BRANCH_TEXT_TAIL=1.
BRANCH_TEXT_TAIL_ALWAYS = os.environ.get("HDIT_BRANCH_TEXT_TAIL", "0") == "1"


class _Branch:
    """`with _Branch(device) as br:` runs the body on a second stream that starts after everything already
    enqueued on the current stream; br.join() makes the current stream wait for it. Used under sequence
    parallelism to run independent work of a block next to its attention, whose peer exchanges leave the
    GPU idle while flags cross NVLink. Tensors made inside the body must stay referenced until join()."""

    def __init__(self, device):
        self.side = _BRANCH_STREAMS.get(device)
        if self.side is None:
            self.side = _BRANCH_STREAMS[device] = torch.cuda.Stream(device=device)
        self.main = torch.cuda.current_stream(device)
        self._ctx = torch.cuda.stream(self.side)

    def __enter__(self):
        self.side.wait_stream(self.main)
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)

    def join(self):
        self.main.wait_stream(self.side)


def _modulate(x, shift, scale):
    return x * (1 + scale[:, None]) + shift[:, None]


class JointBlock(nn.Module):
    """Double-stream block: image and text streams with their own weights, one joint attention."""

    def __init__(self, shape: DiTShape):
        super().__init__()
        d = shape.hidden
        self.norm1 = nn.Module()
        self.norm1.linear = nn.Linear(d, 6 * d)
        self.norm1_context = nn.Module()
        self.norm1_context.linear = nn.Linear(d, 6 * d)
        self.attn = _Wrapped(Attention(shape, joint=True))
        self.ff = _Wrapped(FeedForward(d))
        self.ff_context = _Wrapped(FeedForward(d))
        self.d = d

    def modulation(self, silu_temb):
        """The block's adaLN vectors; they depend on the timestep embedding only."""
        return (self.norm1.linear(silu_temb).chunk(6, dim=-1), self.norm1_context.linear(silu_temb).chunk(6, dim=-1))

    def forward(self, hidden, context, temb, rope, token_offset=0, text_offset=None, text_total=None, mods=None):
        """text_offset / text_total: `context` holds rows [text_offset, ...) of a text stream of text_total
        tokens sharded over the sequence-parallel ranks; None = the whole text stream (reference layout).
        mods: the result of modulation() when the caller has computed it ahead of time."""
        d = self.d
        mod, cmod = mods if mods is not None else self.modulation(F.silu(temb))
        # LayerNorm + modulation and gate + residual are one fused pass each (csrc/elementwise.cu)
        h = kernels.ln_modulate(hidden, mod[0], mod[1])
        c = kernels.ln_modulate(context, cmod[0], cmod[1])
        sp = (ps.get_sequence_parallel_world_size() > 1 or BRANCH_TEXT_TAIL_ALWAYS) and hidden.is_cuda
        # with fused linear layers the gated residual of the image stream rides on the attention's output
        # projection (and the text stream's too, unless its tail runs on the branch stream below)
        fuse = kernels.FUSED_LINEAR and "gate_residual" in kernels.FUSED_LINEAR_TAILS and hidden.is_cuda
        tails = ((hidden, mod[2]) if fuse else None, (context, cmod[2]) if fuse and not sp else None)
        a_img, a_txt = self.attn(h, encoder_hidden_states=c, image_rotary_emb=rope, token_offset=token_offset,
                                 text_len=text_total, text_offset=text_offset, tails=tails)
        if sp:
            # the text stream's tail is independent of the image stream's: under sequence parallelism its
            # GEMMs have few rows and stream their weights, so they run beside the image stream's
            with _Branch(hidden.device) as br:
                ctx_in = context
                context = kernels.gate_residual(ctx_in, cmod[2], a_txt)
                context = self.ff_context(kernels.ln_modulate(context, cmod[3], cmod[4]), residual=context,
                                          gate=cmod[5])
            hidden = a_img if fuse else kernels.gate_residual(hidden, mod[2], a_img)
            hidden = self.ff(kernels.ln_modulate(hidden, mod[3], mod[4]), residual=hidden, gate=mod[5])
            br.join()
            return hidden, context
        hidden = a_img if fuse else kernels.gate_residual(hidden, mod[2], a_img)
        hidden = self.ff(kernels.ln_modulate(hidden, mod[3], mod[4]), residual=hidden, gate=mod[5])
        context = a_txt if fuse else kernels.gate_residual(context, cmod[2], a_txt)
        context = self.ff_context(kernels.ln_modulate(context, cmod[3], cmod[4]), residual=context, gate=cmod[5])
        return hidden, context


class SingleBlock(nn.Module):
    """Single-stream block over [text; image]: attention and MLP in parallel, one output projection."""

    def __init__(self, shape: DiTShape):
        super().__init__()
        d = shape.hidden
        self.norm = nn.Module()
        self.norm.linear = nn.Linear(d, 3 * d)
        self.proj_mlp = nn.Linear(d, 4 * d)
        self.attn = _Wrapped(Attention(shape, joint=False, out_proj=False))
        self.proj_out = nn.Linear(5 * d, d)
        self.d = d

    def modulation(self, silu_temb):
        return self.norm.linear(silu_temb).chunk(3, dim=-1)

    def forward(self, x, temb, rope, text_len, token_offset=0, text_offset=None, text_total=None, mods=None):
        shift, scale, gate = mods if mods is not None else self.modulation(F.silu(temb))
        h = kernels.ln_modulate(x, shift, scale)
        if ps.get_sequence_parallel_world_size() == 1:
            # attention output and GELU(MLP) land side by side in the buffer the output projection reads:
            # no concatenated copy
            B, S, d = x.shape
            buf = torch.empty((B, S, 5 * d), dtype=x.dtype, device=x.device)
            kernels.linear_tail(self.proj_mlp, h, "gelu_tanh", out=buf[..., d:])
            self.attn(h, image_rotary_emb=rope, text_len=text_len, token_offset=token_offset, out=buf[..., :d])
            return kernels.linear_tail(self.proj_out, buf, "gate_residual", residual=x, gate=gate)
        # MLP branch beside the attention: its GEMM fills the SMs that the head-sharded attention grid leaves
        # free and the time the two peer exchanges spend waiting on flags
        B, S, d = x.shape
        buf = torch.empty((B, S, 5 * d), dtype=x.dtype, device=x.device)
        with _Branch(x.device) as br:
            kernels.linear_tail(self.proj_mlp, h, "gelu_tanh", out=buf[..., d:])
        a = self.attn(h, image_rotary_emb=rope, text_len=text_len, token_offset=token_offset, text_offset=text_offset,
                      text_total=text_total)
        buf[..., :d].copy_(a)
        br.join()
        return kernels.linear_tail(self.proj_out, buf, "gate_residual", residual=x, gate=gate)


class CogVideoXBlock(nn.Module):
    """CogVideoX-shaped block: text and video rows share the attention and MLP weights but take their own
    adaLN-Zero vectors (two sets of six: around the attention and around the MLP); attention runs over
    [text; video]."""

    def __init__(self, shape: DiTShape):
        super().__init__()
        d = shape.hidden
        self.norm1 = nn.Module()
        self.norm1.linear = nn.Linear(shape.temb_dim, 6 * d)
        self.attn1 = _Wrapped(Attention(shape, joint=False, out_proj=True))
        self.norm2 = nn.Module()
        self.norm2.linear = nn.Linear(shape.temb_dim, 6 * d)
        self.ff = _Wrapped(FeedForward(d))
        self.d = d

    def modulation(self, silu_temb):
        return self.norm1.linear(silu_temb).chunk(6, dim=-1), self.norm2.linear(silu_temb).chunk(6, dim=-1)

    def forward(self, hidden, context, temb, rope, token_offset=0, mods=None):
        """hidden (B, S_vid, d) video rows of this rank, context (B, S_txt, d) all text rows. Each vector set is
        (shift, scale, gate) for the video rows followed by (shift, scale, gate) for the text rows."""
        m1, m2 = mods if mods is not None else self.modulation(F.silu(temb))
        B, S_vid, d = hidden.shape
        S_txt = context.shape[1]
        x = torch.empty((B, S_txt + S_vid, d), dtype=hidden.dtype, device=hidden.device)
        kernels.ln_modulate(context, m1[3], m1[4], out=x[:, :S_txt])
        kernels.ln_modulate(hidden, m1[0], m1[1], out=x[:, S_txt:])
        attn = self.attn1.module
        a = attn.to_out[0](self.attn1(x, image_rotary_emb=rope, text_len=S_txt, token_offset=token_offset))
        hidden = kernels.gate_residual(hidden, m1[2], a[:, S_txt:])
        context = kernels.gate_residual(context, m1[5], a[:, :S_txt])
        kernels.ln_modulate(context, m2[3], m2[4], out=x[:, :S_txt])
        kernels.ln_modulate(hidden, m2[0], m2[1], out=x[:, S_txt:])
        f = self.ff(x)
        hidden = kernels.gate_residual(hidden, m2[2], f[:, S_txt:])
        context = kernels.gate_residual(context, m2[5], f[:, :S_txt])
        return hidden, context


def rope_tables(ids: torch.Tensor, axes, theta: float = 10000.0):
    """cos / sin tables (S, D) for integer position ids (S, 3); each axis owns axes[i] dims, pairs share a frequency."""
    cos, sin = [], []
    for i, dim in enumerate(axes):
        freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64, device=ids.device) / dim))
        ang = ids[:, i].double()[:, None] * freqs[None]
        cos.append(torch.cos(ang).repeat_interleave(2, dim=-1))
        sin.append(torch.sin(ang).repeat_interleave(2, dim=-1))
    return torch.cat(cos, -1).float().contiguous(), torch.cat(sin, -1).float().contiguous()


class ShapedDiT(nn.Module):
    def __init__(self, shape: DiTShape):
        super().__init__()
        self.shape = shape
        d = shape.hidden
        self.x_embedder = nn.Linear(shape.token_in, d)
        self.context_embedder = nn.Linear(shape.text_dim, d)
        self.time_embed = _MLPEmbed(256, shape.temb_dim)
        self.pooled_embed = _MLPEmbed(shape.pooled_dim, shape.temb_dim) if shape.pooled_dim else None
        self.guidance_embed = _MLPEmbed(256, shape.temb_dim) if shape.guidance_embed else None
        block_cls = CogVideoXBlock if shape.block_kind == "cogvideox" else JointBlock
        self.transformer_blocks = nn.ModuleList([block_cls(shape) for _ in range(shape.n_double)])
        self.single_transformer_blocks = nn.ModuleList([SingleBlock(shape) for _ in range(shape.n_single)])
        # the CogVideoX shape normalises [text; video] once more (with weight and bias) before the output adaLN
        self.norm_final = nn.LayerNorm(d, eps=1e-5) if shape.block_kind == "cogvideox" else None
        self.norm_out = nn.Module()
        self.norm_out.linear = nn.Linear(shape.temb_dim, 2 * d)
        self.proj_out = nn.Linear(d, shape.token_in)
        if shape.rope_axes is None:
            self.pos_embed_max = 192  # learned-position stand-in: sin-cos table cropped to the latent grid
        self._rope_cache = {}
        # shard the text stream over the sequence-parallel ranks when it divides evenly (see forward)
        self.shard_text = True
        # compute every block's adaLN vectors on a second stream, ahead of the blocks (see _modulations_ahead)
        self.modulation_ahead = True
        # under sequence parallelism every rank would stream the same adaLN weights for the same timestep
        # embedding: each rank computes the vectors of every SP-th block and stores them to its peers instead.
        # From this SP degree on (0 = never). Measured at degree 2: 39.7-39.8 ms against 39.55-39.6 ms per
        # Flux-shaped step, i.e. the exchange costs what halving the weight stream saves; the saving grows with
        # the degree (7/8 of 6.4 GB per step at degree 8), the exchange does not.
        self.shard_modulation_from = int(os.environ.get("HDIT_SHARD_MODULATION_FROM", "4"))
        self._mod_stream = {}

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02):
        """Weights ~ N(0, std), biases 0, norm weights 1, from a seeded generator on the parameters' device."""
        gen = torch.Generator(device=self.x_embedder.weight.device).manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("bias"):
                p.zero_()
            elif p.dim() == 1:
                p.fill_(1.0)
            else:
                p.copy_(torch.randn(p.shape, generator=gen, device=p.device, dtype=torch.float32) * std)
        return self

    def register_cache(self):
        """One stale-KV entry per attention layer: the plain cache when the plan has no sequence
        parallelism, the sequence-parallel one otherwise (what the reference's _register_cache does,
        hetu_dit/model_executor/diffusion_executor/models/base_model.py:162-178). Call after a plan switch."""
        from ...core.distributed import parallel_state as ps
        from ...core.resource_manager.cache_manager import get_cache_manager
        if not self.shape.stale_kv:
            return
        kind = "sequence_parallel_attn_cache" if ps.get_sequence_parallel_world_size() > 1 else "naive_cache"
        for m in self.modules():
            if isinstance(m, Attention):
                get_cache_manager().register_cache_entry(m, "attn", kind)

    def _rope(self, text_rows, grid, device):
        """cos / sin tables with `text_rows` zero-angle rows followed by one row per latent token of `grid`
        ((rows, cols) for images, (frames, rows, cols) for video; axis 0 of the ids is the frame index)."""
        grid = tuple(int(g) for g in grid)
        key = (text_rows, grid, str(device))
        if key not in self._rope_cache:
            g3 = grid if len(grid) == 3 else (1,) + grid
            n = g3[0] * g3[1] * g3[2]
            ids = torch.zeros(text_rows + n, 3, device=device)
            tt, yy, xx = torch.meshgrid(*(torch.arange(g, device=device) for g in g3), indexing="ij")
            ids[text_rows:, 0] = tt.flatten()
            ids[text_rows:, 1] = yy.flatten()
            ids[text_rows:, 2] = xx.flatten()
            self._rope_cache[key] = rope_tables(ids, self.shape.rope_axes)
        return self._rope_cache[key]

    def _sincos_pos(self, grid_h, grid_w, device, dtype):
        key = ("pos", grid_h, grid_w, str(device), dtype)
        if key not in self._rope_cache:
            d = self.shape.hidden
            yy, xx = torch.meshgrid(torch.arange(grid_h, device=device, dtype=torch.float32),
                                    torch.arange(grid_w, device=device, dtype=torch.float32), indexing="ij")
            omega = 1.0 / (10000 ** (torch.arange(d // 4, device=device, dtype=torch.float32) / (d // 4)))
            parts = []
            for g in (yy, xx):
                a = g.flatten()[:, None] * omega[None]
                parts += [torch.sin(a), torch.cos(a)]
            self._rope_cache[key] = torch.cat(parts, dim=-1).to(dtype)[None]
        return self._rope_cache[key]

    def forward(self, latent_tokens, text_embeds, pooled, timestep, guidance=None, grid=None, token_offset: int = 0,
                full_grid: Optional[Tuple[int, ...]] = None, token_index: Optional[torch.Tensor] = None):
        """latent_tokens (B, S_img, token_in); text_embeds (B, S_txt, text_dim); pooled (B, pooled_dim) or None;
        timestep, guidance (B,). Returns the predicted noise (B, S_img, token_in).

        Under sequence parallelism a rank passes its share of the latent tokens. `full_grid` is the whole
        latent grid ((rows, cols), or (frames, rows, cols) for video) and selects the rotary / position
        tables; the rank's tokens are either one contiguous range starting at `token_offset` (a band of rows of
        an image, or HunyuanVideo's chunk of the flattened token axis, transformer_hunyuan_video.py:226-231),
        or any subset given by `token_index` (global token ids, e.g. a band of rows of every frame, as the
        reference shards video latents, base_pipeline.py:337-344)."""
        shp = self.shape
        B, S_img, _ = latent_tokens.shape
        S_txt = text_embeds.shape[1]
        if grid is None:
            side = int(math.isqrt(S_img))
            grid = (side, S_img // side)
        dtype = latent_tokens.dtype
        temb = self.time_embed(timestep_embedding(timestep * 1000.0).to(dtype))
        if self.pooled_embed is not None:
            temb = temb + self.pooled_embed(pooled)
        if self.guidance_embed is not None:
            g = guidance if guidance is not None else torch.ones_like(timestep)
            temb = temb + self.guidance_embed(timestep_embedding(g * 1000.0).to(dtype))
        hidden = self.x_embedder(latent_tokens)
        # Text stream: the reference keeps all of it on every sequence-parallel rank. When it divides evenly
        # each rank takes a contiguous shard instead (the result is the same, the text-stream work is not
        # repeated on every rank); PipeFusion stages and the CogVideoX shape keep the reference layout.
        text_offset = text_total = None
        sp = ps.get_sequence_parallel_world_size()
        if self.shard_text and sp > 1 and S_txt % sp == 0 and ps.get_pipeline_parallel_world_size() == 1 and \
                shp.block_kind == "mmdit":
            text_total = S_txt
            S_txt = S_txt // sp
            text_offset = ps.get_sequence_parallel_rank() * S_txt
            text_embeds = text_embeds[:, text_offset:text_offset + S_txt]
        context = self.context_embedder(text_embeds)
        fg = full_grid or grid
        rope = None
        if shp.rope_axes is not None:
            text_rows = (text_total or S_txt) if shp.rope_on_text else 0
            rope = self._rope(text_rows, fg, latent_tokens.device)
            if token_index is not None:
                # the rank's rows of the table, text rows first: a local table addressed from token 0
                rows = token_index + text_rows
                if text_rows:
                    rows = torch.cat([torch.arange(text_rows, device=rows.device), rows])
                rope = (rope[0].index_select(0, rows), rope[1].index_select(0, rows))
                token_offset = 0
        else:
            pos = self._sincos_pos(fg[0], fg[1], latent_tokens.device, dtype)
            hidden = hidden + (pos[:, token_offset:token_offset + S_img] if token_index is None
                               else pos.index_select(1, token_index))
        ahead = self._modulations_ahead(temb) if self.modulation_ahead and temb.is_cuda else None
        main = torch.cuda.current_stream(temb.device) if ahead is not None else None

        def mods_of(i):
            if ahead is None:
                return None
            ev, m = ahead[i]
            main.wait_event(ev)
            return m

        n_double = len(self.transformer_blocks)
        if shp.block_kind == "cogvideox":
            for i, blk in enumerate(self.transformer_blocks):
                hidden, context = blk(hidden, context, temb, rope, token_offset, mods_of(i))
            hidden = self.norm_final(hidden)
        else:
            for i, blk in enumerate(self.transformer_blocks):
                hidden, context = blk(hidden, context, temb, rope, token_offset, text_offset, text_total, mods_of(i))
        if len(self.single_transformer_blocks):
            x = torch.cat([context, hidden] if shp.text_first else [hidden, context], dim=1)
            for i, blk in enumerate(self.single_transformer_blocks):
                x = blk(x, temb, rope, S_txt, token_offset, text_offset, text_total, mods_of(n_double + i))
            hidden = x[:, S_txt:] if shp.text_first else x[:, :S_img]
        if ahead is not None:
            first, second = mods_of(len(ahead) - 1)
            main.wait_stream(self._mod_stream[temb.device])
        else:
            first, second = self.norm_out.linear(F.silu(temb)).chunk(2, dim=-1)
        scale, shift = (first, second) if shp.out_norm_scale_first else (second, first)
        return self.proj_out(kernels.ln_modulate(hidden.contiguous(), shift, scale))

    def forward_graphed(self, latent_tokens, text_embeds, pooled, timestep, guidance=None, grid=None,
                        token_offset: int = 0, full_grid: Optional[Tuple[int, ...]] = None,
                        token_index: Optional[torch.Tensor] = None):
        """forward() replayed from a CUDA graph that is captured on the first call with these shapes under the
        active plan (see step_graph.StepGraphCache). The result is the graph's output buffer: use it before the
        next call with the same shapes. Every rank of a sequence-parallel plan must make the same calls."""
        from ..step_graph import StepGraphCache
        cache = self.__dict__.setdefault("_step_graphs", StepGraphCache())
        if guidance is None:
            guidance = torch.ones_like(timestep)
        key = ("step", tuple(latent_tokens.shape), tuple(text_embeds.shape), latent_tokens.dtype, bool(self.shard_text),
               tuple(grid) if grid is not None else None, int(token_offset),
               tuple(full_grid) if full_grid is not None else None,
               None if token_index is None else (int(token_index.numel()), token_index.data_ptr()))

        def fn(lat, txt, pl, t, g):
            # token_index is read by the replayed graph: the caller keeps that tensor alive and unchanged (it is
            # part of the key by address)
            return self.forward(lat, txt, pl, t, g, grid=grid, token_offset=token_offset, full_grid=full_grid,
                                token_index=token_index)

        return cache.run(key, fn, latent_tokens, text_embeds, pooled, timestep, guidance)

    def _modulations_ahead(self, temb):
        """Every block's adaLN vectors depend only on the timestep embedding, and each is a matrix-vector
        product that streams its weight once from HBM (6.4 GB per step at the Flux shape) while the blocks'
        GEMMs are tensor-bound. They are therefore enqueued on a second stream right after the
        embedding, one event per block, and fill the gaps between the blocks' kernels. Returns
        [(event, vectors)] for the double blocks, the single blocks and the output norm, in that order. The
        caller waits on each event before use and joins the stream at the end, which also keeps the vectors'
        memory from being handed out again while the main stream still reads it."""
        dev = temb.device
        side = self._mod_stream.get(dev)
        if side is None:
            side = self._mod_stream[dev] = torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream(dev)
        side.wait_stream(main)
        out = []
        sp = ps.get_sequence_parallel_world_size()
        if 1 < self.shard_modulation_from <= sp and ps.get_sp_group().heap is not None:
            with torch.cuda.stream(side):
                return self._modulations_sharded(temb, side)
        with torch.cuda.stream(side):
            silu = F.silu(temb)
            for blk in list(self.transformer_blocks) + list(self.single_transformer_blocks):
                m = blk.modulation(silu)
                ev = torch.cuda.Event()
                ev.record(side)
                out.append((ev, m))
            m = self.norm_out.linear(silu).chunk(2, dim=-1)
            ev = torch.cuda.Event()
            ev.record(side)
            out.append((ev, m))
        return out

    _MOD_CHANNEL = 2  # point-to-point flag channel (0: PipeFusion patches, 1: stage hand-off)

    def _modulations_sharded(self, temb, side):
        """_modulations_ahead under sequence parallelism: the timestep embedding is the same on every SP rank, so
        rank r computes the vectors of items r, r + sp, ... (an item = one block, or the output norm), stores
        them into every peer's gathered buffer (one copy launch), raises one flag per peer and waits for the
        peers' flags. Each rank streams 1 / sp of the adaLN weights. The gathered rows are copied out of the
        heap before use: a peer that has finished this step may store the next step's rows while this rank is
        still in the last block (it cannot be earlier than that: every block's exchange barrier needs this rank,
        and the main stream enters the first block only after the copy)."""
        group = ps.get_sp_group()
        heap, me, world = group.heap, group.rank_in_group, group.world_size
        blocks = list(self.transformer_blocks) + list(self.single_transformer_blocks)
        n_items = len(blocks) + 1
        per = (n_items + world - 1) // world
        silu = F.silu(temb)
        B = silu.shape[0]

        def groups_of(m):
            return [m] if torch.is_tensor(m[0]) else list(m)

        rows = []
        for slot, i in enumerate(range(me, n_items, world)):
            m = blocks[i].modulation(silu) if i < len(blocks) else self.norm_out.linear(silu).chunk(2, dim=-1)
            rows.append(torch.cat([t for g in groups_of(m) for t in g], dim=-1))
        width = max(self._mod_width(blocks, i) for i in range(n_items))
        mine = torch.zeros((per, B, width), dtype=silu.dtype, device=silu.device)
        for slot, row in enumerate(rows):
            mine[slot, :, :row.shape[-1]] = row
        gathered, off = heap.alloc((world, per, B, width), silu.dtype, name=f"adaln_gather_{per}x{B}x{width}_{group.ranks}")
        nbytes = mine.numel() * mine.element_size()
        kernels.copy_pieces([(mine.data_ptr(), heap.peer_ptr(r, off) + me * nbytes, 1, 0, 0, 1, 0, 0, nbytes)
                             for r in group.ranks], silu.device)
        for r in group.ranks:
            if r != group.global_rank:
                heap.signal(r, self._MOD_CHANNEL)
        for r in group.ranks:
            if r != group.global_rank:
                heap.wait(r, self._MOD_CHANNEL)
        local = gathered.clone()
        ev = torch.cuda.Event()
        ev.record(side)
        out = []
        d = self.shape.hidden
        for i in range(n_items):
            row = local[i % world, i // world]
            counts = self._mod_counts(blocks, i)
            parts, c0 = [], 0
            for n in counts:
                parts.append(tuple(row[:, c0 + k * d:c0 + (k + 1) * d] for k in range(n)))
                c0 += n * d
            out.append((ev, parts[0] if len(parts) == 1 else tuple(parts)))
        return out

    def _mod_counts(self, blocks, i):
        """How many hidden-sized vectors item i's modulation has, per group (a group = one adaLN linear)."""
        if i >= len(blocks):
            return [2]
        return [3] if isinstance(blocks[i], SingleBlock) else [6, 6]

    def _mod_width(self, blocks, i):
        return sum(self._mod_counts(blocks, i)) * self.shape.hidden

    def flops_per_step(self, s_img: int, s_txt: int, batch: int = 1) -> float:
        """Algorithmic FLOPs of one step: 4*S^2*Dm attention + 2*12*Dm^2*S linear per block."""
        S = s_img + s_txt
        d = self.shape.hidden
        return batch * self.shape.n_blocks * (4.0 * S * S * d + 24.0 * d * d * S)

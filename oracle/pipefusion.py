"""CPU oracle: PipeFusion denoising of the SD3-shaped model (warm-up steps, then the patch pipeline
with stale K/V), fp32, one process.

TEST INFRASTRUCTURE ONLY. Nothing under hetu_dit_b200/ may import this module.

Parity unpinned for the numbers this file's step and patch loops produce: the reference's pipelines subclass
diffusers classes and diffusers is not installed, so a whole denoising run cannot be recorded. Pinned underneath:
the patch index lists and the stale-KV update order (fixtures recorded from the reference's own runtime_state and
CacheManager), attention and the rotary embedding, the scheduler step. The ORDER of events of the loops
(receives, forwards, scheduler steps, sends per stage) and the stage forward of the transformer wrappers are
pinned separately, product against the reference's own loops run on recording stand-ins
(tests/golden/pipefusion_order.json, stage_forward.npz); this file is the sequential model those pipelined
runs must agree with numerically.

Restates the schedule of the reference's SD3 pipeline
(hetu_dit/model_executor/pipelines/pipeline_stable_diffusion_3.py: _sync_pipeline :1352-1467,
_async_pipeline :1515-1678, _backbone_forward with classifier-free guidance :1680-1717) and of its
transformer wrapper (models/transformers/transformer_sd3.py:95-198: positional embedding only on
the first stage, the text stream of a step computed with patch 0 and re-used by the other patches
:131-146). A layer's stale-KV buffer is touched only by the stage that owns the layer and patches
visit stages in order, so running (step, patch, layer) in sequence on one process produces exactly
the values the pipelined execution does, for any number of stages.
"""
import torch
import torch.nn.functional as F

from . import shaped_dit as osd


def flow_match_sigmas(num_steps, shift=3.0):
    """Sigma schedule of a flow-matching Euler scheduler: shifted linear from 1 to 0 (num_steps + 1 values)."""
    s = torch.linspace(1.0, 1.0 / num_steps, num_steps, dtype=torch.float64)
    s = shift * s / (1 + (shift - 1) * s)
    return torch.cat([s, torch.zeros(1, dtype=torch.float64)]).float()


def warmup_cache_order(num_patch_tokens, ulysses):
    """Token order of the stale-KV buffer a warm-up step leaves behind under Ulysses sequence parallelism.

    Rank r holds slice r of every patch. After the head exchange of a whole-image step the gathered K/V is
    ordered rank-major, patch-minor, and the reference stores it in that order
    (core/resource_manager/cache_manager.py:170-184). Patch-mode updates then write the gathered patch p --
    its slices in rank order, i.e. the patch in image order -- at [U * local_start[p], U * local_start[p+1])
    (:186-205), which is the patch's place in *image* order. Until every patch has been refreshed once the
    buffer therefore mixes the two orders: some stale rows are attended twice and some not at all. Returns
    the image-order index of every buffer row after warm-up."""
    starts = [0]
    for n in num_patch_tokens:
        starts.append(starts[-1] + n)
    order = []
    for r in range(ulysses):
        for p, n in enumerate(num_patch_tokens):
            share = n // ulysses
            order.extend(range(starts[p] + r * share, starts[p] + (r + 1) * share))
    return torch.tensor(order, dtype=torch.long)


def denoise(sd, shape, latents, prompt_embeds, pooled, num_steps, guidance_scale, num_patch_tokens, warmup_steps, grid,
            ulysses=1):
    """latents (1, S, token_in); prompt_embeds (2, S_txt, text_dim) = [uncond, cond]; pooled (2, pooled_dim).
    num_patch_tokens: tokens per pipeline patch over all sequence-parallel ranks. ulysses: Ulysses degree of the
    plan being modelled (it changes which stale rows the first patched step sees, see warmup_cache_order).
    Returns the final latents, fp32."""
    sd = {k: v.float() for k, v in sd.items()}
    H, D, d = shape.heads, shape.head_dim, shape.hidden
    sig = flow_match_sigmas(num_steps)
    x = latents.float()
    S = x.shape[1]
    pos = osd.sincos_pos(grid[0], grid[1], d)
    n_layers = shape.n_double
    kv = [None] * n_layers            # per layer stale (K, V) of the image tokens, (2, S, H, D)
    text_cache = [None] * n_layers    # per layer text stream input of the current step
    starts = [0]
    for n in num_patch_tokens:
        starts.append(starts[-1] + n)
    order = warmup_cache_order(num_patch_tokens, ulysses) if ulysses > 1 and len(num_patch_tokens) > 1 else None

    def temb_of(i):
        t = sig[i].expand(2)
        return osd._mlp_embed(sd, "time_embed", osd._timestep_embedding(t * 1000.0)) + osd._mlp_embed(
            sd, "pooled_embed", pooled.float())

    def backbone(tokens, i, patch):
        """tokens (1, n, token_in) -> guided noise prediction (1, n, token_in)."""
        temb = temb_of(i)
        lo = 0 if patch is None else starts[patch]
        n = tokens.shape[1]
        hidden = osd._lin(sd, "x_embedder", torch.cat([tokens, tokens])) + pos[:, lo:lo + n]
        context = osd._lin(sd, "context_embedder", prompt_embeds.float())
        for l in range(n_layers):
            def hook(k, v, l=l):
                if patch is None:
                    kv[l] = (k.clone(), v.clone()) if order is None else (k[:, order].clone(), v[:, order].clone())
                    return k, v
                else:
                    kv[l][0][:, lo:lo + n] = k
                    kv[l][1][:, lo:lo + n] = v
                return kv[l]
            if patch is None:
                hidden, context = osd.joint_block(sd, f"transformer_blocks.{l}", hidden, context, temb, None, H, D,
                                                  "rear", kv_hook=hook)
            elif patch == 0:
                text_cache[l] = context
                hidden, context = osd.joint_block(sd, f"transformer_blocks.{l}", hidden, context, temb, None, H, D,
                                                  "rear", kv_hook=hook)
            else:
                hidden, _ = osd.joint_block(sd, f"transformer_blocks.{l}", hidden, text_cache[l], temb, None, H, D,
                                            "rear", kv_hook=hook)
        first, second = osd._lin(sd, "norm_out.linear", F.silu(temb)).chunk(2, dim=-1)
        scale, shift = (first, second) if shape.out_norm_scale_first else (second, first)
        out = osd._lin(sd, "proj_out", osd._mod(F.layer_norm(hidden, (d,), eps=1e-6), shift, scale))
        uncond, cond = out.chunk(2)
        return uncond + guidance_scale * (cond - uncond)

    for i in range(num_steps):
        dt = sig[i + 1] - sig[i]
        if i < warmup_steps or len(num_patch_tokens) == 1:
            x = x + dt * backbone(x, i, None)
        else:
            new = []
            for p in range(len(num_patch_tokens)):
                xp = x[:, starts[p]:starts[p + 1]]
                new.append(xp + dt * backbone(xp, i, p))
            x = torch.cat(new, dim=1)
    return x


def denoise_flux(sd, shape, latents, prompt_embeds, pooled, num_steps, guidance, num_patch_tokens, warmup_steps, grid,
                 stage_starts=(0,)):
    """PipeFusion denoising of the Flux-shaped model (double + single blocks, rotary positions, embedded
    guidance, no classifier-free batch). latents (1, S, token_in); prompt_embeds (1, S_txt, text_dim); pooled
    (1, pooled_dim); guidance: float. stage_starts: global index (double blocks first, then single blocks) of
    the first block of every pipeline stage.

    Follows the reference's Flux pipeline (hetu_dit/model_executor/pipelines/pipeline_flux.py: _sync_pipeline
    :447-555, _async_pipeline :557-723) and transformer wrapper
    (diffusion_executor/models/transformers/transformer_flux.py:101-206): every patch carries the text stream
    through all blocks of the first stage again; a later stage receives the text stream only with patch 0 of a
    step and re-uses it for the step's other patches (:598-603, :659-663). Stale K/V holds image tokens only."""
    sd = {k: v.float() for k, v in sd.items()}
    H, D, d = shape.heads, shape.head_dim, shape.hidden
    sig = flow_match_sigmas(num_steps)
    x = latents.float()
    S, S_txt = x.shape[1], prompt_embeds.shape[1]
    ids = torch.zeros(S_txt + S, 3)
    yy, xx = torch.meshgrid(torch.arange(grid[0]), torch.arange(grid[1]), indexing="ij")
    ids[S_txt:, 1], ids[S_txt:, 2] = yy.flatten(), xx.flatten()
    rope = osd.rope_tables(ids, shape.rope_axes)
    n_double, n_total = shape.n_double, shape.n_double + shape.n_single
    kv = [None] * n_total
    boundary_text = {}
    starts = [0]
    for n in num_patch_tokens:
        starts.append(starts[-1] + n)
    g_vec = torch.full((1,), float(guidance))

    def backbone(tokens, i, patch):
        t = sig[i].expand(1)
        temb = (osd._mlp_embed(sd, "time_embed", osd._timestep_embedding(t * 1000.0))
                + osd._mlp_embed(sd, "pooled_embed", pooled.float())
                + osd._mlp_embed(sd, "guidance_embed", osd._timestep_embedding(g_vec * 1000.0)))
        lo = 0 if patch is None else starts[patch]
        n = tokens.shape[1]
        hidden = osd._lin(sd, "x_embedder", tokens)
        context = osd._lin(sd, "context_embedder", prompt_embeds.float())
        for g in range(n_total):
            if g > 0 and g in stage_starts and patch is not None:
                if patch == 0:
                    boundary_text[g] = context
                else:
                    context = boundary_text[g]

            def hook(k, v, g=g):
                if patch is None:
                    kv[g] = (k.clone(), v.clone())
                    return k, v
                kv[g][0][:, lo:lo + n] = k
                kv[g][1][:, lo:lo + n] = v
                return kv[g]
            if g < n_double:
                hidden, context = osd.joint_block(sd, f"transformer_blocks.{g}", hidden, context, temb, rope, H, D,
                                                  "front", kv_hook=hook, row0=S_txt + lo)
            else:
                xs = osd.single_block(sd, f"single_transformer_blocks.{g - n_double}", torch.cat([context, hidden], 1),
                                      temb, rope, H, D, text_len=S_txt, row0=S_txt + lo, kv_hook=hook)
                context, hidden = xs[:, :S_txt], xs[:, S_txt:]
        first, second = osd._lin(sd, "norm_out.linear", F.silu(temb)).chunk(2, dim=-1)
        scale, shift = (first, second) if shape.out_norm_scale_first else (second, first)
        return osd._lin(sd, "proj_out", osd._mod(F.layer_norm(hidden, (d,), eps=1e-6), shift, scale))

    for i in range(num_steps):
        dt = sig[i + 1] - sig[i]
        if i < warmup_steps or len(num_patch_tokens) == 1:
            x = x + dt * backbone(x, i, None)
        else:
            new = []
            for p in range(len(num_patch_tokens)):
                xp = x[:, starts[p]:starts[p + 1]]
                new.append(xp + dt * backbone(xp, i, p))
            x = torch.cat(new, dim=1)
    return x

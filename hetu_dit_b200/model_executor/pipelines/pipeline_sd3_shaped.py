"""Denoising stage of the SD3-shaped model with PipeFusion: warm-up steps on the whole image, then
the patch pipeline with stale K/V.

Plays the role of the reference's SD3 pipeline wrapper
(hetu_dit/model_executor/pipelines/pipeline_stable_diffusion_3.py: diffusion_stage :665-900,
_sync_pipeline :1352-1467, _init_async_pipeline :1469-1511, _async_pipeline :1515-1678,
_backbone_forward :1680-1717) and of its transformer wrapper
(models/transformers/transformer_sd3.py:95-198, stage split base_transformer.py:65-148).

The schedule is the reference's: stage s owns a contiguous slice of the blocks; a patch travels
stage to stage, the last stage applies classifier-free guidance and the scheduler step and sends
the new latent patch back to the first stage; the text stream of a step is computed together with
patch 0 and re-used by the other patches. Hand-offs go through the peer-heap coordinator
(group_coordinator.py here): one copy kernel + one flag store per message, no shape handshake per
message, no host synchronisation in steady state. Latents are token-major (B, tokens, 64) -- the
patchified form -- so a pipeline patch is a contiguous token range.
"""
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

from ... import kernels
from ...core.distributed import parallel_state as ps
from ...core.distributed.runtime_state import get_runtime_state
from ..models.shaped_dit import ShapedDiT, _modulate, timestep_embedding


def flow_match_sigmas(num_steps: int, shift: float = 3.0, device=None) -> torch.Tensor:
    """Shifted linear sigma schedule of a flow-matching Euler scheduler, num_steps + 1 values ending at 0."""
    s = torch.linspace(1.0, 1.0 / num_steps, num_steps, dtype=torch.float64)
    s = shift * s / (1 + (shift - 1) * s)
    return torch.cat([s, torch.zeros(1, dtype=torch.float64)]).float().to(device)


def stage_block_range(total_blocks: int, pp_rank: int, pp_world: int,
                      attn_layer_num_for_pp: Optional[List[int]] = None) -> Tuple[int, int]:
    """Blocks [lo, hi) of one stage: explicit per-stage counts, else ceil(total / stages) per stage."""
    if attn_layer_num_for_pp is not None:
        assert sum(attn_layer_num_for_pp) == total_blocks, (
            "Sum of attn_layer_num_for_pp should be equal to the number of all the transformer blocks")
        return sum(attn_layer_num_for_pp[:pp_rank]), sum(attn_layer_num_for_pp[:pp_rank + 1])
    per = (total_blocks + pp_world - 1) // pp_world
    return pp_rank * per, min((pp_rank + 1) * per, total_blocks)


class SD3ShapedPipeline:
    # label of the text-stream message between pipeline stages, in the whole-image steps and in the patch steps
    # (pipeline_stable_diffusion_3.py:1395,1438 and :1502,1560,1632)
    sync_text_message = "encoder_hidden_states"
    async_text_message = "encoder_hidden_states"
    use_cuda_graph = True    # see __init__
    fused_step = True
    _patch_pool = None       # memory pool shared by the per-patch CUDA graphs
    _live_patch_graphs = None

    def __init__(self, model: ShapedDiT, guidance_scale: float = 5.0, grid: Tuple[int, int] = (128, 128)):
        self.model = model
        self.shape = model.shape
        self.guidance_scale = guidance_scale
        self.grid = grid
        self.encoder_hidden_states_cache = {}
        self.sigmas = None
        # True when model.transformer_blocks already holds only this stage's blocks (the worker's block
        # cache placed them); False when the model is whole and the stage's slice is taken here.
        self.stage_sliced = False
        # Replay the whole-image step from a CUDA graph where the step is one self-contained launch sequence:
        # a single pipeline stage without pipeline patches (sequence parallelism included). PipeFusion stages
        # and patched steps run eagerly: their hand-offs and stale-KV updates depend on per-patch host state.
        self.use_cuda_graph = True
        self._graphs = None
        self._patch_pool = None
        self._live_patch_graphs = None
        # guidance + scheduler step (+ wrap-around send) of the last stage as one kernel; False = the eager chain
        self.fused_step = True

    def _stage(self, hidden_states, encoder_hidden_states, pooled, timestep):
        """_transformer(), through a captured CUDA graph when the step qualifies (see use_cuda_graph)."""
        rt = get_runtime_state()
        if not (self.use_cuda_graph and hidden_states.is_cuda and ps.get_pipeline_parallel_world_size() == 1
                and rt.num_pipeline_patch == 1 and not rt.patch_mode):
            return self._transformer(hidden_states, encoder_hidden_states, pooled, timestep)
        from ..step_graph import StepGraphCache
        if self._graphs is None:
            self._graphs = StepGraphCache()
        key = ("stage", tuple(hidden_states.shape), tuple(encoder_hidden_states.shape), hidden_states.dtype,
               tuple(self.grid), float(self.guidance_scale))
        return self._graphs.run(key, self._transformer, hidden_states, encoder_hidden_states, pooled, timestep)

    # ------------------------------------------------------------------ one stage of the backbone
    def _stage_blocks(self):
        blocks = self.model.transformer_blocks
        if self.stage_sliced:
            return list(enumerate(blocks))
        rt = get_runtime_state()
        lo, hi = stage_block_range(len(blocks), ps.get_pipeline_parallel_rank(), ps.get_pipeline_parallel_world_size(),
                                   rt.parallel_config.pp_config.attn_layer_num_for_pp)
        return [(i, blocks[i]) for i in range(lo, hi)]

    def _transformer(self, hidden_states, encoder_hidden_states, pooled, timestep):
        """Stage forward. First stage: latent tokens in, embeddings applied. Last stage: noise tokens out."""
        m, rt = self.model, get_runtime_state()
        d = self.shape.hidden
        dtype = hidden_states.dtype
        temb = m.time_embed(timestep_embedding(timestep * 1000.0).to(dtype)) + m.pooled_embed(pooled)
        if ps.is_pipeline_first_stage():
            hidden_states = m.x_embedder(hidden_states) + self._positions(hidden_states.shape[1],
                                                                          hidden_states.device, dtype)
            encoder_hidden_states = m.context_embedder(encoder_hidden_states)
        for i, block in self._stage_blocks():
            if rt.patch_mode and rt.pipeline_patch_idx == 0:
                self.encoder_hidden_states_cache[i] = encoder_hidden_states
                hidden_states, encoder_hidden_states = block(hidden_states, encoder_hidden_states, temb, None)
            elif rt.patch_mode:
                hidden_states, _ = block(hidden_states, self.encoder_hidden_states_cache[i], temb, None)
            else:
                hidden_states, encoder_hidden_states = block(hidden_states, encoder_hidden_states, temb, None)
        if ps.is_pipeline_last_stage():
            first, second = m.norm_out.linear(F.silu(temb)).chunk(2, dim=-1)
            scale, shift = (first, second) if self.shape.out_norm_scale_first else (second, first)
            hidden_states = m.proj_out(_modulate(F.layer_norm(hidden_states, (d,), eps=1e-6), shift, scale))
        return hidden_states, encoder_hidden_states

    def _positions(self, n, device, dtype):
        """Position embeddings of the tokens this rank holds: the rows of the current patch (patch mode) or
        of all its patches, by their global token index (under sequence parallelism a rank holds one slice of
        every patch, so its tokens are not one contiguous range)."""
        rt = get_runtime_state()
        pos = self.model._sincos_pos(self.grid[0], self.grid[1], device, dtype)
        bounds = rt.pp_patches_token_start_end_idx_global
        if rt.patch_mode:
            s, e = bounds[rt.pipeline_patch_idx]
            out = pos[:, s:e]
        elif ps.get_sequence_parallel_world_size() == 1:
            out = pos[:, :n]
        else:
            out = torch.cat([pos[:, s:e] for s, e in bounds], dim=1)
        if out.shape[1] != n:
            raise ValueError(f"{n} tokens passed, the patch layout of this rank holds {out.shape[1]}")
        return out

    def _sp_local(self, latents):
        """This sequence-parallel rank's tokens: its slice of every pipeline patch, patches in order (the
        reference's _init_sync_pipeline, base_pipeline.py:327-335, on latent rows)."""
        bounds = get_runtime_state().pp_patches_token_start_end_idx_global
        return torch.cat([latents[:, s:e] for s, e in bounds], dim=1)

    def _sp_gather(self, latents):
        """Whole latents from every rank's local ones: gather, then patch by patch the ranks' slices in rank
        order (pipeline_stable_diffusion_3.py:1449-1465, 1660-1677)."""
        rt = get_runtime_state()
        parts = ps.get_sp_group().all_gather(latents, separate_tensors=True)
        starts = rt.pp_patches_token_start_idx_local
        return torch.cat([part[:, starts[p]:starts[p + 1]] for p in range(rt.num_pipeline_patch) for part in parts],
                         dim=1)

    cfg_batch = True  # unconditional + conditional halves go through the backbone as one batch of two

    def _backbone_forward(self, latents, encoder_hidden_states, pooled, t, guide: bool = True):
        """guide=False leaves the last stage's prediction as the two-batch (uncond, cond) tensor: the caller fuses
        the guidance into the scheduler step (_guided_step)."""
        if ps.is_pipeline_first_stage():
            latents = torch.cat([latents] * 2)  # unconditional + conditional through one batch
        timestep = t.expand(latents.shape[0]).contiguous()
        noise_pred, encoder_hidden_states = self._stage(latents, encoder_hidden_states, pooled, timestep)
        if ps.is_pipeline_last_stage() and guide:
            uncond, text = noise_pred.chunk(2)
            latents = uncond + self.guidance_scale * (text - uncond)
        else:
            latents = noise_pred
        return latents, encoder_hidden_states

    def _guided_step(self, noise_pred, last_latents, i, send_as=None, sigmas=None, out=None):
        """Last stage: classifier-free guidance + scheduler step of one (patch of the) latents in a single kernel
        (csrc/elementwise.cu), which also stores the result into the first stage's inbox when `send_as` =
        (name, segment index) names the wrap-around message -- the eager chain and the separate send copy of
        the reference (pipeline_stable_diffusion_3.py:1585-1631, 1703-1713) become one launch plus a flag."""
        if not (self.fused_step and noise_pred.is_cuda and noise_pred.is_contiguous() and last_latents.is_contiguous()
                and last_latents.numel() % 8 == 0):
            if sigmas is not None or out is not None:
                raise RuntimeError("a captured patch step needs the fused guidance + scheduler kernel")
            if self.cfg_batch:
                uncond, text = noise_pred.chunk(2)
                noise_pred = uncond + self.guidance_scale * (text - uncond)
            out = self._scheduler_step(noise_pred, last_latents, i)
            if send_as is not None:
                ps.get_pp_group().pipeline_isend(out, name=send_as[0], segment_idx=send_as[1])
            return out
        peer = None
        pp = ps.get_pp_group() if send_as is not None else None
        if pp is not None:
            peer = pp.reserve_send(last_latents, send_as[0], send_as[1])
        out = kernels.cfg_euler_step(noise_pred, last_latents, self.sigmas if sigmas is None else sigmas, i,
                                     self.guidance_scale, cfg=self.cfg_batch, out=out, out_peer_ptr=peer)
        if pp is not None:
            pp.commit_send()
        return out

    def _scheduler_step(self, noise_pred, last_latents, i):
        """Flow-matching Euler step with the operation order of the reference's scheduler wrapper
        (scheduling_flow_match_euler_discrete.py:86-112, bit-identical to it on its own inputs): the product
        prediction * sigma is rounded to the prediction's 16-bit type, the rest runs in fp32 --
        denoised = sample - product, derivative = (sample - denoised) / sigma, result = sample + derivative * dt --
        and is rounded once. The step index is the caller's, so it advances once per step however many patches the
        step has (the reference gates its scheduler's step counter on the last patch, :119-124)."""
        sigma, sigma_next = self.sigmas[i].float(), self.sigmas[i + 1].float()
        sample = last_latents.float()
        product = (noise_pred.float() * sigma).to(noise_pred.dtype).float()
        denoised = sample - product
        derivative = (sample - denoised) / sigma
        return (sample + derivative * (sigma_next - sigma)).to(last_latents.dtype)

    # ------------------------------------------------------------------ warm-up: whole image per step
    def _sync_pipeline(self, latents, prompt_embeds, pooled, steps: List[int], sync_only: bool = False):
        rt = get_runtime_state()
        rt.set_patched_mode(False)
        pp_world = ps.get_pipeline_parallel_world_size()
        first, last = ps.is_pipeline_first_stage(), ps.is_pipeline_last_stage()
        pp = ps.get_pp_group() if pp_world > 1 else None
        encoder_hidden_states = None
        for k, i in enumerate(steps):
            if last:
                last_timestep_latents = latents
            if pp_world == 1 or (first and k == 0):
                pass
            else:
                latents = pp.pipeline_recv()
                if not first:
                    encoder_hidden_states = pp.pipeline_recv(0, self.sync_text_message)
            latents, encoder_hidden_states = self._backbone_forward(
                latents, prompt_embeds if first else encoder_hidden_states, pooled, self.sigmas[i:i + 1], guide=not last)
            sends = pp_world > 1 and not (sync_only and last and k == len(steps) - 1)
            if last:
                latents = self._guided_step(latents, last_timestep_latents, i, ("latent", -1) if sends else None)
            elif sends:
                pp.pipeline_send(latents)
                pp.pipeline_send(encoder_hidden_states, name=self.sync_text_message)
        return latents

    # ------------------------------------------------------------------ patch pipeline
    def _init_async_pipeline(self, num_timesteps: int, latents, num_pipeline_warmup_steps: int):
        rt = get_runtime_state()
        rt.set_patched_mode(True)
        pp_world = ps.get_pipeline_parallel_world_size()
        first, last = ps.is_pipeline_first_stage(), ps.is_pipeline_last_stage()
        tokens = rt.pp_patches_token_num
        if pp_world == 1:
            return list(latents.split(tokens, dim=1))
        pp = ps.get_pp_group()
        if first:
            # the latents the last stage produced at the end of warm-up
            latents = pp.pipeline_recv() if num_pipeline_warmup_steps > 0 else latents
            patch_latents = list(latents.split(tokens, dim=1))
        elif last:
            patch_latents = list(latents.split(tokens, dim=1))
        else:
            patch_latents = [None] * rt.num_pipeline_patch
        recv_timesteps = num_timesteps - 1 if first else num_timesteps
        for _ in range(recv_timesteps):
            if not first:
                pp.add_pipeline_recv_task(0, self.async_text_message)
            for patch_idx in range(rt.num_pipeline_patch):
                pp.add_pipeline_recv_task(patch_idx)
        return patch_latents

    def _async_pipeline(self, latents, prompt_embeds, pooled, steps: List[int]):
        if len(steps) == 0:
            return latents
        rt = get_runtime_state()
        pp_world = ps.get_pipeline_parallel_world_size()
        first, last = ps.is_pipeline_first_stage(), ps.is_pipeline_last_stage()
        pp = ps.get_pp_group() if pp_world > 1 else None
        patch_latents = self._init_async_pipeline(len(steps), latents, rt.runtime_config.warmup_steps)
        n_patch = rt.num_pipeline_patch
        n_steps = len(steps)
        st = {"last_patch": [None] * n_patch if last else None, "text": None, "first_recv": True}

        def receives(k, p, host_only):
            """Messages patch p of step k starts from. host_only: only the receive-queue bookkeeping (the waits and
            copies themselves are part of a replayed graph)."""
            if last:
                st["last_patch"][p] = patch_latents[p]  # the sample of this step: the previous step's result
            if pp_world == 1 or (first and k == 0):
                return
            if st["first_recv"]:
                if not first and p == 0:
                    pp.recv_next()
                pp.recv_next()
                st["first_recv"] = False
            if not first and p == 0:
                if host_only:
                    pp.pop_received(idx=p, name=self.async_text_message)
                else:
                    # private copy: the text stream serves every patch of this step, while the
                    # sender may refill the inbox slot as soon as patch 0 has gone round the ring
                    st["text"] = pp.get_pipeline_recv_data(idx=p, name=self.async_text_message).clone()
            if host_only:
                pp.pop_received(idx=p)
            else:
                patch_latents[p] = pp.get_pipeline_recv_data(idx=p)

        def posts(k, p):
            """The reference posts its next receives here; with pushed messages only the order is recorded."""
            if pp_world == 1 or (first and k == 0):
                pass
            elif k == n_steps - 1 and p == n_patch - 1:
                pass
            elif first:
                pp.recv_next()
            else:
                if p == n_patch - 1:
                    pp.recv_next()
                pp.recv_next()

        def compute(k, p, i, t, sigmas=None, step_index=None, out=None):
            """Forward of patch p through this stage and what follows it: the guided scheduler step (+ wrap-around
            send) on the last stage, the hand-over to the next stage elsewhere."""
            patch_latents[p], next_text = self._backbone_forward(
                patch_latents[p], prompt_embeds if first else st["text"], pooled, t, guide=not last)
            if last:
                sends = pp_world > 1 and k != n_steps - 1
                patch_latents[p] = self._guided_step(
                    patch_latents[p], st["last_patch"][p].contiguous(), i if step_index is None else step_index,
                    ("latent", p) if sends else None, sigmas=sigmas, out=out)
            elif pp_world > 1:
                if p == 0:
                    pp.pipeline_isend(next_text, name=self.async_text_message)
                pp.pipeline_isend(patch_latents[p], segment_idx=p)

        # Steps 2 .. n - 2 of the patch pipeline enqueue the same launches per patch: they are captured once per
        # patch (at step 2, when every message has been seen once and all lazy set-up is done) and replayed. The
        # first two steps and the last one (no wrap-around send) run eagerly.
        graphed = (self.use_cuda_graph and self.fused_step and pp_world > 1 and latents.is_cuda and n_steps >= 4
                   and rt.runtime_config.warmup_steps > 0)
        graphs = [None] * n_patch
        if graphed:
            dev = latents.device
            t_static = torch.zeros(1, dtype=self.sigmas.dtype, device=dev)
            sig_pair = torch.zeros(2, dtype=self.sigmas.dtype, device=dev)
            static_last = [None] * n_patch
            # one pool for this request's graphs (a pool whose graphs are all gone must not be captured into again)
            self._patch_pool = torch.cuda.graph_pool_handle()
        for k, i in enumerate(steps):
            replay = graphed and 2 <= k <= n_steps - 2
            if replay:
                t_static.copy_(self.sigmas[i:i + 1])
                sig_pair.copy_(self.sigmas[i:i + 2])
            for p in range(n_patch):
                if not replay:
                    receives(k, p, host_only=False)
                    compute(k, p, i, self.sigmas[i:i + 1])
                elif graphs[p] is None:
                    if last:
                        # the sample the scheduler step updates in place from now on
                        static_last[p] = patch_latents[p].contiguous().clone()
                        patch_latents[p] = static_last[p]
                    cur = torch.cuda.current_stream(dev)
                    side = torch.cuda.Stream(device=dev)
                    side.wait_stream(cur)
                    with torch.cuda.stream(side):
                        g = torch.cuda.CUDAGraph()
                        g.capture_begin(pool=self._patch_pool)
                        try:
                            receives(k, p, host_only=False)
                            compute(k, p, i, t_static, sigmas=sig_pair, step_index=0,
                                    out=static_last[p] if last else None)
                        finally:
                            g.capture_end()
                    cur.wait_stream(side)
                    graphs[p] = g
                    g.replay()
                else:
                    receives(k, p, host_only=True)
                    graphs[p].replay()
                posts(k, p)
                rt.next_patch()
        self._live_patch_graphs = graphs  # until the next request: the replays may still be running
        return torch.cat(patch_latents, dim=1) if last else None

    # ------------------------------------------------------------------ entry point
    @torch.no_grad()
    def diffusion_stage(self, latents, prompt_embeds, pooled, num_inference_steps: int):
        """latents (1, S, 64); prompt_embeds (2, S_txt, text_dim) = [negative, positive]; pooled (2, pooled_dim).
        Returns the denoised latents on the last pipeline stage (None elsewhere)."""
        rt = get_runtime_state()
        if rt.ready:
            # the token grid follows the request's resolution (latent pixels / patch size)
            cell = rt.vae_scale_factor * rt.backbone_patch_size
            self.grid = (rt.input_config.height // cell, rt.input_config.width // cell)
        self.sigmas = flow_match_sigmas(num_inference_steps, device=latents.device)
        self.encoder_hidden_states_cache = {}
        warmup = min(rt.runtime_config.warmup_steps, num_inference_steps)
        steps = list(range(num_inference_steps))
        sp = ps.get_sequence_parallel_world_size()
        if sp > 1:
            latents = self._sp_local(latents)
        patched = rt.num_pipeline_patch > 1 and num_inference_steps > warmup
        if patched:
            latents = self._sync_pipeline(latents, prompt_embeds, pooled, steps[:warmup])
            latents = self._async_pipeline(latents, prompt_embeds, pooled, steps[warmup:])
        else:
            latents = self._sync_pipeline(latents, prompt_embeds, pooled, steps, sync_only=True)
            if not ps.is_pipeline_last_stage():
                latents = None
        rt.set_patched_mode(False)
        if sp > 1 and latents is not None:
            latents = self._sp_gather(latents)
        return latents

"""Denoising stage of the Flux-shaped model with PipeFusion.

Plays the role of the reference's Flux pipeline wrapper
(hetu_dit/model_executor/pipelines/pipeline_flux.py: _sync_pipeline :447-555, _init_async_pipeline
:725-773, _async_pipeline :557-723, _backbone_forward :775-800) and of its transformer wrapper
(diffusion_executor/models/transformers/transformer_flux.py:101-206).

The step and patch loops are those of the SD3-shaped pipeline (same hand-off protocol, same
scheduler). What differs is the stage forward: guidance is an embedding instead of a second batch
element, positions are rotary rows selected by the patch's first token, a stage may hold double
blocks, single blocks or both (text and image rows are joined before its single blocks and split
again after them, so that a stage always hands over the two streams separately), and the first
stage carries the text stream through its blocks again for every patch -- only later stages re-use
the text stream that arrived with patch 0 of the step.
"""
import torch
import torch.nn.functional as F

from ... import kernels
from ...core.distributed import parallel_state as ps
from ...core.distributed.runtime_state import get_runtime_state
from ..models.shaped_dit import ShapedDiT, timestep_embedding
from .pipeline_sd3_shaped import SD3ShapedPipeline, stage_block_range


class FluxShapedPipeline(SD3ShapedPipeline):
    # the reference's Flux pipeline labels the text-stream message differently in its two loops
    # (pipeline_flux.py:475,526 against :756,606,668)
    sync_text_message = "encoder_hidden_state"
    async_text_message = "encoder_hidden_states"

    def __init__(self, model: ShapedDiT, guidance_scale: float = 3.5, grid=(64, 64)):
        if model.shape.rope_axes is None or model.guidance_embed is None:
            raise ValueError("FluxShapedPipeline needs a model with rotary positions and a guidance embedding")
        super().__init__(model, guidance_scale=guidance_scale, grid=grid)

    def _stage_blocks(self):
        """(double blocks, single blocks) of this stage; blocks are numbered double first, then single."""
        doubles, singles = list(self.model.transformer_blocks), list(self.model.single_transformer_blocks)
        if self.stage_sliced:
            return doubles, singles
        rt = get_runtime_state()
        lo, hi = stage_block_range(len(doubles) + len(singles), ps.get_pipeline_parallel_rank(),
                                   ps.get_pipeline_parallel_world_size(),
                                   rt.parallel_config.pp_config.attn_layer_num_for_pp)
        nd = len(doubles)
        return doubles[min(lo, nd):min(hi, nd)], singles[max(lo - nd, 0):max(hi - nd, 0)]

    def _rope_and_first_token(self, s_txt, device):
        """Rotary tables and the table row (past the text rows) of the first image token this call holds. A
        patch, or a whole image on one sequence-parallel rank without patches, is one range of rows of the full
        table. A whole-image step under sequence parallelism with several pipeline patches holds one slice of
        every patch: its rows are gathered into a local table (text rows first), addressed from row 0."""
        rt = get_runtime_state()
        rope = self.model._rope(s_txt, self.grid, device)
        bounds = rt.pp_patches_token_start_end_idx_global
        if rt.patch_mode:
            return rope, bounds[rt.pipeline_patch_idx][0]
        if ps.get_sequence_parallel_world_size() == 1:
            return rope, 0
        if len(bounds) == 1:
            return rope, bounds[0][0]
        key = (s_txt, tuple(tuple(b) for b in bounds), tuple(self.grid), str(device))
        cache = self.__dict__.setdefault("_rope_local", {})
        if key not in cache:
            rows = torch.cat([torch.arange(s_txt, device=device)] +
                             [torch.arange(s, e, device=device) + s_txt for s, e in bounds])
            cache[key] = (rope[0].index_select(0, rows), rope[1].index_select(0, rows))
        return cache[key], 0

    def _transformer(self, hidden_states, encoder_hidden_states, pooled, timestep):
        m = self.model
        dtype = hidden_states.dtype
        guidance = torch.full_like(timestep, float(self.guidance_scale))
        temb = (m.time_embed(timestep_embedding(timestep * 1000.0).to(dtype)) + m.pooled_embed(pooled)
                + m.guidance_embed(timestep_embedding(guidance * 1000.0).to(dtype)))
        if ps.is_pipeline_first_stage():
            hidden_states = m.x_embedder(hidden_states)
            encoder_hidden_states = m.context_embedder(encoder_hidden_states)
        s_txt = encoder_hidden_states.shape[1]
        rope, tok0 = self._rope_and_first_token(s_txt, hidden_states.device)
        doubles, singles = self._stage_blocks()
        for block in doubles:
            hidden_states, encoder_hidden_states = block(hidden_states, encoder_hidden_states, temb, rope, tok0)
        if singles:
            x = torch.cat([encoder_hidden_states, hidden_states], dim=1)
            for block in singles:
                x = block(x, temb, rope, s_txt, tok0)
            encoder_hidden_states, hidden_states = x[:, :s_txt], x[:, s_txt:]
        if ps.is_pipeline_last_stage():
            first, second = m.norm_out.linear(F.silu(temb)).chunk(2, dim=-1)
            scale, shift = (first, second) if self.shape.out_norm_scale_first else (second, first)
            hidden_states = m.proj_out(kernels.ln_modulate(hidden_states.contiguous(), shift, scale))
        return hidden_states, encoder_hidden_states

    cfg_batch = False  # guidance-distilled: one batch element, the guidance scale is an embedding

    def _backbone_forward(self, latents, encoder_hidden_states, pooled, t, guide: bool = True):
        return self._stage(latents, encoder_hidden_states, pooled, t.expand(latents.shape[0]).contiguous())

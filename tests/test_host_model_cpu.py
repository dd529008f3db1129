"""Host-side wiring of the -shaped models and the PipeFusion pipelines on CPU, in fp32, against the oracle.

The kernel wrappers are replaced by the torch stand-ins of tests/cpu_stand_ins.py for the duration of a test (the
product itself has no CPU path). In fp32 the comparison is tight (1e-4 of the output's largest magnitude), so a
wiring difference that 16-bit tolerances on the GPU could hide shows up here. The GPU tests remain the parity
tests of the kernels; these cover what is around them.
"""
import pytest
import torch

from oracle import pipefusion as opf
from oracle import shaped_dit as osd
from tests import cpu_stand_ins

TINY = {
    "flux": (("flux-tiny", 2, 3, 512, 4, 128, 64, 256, 96, True, (16, 56, 56), True), {}, (20, 12)),
    "sd3": (("sd3-tiny", 3, 0, 256, 4, 64, 64, 256, 128, False, None, False), {}, (20, 12)),
    "cogvideox": (("cogvideox-tiny", 3, 0, 256, 4, 64, 128, 256, 0, True, (16, 24, 24), False),
                  dict(text_first=True, rope_on_text=False, qk_norm_kind="layer", block_kind="cogvideox", temb_dim=128,
                       out_norm_scale_first=False),
                  (3, 10, 8)),
    "hunyuan": (("hunyuan-tiny", 2, 3, 512, 4, 128, 64, 256, 96, True, (16, 56, 56), True),
                dict(text_first=False, rope_on_text=False), (3, 10, 8)),
}


def _close(got, want, tol=1e-4):
    err = (got.float() - want.float()).abs().max().item()
    assert got.shape == want.shape and err <= tol * want.float().abs().max().item(), err


@pytest.mark.parametrize("kind", sorted(TINY))
def test_model_step_wiring_matches_oracle(kind, monkeypatch):
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.runtime_state import reset_runtime_state
    from hetu_dit_b200.core.resource_manager.cache_manager import reset_cache_manager
    from hetu_dit_b200.model_executor.models.shaped_dit import DiTShape, ShapedDiT
    cpu_stand_ins.install(monkeypatch)
    ps.destroy_model_parallel()
    reset_runtime_state()
    reset_cache_manager()
    args, kw, grid = TINY[kind]
    shape = DiTShape(*args, **kw)
    n_tok = 1
    for g in grid:
        n_tok *= g
    model = ShapedDiT(shape).init_weights(seed=3, std=0.05).float()
    gen = torch.Generator().manual_seed(0)
    lat = torch.randn(1, n_tok, shape.token_in, generator=gen)
    txt = torch.randn(1, 33, shape.text_dim, generator=gen)
    pooled = torch.randn(1, max(shape.pooled_dim, 1), generator=gen)
    t, g = torch.tensor([0.5]), torch.tensor([3.5])
    outs = []
    first = shape.text_first
    hooks = [b.register_forward_hook(lambda _m, _i, out: outs.append(out[0].detach())) for b in model.transformer_blocks]
    hooks += [b.register_forward_hook(lambda _m, _i, out: outs.append(
        (out[:, 33:] if first else out[:, :out.shape[1] - 33]).detach())) for b in model.single_transformer_blocks]
    with torch.no_grad():
        got = model(lat, txt, pooled, t, g, grid=grid)
        want_blocks = []
        want = osd.denoise_step(model.state_dict(), shape, lat, txt, pooled, t, g, grid=grid, block_outputs=want_blocks)
    for h in hooks:
        h.remove()
    assert len(outs) == len(want_blocks) == shape.n_blocks
    for a, b in zip(outs, want_blocks):
        _close(a, b)
    _close(got, want)


def _pipeline_case(flux, monkeypatch):
    from hetu_dit_b200.config import EngineConfig
    from hetu_dit_b200.core.distributed import parallel_state as ps
    from hetu_dit_b200.core.distributed.runtime_state import ModelGeometry, initialize_runtime_state, reset_runtime_state
    from hetu_dit_b200.core.resource_manager.cache_manager import reset_cache_manager
    from hetu_dit_b200.model_executor.models.shaped_dit import DiTShape, ShapedDiT
    from hetu_dit_b200.model_executor.pipelines.pipeline_flux_shaped import FluxShapedPipeline
    from hetu_dit_b200.model_executor.pipelines.pipeline_sd3_shaped import SD3ShapedPipeline
    cpu_stand_ins.install(monkeypatch)
    if flux:
        shape = DiTShape("flux-tiny", 2, 3, 256, 4, 64, 64, 128, 96, True, (16, 24, 24), True)
        batch, scale = 1, 3.5
    else:
        shape = DiTShape("sd3-tiny", 4, 0, 256, 4, 64, 64, 128, 96, False, None, False)
        batch, scale = 2, 4.0
    model = ShapedDiT(shape).init_weights(seed=11, std=0.05).float()
    gen = torch.Generator().manual_seed(12)
    lat = torch.randn(1, 32 * 16, 64, generator=gen)
    prompt = torch.randn(batch, 19, 128, generator=gen)
    pooled = torch.randn(batch, 96, generator=gen)
    ps.destroy_model_parallel()
    reset_cache_manager()
    cfg = EngineConfig()
    cfg.parallel_config.pp_config.num_pipeline_patch = 4
    cfg.runtime_config.warmup_steps = 1
    rt = initialize_runtime_state(ModelGeometry(4, 64), cfg)
    rt.set_input_parameters(height=512, width=256, batch_size=1, num_inference_steps=4)
    assert rt.pp_patches_token_num == [128] * 4
    model.register_cache()
    pipe = (FluxShapedPipeline if flux else SD3ShapedPipeline)(model, guidance_scale=scale, grid=(32, 16))
    oracle = opf.denoise_flux if flux else opf.denoise
    try:
        with torch.no_grad():
            got = pipe.diffusion_stage(lat, prompt, pooled, 4)
            want = oracle(model.state_dict(), shape, lat, prompt, pooled, 4, scale, [128] * 4, 1, (32, 16))
            unpatched = oracle(model.state_dict(), shape, lat, prompt, pooled, 4, scale, [512], 1, (32, 16))
    finally:
        reset_runtime_state()
        reset_cache_manager()
    _close(got, want)
    assert (got - want).abs().max() < 1e-2 * (got - unpatched).abs().max()      # the stale K/V is really in play


def test_sd3_pipefusion_single_stage_wiring_matches_oracle(monkeypatch):
    """Warm-up step, then three steps of the patch pipeline with stale K/V, classifier-free guidance and the
    scheduler step, on one stage."""
    _pipeline_case(False, monkeypatch)


def test_flux_pipefusion_single_stage_wiring_matches_oracle(monkeypatch):
    """The same for the Flux-shaped pipeline: rotary rows per patch, stale K/V in double and single blocks, text
    stream carried through every patch on the first stage."""
    _pipeline_case(True, monkeypatch)

"""Block- and model-level GPU parity of the -shaped DiT against the CPU oracle."""
import pytest
import torch

from oracle import attention as oa
from oracle import shaped_dit as osd

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(shape, s_img, s_txt, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(1, s_img, shape.token_in, generator=gen).bfloat16(),
            torch.randn(1, s_txt, shape.text_dim, generator=gen).bfloat16(),
            torch.randn(1, shape.pooled_dim, generator=gen).bfloat16(), torch.tensor([0.5]), torch.tensor([3.5]))


@pytest.mark.parametrize("kind", ["flux", "sd3"])
def test_tiny_model_step(kind):
    from hetu_dit_b200 import _C
    from hetu_dit_b200.model_executor.models.shaped_dit import DiTShape, ShapedDiT
    if kind == "flux":
        shape = DiTShape("flux-tiny", 2, 3, 512, 4, 128, 64, 256, 96, True, (16, 56, 56), True)
    else:
        shape = DiTShape("sd3-tiny", 3, 0, 256, 4, 64, 64, 256, 128, False, None, False)
    model = ShapedDiT(shape).to(DEV).init_weights(seed=3, std=0.05).bfloat16()
    lat, txt, pooled, t, g = _inputs(shape, 20 * 12, 33)
    with torch.no_grad():
        got = model(lat.to(DEV), txt.to(DEV), pooled.to(DEV), t.to(DEV), g.to(DEV), grid=(20, 12))
        torch.cuda.synchronize()
        assert _C.device_status(0, clear=True)[0] == 0
        sd = {k: v.float().cpu() for k, v in model.state_dict().items()}
        want = osd.denoise_step(sd, shape, lat, txt, pooled, t, g, grid=(20, 12))
    cos, rel = oa.cosine_and_max_rel(got.cpu(), want)
    assert cos >= 0.999 and rel <= 5e-2, (cos, rel)


def test_joint_block_output_tolerance():
    """One Flux-shaped double block at hidden 3072: per-block cosine >= 0.9999, max relative error <= 2e-2."""
    from hetu_dit_b200.model_executor.models.shaped_dit import FLUX_DEV, JointBlock, rope_tables
    torch.manual_seed(0)
    blk = JointBlock(FLUX_DEV).to(DEV)
    gen = torch.Generator(device=DEV).manual_seed(5)
    with torch.no_grad():
        for n, p in blk.named_parameters():
            if p.dim() > 1:
                p.copy_(torch.randn(p.shape, generator=gen, device=DEV) * 0.02)
            elif n.endswith("bias"):
                p.zero_()
    blk = blk.bfloat16()
    S_txt, gh, gw = 64, 16, 24
    g2 = torch.Generator().manual_seed(6)
    hidden = torch.randn(1, gh * gw, 3072, generator=g2).bfloat16()
    context = torch.randn(1, S_txt, 3072, generator=g2).bfloat16()
    temb = torch.randn(1, 3072, generator=g2).bfloat16()
    ids = torch.zeros(S_txt + gh * gw, 3)
    yy, xx = torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij")
    ids[S_txt:, 1], ids[S_txt:, 2] = yy.flatten(), xx.flatten()
    rope = rope_tables(ids, FLUX_DEV.rope_axes)
    with torch.no_grad():
        h, c = blk(hidden.to(DEV), context.to(DEV), temb.to(DEV), (rope[0].to(DEV), rope[1].to(DEV)))
        torch.cuda.synchronize()
        sd = {"b." + k: v.float().cpu() for k, v in blk.state_dict().items()}
        wh, wc = osd.joint_block(sd, "b", hidden.float(), context.float(), temb.float(), rope, 24, 128, "front")
    for got, want in ((h, wh), (c, wc)):
        cos, rel = oa.cosine_and_max_rel(got.cpu(), want)
        assert cos >= 0.9999 and rel <= 2e-2, (cos, rel)

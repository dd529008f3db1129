"""GPU parity of the movement kernels (C ABI) against the CPU oracle: bit-exact for byte movement."""
import os

import numpy as np
import pytest
import torch

from oracle import attention as oa
from oracle import bookkeeping as ob

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("shift,cols", [(0, 64), (8, 64), (4, 30), (2, 31), (1, 33)])
def test_copy_pieces_alignments(shift, cols):
    """Every vector width (16/8/4/2/1 bytes) moves exactly the requested bytes and nothing else."""
    from hetu_dit_b200 import kernels
    gen = torch.Generator().manual_seed(shift * 100 + cols)
    src = torch.randint(0, 255, (5, 37, 256), dtype=torch.uint8, generator=gen).to(DEV)
    dst = torch.zeros(5, 64, 300, dtype=torch.uint8, device=DEV)
    want = dst.clone()
    sv = src[:, 3:30, shift:shift + cols]
    kernels.copy_pieces([(sv.data_ptr(), dst[:, 10:37, shift:shift + cols].data_ptr(), 5, 37 * 256, 64 * 300, 27, 256,
                          300, cols)], torch.device(DEV))
    want[:, 10:37, shift:shift + cols] = sv
    torch.cuda.synchronize()
    assert torch.equal(dst, want)


def test_copy_many_pieces_and_empty():
    from hetu_dit_b200 import kernels
    src = torch.arange(100 * 1024, dtype=torch.int32, device=DEV).reshape(100, 1024)
    dst = torch.zeros_like(src)
    pieces = [(src[i].data_ptr(), dst[99 - i].data_ptr(), 1, 0, 0, 1, 0, 0, 4096) for i in range(100)]
    pieces.append((src.data_ptr(), dst.data_ptr(), 1, 0, 0, 0, 0, 0, 4096))  # zero rows: ignored
    kernels.copy_pieces(pieces, torch.device(DEV))
    kernels.copy_pieces([], torch.device(DEV))
    torch.cuda.synchronize()
    assert torch.equal(dst, src.flip(0))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_kv_scatter_matches_cache_update(dtype):
    """PipeFusion stale-KV scatter for every patch of an SD3-shaped layer, bit for bit."""
    from hetu_dit_b200 import kernels
    B, H, D = 2, 24, 64
    meta = ob.calc_patches_metadata(512, 512, 8, 2, 4, 1, 0)
    tok = meta["pp_patches_token_start_idx_local"]
    S = tok[-1]
    gen = torch.Generator().manual_seed(3)
    cache_cpu = torch.randn(B, S, 2 * H * D, generator=gen).to(dtype)
    cache = cache_cpu.clone().to(DEV)
    for p in range(meta["num_pipeline_patch"]):
        n = tok[p + 1] - tok[p]
        k = torch.randn(B, n, H * D, generator=gen).to(dtype)
        v = torch.randn(B, n, H * D, generator=gen).to(dtype)
        want = oa.kv_cache_update(cache_cpu, torch.cat([k, v], -1), True, meta["num_pipeline_patch"], p, tok)
        kernels.kv_scatter(cache, k.to(DEV), v.to(DEV), tok[p])
        torch.cuda.synchronize()
        assert torch.equal(cache.cpu(), want)
        kc, vc = torch.chunk(cache, 2, dim=-1)
        assert torch.equal(kc[:, tok[p]:tok[p + 1]].cpu(), k) and torch.equal(vc[:, tok[p]:tok[p + 1]].cpu(), v)


def test_kv_scatter_range_error():
    from hetu_dit_b200 import _C, kernels
    cache = torch.zeros(1, 16, 128, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(1, 8, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(_C.HditError) as e:
        kernels.kv_scatter(cache, k, k, 12)
    assert e.value.code == _C.HDIT_ERR_SHAPE


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_norm_rope_matches_oracle(D, dtype):
    from hetu_dit_b200 import kernels
    gen = torch.Generator().manual_seed(D)
    B, S, H, S_txt = 2, 75, 5, 11
    q = torch.randn(B, S, H, D, generator=gen).to(dtype)
    k = torch.randn(B, S, H, D, generator=gen).to(dtype)
    wq = (1 + 0.1 * torch.randn(D, generator=gen)).to(dtype)
    wk = (1 + 0.1 * torch.randn(D, generator=gen)).to(dtype)
    ang = torch.rand(S - S_txt, D // 2, generator=gen) * 6.28
    cos = torch.cos(ang).repeat_interleave(2, -1).contiguous()
    sin = torch.sin(ang).repeat_interleave(2, -1).contiguous()

    def want(x, w):
        y = oa.rms_norm(x, w, 1e-6)
        rot = oa.apply_rotary_emb(y[:, S_txt:].transpose(1, 2), cos, sin).transpose(1, 2)
        return torch.cat([y[:, :S_txt], rot], 1)

    qd, kd = q.to(DEV), k.to(DEV)
    kernels.qk_norm_rope([(qd, wq.to(DEV), True, True), (kd, wk.to(DEV), True, True)], eps=1e-6, cos=cos.to(DEV),
                         sin=sin.to(DEV), rope_seq_start=S_txt)
    torch.cuda.synchronize()
    for got, ref in ((qd, want(q, wq)), (kd, want(k, wk))):
        # Same rounding sequence as the reference; only the fp32 reduction order of the variance may
        # differ, which can move an intermediate by one unit in the last place before the rotation
        # mixes two such values: bound = 2 ulp of the largest magnitude.
        ulp = 2 ** -8 if dtype == torch.bfloat16 else 2 ** -11
        diff = (got.cpu().float() - ref.float()).abs()
        assert diff.max().item() <= 2 * ulp * ref.float().abs().max().item()
        assert (diff == 0).float().mean().item() > 0.99


@pytest.mark.parametrize("D", [64, 128])
def test_layer_norm_rope_matches_torch(D):
    """LayerNorm over the head dimension (the QK norm of the CogVideoX shape) + rotary embedding on the rows
    past the text prefix, against torch's layer_norm on the same 16-bit inputs."""
    from hetu_dit_b200 import kernels
    gen = torch.Generator().manual_seed(3 * D)
    B, S, H, S_txt = 2, 61, 3, 9
    dtype = torch.bfloat16
    q = torch.randn(B, S, H, D, generator=gen).to(dtype)
    k = torch.randn(B, S, H, D, generator=gen).to(dtype)
    w = (1 + 0.1 * torch.randn(D, generator=gen)).to(dtype)
    bias = (0.1 * torch.randn(D, generator=gen)).to(dtype)
    ang = torch.rand(S - S_txt, D // 2, generator=gen) * 6.28
    cos = torch.cos(ang).repeat_interleave(2, -1).contiguous()
    sin = torch.sin(ang).repeat_interleave(2, -1).contiguous()

    def want(x):
        y = torch.nn.functional.layer_norm(x.float(), (D,), w.float(), bias.float(), 1e-6).to(dtype)
        rot = oa.apply_rotary_emb(y[:, S_txt:].transpose(1, 2), cos, sin).transpose(1, 2)
        return torch.cat([y[:, :S_txt], rot.to(dtype)], 1)

    qd, kd = q.to(DEV), k.to(DEV)
    kernels.qk_norm_rope([(qd, w.to(DEV), 2, True, bias.to(DEV)), (kd, w.to(DEV), 2, True, bias.to(DEV))], eps=1e-6,
                         cos=cos.to(DEV), sin=sin.to(DEV), rope_seq_start=S_txt)
    torch.cuda.synchronize()
    for got, ref in ((qd, want(q)), (kd, want(k))):
        diff = (got.cpu().float() - ref.float()).abs()
        assert diff.max().item() <= 2 * 2 ** -8 * ref.float().abs().max().item()
        assert (diff == 0).float().mean().item() > 0.97


def test_rope_golden(golden_dir):
    """apply_rotary_emb outputs recorded from the reference function."""
    from hetu_dit_b200 import kernels
    with np.load(os.path.join(golden_dir, "rope.npz")) as f:
        for i in range(2):
            x = torch.from_numpy(f[f"x{i}"]).to(torch.bfloat16)  # (B, H, S, D)
            cos, sin = torch.from_numpy(f[f"cos{i}"]).to(DEV), torch.from_numpy(f[f"sin{i}"]).to(DEV)
            xd = x.transpose(1, 2).contiguous().to(DEV)
            kernels.qk_norm_rope([(xd, None, False, True)], cos=cos, sin=sin)
            torch.cuda.synchronize()
            assert torch.equal(xd.transpose(1, 2).cpu().float(), torch.from_numpy(f[f"yb{i}"]))


def test_norm_rope_head_scatter():
    """Head-sliced destinations at a sequence offset == the Ulysses all-to-all layout."""
    from hetu_dit_b200 import kernels
    gen = torch.Generator().manual_seed(9)
    B, S, H, D, U = 1, 40, 8, 64, 4
    x = torch.randn(B, S, H, D, generator=gen).to(torch.bfloat16)
    w = torch.ones(D, dtype=torch.bfloat16)
    dsts = [torch.zeros(B, 3 * S, H // U, D, dtype=torch.bfloat16, device=DEV) for _ in range(U)]
    kernels.qk_norm_rope([(x.to(DEV), w.to(DEV), True, False)], dsts=[dsts], dst_seq_offset=S)
    torch.cuda.synchronize()
    y = oa.rms_norm(x, w, 1e-6)
    for u in range(U):
        got = dsts[u].cpu()
        assert torch.equal(got[:, S:2 * S], y[:, :, u * 2:(u + 1) * 2])
        assert got[:, :S].abs().sum() == 0 and got[:, 2 * S:].abs().sum() == 0


@pytest.mark.parametrize("dim", [256, 1536, 3072])
def test_ln_modulate_and_gate_residual(dim):
    from hetu_dit_b200 import kernels
    gen = torch.Generator().manual_seed(dim)
    B, S = 2, 37
    x = torch.randn(B, S, dim, generator=gen).bfloat16()
    y = torch.randn(B, S, dim, generator=gen).bfloat16()
    mod = (0.3 * torch.randn(B, 3 * dim, generator=gen)).bfloat16()
    shift, scale, gate = mod.chunk(3, dim=-1)
    xd, yd, md = x.to(DEV), y.to(DEV), mod.to(DEV)
    sh, sc, ga = md.chunk(3, dim=-1)
    got = kernels.ln_modulate(xd, sh, sc)
    want = torch.nn.functional.layer_norm(x.float(), (dim,), eps=1e-6) * (1 + scale.float()[:, None]) + shift.float()[:, None]
    assert (got.cpu().float() - want).abs().max().item() <= 2 ** -7 * want.abs().max().item()
    got = kernels.gate_residual(xd, ga, yd)
    want = x.float() + gate.float()[:, None] * y.float()
    assert torch.equal(got.cpu(), want.bfloat16())
    # strided rows (a slice of a longer sequence) work too
    got = kernels.gate_residual(xd[:, 5:20], ga, yd[:, 5:20])
    assert torch.equal(got.cpu(), want[:, 5:20].bfloat16())


def test_gelu_tanh_matches_torch():
    from hetu_dit_b200 import kernels
    gen = torch.Generator().manual_seed(4)
    x = (3 * torch.randn(2, 33, 512, generator=gen)).bfloat16()
    want = torch.nn.functional.gelu(x.float(), approximate="tanh")
    xd = x.to(DEV)
    got = kernels.gelu_tanh(xd)
    assert (got.cpu().float() - want).abs().max().item() <= 2 ** -7 * want.abs().max().item()
    wide = torch.zeros(2, 33, 640, dtype=torch.bfloat16, device=DEV)
    kernels.gelu_tanh(xd, out=wide[..., 128:])
    assert torch.equal(wide[..., 128:], got) and wide[..., :128].abs().sum() == 0
    kernels.gelu_tanh(xd, out=xd)  # in place
    assert torch.equal(xd, got)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cfg", [True, False])
def test_cfg_euler_step_matches_the_eager_chain_bit_for_bit(dtype, cfg):
    """Guidance combine + flow-matching Euler step in one kernel against the eager sequence it replaces (16-bit
    guidance arithmetic with one rounding per operation, the step in the reference scheduler's operation order), and
    the second destination."""
    from hetu_dit_b200 import kernels
    gen = torch.Generator().manual_seed(17)
    n = (1, 384, 64)
    pred = torch.randn((2 if cfg else 1,) + n[1:], generator=gen).to(dtype).to(DEV)
    sample = torch.randn(n, generator=gen).to(dtype).to(DEV)
    sigmas = torch.linspace(1.0, 0.0, 9).to(DEV)
    scale, step = 4.5, 3
    if cfg:
        uncond, text = pred.chunk(2)
        guided = uncond + scale * (text - uncond)
    else:
        guided = pred
    # the step in the operation order of the reference's scheduler wrapper (pinned against its recorded outputs in
    # tests/test_host_logic.py::test_scheduler_step_matches_reference_wrapper)
    sigma, x = sigmas[step], sample.float()
    product = (guided.float() * sigma).to(dtype).float()
    want = (x + ((x - (x - product)) / sigma) * (sigmas[step + 1] - sigma)).to(dtype)
    peer = torch.zeros_like(sample)
    got = kernels.cfg_euler_step(pred, sample, sigmas, step, scale, cfg=cfg, out_peer_ptr=peer.data_ptr())
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.equal(peer, want)


def test_norm_rope_two_row_ranges_in_one_launch_and_folded_signal():
    """One launch over [text; image] rows with their own norm weights and rotary rows equals two launches, bit
    for bit; and the launch's last CTA publishes the next epoch to the peers' flags (here: flags in local memory
    standing in for two peers), advancing the device-side epoch counter once per launch."""
    from hetu_dit_b200 import kernels
    gen = torch.Generator().manual_seed(23)
    B, S, H, D, T = 2, 90, 4, 128, 26
    dtype = torch.bfloat16
    q = torch.randn(B, S, H, D, generator=gen).to(dtype).to(DEV)
    k = torch.randn(B, S, H, D, generator=gen).to(dtype).to(DEV)
    v = torch.randn(B, S, H, D, generator=gen).to(dtype).to(DEV)
    w = [(1 + 0.1 * torch.randn(D, generator=gen)).to(dtype).to(DEV) for _ in range(4)]
    ang = torch.rand(200, D // 2, generator=gen) * 6.28
    cos = torch.cos(ang).repeat_interleave(2, -1).contiguous().to(DEV)
    sin = torch.sin(ang).repeat_interleave(2, -1).contiguous().to(DEV)

    def outs():
        return [torch.zeros(B, S + 5, H, D, dtype=dtype, device=DEV) for _ in range(3)]

    two = outs()
    kernels.qk_norm_rope([(q[:, :T], w[0], True, True), (k[:, :T], w[1], True, True), (v[:, :T], None, False, False)],
                         cos=cos, sin=sin, rope_row0=7, dsts=[[o] for o in two], dst_seq_offset=5)
    kernels.qk_norm_rope([(q[:, T:], w[2], True, True), (k[:, T:], w[3], True, True), (v[:, T:], None, False, False)],
                         cos=cos, sin=sin, rope_row0=100, dsts=[[o] for o in two], dst_seq_offset=5 + T)
    flags = torch.zeros(64, dtype=torch.int32, device=DEV)   # [0..2]: peers' slots, [8]: epoch counter, [9]: ticket
    base = flags.data_ptr()
    signal = kernels.FlagSignal([base + 0, None, base + 8], 1, base + 32, base + 36)
    for launch in (1, 2):
        one = outs()
        kernels.qk_norm_rope([(q, w[0], True, True), (k, w[1], True, True), (v, None, False, False)], cos=cos, sin=sin,
                             rope_row0=7, dsts=[[o] for o in one], dst_seq_offset=5,
                             range2=(T, [(w[2], True), (w[3], True), (None, False)], 100), signal=signal)
        torch.cuda.synchronize()
        for a, b in zip(one, two):
            assert torch.equal(a, b)
        f = flags.cpu().tolist()
        assert f[0] == launch and f[2] == launch and f[1] == 0 and f[8] == launch and f[9] == 0, f[:10]


def test_attention_waits_for_peer_flags_and_reports_a_silent_peer():
    """The attention kernel's loader waits for the flags its peers bump: with the flags at the awaited epoch the
    result is the ordinary one; with a flag that nothing sets the bounded wait runs out, the kernel reports
    HDIT_ERR_PEER_TIMEOUT (where = 9, the silent peer's index) and returns -- the context stays usable."""
    from hetu_dit_b200 import _C, kernels
    gen = torch.Generator().manual_seed(29)
    q, k, v = (torch.randn(1, 200, 2, 64, generator=gen).bfloat16().to(DEV) for _ in range(3))
    want = kernels.attn_fwd([q], [k], [v])
    flags = torch.zeros(16, dtype=torch.int32, device=DEV)
    flags[0], flags[2], flags[8] = 5, 6, 5     # peers 0 and 2 have reached epoch 5 (one is already ahead)
    base = flags.data_ptr()
    wait = kernels.FlagWait([base + 0, None, base + 8], base + 32, max_spins=20000)
    got = kernels.attn_fwd([q], [k], [v], wait_flags=wait)
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0 and torch.equal(got, want)
    flags[2] = 4                               # peer 2 has not arrived
    kernels.attn_fwd([q], [k], [v], wait_flags=wait)
    torch.cuda.synchronize()
    code, _, where, who = _C.device_status(0, clear=True)
    assert (code, where, who) == (_C.HDIT_ERR_PEER_TIMEOUT, 9, 2)
    assert torch.equal(kernels.attn_fwd([q], [k], [v]), want)   # the next launch is unaffected
    torch.cuda.synchronize()
    assert _C.device_status(0, clear=True)[0] == 0


def test_peer_heap_mark_and_rewind():
    """Buffers allocated after mark() go away on rewind() and the same names come back at the same offsets;
    buffers from before the mark stay where they are."""
    from hetu_dit_b200.core.distributed.peer import PeerHeap
    heap = PeerHeap(8 << 20, 0, 1, torch.device(DEV))
    inbox, off_inbox = heap.alloc((1024,), torch.uint8, name="pp_inbox")
    mark = heap.mark()
    a, off_a = heap.alloc((4, 256), torch.bfloat16, name="usp_q_a")
    b, off_b = heap.alloc((1000,), torch.float32, name="usp_k_a")
    assert heap.alloc((4, 256), torch.bfloat16, name="usp_q_a")[1] == off_a
    heap.rewind(mark)
    c, off_c = heap.alloc((8, 256), torch.bfloat16, name="usp_q_b")     # another shape takes the space
    assert off_c == off_a and c.data_ptr() == a.data_ptr()
    assert heap.alloc((1024,), torch.uint8, name="pp_inbox")[1] == off_inbox
    heap.rewind(mark)
    assert heap.alloc((4, 256), torch.bfloat16, name="usp_q_a")[1] == off_a
    assert heap.alloc((1000,), torch.float32, name="usp_k_a")[1] == off_b

"""Torch stand-ins for the kernel wrappers of hetu_dit_b200.kernels -- TEST INFRASTRUCTURE ONLY.

The product has no CPU path (kernels.py raises on CPU tensors). These functions restate the wrappers' documented
contracts (include/hdit.h, kernels.py docstrings) in plain torch so that the HOST code above them -- model wiring,
pipelines, stale-KV bookkeeping -- can run on a machine without a GPU and be compared with the oracle in fp32,
where a wiring mistake (a wrong residual, text source, row order or modulation vector) is not hidden by 16-bit
rounding. install(monkeypatch) swaps them in for the duration of one test. Single rank only: no peer destinations,
no partial / merge modes, no flags.
"""
import torch
import torch.nn.functional as F

from oracle import attention as oa


def attn_fwd(q_segs, k_segs, v_segs, *, softmax_scale=None, out=None, return_lse=False, mode=0, acc_out=None,
             acc_lse=None, kv_split=None, kv_interleave=0, out_dsts=None, q_rows_per_dst=None, q_dst_row0=None,
             wait_flags=None):
    if mode != 0 or out_dsts is not None or wait_flags is not None:
        raise NotImplementedError("the stand-in covers single-rank FINAL-mode calls only")
    q, k, v = (torch.cat(list(x), dim=1) for x in (q_segs, k_segs, v_segs))
    res, lse = oa.attention_with_lse(q, k, v, softmax_scale)
    res = res.to(q.dtype)
    if out is not None:
        out.copy_(res)
        res = out
    return (res, lse) if return_lse else res


def _norm(x, w, kind, bias, eps):
    if kind in (True, 1):
        return oa.rms_norm(x, w, eps)
    if kind == 2:
        return F.layer_norm(x.float(), (x.shape[-1],), None if w is None else w.float(),
                            None if bias is None else bias.float(), eps).to(x.dtype)
    return x


def _rope_rows(x, cos, sin, row0):
    n = x.shape[1]
    return oa.apply_rotary_emb(x.transpose(1, 2), cos[row0:row0 + n], sin[row0:row0 + n]).transpose(1, 2)


def qk_norm_rope(tensors, *, eps=1e-6, cos=None, sin=None, rope_seq_start=0, rope_row0=0, dsts=None,
                 dst_seq_offset=0, range2=None, signal=None):
    if dsts is not None or signal is not None:
        raise NotImplementedError("the stand-in works in place on one rank")
    for i, (x, w, do_norm, do_rope, *rest) in enumerate(tensors):
        bias = rest[0] if rest else None
        S = x.shape[1]
        end1 = S
        if range2 is not None and 0 < range2[0] < S:
            end1 = int(range2[0])
            w2, rope2, *rest2 = range2[1][i]
            part = _norm(x[:, end1:], w2, do_norm, rest2[0] if rest2 else None, eps)
            if rope2:
                part = _rope_rows(part, cos, sin, int(range2[2]))
            new2 = part
        first = _norm(x[:, :end1], w, do_norm, bias, eps)
        if do_rope:
            s0 = min(max(int(rope_seq_start), 0), end1)
            first = torch.cat([first[:, :s0], _rope_rows(first[:, s0:], cos, sin, int(rope_row0))], dim=1)
        x[:, :end1] = first
        if end1 < S:
            x[:, end1:] = new2


def ln_modulate(x, shift, scale, eps=1e-6, out=None):
    y = (F.layer_norm(x.float(), (x.shape[-1],), eps=eps) * (1 + scale[:, None].float()) + shift[:, None].float()).to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def gate_residual(x, gate, y, out=None):
    r = (x.float() + gate[:, None].float() * y.float()).to(x.dtype)
    if out is not None:
        out.copy_(r)
        return out
    return r


def gelu_tanh(x, out=None):
    r = F.gelu(x.float(), approximate="tanh").to(x.dtype)
    if out is not None:
        out.copy_(r)
        return out
    return r


def linear_tail(linear, x, epilogue, residual=None, gate=None, out=None):
    y = linear(x)
    if epilogue == "gelu_tanh":
        return gelu_tanh(y, out=out)
    if epilogue == "gate_residual":
        return gate_residual(residual, gate, y, out=out)
    raise ValueError(epilogue)


def kv_scatter(kv_cache, new_k, new_v, token_start):
    B = kv_cache.shape[0]
    nk, nv = new_k.reshape(B, new_k.shape[1], -1), new_v.reshape(B, new_v.shape[1], -1)
    n, R = nk.shape[1], nk.shape[2]
    kv_cache[:, token_start:token_start + n, :R] = nk
    kv_cache[:, token_start:token_start + n, R:] = nv


def install(monkeypatch):
    from hetu_dit_b200 import kernels
    for name in ("attn_fwd", "qk_norm_rope", "ln_modulate", "gate_residual", "gelu_tanh", "linear_tail", "kv_scatter"):
        monkeypatch.setattr(kernels, name, globals()[name])

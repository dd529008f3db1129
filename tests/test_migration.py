"""Parameter-slice migration: plans bit-exact against the reference-recorded fixtures (CPU), and the
pulled / back-filled weights bit-exact against the CPU master copy (GPU)."""
import json
import os

import pytest
import torch
import torch.nn as nn


class _Wrapped(nn.Module):
    def __init__(self, module):
        super().__init__()
        self.module = module


class _Proj(nn.Module):
    def __init__(self, i, o):
        super().__init__()
        self.proj = nn.Linear(i, o)


def _block_from_spec(spec, device="meta"):
    """A block whose named_modules() yields Linear layers under the given dotted names."""
    root = nn.Module()
    with torch.device(device):
        for path, out_f, in_f, bias in spec:
            parts = path.split(".")
            mod = root
            for p in parts[:-1]:
                if not hasattr(mod, p):
                    mod.add_module(p, nn.Module())
                mod = getattr(mod, p)
            mod.add_module(parts[-1], nn.Linear(in_f, out_f, bias=bias))
    return root


class _Model(nn.Module):
    def __init__(self, blocks):
        super().__init__()
        self.transformer_blocks = nn.ModuleList(blocks)


def test_plans_match_reference(golden_dir):
    from hetu_dit_b200.model_executor.cache.transformer_cache import TransformerBlockCache
    with open(os.path.join(golden_dir, "bookkeeping.json")) as f:
        cases = json.load(f)["migration_plans"]
    assert len(cases) >= 8
    for c in cases:
        model = _Model([_block_from_spec([tuple(l) for l in c["linears"]]) for _ in range(c["num_blocks"])])
        cache = TransformerBlockCache(device="cpu")
        for k, v in c["cached"].items():
            cache.cache[int(k)] = (None, tuple(v))
        lo, hi = cache.range_to_indices(c["new_pp"], c["num_blocks"])
        _, pieces = cache.plan_needed_pieces(list(range(lo, hi)), model, tuple(c["target_tp"]), c["slice_bias"])
        got = [{k: getattr(p, k) for k in ("uid", "block_index", "layer_path", "tensor_type", "split_dim", "full_size",
                                           "abs_start_idx", "abs_end_idx", "dest_offset")} for p in pieces]
        assert got == c["pieces"], c["kind"]


def test_piece_copy_descriptors_match_oracle():
    """The strided boxes built for a piece equal the (source, destination) descriptors of the reference."""
    from oracle import bookkeeping as ob
    from hetu_dit_b200.model_executor.cache.base_cache import NeededPiece
    from hetu_dit_b200.model_executor.cache.transformer_cache import TransformerBlockCache
    cache = TransformerBlockCache(device="cpu")
    es = 2
    for (split_dim, ttype, full, holder_tp, a, b, dest_off, src_shape, dst_shape) in [
        (0, "weight", 3072, (0.0, 0.5), 512, 1536, 512, (1536, 3072), (3072, 3072)),
        (1, "weight", 3072, (0.5, 1.0), 2048, 3072, 1024, (3072, 1536), (3072, 2048)),
        (0, "bias", 3072, (0.25, 1.0), 1000, 1100, 232, (2304,), (1000,)),
        (1, "weight", 1000, (1.0 / 3, 1.0), 400, 777, 67, (64, 667), (64, 500)),
    ]:
        p = NeededPiece(1, 0, "attn.module.to_q", ttype, split_dim, full, a, b, dest_off)
        src = torch.empty(src_shape, dtype=torch.bfloat16)
        dst = torch.empty(dst_shape, dtype=torch.bfloat16)
        entry = {"tp_range": holder_tp, "tensors": {"attn.module.to_q": {
            ttype: (src.data_ptr(), tuple(src.shape), src.stride(0) if src.dim() > 1 else 1, es)}}}
        box = cache.piece_copy(p, entry, dst)
        want = ob.piece_copy_descriptor(dict(tensor_type=ttype, split_dim=split_dim, full_size=full, abs_start_idx=a,
                                             abs_end_idx=b, dest_offset=dest_off), holder_tp, src_shape, dst_shape, es)
        s_off, d_off, rows, row_bytes, s_pitch, d_pitch = want
        assert box[0] - src.data_ptr() == s_off and box[1] - dst.data_ptr() == d_off
        assert box[2] * box[5] * box[8] == rows * row_bytes  # same bytes
        if rows > 1:
            assert (box[5], box[6], box[7], box[8]) == (rows, s_pitch, d_pitch, row_bytes)


def _tiny_block(hidden, seed):
    torch.manual_seed(seed)
    blk = nn.Module()
    attn = nn.Module()
    attn.to_q, attn.to_k, attn.to_v = nn.Linear(hidden, hidden), nn.Linear(hidden, hidden, bias=False), nn.Linear(hidden, hidden)
    attn.to_out = nn.ModuleList([nn.Linear(hidden, hidden), nn.Identity()])
    blk.attn = _Wrapped(attn)
    ff = nn.Module()
    ff.net = nn.ModuleList([_Proj(hidden, 4 * hidden), nn.Identity(), nn.Linear(4 * hidden, hidden)])
    blk.ff = _Wrapped(ff)
    blk.norm1 = nn.Module()
    blk.norm1.linear = nn.Linear(hidden, 6 * hidden)  # never split
    return blk.to(torch.bfloat16)


def _adjust(cache, *args, **kwargs):
    """The cache's public entry point is a coroutine, as in the reference (base_cache.py:243)."""
    import asyncio
    return asyncio.run(cache.adjust_pipeline(*args, **kwargs))


@pytest.mark.gpu
@pytest.mark.parametrize("hidden", [128, 200])
def test_migration_pull_and_backfill_bit_exact(hidden):
    """Pieces pulled from a 'peer' cache (same GPU, raw pointers) and gaps back-filled from the CPU master:
    every target slice equals the master's slice bit for bit."""
    from hetu_dit_b200.model_executor.cache.transformer_cache import TransformerBlockCache
    dev = torch.device("cuda:0")
    master = _Model([_tiny_block(hidden, s) for s in range(4)])
    peer = TransformerBlockCache(device=dev)
    peer_model = _Model([])
    _adjust(peer, peer_model, master, (0, 0), (0.0, 0.75), (0.0, 1.0), (0.0, 1.0))  # holds blocks 0-2 fully
    assert peer.active_block_indices == [0, 1, 2]
    me = TransformerBlockCache(device=dev)
    my_model = _Model([])
    _adjust(me, my_model, master, (0, 0), (0.0, 0.5), (0.0, 0.5), (0.0, 0.5))  # blocks 0-1, lower half
    torch.cuda.synchronize()
    # switch: all four blocks, TP range (0.25, 1.0): overlap reused, rest pulled from the peer, block 3 from CPU
    dirs = {1: peer.directory()}
    _adjust(me, my_model, master, (0.0, 0.5), (0.0, 1.0), (0.0, 0.5), (0.25, 1.0), peer_directories=dirs)
    torch.cuda.synchronize()
    pieces = me._last_p2p_all_pieces
    assert {p.source_rank for p in pieces if p.block_index < 3} == {1}
    assert {p.source_rank for p in pieces if p.block_index == 3} == {-1}
    assert len(my_model.transformer_blocks) == 4
    for i, blk in enumerate(my_model.transformer_blocks):
        ref = master.transformer_blocks[i]
        for name, sub in blk.named_modules():
            if not isinstance(sub, nn.Linear):
                continue
            r = ref.get_submodule(name)
            kind = me.choose_tp_split_type(name)
            if kind is None:
                assert torch.equal(sub.weight.cpu(), r.weight)
            elif kind == "row":
                lo, hi = me.range_to_indices((0.25, 1.0), r.weight.shape[0])
                assert torch.equal(sub.weight.cpu(), r.weight[lo:hi]), (i, name)
                if r.bias is not None:
                    assert torch.equal(sub.bias.cpu(), r.bias[lo:hi]), (i, name)
            else:
                lo, hi = me.range_to_indices((0.25, 1.0), r.weight.shape[1])
                assert torch.equal(sub.weight.cpu(), r.weight[:, lo:hi]), (i, name)
                assert torch.equal(sub.bias.cpu(), r.bias)
    # an unchanged plan is a no-op; the LRU keeps what the plan needs
    before = [id(b) for b in my_model.transformer_blocks]
    _adjust(me, my_model, master, (0.0, 1.0), (0.0, 1.0), (0.25, 1.0), (0.25, 1.0))
    assert [id(b) for b in my_model.transformer_blocks] == before
    assert peer.find_sources(pieces) and set(peer.find_sources(pieces)) <= {p.uid for p in pieces if p.block_index < 3}

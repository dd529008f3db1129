"""Parameter-slice migration: which pieces of which Linear layers a GPU is missing after a plan
switch, who can supply them, and the byte copies that fetch them.

Interface of the reference's hetu_dit/model_executor/cache/base_cache.py (NeededPiece :20,
DataReconstructionPlan :41, BaseBlockCache :50 with range_to_indices :213, adjust_pipeline :243,
_adjust_pipeline_legacy :284, _source_needed_pieces_from_peers :1132, _create_skeleton_block :1181,
_fill_plan_cpu_gaps :1238, _evict :108) and of the peer side in worker/worker.py
(rpc_find_sources :2079, rpc_nixl_send_data :2139).

The plan (list of NeededPiece) is computed exactly as the reference does. The transport differs:
the reference asks every peer over Ray which pieces it can serve, then has the source issue NIXL/UCX
WRITEs built from one descriptor per piece (one per weight *row* for column splits). Here every rank
publishes a directory of its cached blocks (TP range + device address of each weight in peer-mapped
memory); the requester matches pieces against the directories itself and *pulls* all of them with
one strided-copy launch per 40 pieces. What no peer holds comes from the CPU master copy.
"""
import copy
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ... import kernels


@dataclass(eq=True)
class NeededPiece:
    uid: int
    block_index: int
    layer_path: str
    tensor_type: str        # "weight" | "bias"
    split_dim: int
    full_size: int
    abs_start_idx: int
    abs_end_idx: int
    dest_offset: int
    source_rank: int = field(default=-1)
    status: str = field(default="needed")  # needed | sourced | done
    component: Optional[str] = field(default=None, compare=False)


@dataclass
class DataReconstructionPlan:
    block_index: int
    target_tp_range: Tuple[float, float]
    skeleton_block: Optional[nn.Module]
    pieces: List[NeededPiece] = field(default_factory=list)


def _resolve(module: nn.Module, path: str) -> nn.Module:
    for part in path.split("."):
        module = getattr(module, part)
    return module


class BaseBlockCache:
    """LRU cache of GPU-resident transformer blocks, each tagged with the TP range its split Linears hold."""

    def __init__(self, max_num_cached_blocks: int = 1 << 30, device: Optional[torch.device] = None, allocator=None,
                 deallocator=None):
        self.max_num_cached_blocks = max_num_cached_blocks
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        # allocator(shape, dtype) -> tensor: where migrated parameters live (peer-mapped memory when peers must
        # be able to pull them); default: ordinary device memory.
        self.allocator = allocator or (lambda shape, dtype: torch.empty(shape, dtype=dtype, device=self.device))
        self.deallocator = deallocator  # deallocator(tensor): gives evicted parameters back to the arena
        self.defer_release = False      # see _release()
        self._pending_release: List[torch.Tensor] = []
        self.cache: "OrderedDict[int, Tuple[nn.Module, Tuple[float, float]]]" = OrderedDict()
        self.active_block_indices: List[int] = []
        self._last_p2p_preplans: Dict[int, DataReconstructionPlan] = {}
        self._last_p2p_all_pieces: List[NeededPiece] = []

    # ---- model-specific hooks -----------------------------------------------------------------
    def choose_tp_split_type(self, name: str) -> Optional[str]:
        raise NotImplementedError

    def block_lists(self, model: nn.Module) -> List[nn.ModuleList]:
        raise NotImplementedError

    def get_total_blocks(self, model: nn.Module) -> int:
        return sum(len(l) for l in self.block_lists(model))

    def get_cpu_block_for_index(self, cpu_full_model: nn.Module, idx: int) -> nn.Module:
        for blocks in self.block_lists(cpu_full_model):
            if idx < len(blocks):
                return blocks[idx]
            idx -= len(blocks)
        raise IndexError(idx)

    # ---- ranges ---------------------------------------------------------------------------------
    def range_to_indices(self, rng: Tuple[float, float], total_size: int) -> Tuple[int, int]:
        """Fractional range -> [start, end): truncation, clamping, and an end of exactly 1.0 snaps to the size."""
        if total_size == 0:
            return 0, 0
        start = max(0, min(int(rng[0] * total_size), total_size))
        end = max(0, min(int(rng[1] * total_size), total_size))
        if start > end:
            end = start
        elif rng[1] == 1.0 and end < total_size:
            end = total_size
        return start, end

    # ---- plan -------------------------------------------------------------------------------------
    def plan_needed_pieces(self, new_required_indices: List[int], cpu_full_model: nn.Module,
                           target_tp: Tuple[float, float], slice_bias: bool = True, component_name=None):
        """For every required block and every split Linear in it: the parts of the target range that the
        cached copy (if any) does not cover, as NeededPieces (weights, plus biases of row splits)."""
        plans: Dict[int, DataReconstructionPlan] = {}
        pieces: List[NeededPiece] = []
        uid = 0
        for idx in new_required_indices:
            cpu_block = self.get_cpu_block_for_index(cpu_full_model, idx)
            cached = self.cache.get(idx)
            cached_tp = cached[1] if cached is not None else None
            plan = DataReconstructionPlan(idx, target_tp, None, [])
            for name, sub in cpu_block.named_modules():
                if not isinstance(sub, nn.Linear):
                    continue
                kind = self.choose_tp_split_type(name)
                if kind is None:
                    continue
                split_dim = 0 if kind == "row" else 1
                full = sub.weight.size(split_dim)
                lo, hi = self.range_to_indices(target_tp, full)
                if hi <= lo:
                    continue
                if cached_tp is not None:
                    c_lo, c_hi = self.range_to_indices(cached_tp, full)
                    keep_lo, keep_hi = max(lo, c_lo), min(hi, c_hi)
                else:
                    keep_lo = keep_hi = lo
                gaps = []
                if keep_lo > lo:
                    gaps.append((lo, keep_lo))
                if keep_hi < hi:
                    gaps.append((keep_hi, hi))
                for g_lo, g_hi in gaps:
                    if g_hi <= g_lo:
                        continue
                    uid += 1
                    plan.pieces.append(NeededPiece(uid, idx, name, "weight", split_dim, full, g_lo, g_hi, g_lo - lo,
                                                   component=component_name))
                    if slice_bias and kind == "row" and sub.bias is not None:
                        b_full = sub.bias.size(0)
                        b_lo, _ = self.range_to_indices(target_tp, b_full)
                        s = b_lo + (g_lo - lo)
                        e = s + (g_hi - g_lo)
                        if e > s:
                            uid += 1
                            plan.pieces.append(NeededPiece(uid, idx, name, "bias", split_dim, b_full, s, e, s - b_lo,
                                                           component=component_name))
            plans[idx] = plan
            pieces.extend(plan.pieces)
        self._last_p2p_preplans, self._last_p2p_all_pieces = plans, pieces
        return plans, pieces

    # ---- peer side ----------------------------------------------------------------------------------
    def find_sources(self, pieces: List[NeededPiece]) -> List[int]:
        """uids of the pieces this cache can serve: the block is cached and its slice covers the whole span."""
        out = []
        for p in pieces:
            entry = self.cache.get(p.block_index)
            if entry is None:
                continue
            lo, hi = self.range_to_indices(entry[1], p.full_size)
            if lo <= p.abs_start_idx and hi >= p.abs_end_idx:
                out.append(p.uid)
        return out

    def directory(self, ptr_of=None) -> Dict[int, dict]:
        """What a peer needs to pull from this cache: per cached block its TP range and, per split Linear,
        address / shape / row stride of weight and bias. `ptr_of(tensor)` maps a local tensor to the address
        peers use (heap offset, or the raw pointer inside one process)."""
        ptr_of = ptr_of or (lambda t: t.data_ptr())
        out = {}
        for idx, (block, tp) in self.cache.items():
            tensors = {}
            for name, sub in block.named_modules():
                if isinstance(sub, nn.Linear) and self.choose_tp_split_type(name) is not None:
                    tensors[name] = {"weight": (ptr_of(sub.weight.data), tuple(sub.weight.shape), sub.weight.stride(0),
                                                sub.weight.element_size())}
                    if sub.bias is not None:
                        tensors[name]["bias"] = (ptr_of(sub.bias.data), tuple(sub.bias.shape), 1, sub.bias.element_size())
            out[idx] = {"tp_range": tuple(tp), "tensors": tensors}
        return out

    # ---- requester side -------------------------------------------------------------------------------
    def _source_needed_pieces_from_peers(self, pieces: List[NeededPiece], peer_directories: Dict[int, Dict[int, dict]]):
        """First peer (lowest rank) whose cached slice fully covers a piece wins (worker.py:2129-2132)."""
        for p in pieces:
            for rank in sorted(peer_directories):
                entry = peer_directories[rank].get(p.block_index)
                if entry is None or p.layer_path not in entry["tensors"]:
                    continue
                lo, hi = self.range_to_indices(entry["tp_range"], p.full_size)
                if lo <= p.abs_start_idx and hi >= p.abs_end_idx and p.tensor_type in entry["tensors"][p.layer_path]:
                    p.source_rank, p.status = rank, "sourced"
                    break

    def piece_copy(self, p: NeededPiece, src_entry: dict, dst_tensor: torch.Tensor, resolve_ptr=None):
        """The strided box (bytes) that moves one piece from a source slice into the skeleton tensor."""
        src_ptr, src_shape, src_row_stride, es = src_entry["tensors"][p.layer_path][p.tensor_type]
        if resolve_ptr is not None:
            src_ptr = resolve_ptr(src_ptr)
        my_lo, _ = self.range_to_indices(src_entry["tp_range"], p.full_size)
        rel = p.abs_start_idx - my_lo
        span = p.abs_end_idx - p.abs_start_idx
        dst_ptr = dst_tensor.data_ptr()
        if p.tensor_type == "bias":
            return (src_ptr + rel * es, dst_ptr + p.dest_offset * es, 1, 0, 0, 1, 0, 0, span * es)
        src_pitch = src_row_stride * es
        dst_pitch = dst_tensor.stride(0) * es
        if p.split_dim == 0:
            row_bytes = dst_tensor.shape[1] * es
            if src_pitch == row_bytes and dst_pitch == row_bytes:
                return (src_ptr + rel * src_pitch, dst_ptr + p.dest_offset * dst_pitch, 1, 0, 0, 1, 0, 0, span * row_bytes)
            return (src_ptr + rel * src_pitch, dst_ptr + p.dest_offset * dst_pitch, 1, 0, 0, span, src_pitch, dst_pitch,
                    row_bytes)
        return (src_ptr + rel * es, dst_ptr + p.dest_offset * es, 1, 0, 0, dst_tensor.shape[0], src_pitch, dst_pitch,
                span * es)

    def _create_skeleton_block(self, idx: int, cpu_full_model: nn.Module, target_tp: Tuple[float, float],
                               slice_bias: bool = True) -> nn.Module:
        """A GPU copy of block `idx` whose split Linears have the target slice's shape but no data yet;
        everything that is not split (norms, modulation, unsplit Linears, column-split biases) is copied from
        the CPU master."""
        cpu_block = self.get_cpu_block_for_index(cpu_full_model, idx)
        split = {n: self.choose_tp_split_type(n) for n, m in cpu_block.named_modules() if isinstance(m, nn.Linear)}
        block = copy.deepcopy(cpu_block).to("meta")
        for name, sub in cpu_block.named_modules():
            tgt = _resolve(block, name) if name else block
            for pname, prm in sub.named_parameters(recurse=False):
                kind = split.get(name) if isinstance(sub, nn.Linear) else None
                if kind is not None and pname == "weight":
                    dim = 0 if kind == "row" else 1
                    lo, hi = self.range_to_indices(target_tp, prm.size(dim))
                    shape = list(prm.shape)
                    shape[dim] = hi - lo
                    new = self.allocator(tuple(shape), prm.dtype)
                elif kind == "row" and pname == "bias" and slice_bias:
                    lo, hi = self.range_to_indices(target_tp, prm.size(0))
                    new = self.allocator((hi - lo,), prm.dtype)
                else:
                    new = self.allocator(tuple(prm.shape), prm.dtype)
                    new.copy_(prm.data, non_blocking=True)
                setattr(tgt, pname, nn.Parameter(new, requires_grad=False))
            for bname, buf in sub.named_buffers(recurse=False):
                setattr(tgt, bname, buf.to(self.device))
        return block

    def _fill_plan_cpu_gaps(self, plan: DataReconstructionPlan, cpu_full_model: nn.Module, slice_bias: bool = True):
        """H2D copy of every piece no peer delivered, from the CPU master copy."""
        cpu_block = self.get_cpu_block_for_index(cpu_full_model, plan.block_index)
        for p in plan.pieces:
            if p.status == "done":
                continue
            src = getattr(_resolve(cpu_block, p.layer_path), p.tensor_type).data
            dst = getattr(_resolve(plan.skeleton_block, p.layer_path), p.tensor_type).data
            span = p.abs_end_idx - p.abs_start_idx
            if p.tensor_type == "bias" or p.split_dim == 0:
                dst[p.dest_offset:p.dest_offset + span].copy_(src[p.abs_start_idx:p.abs_end_idx], non_blocking=True)
            else:
                dst[:, p.dest_offset:p.dest_offset + span].copy_(src[:, p.abs_start_idx:p.abs_end_idx], non_blocking=True)
            p.status = "done"

    def _reuse_overlap(self, plan: DataReconstructionPlan, old_block: nn.Module, old_tp: Tuple[float, float],
                       cpu_block: Optional[nn.Module] = None):
        """Device copies of the part of the target range the previously cached slice already holds. The unsplit
        sizes come from the CPU master block when it is given (always, from adjust_pipeline); a slice whose shape
        disagrees with its range raises instead of being copied at a wrong offset."""
        boxes = []
        for name, sub in plan.skeleton_block.named_modules():
            if not isinstance(sub, nn.Linear):
                continue
            kind = self.choose_tp_split_type(name)
            if kind is None:
                continue
            old = _resolve(old_block, name)
            dim = 0 if kind == "row" else 1
            tensors = [("weight", dim)]
            if kind == "row" and sub.bias is not None:
                tensors.append(("bias", 0))
            for tname, d in tensors:
                new_t, old_t = getattr(sub, tname).data, getattr(old, tname).data
                if cpu_block is not None:
                    full = getattr(_resolve(cpu_block, name), tname).shape[d if new_t.dim() > 1 else 0]
                else:
                    full = _full_size(new_t, old_t, d, plan.target_tp_range, old_tp, self)
                lo, hi = self.range_to_indices(plan.target_tp_range, full)
                o_lo, o_hi = self.range_to_indices(old_tp, full)
                dd = d if new_t.dim() > 1 else 0
                if new_t.shape[dd] != hi - lo or old_t.shape[dd] != o_hi - o_lo:
                    raise RuntimeError(
                        f"{name}.{tname}: slices of {old_t.shape[dd]} / {new_t.shape[dd]} along dim {dd} do not match "
                        f"the ranges {old_tp} / {plan.target_tp_range} of a dimension of {full}")
                k_lo, k_hi = max(lo, o_lo), min(hi, o_hi)
                if k_hi <= k_lo:
                    continue
                if new_t.dim() == 1 or d == 0:
                    kernels.copy_2d(new_t[k_lo - lo:k_hi - lo], old_t[k_lo - o_lo:k_hi - o_lo])
                else:
                    kernels.copy_2d(new_t[:, k_lo - lo:k_hi - lo], old_t[:, k_lo - o_lo:k_hi - o_lo])
        return boxes

    # ---- LRU ---------------------------------------------------------------------------------------------
    def _release(self, block: Optional[nn.Module]):
        """Hands a block's parameter memory back. While `defer_release` is set the memory only goes on a list:
        during a plan switch peers may still pull from a block this rank has already replaced or evicted (they
        read the directory exchanged before the switch), so the region must not be handed out again until
        every rank's pulls have completed -- the worker calls flush_released() after that point."""
        if block is not None and self.deallocator is not None:
            for prm in block.parameters():
                if self.defer_release:
                    self._pending_release.append(prm.data)
                else:
                    self.deallocator(prm.data)

    def flush_released(self) -> int:
        """Deallocates everything released while `defer_release` was set; returns how many tensors."""
        n = len(self._pending_release)
        for t in self._pending_release:
            self.deallocator(t)
        self._pending_release = []
        return n

    def _add_or_update(self, idx: int, block: nn.Module, tp_range: Tuple[float, float]):
        old = self.cache.get(idx)
        if old is not None and old[0] is not block:
            self._release(old[0])
        self.cache[idx] = (block, tuple(tp_range))
        self.cache.move_to_end(idx)

    def _evict(self, keep: Optional[set] = None):
        keep = keep or set()
        while len(self.cache) > self.max_num_cached_blocks:
            victim = next((i for i in self.cache if i not in keep), None)
            if victim is None:
                break
            self._release(self.cache.pop(victim)[0])

    # ---- the plan switch -----------------------------------------------------------------------------------
    async def adjust_pipeline(self, transformer: Optional[nn.Module] = None,
                              cpu_full_transformer: Optional[nn.Module] = None, old_pp_range: tuple = None,
                              new_pp_range: tuple = None, old_tp_range: tuple = None, new_tp_range: tuple = None,
                              slice_bias: bool = True, text_encoder: Optional[nn.Module] = None,
                              cpu_full_text_encoder: Optional[nn.Module] = None, model: Optional[nn.Module] = None,
                              cpu_full_model: Optional[nn.Module] = None, peer_directories=None, resolve_ptr=None,
                              **kwargs) -> nn.Module:
        """The reference's entry point (model_executor/cache/base_cache.py:243-282): a coroutine taking the model as
        (transformer, cpu_full_transformer), (text_encoder, cpu_full_text_encoder) or (model, cpu_full_model), by
        keyword or in this order. `peer_directories` and `resolve_ptr` are this repository's additions (where the
        reference asks its peers over RPC, the caller passes what the peers published). The work is synchronous
        GPU / host work: adjust_pipeline_sync()."""
        component_name = kwargs.pop("component_name", None)
        if model is None or cpu_full_model is None:
            if transformer is not None and cpu_full_transformer is not None:
                model, cpu_full_model, component_name = transformer, cpu_full_transformer, "Transformer"
            elif text_encoder is not None and cpu_full_text_encoder is not None:
                model, cpu_full_model, component_name = text_encoder, cpu_full_text_encoder, "TextEncoder"
            else:
                raise TypeError("adjust_pipeline requires either (transformer, cpu_full_transformer) or "
                                "(text_encoder, cpu_full_text_encoder) or (model, cpu_full_model)")
        return self.adjust_pipeline_sync(model, cpu_full_model, old_pp_range, new_pp_range, old_tp_range,
                                         new_tp_range, slice_bias=slice_bias, peer_directories=peer_directories,
                                         resolve_ptr=resolve_ptr, component_name=component_name)

    def adjust_pipeline_sync(self, transformer: nn.Module, cpu_full_transformer: nn.Module, old_pp_range,
                             new_pp_range, old_tp_range, new_tp_range=None, slice_bias: bool = True,
                             peer_directories=None, resolve_ptr=None, component_name=None) -> nn.Module:
        """Brings `transformer`'s block lists to the new (PP, TP) ranges: reuse what is cached, pull what peers
        hold, read the rest from the CPU master copy. `peer_directories` = {rank: directory()} of the peers."""
        total = self.get_total_blocks(cpu_full_transformer)
        lo, hi = self.range_to_indices(new_pp_range, total)
        required = list(range(lo, hi))
        target_tp = tuple(new_tp_range) if new_tp_range is not None else tuple(old_tp_range)
        if set(self.active_block_indices) == set(required) and tuple(old_tp_range) == target_tp and all(
                i in self.cache and self.cache[i][1] == target_tp for i in required):
            self._last_p2p_preplans, self._last_p2p_all_pieces = {}, []   # nothing was needed
            return transformer
        plans, pieces = self.plan_needed_pieces(required, cpu_full_transformer, target_tp, slice_bias, component_name)
        if peer_directories:
            self._source_needed_pieces_from_peers(pieces, peer_directories)
        boxes = []
        for idx in required:
            cached = self.cache.get(idx)
            if cached is not None and cached[1] == target_tp:
                self.cache.move_to_end(idx)
                continue
            plan = plans[idx]
            plan.skeleton_block = self._create_skeleton_block(idx, cpu_full_transformer, target_tp, slice_bias)
            if cached is not None:
                self._reuse_overlap(plan, cached[0], cached[1], self.get_cpu_block_for_index(cpu_full_transformer, idx))
            for p in plan.pieces:
                if p.status == "sourced":
                    dst = getattr(_resolve(plan.skeleton_block, p.layer_path), p.tensor_type).data
                    boxes.append(self.piece_copy(p, peer_directories[p.source_rank][p.block_index], dst, resolve_ptr))
                    p.status = "done"
            self._fill_plan_cpu_gaps(plan, cpu_full_transformer, slice_bias)
            self._add_or_update(idx, plan.skeleton_block, target_tp)
        kernels.copy_pieces(boxes, self.device)
        self.place_blocks_on_model(transformer, [self.cache[i][0] for i in required], required, cpu_full_transformer)
        self.active_block_indices = required
        self._evict(keep=set(required))
        return transformer

    def place_blocks_on_model(self, model: nn.Module, blocks_list: List[nn.Module], required_indices: List[int],
                              cpu_full_model: nn.Module):
        """Distributes the global block indices back onto the model's block lists."""
        lists = self.block_lists(cpu_full_model)
        names = self.block_list_names()
        out = {n: [] for n in names}
        bounds, acc = [], 0
        for l in lists:
            bounds.append((acc, acc + len(l)))
            acc += len(l)
        for blk, gi in zip(blocks_list, required_indices):
            for n, (a, b) in zip(names, bounds):
                if a <= gi < b:
                    out[n].append(blk)
        for n in names:
            setattr(model, n, nn.ModuleList(out[n]))

    def block_list_names(self) -> List[str]:
        raise NotImplementedError


def _full_size(new_t, old_t, dim, new_tp, old_tp, cache) -> int:
    """Size of the unsplit dimension, recovered from a slice and its fractional range."""
    n = new_t.shape[dim] if new_t.dim() > 1 else new_t.shape[0]
    frac = new_tp[1] - new_tp[0]
    guess = int(round(n / frac)) if frac > 0 else n
    for cand in (guess, guess - 1, guess + 1):
        lo, hi = cache.range_to_indices(new_tp, cand)
        if hi - lo == n:
            return cand
    return guess

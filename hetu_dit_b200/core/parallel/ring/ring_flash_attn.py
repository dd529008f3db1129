"""Ring (context-parallel) attention with the log-sum-exp merge done inside the attention kernel.

Interface of the reference's hetu_dit/core/parallel/ring/ring_flash_attn.py:
ring_flash_attn_forward (:9-97) and ring_flash_attn_func (:155-188).

The reference rotates K and V around the ring with NCCL isend/irecv, calls
flash-attn once per step and merges partial results with eager fp32 kernels.
Here every rank's K/V block lives in the node's peer heap, so a rank *pulls* the
R-1 remote blocks into local staging memory with one coalesced copy kernel each
(on a side stream, crossing NVLink exactly once) while the tensor cores work on
the local block; the remaining blocks are then consumed by a single launch whose
epilogue merges with the first partial result by log-sum-exp. Joint (text) K/V
joins the block list at the position the reference's step index implies:
first for "front", last for "rear". Attention is invariant to the order in
which KV blocks are visited, so results agree with the reference's rotation.
"""
from typing import Optional

import torch

from .... import _C, kernels
from ...distributed.peer import PeerGroup
from ...resource_manager.cache_manager import get_cache_manager

_SUPPORTED_JOINT = ["none", "front", "rear"]


def _ring_state(heap, device):
    """Side stream and staging buffers of the ring pulls, owned by the heap (one per plan group) and keyed by
    the stream the caller runs on: two models, or two streams, in one process do not share them."""
    state = heap.__dict__.setdefault("_ring_state", {})
    key = torch.cuda.current_stream(device).cuda_stream
    if key not in state:
        state[key] = {"side": torch.cuda.Stream(device=device), "staging": {}}
    return state[key]


def _in_heap(heap, t: torch.Tensor) -> bool:
    off = t.data_ptr() - heap.base
    return 0 <= off < heap.nbytes and t.is_contiguous()


def _publish(heap, t: torch.Tensor, tag: str) -> torch.Tensor:
    """A contiguous copy of `t` inside the peer heap (no copy when it already lives there)."""
    if _in_heap(heap, t):
        return t
    buf, _ = heap.alloc(t.shape, t.dtype, name=f"ring_{tag}_{tuple(t.shape)}_{t.dtype}")
    kernels.copy_2d(buf, t)
    return buf


def ring_flash_attn_forward(process_group: Optional[PeerGroup], q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                            softmax_scale, dropout_p=0, causal=True, window_size=(-1, -1), alibi_slopes=None,
                            deterministic=False, attn_layer=None, joint_tensor_key=None, joint_tensor_value=None,
                            joint_strategy="none", joint_tensor_query=None, out_scatter=None, wait_flags=None):
    """(out in q.dtype, lse (B, H, Sq) fp32) for this rank's queries against the whole ring's K/V.

    joint_tensor_query (not in the reference's signature): joint queries kept as their own segment
    instead of being concatenated into `q` by the caller; output rows are [joint; q] for "front" and
    [q; joint] for "rear", exactly as if they had been concatenated.

    out_scatter (not in the reference's signature): dict(dsts=RawDst, q=(rows per destination, first row),
    joint=(...)) -- the launch that produces the final result stores its rows into these destination buffers
    (the Ulysses reverse all-to-all from the attention epilogue) and `out` is returned as None.

    wait_flags (a kernels.FlagWait, ring of one only): the attention kernel waits for these peer flags before it
    loads q, k, v (the barrier after the Ulysses head exchange, folded into the consumer)."""
    if joint_strategy not in _SUPPORTED_JOINT:
        raise ValueError(
            f"joint_strategy: {joint_strategy} not supprted. supported joint strategy: {_SUPPORTED_JOINT}")
    if joint_strategy != "none" and (joint_tensor_key is None or joint_tensor_value is None):
        raise ValueError("joint_tensor_key & joint_tensor_value must not be None when joint_strategy is not None")
    if causal or dropout_p != 0:
        raise NotImplementedError("the DiT denoising path is non-causal and dropout-free")

    if attn_layer is not None:
        k, v = get_cache_manager().update_and_get_kv_cache(new_kv=[k, v], layer=attn_layer, slice_dim=1,
                                                           layer_type="attn")

    world = 1 if process_group is None else process_group.world_size
    front = [joint_tensor_key], [joint_tensor_value]
    q_segs = [q]
    roles = ["q"]
    if joint_tensor_query is not None:
        front_q = joint_strategy == "front"
        q_segs = [joint_tensor_query, q] if front_q else [q, joint_tensor_query]
        roles = ["joint", "q"] if front_q else ["q", "joint"]
    scatter_kw = {}
    if out_scatter is not None:
        scatter_kw = dict(out_dsts=out_scatter["dsts"], q_rows_per_dst=[out_scatter[r][0] for r in roles],
                          q_dst_row0=[out_scatter[r][1] for r in roles])
    if world == 1:
        ks, vs = [k], [v]
        if joint_strategy == "rear":
            ks, vs = [k, joint_tensor_key], [v, joint_tensor_value]
        elif joint_strategy == "front":
            ks, vs = [joint_tensor_key, k], [joint_tensor_value, v]
        res = kernels.attn_fwd(q_segs, ks, vs, softmax_scale=softmax_scale, return_lse=True, wait_flags=wait_flags,
                               **scatter_kw)
        return (None, res) if out_scatter is not None else res
    if wait_flags is not None:
        raise ValueError("wait_flags need a ring of one: the ring pull reads K / V before attention does")

    heap = process_group.heap
    if heap is None:
        raise RuntimeError("ring attention across ranks needs the peer heap")
    dev = q.device
    k_pub, v_pub = _publish(heap, k, "k"), _publish(heap, v, "v")
    k_off, v_off = heap.offset_of(k_pub), heap.offset_of(v_pub)
    process_group.barrier()  # every rank's block is in place (and last layer's readers are done)

    me = process_group.rank_in_group
    B, S_blk, H, D = k_pub.shape
    state = _ring_state(heap, dev)
    key = (world, tuple(k_pub.shape), k_pub.dtype)
    if key not in state["staging"]:
        state["staging"][key] = torch.empty((2, world - 1) + tuple(k_pub.shape), dtype=k_pub.dtype, device=dev)
    stage = state["staging"][key]
    nbytes = k_pub.numel() * k_pub.element_size()

    # pull the R-1 remote blocks on the side stream, in the order the ring would deliver them
    side = state["side"]
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        pieces = []
        for step in range(1, world):
            src = process_group.ranks[(me - step) % world]
            pieces.append((heap.peer_ptr(src, k_off), stage[0, step - 1].data_ptr(), 1, 0, 0, 1, 0, 0, nbytes))
            pieces.append((heap.peer_ptr(src, v_off), stage[1, step - 1].data_ptr(), 1, 0, 0, 1, 0, 0, nbytes))
        kernels.copy_pieces(pieces, dev)
        pulled = torch.cuda.Event()
        pulled.record(side)

    sq = sum(t.shape[1] for t in q_segs)
    acc = torch.empty((B, sq, H, D), dtype=torch.float32, device=dev)
    acc_lse = torch.empty((B, H, sq), dtype=torch.float32, device=dev)
    ks, vs = [k_pub], [v_pub]
    if joint_strategy == "front":
        ks, vs = front[0] + ks, front[1] + vs
    kernels.attn_fwd(q_segs, ks, vs, softmax_scale=softmax_scale, mode=_C.ATTN_PARTIAL_FIRST, acc_out=acc,
                     acc_lse=acc_lse)

    torch.cuda.current_stream(dev).wait_event(pulled)
    ks = [stage[0, i] for i in range(world - 1)]
    vs = [stage[1, i] for i in range(world - 1)]
    if joint_strategy == "rear":
        ks, vs = ks + [joint_tensor_key], vs + [joint_tensor_value]
    res = kernels.attn_fwd(q_segs, ks, vs, softmax_scale=softmax_scale, mode=_C.ATTN_MERGE_FINAL, acc_out=acc,
                           acc_lse=acc_lse, return_lse=True, **scatter_kw)
    out, lse = (None, res) if out_scatter is not None else res
    process_group.barrier()  # peers have finished pulling this rank's block
    return out, lse


def ring_flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                         alibi_slopes=None, deterministic=False, return_attn_probs=False, group=None, attn_layer=None,
                         joint_tensor_key=None, joint_tensor_value=None, joint_strategy="none", joint_tensor_query=None,
                         out_scatter=None, wait_flags=None):
    """Forward only (inference): returns out, or (out, lse, None) when return_attn_probs is set."""
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    assert alibi_slopes is None
    out, lse = ring_flash_attn_forward(group, q, k, v, softmax_scale=softmax_scale, dropout_p=dropout_p, causal=causal,
                                       window_size=window_size, alibi_slopes=alibi_slopes, deterministic=False,
                                       attn_layer=attn_layer, joint_tensor_key=joint_tensor_key,
                                       joint_tensor_value=joint_tensor_value, joint_strategy=joint_strategy,
                                       joint_tensor_query=joint_tensor_query, out_scatter=out_scatter,
                                       wait_flags=wait_flags)
    return out if not return_attn_probs else (out, lse, None)

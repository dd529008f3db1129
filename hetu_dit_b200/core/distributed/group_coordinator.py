"""PipeFusion stage-to-stage patch hand-off over peer memory.

Interface of the reference's PipelineGroupCoordinator
(hetu_dit/core/distributed/group_coordinator.py:630-1002): set_config,
reset_buffer, pipeline_send / pipeline_isend, pipeline_recv,
add_pipeline_recv_task / recv_next / get_pipeline_recv_data, next_rank /
prev_rank on a ring of stages.

The reference posts NCCL isend/irecv pairs and learns every new message shape
with a two-round int64 handshake plus two device synchronisations
(:848-929). Here the sender *pushes*: one coalesced copy kernel writes the
payload straight into the receiver's inbox (a fixed region of the receiver's
peer heap) and a release-store bumps the link's sequence counter; the receiver
enqueues a bounded wait on that counter. Messages of a link are FIFO. The
first message of each (name, segment) carries a 256-byte header (dims, dtype)
that the receiver reads once; inbox offsets are bump-allocated in first-use
order, which is the same on both ends of a FIFO link, so no address exchange
is needed.

A stage may overwrite (name, segment) in its successor's inbox only after the
successor has consumed the previous content. The PipeFusion schedule guarantees
it: stages form a ring and patch p of step t+1 reaches a stage only after
patch p of step t has travelled through every other stage.
"""
from typing import Dict, List, Optional, Tuple

import torch

from ... import kernels
from .peer import PeerGroup

_HEADER_BYTES = 256
_MAGIC = 0x48444954  # "HDIT"
_DTYPES = [torch.float16, torch.bfloat16, torch.float32, torch.int64, torch.int32, torch.uint8]
INBOX_BYTES_DEFAULT = 192 * 1024 * 1024
_CHANNEL = 0


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PipelineGroupCoordinator:
    def __init__(self, group: PeerGroup, inbox_bytes: int = INBOX_BYTES_DEFAULT):
        self.group = group
        self.ranks = group.ranks
        self.world_size = group.world_size
        self.rank_in_group = group.rank_in_group
        self.rank = group.global_rank
        self.heap = group.heap
        self.dtype: Optional[torch.dtype] = None
        self.inbox = None
        self.inbox_offset = 0
        self.inbox_bytes = inbox_bytes
        self.max_spins = None  # None: the heap's bound (PeerHeap.max_spins)
        if self.world_size > 1:
            if self.heap is None:
                raise RuntimeError("PipeFusion across ranks needs the peer heap")
            # First allocation after a plan switch on every stage -> same offset everywhere. At most
            # half of the heap, so the sequence-parallel buffers of the same plan still fit.
            inbox_bytes = min(inbox_bytes, (self.heap._limit // 2) // 4096 * 4096)
            self.inbox_bytes = inbox_bytes
            self.inbox, self.inbox_offset = self.heap.alloc((inbox_bytes,), torch.uint8, name="pp_inbox")
        self.reset_buffer()

    # ring neighbours (group_coordinator.py:171-185)
    @property
    def next_rank(self) -> int:
        return self.ranks[(self.rank_in_group + 1) % self.world_size]

    @property
    def prev_rank(self) -> int:
        return self.ranks[(self.rank_in_group - 1) % self.world_size]

    @property
    def is_first_rank(self) -> bool:
        return self.rank_in_group == 0

    @property
    def is_last_rank(self) -> bool:
        return self.rank_in_group == self.world_size - 1

    def set_config(self, dtype: torch.dtype):
        self.dtype = dtype

    def reset_buffer(self):
        """Forget message shapes and inbox layout (new request shape). Both ends of every link
        must call it between the same two messages."""
        self.recv_tasks_queue: List[Tuple[str, int]] = []
        self.receiving_tasks: List[Tuple[str, int]] = []
        self.recv_shape: Dict[str, Dict[int, torch.Size]] = {}
        self.send_shape: Dict[str, Dict[int, torch.Size]] = {}
        self.recv_buffer: Dict[str, Dict[int, torch.Tensor]] = {}
        self._send_slot: Dict[Tuple[str, int], Tuple[int, torch.Size, torch.dtype]] = {}
        self._send_cursor = 0
        self._recv_cursor = 0

    # ------------------------------------------------------------------ send
    def _header(self, t: torch.Tensor) -> torch.Tensor:
        words = [_MAGIC, t.dim(), _DTYPES.index(t.dtype)] + list(t.shape)
        words += [0] * (_HEADER_BYTES // 8 - len(words))
        return torch.tensor(words, dtype=torch.int64, device=t.device)

    def _slot(self, tensor: torch.Tensor, name: str, segment_idx: int):
        """(payload address in the successor's inbox, header piece or None) of message (name, segment_idx)."""
        key = (name, segment_idx)
        nbytes = tensor.numel() * tensor.element_size()
        dst_base = self.heap.peer_ptr(self.next_rank, self.inbox_offset)
        slot = self._send_slot.get(key)
        header = None
        if slot is None or slot[1] != tensor.shape or slot[2] != tensor.dtype:
            if slot is not None:
                raise RuntimeError(f"message {key} changed shape without reset_buffer()")
            off = self._send_cursor
            if off + _HEADER_BYTES + nbytes > self.inbox_bytes:
                raise MemoryError("PipeFusion inbox too small for this request shape")
            self._send_cursor = off + _HEADER_BYTES + _align(nbytes)
            self._send_slot[key] = (off, tensor.shape, tensor.dtype)
            self.send_shape.setdefault(name, {})[segment_idx] = tensor.shape
            hdr = self._header(tensor)
            header = (hdr.data_ptr(), dst_base + off, 1, 0, 0, 1, 0, 0, _HEADER_BYTES)
            self._keep_alive = hdr  # until the copy below has been enqueued behind it on the same stream
        else:
            off = slot[0]
        return dst_base + off + _HEADER_BYTES, header

    def _push(self, tensor: torch.Tensor, name: str, segment_idx: int):
        nbytes = tensor.numel() * tensor.element_size()
        dst, header = self._slot(tensor, name, segment_idx)
        pieces = [header] if header is not None else []
        if nbytes:
            pieces.append((tensor.data_ptr(), dst, 1, 0, 0, 1, 0, 0, nbytes))
        kernels.copy_pieces(pieces, tensor.device)
        self.heap.signal(self.next_rank, _CHANNEL)

    def reserve_send(self, like: torch.Tensor, name: str = "latent", segment_idx: int = -1) -> int:
        """For a producer kernel that writes the message itself: the address in the successor's inbox where the
        payload of a tensor shaped like `like` belongs (the header goes out now if this is the first message of
        the slot). The caller's kernel stores the payload there and then calls commit_send()."""
        dst, header = self._slot(like, name or "latent", segment_idx)
        if header is not None:
            kernels.copy_pieces([header], like.device)
        return dst

    def commit_send(self):
        """Publishes the message whose payload a kernel has stored at the address reserve_send() returned."""
        self.heap.signal(self.next_rank, _CHANNEL)

    def pipeline_isend(self, tensor: torch.Tensor, name: str = "latent", segment_idx: int = -1) -> None:
        self._push(tensor.contiguous(), name or "latent", segment_idx)

    def pipeline_send(self, tensor: torch.Tensor, name: str = "latent", segment_idx: int = -1) -> None:
        # Stream-ordered like pipeline_isend: the copy has been enqueued behind the producer of
        # `tensor`, which is all the reference's blocking variant guarantees to later stream work.
        self._push(tensor.contiguous(), name or "latent", segment_idx)

    # ------------------------------------------------------------------ receive
    def _await_message(self, name: str, idx: int) -> torch.Tensor:
        self.heap.wait(self.prev_rank, _CHANNEL, self.max_spins)
        buf = self.recv_buffer.get(name, {}).get(idx)
        if buf is not None:
            return buf
        # First message of this (name, idx): read its header once (one synchronisation, as the
        # reference's shape handshake has) and fix its place in the inbox.
        self.heap.check()
        off = self._recv_cursor
        hdr = self.inbox[off:off + _HEADER_BYTES].view(torch.int64).cpu().tolist()
        if hdr[0] != _MAGIC:
            raise RuntimeError(f"PipeFusion inbox corrupt at offset {off} while receiving ({name}, {idx})")
        ndim, dtype = hdr[1], _DTYPES[hdr[2]]
        shape = torch.Size(hdr[3:3 + ndim])
        nbytes = shape.numel() * torch.empty((), dtype=dtype).element_size()
        self._recv_cursor = off + _HEADER_BYTES + _align(nbytes)
        buf = self.inbox[off + _HEADER_BYTES:off + _HEADER_BYTES + nbytes].view(dtype).view(shape)
        self.recv_shape.setdefault(name, {})[idx] = shape
        self.recv_buffer.setdefault(name, {})[idx] = buf
        return buf

    def pipeline_recv(self, idx: int = -1, name: str = "latent") -> torch.Tensor:
        return self._await_message(name or "latent", idx)

    def add_pipeline_recv_task(self, idx: int = -1, name: str = "latent"):
        self.recv_tasks_queue.append((name or "latent", idx))

    def recv_next(self):
        """The reference posts the next irecv here; with pushed messages only the order is recorded."""
        if not self.recv_tasks_queue:
            raise ValueError("No more tasks to receive")
        self.receiving_tasks.append(self.recv_tasks_queue.pop(0))

    def pop_received(self, idx: int = -1, name: str = "latent") -> None:
        """The bookkeeping half of get_pipeline_recv_data(): the wait itself is part of a replayed CUDA graph."""
        assert len(self.receiving_tasks) > 0, "No tasks to receive, call add_pipeline_recv_task first"
        got_name, got_idx = self.receiving_tasks.pop(0)
        assert got_name == (name or "latent") and got_idx == idx, "Received tensor does not match the requested"

    def get_pipeline_recv_data(self, idx: int = -1, name: str = "latent") -> torch.Tensor:
        assert len(self.receiving_tasks) > 0, "No tasks to receive, call add_pipeline_recv_task first"
        got_name, got_idx = self.receiving_tasks.pop(0)
        assert got_name == (name or "latent") and got_idx == idx, "Received tensor does not match the requested"
        return self._await_message(got_name, got_idx)

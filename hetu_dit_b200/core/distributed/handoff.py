"""Stage hand-off of the denoised latents to the decode worker, GPU to GPU.

In the reference the diffusion stage's result leaves the GPU (`latents.to("cpu")`,
hetu_dit/model_executor/pipelines/pipeline_stable_diffusion_3.py:898), travels through the Ray object store to
the engine (hetu_dit/engine/async_serving_engine.py:553-590) and is uploaded again by the decode executor
(hetu_dit/worker/worker.py:812-867): a device-to-host copy, a pickle and a host-to-device copy per request. When
both workers sit in one NVSwitch domain the wire format can be the tensor itself: the sender stores a 256-byte
header (magic, rank, dtype, shape) and the payload into the receiver's hand-off slot in its peer heap with one
copy launch and bumps a sequence flag; the receiver waits on the flag (bounded), reads the header and gets a view
of its own memory.

The slots live at the top of every rank's heap (reserved once, before any plan allocates), one per source rank,
so they survive plan switches. A slot is overwritten by the next send from the same source: the receiver copies
or consumes the tensor before it accepts the next request from that source.
"""
from typing import Optional

import torch

from ... import kernels
from .peer import PeerHeap

_HEADER_BYTES = 256
_MAGIC = 0x4844484F  # "HDHO"
_DTYPES = [torch.float16, torch.bfloat16, torch.float32]
HANDOFF_CHANNEL = 1   # point-to-point flag channel (0 carries the PipeFusion patches)


class StageHandoff:
    def __init__(self, heap: PeerHeap, slot_bytes: int = 16 << 20):
        self.heap = heap
        self.slot_bytes = (int(slot_bytes) + 255) // 256 * 256
        self.base = heap.reserve_tail((self.slot_bytes + _HEADER_BYTES) * heap.world_size)

    def _slot(self, src_rank: int) -> int:
        return self.base + src_rank * (self.slot_bytes + _HEADER_BYTES)

    def send(self, dst_rank: int, tensor: torch.Tensor) -> None:
        """Enqueues the transfer on the current stream of the sender."""
        t = tensor.contiguous()
        nbytes = t.numel() * t.element_size()
        if nbytes > self.slot_bytes:
            raise MemoryError(f"hand-off of {nbytes} bytes exceeds the {self.slot_bytes}-byte slot")
        words = [_MAGIC, self.heap.rank, _DTYPES.index(t.dtype), t.dim()] + list(t.shape)
        hdr = torch.tensor(words + [0] * (_HEADER_BYTES // 8 - len(words)), dtype=torch.int64, device=t.device)
        dst = self.heap.peer_ptr(dst_rank, self._slot(self.heap.rank))
        pieces = [(hdr.data_ptr(), dst, 1, 0, 0, 1, 0, 0, _HEADER_BYTES)]
        if nbytes:
            pieces.append((t.data_ptr(), dst + _HEADER_BYTES, 1, 0, 0, 1, 0, 0, nbytes))
        kernels.copy_pieces(pieces, t.device)
        self.heap.signal(dst_rank, HANDOFF_CHANNEL)

    def recv(self, src_rank: int, max_spins: Optional[int] = None) -> torch.Tensor:
        """The tensor `src_rank` sent, as a view of this rank's slot (synchronises: the header is read on the
        host). Raises HditError(HDIT_ERR_PEER_TIMEOUT) when nothing arrives within the bound."""
        self.heap.wait(src_rank, HANDOFF_CHANNEL, max_spins)
        self.heap.check()
        off = self._slot(src_rank)
        hdr = self.heap._bytes[off:off + _HEADER_BYTES].view(torch.int64).cpu().tolist()
        if hdr[0] != _MAGIC or hdr[1] != src_rank:
            raise RuntimeError(f"hand-off slot of rank {src_rank} holds no message from it")
        dtype, ndim = _DTYPES[hdr[2]], hdr[3]
        shape = torch.Size(hdr[4:4 + ndim])
        nbytes = shape.numel() * torch.empty((), dtype=dtype).element_size()
        return self.heap._bytes[off + _HEADER_BYTES:off + _HEADER_BYTES + nbytes].view(dtype).view(shape)

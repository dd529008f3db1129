"""Symmetric peer heap of one NVSwitch domain and the groups built on it.

Every rank (one process per GPU) owns one heap allocated by the C library and
maps every other rank's heap once through CUDA IPC. A buffer that peers write
into, or read from, is carved from the heap at the same offset on every rank of
the communicating group, so `peer_ptr(rank, offset)` is all a kernel needs. This
replaces the reference's pool of NCCL communicators for every rank subset
(hetu_dit/core/distributed/parallel_state.py:1126-1510): activating a plan only
selects which ranks' base pointers are used.
"""
import ctypes
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ... import _C

FLAG_BYTES = 64 * 1024          # head of the heap: int32 counters
MAX_RANKS_PER_NODE = 8
_BARRIER_SLOTS = 256 * MAX_RANKS_PER_NODE  # one row of 8 counters per rank subset (bit mask of members)
_P2P_BASE = _BARRIER_SLOTS      # then 8 x 8 x 16 point-to-point sequence counters
_EPOCH_BASE = _P2P_BASE + 8 * 8 * 16  # then one barrier epoch counter per rank subset (device-side)
_P2P_SENT_BASE = _EPOCH_BASE + 256    # then, per link and channel, how many messages this rank has signalled ...
_P2P_EXPECT_BASE = _P2P_SENT_BASE + 8 * 8 * 16  # ... and how many it has waited for (device-side, graph-replayable)
_FOLD_BASE = _P2P_EXPECT_BASE + 8 * 8 * 16  # then, per rank subset, 8 arrival flags of the folded exchange barrier,
_FOLD_EPOCH_BASE = _FOLD_BASE + _BARRIER_SLOTS  # its epoch counter (device-side) ...
_FOLD_TICKET_BASE = _FOLD_EPOCH_BASE + 256      # ... and the ticket word of the signalling kernel
DEFAULT_MAX_SPINS = 20_000_000  # about two seconds of polling


class _RawCuda:
    """Minimal __cuda_array_interface__ carrier so torch can view heap memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerHeap:
    def __init__(self, nbytes: int, rank: int, world_size: int, device: torch.device,
                 all_gather_bytes: Optional[Callable[[bytes], List[bytes]]] = None):
        """all_gather_bytes(my_handle) -> every rank's handle in rank order (any host channel,
        e.g. torch.distributed.all_gather_object); None for a single rank."""
        if nbytes <= FLAG_BYTES:
            raise ValueError("heap too small")
        self.nbytes = int(nbytes)
        self.rank, self.world_size, self.device = rank, world_size, torch.device(device)
        self._cursor = FLAG_BYTES
        self._limit = self.nbytes   # allocations end here; reserve_tail() lowers it
        self.max_spins = DEFAULT_MAX_SPINS  # default bound of every device-side wait; a plan may raise it
        self._named: Dict[str, tuple] = {}
        self._epochs: Dict[int, int] = {}
        self._flip: Dict[str, int] = {}
        lib = _C.lib()
        with torch.cuda.device(self.device):
            base = ctypes.c_void_p()
            _C.check(lib.hdit_heap_alloc(self.nbytes, ctypes.byref(base)))
            self.base = base.value
            self.peer_base: List[Optional[int]] = [None] * world_size
            self.peer_base[rank] = self.base
            if world_size > 1:
                if all_gather_bytes is None:
                    raise ValueError("a multi-rank heap needs a host channel to exchange IPC handles")
                handle = ctypes.create_string_buffer(64)
                _C.check(lib.hdit_ipc_export(self.base, handle))
                handles = all_gather_bytes(handle.raw)
                for r, h in enumerate(handles):
                    if r == rank:
                        continue
                    p = ctypes.c_void_p()
                    _C.check(lib.hdit_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)))
                    self.peer_base[r] = p.value
        self._bytes = torch.as_tensor(_RawCuda(self.base, self.nbytes), device=self.device)

    # ------------------------------------------------------------------ allocation
    def reset(self):
        """Forget every buffer (plan switch). Ranks of a new group then allocate from the same offset."""
        self._cursor = FLAG_BYTES
        self._named.clear()
        self._flip.clear()

    def mark(self):
        """The allocation state right now, for rewind()."""
        return self._cursor, frozenset(self._named)

    def rewind(self, mark):
        """Forget every buffer allocated since mark() (a request of a new shape on the same plan: exchange
        buffers are named by shape, and a bump allocator can only give memory back from its end). Every rank of
        the plan must rewind between the same two requests; CUDA graphs that captured the forgotten buffers'
        addresses are void afterwards."""
        cursor, names = mark
        self._cursor = cursor
        for name in [n for n in self._named if n not in names]:
            del self._named[name]

    def reserve_tail(self, nbytes: int) -> int:
        """Sets `nbytes` at the top of the heap aside for good (it survives reset()) and returns its offset. Every
        rank must make the same reservations in the same order, before the plans start to allocate."""
        nbytes = (int(nbytes) + 255) // 256 * 256
        if self._cursor + nbytes > self._limit:
            raise MemoryError("peer heap too small for this reservation")
        self._limit -= nbytes
        return self._limit

    def alloc(self, shape: Sequence[int], dtype: torch.dtype, name: Optional[str] = None):
        """(tensor, offset): a zero-copy view of `shape` at a 256-byte aligned heap offset. A `name`
        makes the buffer persistent: asking again with the same name, shape and dtype returns it."""
        shape = tuple(int(s) for s in shape)
        if name is not None and name in self._named:
            t, off = self._named[name]
            if tuple(t.shape) == shape and t.dtype == dtype:
                return t, off
            raise ValueError(f"heap buffer {name!r} exists with shape {tuple(t.shape)}, asked for {shape}")
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = (self._cursor + 255) // 256 * 256
        if off + nbytes > self._limit:
            raise MemoryError(f"peer heap exhausted: need {nbytes} bytes at offset {off} of {self._limit}")
        self._cursor = off + nbytes
        t = self._bytes[off:off + nbytes].view(dtype).view(shape)
        if name is not None:
            self._named[name] = (t, off)
        return t, off

    def flip(self, name: str) -> int:
        """0, 1, 0, ... per name: which of two alternately used buffers the next exchange of that name takes.
        Every rank of a group calls it once per exchange, so the ranks agree."""
        v = self._flip[name] = 1 - self._flip.get(name, 1)
        return v

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base
        if off < 0 or off >= self.nbytes:
            raise ValueError("tensor does not live in the peer heap")
        return off

    def peer_ptr(self, rank: int, offset: int) -> int:
        base = self.peer_base[rank]
        if base is None:
            raise RuntimeError(f"rank {rank} is not mapped")
        return base + offset

    # ------------------------------------------------------------------ flags
    def _flag_ptr(self, rank: int, index: int) -> int:
        return self.peer_ptr(rank, index * 4)

    def barrier(self, ranks: Sequence[int], max_spins: Optional[int] = None):
        """Stream-ordered barrier among `ranks` (global ranks of this node, this rank included)."""
        max_spins = self.max_spins if max_spins is None else max_spins
        ranks = list(ranks)
        n = len(ranks)
        if n == 1:
            return
        me = ranks.index(self.rank)
        mask = 0
        for r in ranks:
            mask |= 1 << (r % MAX_RANKS_PER_NODE)
        # the epoch lives in this rank's heap and is advanced by the barrier kernel itself, so the
        # call can be captured in a CUDA graph and replayed
        counter = self._flag_ptr(self.rank, _EPOCH_BASE + mask)
        peer_slots = (ctypes.c_void_p * n)()
        my_slots = (ctypes.c_void_p * n)()
        for i, r in enumerate(ranks):
            if i == me:
                continue
            peer_slots[i] = self._flag_ptr(r, mask * MAX_RANKS_PER_NODE + me)      # in r's heap, row of this group
            my_slots[i] = self._flag_ptr(self.rank, mask * MAX_RANKS_PER_NODE + i)  # in my heap, written by r
        with torch.cuda.device(self.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            _C.check(_C.lib().hdit_peer_barrier(peer_slots, my_slots, n, me, 0, counter, max_spins, stream))

    def folded_barrier(self, ranks: Sequence[int]):
        """(FlagSignal, FlagWait) of a barrier whose signalling half runs in the tail of a producer kernel and
        whose waiting half runs in the head of the consumer kernel (both of this library): the producer's last
        CTA bumps this rank's flag in every peer's heap, the consumer polls the flags the peers bump here. Only
        "the producers' stores are visible to the consumer" is guaranteed -- unlike barrier(), it does not hold
        this rank back until the peers have arrived."""
        from ... import kernels
        ranks = list(ranks)
        me = ranks.index(self.rank)
        mask = 0
        for r in ranks:
            mask |= 1 << (r % MAX_RANKS_PER_NODE)
        row = _FOLD_BASE + mask * MAX_RANKS_PER_NODE
        epoch = self._flag_ptr(self.rank, _FOLD_EPOCH_BASE + mask)
        ticket = self._flag_ptr(self.rank, _FOLD_TICKET_BASE + mask)
        sig = kernels.FlagSignal([None if i == me else self._flag_ptr(r, row + me) for i, r in enumerate(ranks)], me,
                                 epoch, ticket)
        wait = kernels.FlagWait([None if i == me else self._flag_ptr(self.rank, row + i) for i in range(len(ranks))],
                                epoch, self.max_spins)
        return sig, wait

    def p2p_flag_index(self, src: int, dst: int, channel: int) -> int:
        return _P2P_BASE + ((src % 8) * 8 + (dst % 8)) * 16 + channel

    def signal(self, dst: int, channel: int):
        """Bump the (me -> dst, channel) sequence counter in dst's heap after all earlier stream work. The
        sequence number lives in this rank's heap and is advanced by the kernel, so the call can be captured
        in a CUDA graph and replayed."""
        idx = self.p2p_flag_index(self.rank, dst, channel)
        counter = self._flag_ptr(self.rank, _P2P_SENT_BASE + idx - _P2P_BASE)
        with torch.cuda.device(self.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            _C.check(_C.lib().hdit_peer_signal(self._flag_ptr(dst, idx), 0, counter, stream))

    def wait(self, src: int, channel: int, max_spins: Optional[int] = None):
        """Hold the stream until the next (src -> me, channel) message has been signalled (bounded: on expiry
        the kernel records HDIT_ERR_PEER_TIMEOUT and the stream moves on; check() raises it)."""
        max_spins = self.max_spins if max_spins is None else max_spins
        idx = self.p2p_flag_index(src, self.rank, channel)
        counter = self._flag_ptr(self.rank, _P2P_EXPECT_BASE + idx - _P2P_BASE)
        with torch.cuda.device(self.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            _C.check(_C.lib().hdit_peer_wait(self._flag_ptr(self.rank, idx), 0, counter, max_spins, src * 16 + channel,
                                             stream))

    def resync_flags(self, host_barrier: Callable[[], None]):
        """After a reported timeout the counters of the ranks no longer agree. Collective over all ranks of the
        node: every rank drains its GPU, all meet on the host, every rank zeroes its own flag block (barrier
        rows, point-to-point flags and every device-side counter), all meet again."""
        torch.cuda.synchronize(self.device)
        host_barrier()
        self._bytes[:FLAG_BYTES].zero_()
        torch.cuda.synchronize(self.device)
        host_barrier()

    def check(self):
        """Synchronise and raise if a bounded device-side wait ran out since the last check."""
        torch.cuda.synchronize(self.device)
        code, blk, where, it = _C.device_status(self.device.index or 0, clear=True)
        if code != 0:
            raise _C.HditError(code, f"device-side wait timed out (where={where}, detail={it}, block={blk})")


class PeerGroup:
    """An ordered set of global ranks sharing the heap; the stand-in for a torch ProcessGroup
    handed to the attention operators (ULYSSES_PG / RING_PG) and coordinators."""

    def __init__(self, ranks: Sequence[int], my_global_rank: int, heap: Optional[PeerHeap]):
        self.ranks = list(ranks)
        self.world_size = len(self.ranks)
        self.rank_in_group = self.ranks.index(my_global_rank) if my_global_rank in self.ranks else -1
        self.global_rank = my_global_rank
        self.heap = heap
        self._gather_parity = {}

    @property
    def rank(self):
        return self.rank_in_group

    def barrier(self, max_spins: Optional[int] = None):
        if self.world_size > 1:
            if self.heap is None:
                raise RuntimeError("a multi-rank group needs the peer heap")
            self.heap.barrier(self.ranks, max_spins)

    def all_gather(self, input_: torch.Tensor, dim: int = 0, separate_tensors: bool = False):
        """GroupCoordinator.all_gather of the reference (core/distributed/group_coordinator.py:225-264): the
        group's tensors concatenated along `dim` in group-rank order, or as a list when separate_tensors is
        set. Used once per request for the sequence-parallel latents
        (pipeline_stable_diffusion_3.py:1449,1660) and for the CFG halves (:1708).

        Every rank stores its tensor into its slot of a gathered buffer in each peer's heap (one copy
        launch), then a flag barrier. The result is copied out of the heap; two gathered buffers per shape
        are used alternately, because a fast peer may start the next gather of the same shape before this
        rank has copied the current one out (it cannot get two ahead: the barrier in between needs this
        rank)."""
        world = self.world_size
        if world == 1:
            return input_
        if not -input_.dim() <= dim < input_.dim():
            raise ValueError(f"Invalid dim ({dim}) for input tensor with shape {tuple(input_.size())}")
        if self.heap is None:
            raise RuntimeError("a multi-rank group needs the peer heap")
        from ... import kernels
        if dim < 0:
            dim += input_.dim()
        x = input_.contiguous()
        key = (tuple(x.shape), x.dtype)
        parity = self._gather_parity[key] = 1 - self._gather_parity.get(key, 0)
        buf, off = self.heap.alloc((world,) + tuple(x.shape), x.dtype, name=f"all_gather{parity}_{key}_{self.ranks}")
        nbytes = x.numel() * x.element_size()
        if nbytes:
            me = self.rank_in_group
            kernels.copy_pieces([(x.data_ptr(), self.heap.peer_ptr(r, off) + me * nbytes, 1, 0, 0, 1, 0, 0, nbytes)
                                 for r in self.ranks], x.device)
        self.barrier()
        out = buf.clone()
        if separate_tensors:
            return [out[i] for i in range(world)]
        if dim != 0:
            out = out.movedim(0, dim)
        size = list(x.shape)
        size[dim] *= world
        return out.reshape(size)

    def next_rank(self):
        return self.ranks[(self.rank_in_group + 1) % self.world_size]

    def prev_rank(self):
        return self.ranks[(self.rank_in_group - 1) % self.world_size]

    def __repr__(self):
        return f"PeerGroup(ranks={self.ranks}, rank={self.rank_in_group})"


class ParamArena:
    """Peer-mapped memory for model parameters that other ranks may pull during a plan switch.

    Unlike the activation heap it survives plan switches, so it has a first-fit free list instead of a
    bump pointer. Offsets are private to the owning rank; a peer learns them from the owner's block
    directory and turns them into addresses with peer_ptr()."""

    def __init__(self, nbytes: int, rank: int, world_size: int, device, all_gather_bytes=None):
        self.heap = PeerHeap(nbytes + FLAG_BYTES, rank, world_size, device, all_gather_bytes)
        self.rank = rank
        self._free = [(FLAG_BYTES, nbytes)]  # (offset, size), sorted by offset
        self._used = {}                      # offset -> size

    def alloc(self, shape, dtype) -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        size = max(256, (n * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256)
        for i, (off, avail) in enumerate(self._free):
            if avail >= size:
                if avail == size:
                    self._free.pop(i)
                else:
                    self._free[i] = (off + size, avail - size)
                self._used[off] = size
                nbytes = n * torch.empty((), dtype=dtype).element_size()
                return self.heap._bytes[off:off + nbytes].view(dtype).view(shape)
        raise MemoryError(f"parameter arena exhausted ({size} bytes requested)")

    def free(self, t: torch.Tensor):
        off = t.data_ptr() - self.heap.base
        size = self._used.pop(off, None)
        if size is None:
            return
        self._free.append((off, size))
        self._free.sort()
        merged = []
        for o, s in self._free:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + s)
            else:
                merged.append((o, s))
        self._free = merged

    def flip(self, name: str) -> int:
        """0, 1, 0, ... per name: which of two alternately used buffers the next exchange of that name takes.
        Every rank of a group calls it once per exchange, so the ranks agree."""
        v = self._flip[name] = 1 - self._flip.get(name, 1)
        return v

    def offset_of(self, t: torch.Tensor) -> int:
        return t.data_ptr() - self.heap.base

    def peer_ptr(self, rank: int, offset: int) -> int:
        return self.heap.peer_ptr(rank, offset)

    def bytes_in_use(self) -> int:
        return sum(self._used.values())

"""Denoising steps as replayed CUDA graphs.

One step of a DiT is about a thousand kernel launches; at 8 GPUs each is a few microseconds long, so enqueueing
them from Python takes longer than running them. A step's launch sequence is the same from step to step as long
as the plan, the shapes and the patch index are the same, so it is captured once and replayed.

What makes this safe here: every buffer the exchange kernels use lives at a fixed address in the peer heap
(named allocations), barrier epochs and point-to-point sequence numbers are kept in device memory and advanced by
the kernels themselves, and the attention wrapper's scratch comes from the graph's private pool. A plan switch
resets the heap, so graphs are keyed by the plan epoch and dropped when it changes.

The first call with a key runs the step eagerly and returns that result: it doubles as the warm-up every capture
needs (lazy set-up, heap buffers of that shape, library workspaces), so no step is executed only to be thrown
away, and a key that never comes back costs nothing extra. The second call captures and replays. All ranks of a
plan must call run() with the same key sequence (they do: the pipelines are SPMD).

Captures go through CUDAGraph.capture_begin / capture_end on a side stream with one memory pool shared by all
graphs of the cache: the torch.cuda.graph context manager would synchronise the device, run the garbage
collector and empty the allocator cache on every capture, which costs more than the step it captures when every
request brings a new text length. Sharing the pool is safe because the graphs of a cache never run concurrently
and their static inputs and outputs stay referenced (only dead temporaries are reused between graphs).
"""
from typing import Callable, Dict, Hashable, Optional, Tuple

import torch

from ..core.distributed import parallel_state as ps


class StepGraphCache:
    def __init__(self, max_entries: int = 32):
        # key -> None (seen once, ran eagerly) or (graph, static inputs, static output)
        self._entries: Dict[Hashable, Optional[Tuple[torch.cuda.CUDAGraph, list, object]]] = {}
        self._epoch = -1
        self.max_entries = max_entries
        self.captures = 0
        self.replays = 0
        self._pool = None

    def clear(self):
        self._entries.clear()
        self._pool = None  # a pool whose graphs are all gone must not be captured into again

    def run(self, key: Hashable, fn: Callable, *inputs):
        """fn(*inputs): eagerly on the first use of `key`, through a CUDA graph captured on its second use from
        then on. Tensor inputs are copied into the graph's static input buffers; a replayed result is the graph's
        static output (valid until the next run() with the same key). Non-tensor inputs must be part of `key`."""
        epoch = ps.get_parallel_groups().plan_epoch
        if epoch != self._epoch:
            self.clear()
            self._epoch = epoch
        ent = self._entries.get(key, False)
        if ent is False:
            # first use: the eager step is the warm-up; remember that the key has been seen
            if len(self._entries) >= self.max_entries:
                self._entries.pop(next(iter(self._entries)))
            self._entries[key] = None
            return fn(*inputs)
        if ent is None:
            dev = next(x.device for x in inputs if isinstance(x, torch.Tensor))
            static = [x.clone() if isinstance(x, torch.Tensor) else x for x in inputs]
            cur = torch.cuda.current_stream(dev)
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                if self._pool is None or not any(e is not None for e in self._entries.values()):
                    # no live graph holds the pool any more (all evicted): it must not be captured into again
                    self._pool = torch.cuda.graph_pool_handle()
                graph = torch.cuda.CUDAGraph()
                graph.capture_begin(pool=self._pool)
                try:
                    out = fn(*static)
                finally:
                    graph.capture_end()
            cur.wait_stream(side)
            ent = self._entries[key] = (graph, static, out)
            self.captures += 1
        else:
            graph, static, out = ent
            for dst, src in zip(static, inputs):
                if isinstance(dst, torch.Tensor) and dst.data_ptr() != src.data_ptr():
                    dst.copy_(src, non_blocking=True)
        ent[0].replay()
        self.replays += 1
        return ent[2]

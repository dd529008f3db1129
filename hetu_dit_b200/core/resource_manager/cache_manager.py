"""Stale-KV cache of PipeFusion.

Interface of the reference's CacheManager
(hetu_dit/core/resource_manager/cache_manager.py:38-254): register_cache_entry,
update_and_get_kv_cache(new_kv=[k, v], layer, slice_dim, layer_type) -> (k, v),
get_cache_manager, reset_cache_manager.

Layout kept from the reference: one buffer per attention layer holding
[K || V] concatenated on the last dim; the returned K and V are the two halves
of that buffer (views). What changes is how it is filled: the reference
materialises torch.cat([k, v], -1) for every call, assigns the slice and later
makes the halves contiguous again; here one scatter kernel writes the fresh K
and V rows straight into their place in the stale buffer and attention reads
the halves through strided TMA descriptors.
"""
from typing import Any, Dict, List, Optional, Tuple, Union

import torch

from ... import kernels
from ..distributed import parallel_state as ps
from ..distributed.runtime_state import get_runtime_state, runtime_state_is_initialized


class CacheEntry:
    def __init__(self, cache_type: str, num_cache_tensors: int = 1):
        self.cache_type = cache_type
        self.tensors: List[Optional[torch.Tensor]] = [None] * num_cache_tensors


class CacheManager:
    supported_layer = ["attn"]
    supported_cache_type = ["naive_cache", "sequence_parallel_attn_cache"]

    def __init__(self):
        self.cache: Dict[Tuple[str, Any], CacheEntry] = {}

    def register_cache_entry(self, layer, layer_type: str, cache_type: str = "naive_cache"):
        if layer_type not in self.supported_layer:
            raise ValueError(
                f"Layer type: {layer_type} is not supported. Supported layer type: {self.supported_layer}")
        if cache_type not in self.supported_cache_type:
            raise ValueError(
                f"Cache type: {cache_type} is not supported. Supported cache type: {self.supported_cache_type}")
        self.cache[layer_type, layer] = CacheEntry(cache_type)

    # ------------------------------------------------------------------------------------------
    def update_and_get_kv_cache(self, new_kv: Union[torch.Tensor, List[torch.Tensor]], layer: Any, slice_dim: int = 1,
                                layer_type: str = "attn", custom_get_kv=None, **kwargs):
        if custom_get_kv is not None:
            packed = torch.cat(new_kv, dim=-1) if isinstance(new_kv, (list, tuple)) else new_kv
            return custom_get_kv(self, packed, layer, slice_dim, layer_type, **kwargs)
        entry = self.cache[layer_type, layer]
        as_list = isinstance(new_kv, (list, tuple))
        if as_list:
            k, v = new_kv
        else:
            k, v = torch.chunk(new_kv, 2, dim=-1)
        if entry.cache_type == "naive_cache":
            scale = 1
        else:
            scale = ps.get_ulysses_parallel_world_size()
        kv = self._update(entry, k, v, slice_dim, scale, sequence_parallel=entry.cache_type != "naive_cache")
        if kv is None:
            # nothing is cached in this mode (single patch): the fresh tensors are the answer
            return (k, v) if as_list else new_kv
        return torch.chunk(kv, 2, dim=-1) if as_list else kv

    def _update(self, entry: CacheEntry, k: torch.Tensor, v: torch.Tensor, slice_dim: int, scale: int,
                sequence_parallel: bool) -> Optional[torch.Tensor]:
        if slice_dim < 0:
            slice_dim += k.dim()
        if not runtime_state_is_initialized() or get_runtime_state().num_pipeline_patch == 1:
            entry.tensors[0] = None
            return None
        rt = get_runtime_state()
        if not rt.patch_mode:
            # warm-up step: the whole sequence is fresh; (re)build the stale buffer from it. For the
            # sequence-parallel cache the reference re-concatenates per-rank chunks rank-major,
            # patch-minor (cache_manager.py:172-183), which is the order they already have.
            shape = list(k.shape)
            shape[-1] *= 2
            buf = entry.tensors[0]
            if buf is None or list(buf.shape) != shape or buf.dtype != k.dtype or buf.device != k.device:
                buf = torch.empty(shape, dtype=k.dtype, device=k.device)
                entry.tensors[0] = buf
            self._scatter(buf, k, v, slice_dim, 0)
            return buf
        buf = entry.tensors[0]
        if buf is None:
            raise RuntimeError("patch-mode KV update before any warm-up step filled the stale buffer")
        starts = rt.pp_patches_token_start_idx_local
        p = rt.pipeline_patch_idx
        start, end = scale * starts[p], scale * starts[p + 1]
        if end - start != k.shape[slice_dim]:
            raise ValueError(
                f"patch {p} covers tokens [{start}, {end}) but the fresh K/V holds {k.shape[slice_dim]} tokens")
        self._scatter(buf, k, v, slice_dim, start)
        return buf

    @staticmethod
    def _scatter(buf: torch.Tensor, k: torch.Tensor, v: torch.Tensor, slice_dim: int, start: int):
        """buf[..., start:start+n, ..., :R] = k and buf[..., start:start+n, ..., R:] = v along `slice_dim`,
        R being the size of the last dim (the halves interleave per row of the last dim, exactly
        as torch.cat([k, v], dim=-1) lays them out)."""
        lead = 1
        for s in k.shape[:slice_dim]:
            lead *= s
        n = k.shape[slice_dim]
        mid = 1
        for s in k.shape[slice_dim + 1:-1]:
            mid *= s
        row = k.shape[-1] if slice_dim != k.dim() - 1 else 1
        if slice_dim == k.dim() - 1:
            raise ValueError("the K/V cache cannot be sliced along the last dimension")
        if not k.is_contiguous():
            k = k.contiguous()
        if not v.is_contiguous():
            v = v.contiguous()
        total = buf.shape[slice_dim]
        kernels.kv_scatter(buf.view(lead, total * mid, 2 * row), k.view(lead, n * mid, row), v.view(lead, n * mid, row),
                           start * mid)

    def _reset_cache(self):
        """Plan switch / new request shape: every stale buffer is dropped (cache_manager.py:233-238)."""
        self.cache = {}


_CACHE_MGR = CacheManager()


def get_cache_manager() -> CacheManager:
    return _CACHE_MGR


def reset_cache_manager():
    _CACHE_MGR._reset_cache()

"""Plan arithmetic shared by the worker and the block cache.

Mirrors the reference's hetu_dit/utils.py: get_gpu_metadata (:788-828) and the
round()-based range_to_indices of the `base` adjust strategy (:437-441).
"""
from typing import Dict, Tuple


def get_gpu_metadata(pipeline_parallel_rank: int, pipeline_parallel_world_size: int, tensor_model_parallel_rank: int,
                     tensor_model_parallel_world_size: int) -> Dict[str, Tuple[float, float]]:
    """Fractional [start, end) ranges of the blocks (pipeline) and of every split Linear (tensor) a rank owns."""
    t = 1.0 / tensor_model_parallel_world_size
    t0 = tensor_model_parallel_rank * t
    p = 1.0 / pipeline_parallel_world_size
    p0 = pipeline_parallel_rank * p
    return {"tensor_parallel": (t0, t0 + t), "pipeline_parallel": (p0, p0 + p)}


def range_to_indices(rng, total_size):
    start_prop, end_prop = rng
    return round(start_prop * total_size), round(end_prop * total_size)

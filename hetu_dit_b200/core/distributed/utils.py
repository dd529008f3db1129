"""Rank arithmetic for orthogonal parallel axes.

Mirrors the interface of the reference's hetu_dit/core/distributed/utils.py
(generate_masked_orthogonal_rank_groups :4-110, RankGenerator :113-188): a
global rank is a mixed-radix number whose digits are the per-axis ranks in the
order "tp-sp-pp-cfg-dp" (tp fastest).
"""
from typing import List, Sequence


def _digits_to_rank(index: int, axes) -> int:
    """Spread `index` (mixed radix over the sizes in `axes`) onto the axes' global strides."""
    total = 0
    for size, stride in axes:
        total += (index % size) * stride
        index //= size
    return total


def generate_masked_orthogonal_rank_groups(world_size: int, parallel_size: Sequence[int],
                                           mask: Sequence[bool]) -> List[List[int]]:
    """All groups whose members differ exactly in the axes selected by `mask`."""
    strides, acc = [], 1
    for s in parallel_size:
        strides.append(acc)
        acc *= s
    inside = [(s, st) for s, st, m in zip(parallel_size, strides, mask) if m]
    outside = [(s, st) for s, st, m in zip(parallel_size, strides, mask) if not m]
    group_size = 1
    for s, _ in inside:
        group_size *= s
    return [[_digits_to_rank(r, inside) + _digits_to_rank(g, outside) for r in range(group_size)]
            for g in range(world_size // group_size)]


class RankGenerator:
    AXES = ("tp", "sp", "pp", "cfg", "dp")

    def __init__(self, tp: int, sp: int, pp: int, cfg: int, dp: int, order: str, rank_offset: int = 0) -> None:
        self.tp, self.sp, self.pp, self.cfg, self.dp = tp, sp, pp, cfg, dp
        self.rank_offset = rank_offset
        self.world_size = tp * sp * pp * cfg * dp
        self.name_to_size = dict(zip(self.AXES, (tp, sp, pp, cfg, dp)))
        tokens = order.lower().split("-")
        for name in self.AXES:
            if name not in tokens:
                if self.name_to_size[name] != 1:
                    raise RuntimeError(
                        f"The size of ({name}) is ({self.name_to_size[name]}), but you haven't specified the order ({order}).")
                tokens.append(name)
        self.order = "-".join(tokens)
        self.ordered_size = [self.name_to_size[t] for t in tokens]

    def get_mask(self, order: str, token: str) -> List[bool]:
        wanted = set(token.split("-"))
        return [t in wanted for t in order.split("-")]

    def get_ranks(self, token: str) -> List[List[int]]:
        """Rank groups of one axis ("sp") or a product of axes ("tp-sp")."""
        groups = generate_masked_orthogonal_rank_groups(self.world_size, self.ordered_size,
                                                        self.get_mask(self.order, token))
        if self.rank_offset:
            groups = [[r + self.rank_offset for r in g] for g in groups]
        return groups

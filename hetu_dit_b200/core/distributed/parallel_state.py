"""Which ranks form the world / TP / SP (Ulysses x ring) / PP / CFG / DP groups of the active plan.

Interface of the reference's hetu_dit/core/distributed/parallel_state.py: the
getters (:39-227), initialize_model_parallel (:357), set_seq_parallel_pg (:642)
and ParallelGroups with its set_activate_* switches (:752-1534). The reference
pre-creates an NCCL communicator for every subset and partition of the 8 ranks
of a node so that a plan switch is a dictionary lookup; here a group is just a
rank list over the node's symmetric peer heap, so "activation" is arithmetic.

Rank order inside a plan is "tp-sp-pp-cfg-dp" (tp fastest); inside the SP axis
Ulysses groups are consecutive ranks and ring groups have stride `ulysses`.
A plan may sit on any sorted subset of the node's ranks: position i of the
sorted list plays local rank i (worker.py:507 `rank_map`).
"""
from itertools import combinations, count
from typing import Dict, List, Optional, Sequence, Tuple

from .peer import PeerGroup, PeerHeap
from .utils import RankGenerator


class _ProcessGroupSlots:
    """Stand-in for yunchang.globals.PROCESS_GROUP, which the attention operators read on
    every forward (hybrid/attn_layer.py:89-90)."""
    ULYSSES_PG: Optional[PeerGroup] = None
    RING_PG: Optional[PeerGroup] = None


PROCESS_GROUP = _ProcessGroupSlots
_PLAN_EPOCHS = count(1)  # process-wide, so that an epoch value is never seen twice


def seq_parallel_rank_lists(sp_ulysses_degree: int, sp_ring_degree: int, world_size: int, ranks: Sequence[int],
                            use_ulysses_low: bool = True) -> Tuple[List[List[int]], List[List[int]]]:
    """Rank lists set_seq_parallel_pg (parallel_state.py:642-749) would create, in creation order."""
    sp = sp_ulysses_degree * sp_ring_degree
    assert world_size % sp == 0, f"world_size {world_size} % sp_degree {sp} == 0"
    lut = sorted(ranks)
    ulysses_groups, ring_groups = [], []
    for base in range(0, world_size, sp):
        if use_ulysses_low:
            ulysses_groups += [[lut[base + i * sp_ulysses_degree + j] for j in range(sp_ulysses_degree)]
                               for i in range(sp_ring_degree)]
            ring_groups += [[lut[base + i + j * sp_ulysses_degree] for j in range(sp_ring_degree)]
                            for i in range(sp_ulysses_degree)]
        else:
            ring_groups += [[lut[base + i * sp_ring_degree + j] for j in range(sp_ring_degree)]
                            for i in range(sp_ulysses_degree)]
            ulysses_groups += [[lut[base + i + j * sp_ring_degree] for j in range(sp_ulysses_degree)]
                               for i in range(sp_ring_degree)]
    return ulysses_groups, ring_groups


def set_seq_parallel_pg(sp_ulysses_degree, sp_ring_degree, rank, world_size, ranks: List[int], use_ulysses_low=True,
                        is_serving=False, comm_pools=None, heap: Optional[PeerHeap] = None):
    """Returns (ulysses_pg, ring_pg) of `rank` as PeerGroups."""
    ug, rg = seq_parallel_rank_lists(sp_ulysses_degree, sp_ring_degree, world_size, ranks, use_ulysses_low)
    mine_u = next(g for g in ug if rank in g)
    mine_r = next(g for g in rg if rank in g)
    return PeerGroup(mine_u, rank, heap), PeerGroup(mine_r, rank, heap)


class SequenceParallelGroup(PeerGroup):
    """SP group with its Ulysses and ring sub-groups (group_coordinator.py:1068-1105)."""

    def __init__(self, ranks, my_global_rank, heap, ulysses_group: PeerGroup, ring_group: PeerGroup):
        super().__init__(ranks, my_global_rank, heap)
        self.ulysses_group, self.ring_group = ulysses_group, ring_group
        self.ulysses_world_size, self.ulysses_rank = ulysses_group.world_size, ulysses_group.rank_in_group
        self.ring_world_size, self.ring_rank = ring_group.world_size, ring_group.rank_in_group


class ParallelGroups:
    valid_degrees = [1, 2, 4, 8]

    def __init__(self, rank: int, world_size: int, heap: Optional[PeerHeap] = None, gpus_per_node: int = 8):
        self.rank, self.world_size, self.heap = rank, world_size, heap
        self.gpus_per_node = gpus_per_node
        self.rank_map: List[int] = list(range(world_size))
        self.degrees: Dict[str, int] = dict(tp=1, ulysses=1, ring=1, pp=1, cfg=1, dp=1)
        self._groups: Dict[str, PeerGroup] = {}
        self._pp_coordinator = None
        self.plan_epoch = next(_PLAN_EPOCHS)  # new value whenever a group is re-bound: captured CUDA graphs of older plans are void
        self.activate_plan(list(range(world_size)) if world_size == 1 else [rank])

    def void_captured_graphs(self):
        """New plan epoch without a new plan: addresses that captured CUDA graphs hold are no longer valid."""
        self.plan_epoch = next(_PLAN_EPOCHS)

    # -- enumeration the reference uses to size its communicator pool -------------------
    def _generate_rank_combinations(self, world_size: int, base_num: int = 0) -> List[List[int]]:
        out = []
        for degree in self.valid_degrees:
            if degree <= world_size:
                out += [[r + base_num for r in c] for c in combinations(range(world_size), degree)]
        return out

    def _generate_group_ranks(self, ranks: List[int]) -> List[List[List[int]]]:
        """Every way to cut `ranks` into equal groups of a power-of-two size."""
        def cut(rs, size):
            if len(rs) == size:
                return [[list(rs)]]
            res = []
            for others in combinations(rs[1:], size - 1):
                head = [rs[0], *others]
                rest = [r for r in rs if r not in head]
                res += [[head] + tail for tail in cut(rest, size)]
            return res

        n = len(ranks)
        if n == 1:
            return [[list(ranks)]]
        out, size = [], 1
        while size <= n:
            if n % size == 0:
                out += cut(list(ranks), size)
            size <<= 1
        return out

    # -- plan activation ----------------------------------------------------------------
    def activate_plan(self, ranks: Sequence[int], tp: int = 1, ulysses: int = 1, ring: int = 1, pp: int = 1,
                      cfg: int = 1, dp: int = 1):
        """Everything switch_parallel_env does to the groups (worker.py:480-586) in one call."""
        lut = sorted(ranks)
        n = len(lut)
        sp = ulysses * ring
        self.plan_epoch = next(_PLAN_EPOCHS)
        if tp * sp * pp * cfg * dp != n:
            raise ValueError(f"degrees tp={tp} sp={sp} pp={pp} cfg={cfg} dp={dp} do not multiply to {n} ranks")
        if self.rank not in lut:
            raise ValueError(f"rank {self.rank} is not part of the plan {lut}")
        self.rank_map = lut
        self.degrees = dict(tp=tp, ulysses=ulysses, ring=ring, pp=pp, cfg=cfg, dp=dp)
        gen = RankGenerator(tp, sp, pp, cfg, dp, "tp-sp-pp-cfg-dp")
        self._groups = {"world": PeerGroup(lut, self.rank, self.heap)}
        for axis in ("tp", "sp", "pp", "cfg", "dp"):
            for local in gen.get_ranks(axis):
                members = [lut[i] for i in local]
                if self.rank in members:
                    self._groups[axis] = PeerGroup(members, self.rank, self.heap)
        sp_ranks = self._groups["sp"].ranks
        upg, rpg = set_seq_parallel_pg(ulysses, ring, self.rank, len(sp_ranks), sp_ranks, heap=self.heap)
        self._groups["sp"] = SequenceParallelGroup(sp_ranks, self.rank, self.heap, upg, rpg)
        PROCESS_GROUP.ULYSSES_PG, PROCESS_GROUP.RING_PG = upg, rpg
        self._pp_coordinator = None

    # reference-named switches (parallel_state.py:977-1124), called by Worker.switch_parallel_env the way the
    # reference calls them: set_activate_<axis>_group(degree, ranks, group_ranks[, ...]) where `ranks` are the
    # plan's global ranks and `group_ranks` the partition of them along that axis; this rank's group is the
    # member list that contains it. The old one-argument forms (just this rank's member list) still work.
    def _mine(self, ranks, group_ranks):
        if group_ranks is None:
            return list(ranks)
        for g in group_ranks:
            if self.rank in g:
                return list(g)
        raise ValueError(f"rank {self.rank} is in none of the groups {group_ranks}")

    def set_activate_world_group(self, degree=None, ranks=None, group_ranks=None):
        if ranks is None:            # one-argument form: set_activate_world_group(ranks)
            degree, ranks = None, degree
        self.plan_epoch = next(_PLAN_EPOCHS)
        self.rank_map = sorted(ranks)
        self._groups["world"] = PeerGroup(self.rank_map, self.rank, self.heap)
        self.activate_world_groups = [list(g) for g in (group_ranks or [self.rank_map])]

    def set_activate_sp_group(self, degree=None, ranks=None, group_ranks=None, ulysses_degree=1, ring_degree=1):
        if not isinstance(degree, int) or ranks is None or isinstance(ranks, int):
            # old form: set_activate_sp_group(member_ranks, ulysses_degree, ring_degree)
            members, ulysses_degree, ring_degree = list(degree), ranks, group_ranks
        else:
            members = self._mine(ranks, group_ranks)
        self.plan_epoch = next(_PLAN_EPOCHS)
        upg, rpg = set_seq_parallel_pg(ulysses_degree, ring_degree, self.rank, len(members), list(members),
                                       heap=self.heap)
        self._groups["sp"] = SequenceParallelGroup(sorted(members), self.rank, self.heap, upg, rpg)
        self.degrees["ulysses"], self.degrees["ring"] = ulysses_degree, ring_degree
        PROCESS_GROUP.ULYSSES_PG, PROCESS_GROUP.RING_PG = upg, rpg

    def _set_axis(self, axis: str, degree, ranks, group_ranks):
        if ranks is None:            # one-argument form: the member list itself
            members = list(degree)
        else:
            members = self._mine(ranks, group_ranks)
        self.plan_epoch = next(_PLAN_EPOCHS)
        self._groups[axis] = PeerGroup(members, self.rank, self.heap)
        self.degrees[axis] = len(members)
        if axis == "pp":
            self._pp_coordinator = None

    def set_activate_tp_group(self, degree=None, ranks=None, group_ranks=None):
        self._set_axis("tp", degree, ranks, group_ranks)

    def set_activate_pp_group(self, degree=None, ranks=None, group_ranks=None):
        self._set_axis("pp", degree, ranks, group_ranks)

    def set_activate_cfg_group(self, degree=None, ranks=None, group_ranks=None):
        self._set_axis("cfg", degree, ranks, group_ranks)

    def set_activate_dp_group(self, degree=None, ranks=None, group_ranks=None):
        self._set_axis("dp", degree, ranks, group_ranks)

    def group(self, axis: str) -> PeerGroup:
        return self._groups[axis]

    def pp_coordinator(self):
        if self._pp_coordinator is None:
            from .group_coordinator import PipelineGroupCoordinator
            self._pp_coordinator = PipelineGroupCoordinator(self._groups["pp"])
        return self._pp_coordinator


_PARALLEL_GROUPS: Optional[ParallelGroups] = None


def init_distributed_environment(rank: int = 0, world_size: int = 1, heap: Optional[PeerHeap] = None) -> ParallelGroups:
    global _PARALLEL_GROUPS
    _PARALLEL_GROUPS = ParallelGroups(rank, world_size, heap)
    return _PARALLEL_GROUPS


def initialize_model_parallel(data_parallel_degree: int = 1, classifier_free_guidance_degree: int = 1,
                              sequence_parallel_degree: int = 1, ulysses_degree: int = 1, ring_degree: int = 1,
                              tensor_parallel_degree: int = 1, pipeline_parallel_degree: int = 1,
                              ranks: Optional[Sequence[int]] = None):
    """Static (non-serving) set-up over the whole world (parallel_state.py:357-505)."""
    pg = get_parallel_groups()
    if sequence_parallel_degree != ulysses_degree * ring_degree:
        raise ValueError("sequence_parallel_degree must equal ulysses_degree * ring_degree")
    pg.activate_plan(list(ranks) if ranks is not None else list(range(pg.world_size)), tp=tensor_parallel_degree,
                     ulysses=ulysses_degree, ring=ring_degree, pp=pipeline_parallel_degree,
                     cfg=classifier_free_guidance_degree, dp=data_parallel_degree)


def model_parallel_is_initialized() -> bool:
    return _PARALLEL_GROUPS is not None


def get_parallel_groups() -> ParallelGroups:
    global _PARALLEL_GROUPS
    if _PARALLEL_GROUPS is None:
        _PARALLEL_GROUPS = ParallelGroups(0, 1, None)
    return _PARALLEL_GROUPS


def destroy_model_parallel():
    global _PARALLEL_GROUPS
    _PARALLEL_GROUPS = None
    PROCESS_GROUP.ULYSSES_PG = PROCESS_GROUP.RING_PG = None


def get_world_group() -> PeerGroup:
    return get_parallel_groups().group("world")


def get_tp_group() -> PeerGroup:
    return get_parallel_groups().group("tp")


def get_sp_group() -> SequenceParallelGroup:
    return get_parallel_groups().group("sp")


def get_pp_group():
    """The PipeFusion patch coordinator of the active plan."""
    return get_parallel_groups().pp_coordinator()


def get_pp_group_or_none():
    return _PARALLEL_GROUPS.pp_coordinator() if _PARALLEL_GROUPS is not None else None


def get_cfg_group() -> PeerGroup:
    return get_parallel_groups().group("cfg")


def get_dp_group() -> PeerGroup:
    return get_parallel_groups().group("dp")


def get_world_group_world_size() -> int:
    return get_world_group().world_size


def get_world_group_rank() -> int:
    return get_world_group().rank_in_group


def get_tensor_model_parallel_world_size() -> int:
    return get_tp_group().world_size


def get_tensor_model_parallel_rank() -> int:
    return get_tp_group().rank_in_group


def get_sequence_parallel_world_size() -> int:
    return get_sp_group().world_size


def get_sequence_parallel_rank() -> int:
    return get_sp_group().rank_in_group


def get_ulysses_parallel_world_size() -> int:
    return get_sp_group().ulysses_world_size


def get_ulysses_parallel_rank() -> int:
    return get_sp_group().ulysses_rank


def get_ring_parallel_world_size() -> int:
    return get_sp_group().ring_world_size


def get_ring_parallel_rank() -> int:
    return get_sp_group().ring_rank


def get_pipeline_parallel_world_size() -> int:
    return get_parallel_groups().group("pp").world_size


def get_pipeline_parallel_rank() -> int:
    return get_parallel_groups().group("pp").rank_in_group


def is_pipeline_first_stage() -> bool:
    return get_pipeline_parallel_rank() == 0


def is_pipeline_last_stage() -> bool:
    return get_pipeline_parallel_rank() == get_pipeline_parallel_world_size() - 1


def get_classifier_free_guidance_world_size() -> int:
    return get_cfg_group().world_size


def get_classifier_free_guidance_rank() -> int:
    return get_cfg_group().rank_in_group


def get_data_parallel_world_size() -> int:
    return get_dp_group().world_size


def get_data_parallel_rank() -> int:
    return get_dp_group().rank_in_group

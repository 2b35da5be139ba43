"""Process mesh and process groups.

``world = dp * pp * cp * tp`` with TP innermost: ``rank = ((dp*PP + pp)*CP + cp)*TP + tp``. EP is not a mesh
factor: expert-parallel groups re-use ranks of TP / CP / DP (in that priority, as allowed by the plan), and two
derived axes exist: DCP (= DP x CP, the shard group of non-expert ZeRO state) and EREP (ranks holding replicas
of the same experts). Semantics follow the reference's ``runtime/mesh.py:22-410``; here every family of groups
is produced by one generic enumerator over mesh coordinates instead of one hand-written loop nest per regime.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from enum import Enum

import torch.distributed as dist

from maltos_b200.parallel.plan import ParallelPlan


class MeshAxis(str, Enum):
    DP = "dp"
    TP = "tp"
    PP = "pp"
    CP = "cp"
    EP = "ep"
    DCP = "dcp"
    EREP = "erep"


@dataclass(frozen=True)
class MeshConfig:
    dp: int = 1
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1

    def __post_init__(self) -> None:
        for name in ("dp", "tp", "pp", "cp", "ep"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1, got {getattr(self, name)}")

    @property
    def world_size(self) -> int:
        return self.dp * self.tp * self.pp * self.cp

    def rank_coordinates(self, rank_id: int) -> tuple[int, int, int, int]:
        """rank -> (dp, pp, cp, tp)."""
        if not 0 <= rank_id < self.world_size:
            raise ValueError(f"rank_id must be in [0, {self.world_size}), got {rank_id}")
        rest, tp = divmod(rank_id, self.tp)
        rest, cp = divmod(rest, self.cp)
        dp, pp = divmod(rest, self.pp)
        return dp, pp, cp, tp

    def rank_id(self, *, dp: int, pp: int, cp: int, tp: int) -> int:
        if not (0 <= dp < self.dp and 0 <= pp < self.pp and 0 <= cp < self.cp and 0 <= tp < self.tp):
            raise ValueError(f"invalid mesh coordinates: dp={dp}, pp={pp}, cp={cp}, tp={tp}")
        return ((dp * self.pp + pp) * self.cp + cp) * self.tp + tp

    def infer_checkpoint_rank(self, rank_id: int, *, plan: ParallelPlan, replicated_axes: set[MeshAxis]) -> int:
        """Rank that stores a tensor replicated along ``replicated_axes``: index 0 of every such axis."""
        dp, pp, cp, tp = self.rank_coordinates(rank_id)
        axes = set(replicated_axes)
        if axes & {MeshAxis.DP, MeshAxis.DCP}:
            dp = 0
        if axes & {MeshAxis.CP, MeshAxis.DCP}:
            cp = 0
        if MeshAxis.PP in axes:
            pp = 0
        if MeshAxis.TP in axes:
            tp = 0
        if MeshAxis.EREP in axes and self.ep > 1:
            dp, cp, tp = _first_expert_replica(self, plan, dp, cp, tp)
        return self.rank_id(dp=dp, pp=pp, cp=cp, tp=tp)


# --------------------------------------------------------------------------- expert-parallel geometry
def _ep_span(mesh: MeshConfig, reuse_tp: bool, reuse_cp: bool) -> list[tuple[str, int]]:
    """Axes an EP group may span, innermost first."""
    span = []
    if reuse_tp:
        span.append(("tp", mesh.tp))
    if reuse_cp:
        span.append(("cp", mesh.cp))
    span.append(("dp", mesh.dp))
    return span


def _ep_flat_index(mesh: MeshConfig, reuse_tp: bool, reuse_cp: bool, dp: int, cp: int, tp: int) -> int:
    coord = {"dp": dp, "cp": cp, "tp": tp}
    flat, mult = 0, 1
    for name, size in _ep_span(mesh, reuse_tp, reuse_cp):
        flat += coord[name] * mult
        mult *= size
    return flat


def _ep_unflatten(mesh: MeshConfig, reuse_tp: bool, reuse_cp: bool, flat: int, dp: int, cp: int, tp: int) -> tuple[int, int, int]:
    coord = {"dp": dp, "cp": cp, "tp": tp}
    for name, size in _ep_span(mesh, reuse_tp, reuse_cp):
        flat, coord[name] = divmod(flat, size)
    return coord["dp"], coord["cp"], coord["tp"]


def validate_expert_parallel(mesh: MeshConfig, *, reuse_tp: bool, reuse_cp: bool) -> None:
    """EP must tile the spanned axes: fill the innermost axis completely before touching the next one."""
    ep = mesh.ep
    if ep == 1:
        return
    span = _ep_span(mesh, reuse_tp, reuse_cp)
    label = "*".join(n.upper() for n, _ in span)
    space = 1
    for _, size in span:
        space *= size
    if ep > space:
        raise ValueError(f"EP must be <= {label}={space}, got ep={ep}")
    if space % ep:
        raise ValueError(f"{label}={space} must be divisible by EP={ep}")
    covered = 1
    for name, size in span:
        if ep <= covered * size:
            need = ep // covered if ep % covered == 0 else None
            if need is None:
                raise ValueError(f"EP={ep} must be divisible by the product of the inner axes ({covered})")
            if size % need:
                raise ValueError(f"{name.upper()}={size} must be divisible by EP share {need} (ep={ep})")
            return
        if ep % (covered * size):
            raise ValueError(f"EP={ep} must be divisible by {covered * size} to span axis {name.upper()} fully")
        covered *= size


_validate_ep_for_plan = validate_expert_parallel  # name used by callers written against the reference


def _first_expert_replica(mesh: MeshConfig, plan: ParallelPlan, dp: int, cp: int, tp: int) -> tuple[int, int, int]:
    reuse_tp, reuse_cp = plan.reuse_tp_for_ep, plan.reuse_cp_for_ep
    local = _ep_flat_index(mesh, reuse_tp, reuse_cp, dp, cp, tp) % mesh.ep
    return _ep_unflatten(mesh, reuse_tp, reuse_cp, local, dp, cp, tp)


def enumerate_axis_groups(mesh: MeshConfig, plan: ParallelPlan) -> list[tuple[MeshAxis, list[int]]]:
    """Every process group of the mesh as (axis, global ranks), in the creation order all ranks must follow."""
    out: list[tuple[MeshAxis, list[int]]] = []
    DP, PP, CP, TP = range(mesh.dp), range(mesh.pp), range(mesh.cp), range(mesh.tp)
    rid = lambda d, p, c, t: mesh.rank_id(dp=d, pp=p, cp=c, tp=t)  # noqa: E731

    for d, p, c in itertools.product(DP, PP, CP):
        out.append((MeshAxis.TP, [rid(d, p, c, t) for t in TP]))
    if mesh.ep > 1:
        reuse_tp, reuse_cp = plan.reuse_tp_for_ep, plan.reuse_cp_for_ep
        fixed_t = [None] if reuse_tp else list(TP)
        fixed_c = [None] if reuse_cp else list(CP)
        for by_block in (True, False):  # True: EP groups (same block of ep consecutive flats); False: EREP groups
            axis = MeshAxis.EP if by_block else MeshAxis.EREP
            for ft, fc, p in itertools.product(fixed_t, fixed_c, PP):
                buckets: dict[int, list[int]] = {}
                for d, c, t in itertools.product(DP, CP, TP):
                    if (ft is not None and t != ft) or (fc is not None and c != fc):
                        continue
                    flat = _ep_flat_index(mesh, reuse_tp, reuse_cp, d, c, t)
                    key = flat // mesh.ep if by_block else flat % mesh.ep
                    buckets.setdefault(key, []).append(rid(d, p, c, t))
                for key in sorted(buckets):
                    out.append((axis, buckets[key]))
    for d, p, t in itertools.product(DP, PP, TP):
        out.append((MeshAxis.CP, [rid(d, p, c, t) for c in CP]))
    for d, c, t in itertools.product(DP, CP, TP):
        out.append((MeshAxis.PP, [rid(d, p, c, t) for p in PP]))
    for p, c, t in itertools.product(PP, CP, TP):
        out.append((MeshAxis.DP, [rid(d, p, c, t) for d in DP]))
    for p, t in itertools.product(PP, TP):
        out.append((MeshAxis.DCP, [rid(d, p, c, t) for d in DP for c in CP]))
    return out


@dataclass
class ProcessGroupManager:
    mesh: MeshConfig
    plan: ParallelPlan
    groups: dict[MeshAxis, "dist.ProcessGroup | None"] = field(default_factory=dict)
    group_ranks: dict[MeshAxis, list[int]] = field(default_factory=dict)

    @classmethod
    def from_plan(cls, plan: ParallelPlan, mesh: MeshConfig) -> "ProcessGroupManager":
        validate_expert_parallel(mesh, reuse_tp=plan.reuse_tp_for_ep, reuse_cp=plan.reuse_cp_for_ep)
        mgr = cls(mesh=mesh, plan=plan)
        mgr.initialize_groups()
        return mgr

    @property
    def world_size(self) -> int:
        return self.mesh.world_size

    def initialize_groups(self) -> None:
        self.groups = {axis: None for axis in MeshAxis}
        self.group_ranks = {}
        if not dist.is_initialized():
            return
        if dist.get_world_size() != self.mesh.world_size:
            raise ValueError(f"mesh world size {self.mesh.world_size} != distributed world size {dist.get_world_size()}")
        me = dist.get_rank()
        for axis, ranks in enumerate_axis_groups(self.mesh, self.plan):
            handle = dist.new_group(ranks)  # collective over the default group: every rank creates every group
            if me in ranks:
                self.group_ranks[axis] = ranks
                if len(ranks) > 1 or axis is MeshAxis.EP:
                    self.groups[axis] = handle

    def get_group(self, axis: MeshAxis):
        return self.groups.get(axis)

    def get_group_ranks(self, axis: MeshAxis) -> list[int]:
        return self.group_ranks.get(axis, [dist.get_rank() if dist.is_initialized() else 0])

    def close(self) -> None:
        if dist.is_initialized():
            done: set[int] = set()
            for handle in self.groups.values():
                if handle is None or id(handle) in done:
                    continue
                done.add(id(handle))
                from maltos_b200.ops import comm

                comm.release_context(handle)
                dist.destroy_process_group(handle)
        self.groups = {axis: None for axis in MeshAxis}

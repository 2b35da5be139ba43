"""Shared machinery of the data-parallel family (bucketed DDP, ZeRO-1/2/3, expert-gradient sync).

* ``ChainedWork``: a chain of asynchronous collectives fired back to back; between links the next collective is
  ordered after the previous one by a stream dependency (NCCL) or a blocking wait (gloo); persistent chains can be
  fired again every step (reference ``runtime/plugins/zero_common.py:16-81``).
* flat buckets, shard-group contexts (DCP for shared parameters with a ``x cp`` correction because AVG divides by
  ``dp*cp`` where ``/dp`` is wanted; EREP for experts), fp64 global-norm clipping with a non-finite guard.

On CUDA the bucket reduce-scatter, the cast/scale, the squared-norm partial and the AdamW update are one fused pass
over the shard (``maltos_b200.ops.comm`` + ``maltos_b200.ops.optim``); the torch.distributed path here is the gloo /
oracle implementation.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import ParamRole
from maltos_b200.utils.distributed import CompletedWork  # noqa: F401  (re-exported)


class ChainedWork:
    def __init__(self, parent: "ChainedWork | None", functor: Callable[[], object], *, blocks_by_stream: bool = True) -> None:
        self.parent = parent
        self.functor = functor
        self.blocks_by_stream = blocks_by_stream
        self.handle = None

    def fire(self) -> None:
        if self.parent is not None:
            # a persistent chain is replayed from its root on every fire; old handles describe the previous round
            self.parent.fire()
            if self.parent.blocks_by_stream:
                self.parent.handle.block_current_stream()
            else:
                self.parent.handle.wait()
        self.handle = self.functor()

    def wait(self) -> None:
        if self.handle is None:
            self.fire()
        self.handle.wait()


class LocalCopyWork(CompletedWork):
    """No collective needed (single-rank group): copy synchronously."""

    def __init__(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        dst.copy_(src)


class NarrowShardWork:
    """All-reduce of a full buffer standing in for a reduce-scatter: on wait, this rank's slice lands in ``local_grad``."""

    def __init__(self, work, grad_buffer, local_grad, shard_start: int, shard_end: int, *, accumulate: bool = False) -> None:
        self.work, self.grad_buffer, self.local_grad = work, grad_buffer, local_grad
        self.shard_start, self.shard_end, self.accumulate = shard_start, shard_end, accumulate

    def block_current_stream(self) -> None:
        self.work.block_current_stream()

    def wait(self) -> None:
        self.work.wait()
        piece = self.grad_buffer[self.shard_start:self.shard_end]
        if self.accumulate:
            self.local_grad.add_(piece)
        else:
            self.local_grad.copy_(piece)


def expert_erep_correction(*, tp: int, cp: int, ep: int, reuse_tp: bool, reuse_cp: bool) -> float:
    """Factor that turns AVG over EREP into the right reduction: EREP members that hold *different tokens* (EP placed
    inside TP/CP) must be summed, genuine data-parallel replicas averaged."""
    inner = (tp if reuse_tp else 1) * (cp if reuse_cp else 1)
    return float(inner // ep) if ep <= inner else 1.0


def expert_data_shards(*, tp: int, cp: int, ep: int, reuse_tp: bool, reuse_cp: bool) -> int:
    """How many different data-parallel shards feed one expert through the EP all-to-all. The global loss is the MEAN
    over data shards, and an expert accumulates the SUM of the gradients sent back by all of them, so expert
    gradients are divided by this number (tokens of TP/CP ranks inside the group belong to the same shard)."""
    inner = (tp if reuse_tp else 1) * (cp if reuse_cp else 1)
    return max(ep // inner, 1) if ep > inner else 1


def expert_token_copies(runtime) -> int:
    """How many times one token reaches an expert through the EP all-to-all. With tensor parallelism WITHOUT sequence
    parallelism the activations in front of the MoE layer are replicated over the TP ranks; when the expert group reuses those
    ranks, every one of them dispatches the same tokens, the expert sees each token ``tp`` times and its gradient comes out
    ``tp`` times too large (AdamW hides the factor, clipping and the reported norm do not). Expert gradients are divided by
    this number."""
    mesh, plan = runtime.mesh, runtime.plan
    if mesh.tp > 1 and mesh.ep > 1 and plan.reuse_tp_for_ep and runtime.has_plugin(PluginId.TP) and not runtime.has_plugin(PluginId.TP_SP):
        return mesh.tp
    return 1


def rearm_bucket_pending(num_params: int, *, grad_accum_end: bool) -> int:
    """Pending-hook count for a bucket at the start of a backward: only the window-closing micro-step may reach 0."""
    return num_params if grad_accum_end else 0


def build_param_buckets(params: list[nn.Parameter], bucket_byte_size: int) -> list[list[nn.Parameter]]:
    buckets: list[list[nn.Parameter]] = []
    cur: list[nn.Parameter] = []
    size = 0
    for p in params:
        nbytes = p.numel() * p.element_size()
        if cur and size + nbytes > bucket_byte_size:
            buckets.append(cur)
            cur, size = [], 0
        cur.append(p)
        size += nbytes
    if cur:
        buckets.append(cur)
    return buckets


@dataclass(frozen=True)
class GroupContext:
    group: "dist.ProcessGroup | None"
    world_size: int
    rank: int
    correction: float = 1.0   # multiply after AVG: world_size / wanted divisor

    @property
    def is_gloo(self) -> bool:
        return self.group is not None and dist.get_backend(self.group) == "gloo"

    @property
    def supports_async_overlap(self) -> bool:
        return self.group is not None and not self.is_gloo


def padded_len(numel: int, world: int) -> int:
    return (numel + world - 1) // world * world


def global_grad_norm(local_sq: torch.Tensor) -> torch.Tensor:
    """sqrt of the world-wide sum of ``local_sq`` (fp64 device scalar)."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(local_sq, op=dist.ReduceOp.SUM)
    return local_sq.sqrt()


class ZeroPluginBase(RuntimePlugin):
    def __init__(self, *, id: PluginId, name: str, owns_optimizer: bool, owns_model_state: bool = False,
                 runs_after: set[PluginId], bucket_mb_size: int = 25) -> None:
        super().__init__(id=id, name=name, owns_optimizer=owns_optimizer, owns_model_state=owns_model_state, runs_after=runs_after)
        self.bucket_byte_size = bucket_mb_size * 1024 * 1024
        self.dp_group = None
        self.world_size = 1
        self.rank = 0
        self.buckets: list = []
        self.optimizer = None
        self.scheduler = None
        self._chained_work_wrappers: list = []

    def optimizer_state_source_rank(self, rank_id: int) -> int:
        return rank_id

    def wrap_chained_work(self, wrap, *, role_filter: ParamRole | None = None) -> None:
        """Other plugins (CP, EP) append reduction links to the bucket chains created from now on."""
        self._chained_work_wrappers.append((wrap, role_filter))

    def _apply_chained_work_wrappers(self, work: ChainedWork, tensor: torch.Tensor, role: ParamRole) -> ChainedWork:
        for wrap, only in self._chained_work_wrappers:
            if only is None or only == role:
                work = wrap(work, tensor)
        return work

    def _group_context_for_role(self, role: ParamRole) -> GroupContext:
        rt = self.runtime
        mesh = rt.mesh
        if role == ParamRole.EXPERT:
            group = rt.get_group(MeshAxis.EREP)
            copies = expert_token_copies(rt)
            if group is None:
                shards = expert_data_shards(tp=mesh.tp, cp=mesh.cp, ep=mesh.ep, reuse_tp=rt.plan.reuse_tp_for_ep, reuse_cp=rt.plan.reuse_cp_for_ep)
                return GroupContext(None, 1, 0, correction=1.0 / (shards * copies))
            corr = expert_erep_correction(tp=mesh.tp, cp=mesh.cp, ep=mesh.ep, reuse_tp=rt.plan.reuse_tp_for_ep, reuse_cp=rt.plan.reuse_cp_for_ep)
            corr /= expert_data_shards(tp=mesh.tp, cp=mesh.cp, ep=mesh.ep, reuse_tp=rt.plan.reuse_tp_for_ep, reuse_cp=rt.plan.reuse_cp_for_ep) * copies
            return GroupContext(group, dist.get_world_size(group), dist.get_rank(group), correction=corr)
        group = rt.get_group(MeshAxis.DCP)
        if group is None:
            return GroupContext(self.dp_group, self.world_size, self.rank)
        return GroupContext(group, dist.get_world_size(group), dist.get_rank(group), correction=float(mesh.cp))

    def _padded_len(self, numel: int, world_size: int) -> int:
        return padded_len(numel, world_size)

    def _role_params(self, model: nn.Module, role: ParamRole) -> list[nn.Parameter]:
        rt = self.runtime
        seen: set[int] = set()
        out = []
        for p in model.parameters():
            if p.requires_grad and id(p) not in seen and rt.get_param_role(p) == role:
                seen.add(id(p))
                out.append(p)
        return out[::-1]

    def _build_param_buckets(self, params):
        return build_param_buckets(params, self.bucket_byte_size)

    # ---- clipping on local shards
    def _shard_replica_factor(self, param: nn.Parameter) -> int:
        """Replication of a SHARD of ``param``'s gradient: the ranks of the shard group (data x context parallel ranks for
        shared parameters, the expert replicas for expert parameters) hold different pieces, so replication along those axes
        does not count - only copies on other axes (unsharded weights under tensor parallelism) do. Counting the shard-group
        axes as well (the reference does) under-reports the global norm by sqrt(cp) or sqrt(expert replicas)."""
        rt = self.runtime
        if rt.get_param_role(param) == ParamRole.EXPERT:
            over = frozenset({MeshAxis.EREP, MeshAxis.DP, MeshAxis.CP, MeshAxis.DCP})
        else:
            over = frozenset({MeshAxis.DP, MeshAxis.CP, MeshAxis.DCP})
        return rt.grad_norm_replica_factor(param, sharded_over=over)

    def _bucket_local_sq(self, bucket) -> torch.Tensor:
        raise NotImplementedError

    def _maybe_clip_local_shards(self) -> None:
        rt = self.runtime
        max_norm = rt.grad_clip_max_norm
        if max_norm is None or not self.buckets:
            return
        grads = [b.local_param.grad for b in self.buckets if getattr(b.local_param, "grad", None) is not None]
        if not grads:
            return
        local_sq = torch.zeros((), dtype=torch.float64, device=grads[0].device)
        for b in self.buckets:
            local_sq.add_(self._bucket_local_sq(b))
        norm = float(global_grad_norm(local_sq).item())
        scaler = rt.state.scaler
        if scaler is not None:
            # fp16: the shards still carry the loss scale (the scaler divides it out inside its step), and an overflow is an
            # ordinary event - the scaler skips the step on every rank and backs the scale off; nothing to clip then
            if not math.isfinite(norm):
                rt.state.metadata["grad_norm"] = norm
                return
            norm /= float(scaler.get_scale())
        if not math.isfinite(norm):
            bad = []
            for b in self.buckets:
                g = getattr(b.local_param, "grad", None)
                if g is not None and not torch.isfinite(g).all():
                    bad.append(f"bucket={getattr(b, 'index', '?')} names={list(getattr(b, 'logical_names', ()))[:4]}")
            raise FloatingPointError("non-finite ZeRO gradient norm; refusing optimizer step to avoid inf * 0 -> NaN. "
                                     f"Affected local shards: {'; '.join(bad[:8]) or 'no local non-finite shard found'}")
        coef = float(max_norm) / (norm + 1e-6)
        if coef < 1.0:
            for g in grads:
                g.mul_(coef)
        rt.state.metadata["grad_norm"] = norm

    def collect_metrics(self) -> dict[str, float]:
        norm = self.runtime.state.metadata.get("grad_norm")
        max_norm = self.runtime.grad_clip_max_norm
        if norm is None or max_norm is None:
            return {}
        return {"grad_norm": float(norm), "max_norm": float(max_norm)}

"""ZeRO stage 1 and 2: optimizer state (and, for stage 2, gradients) sharded over the data-parallel group.

Parameters of one role (shared / expert), in reverse order, are packed into flat buckets padded to the shard-group
size; ``param.data`` become views of the flat data buffer and the optimizer owns one parameter per bucket = this
rank's ``1/N`` slice. When the last gradient of a bucket arrives on the window-closing micro-step its
reduce-scatter(AVG) starts, overlapped with the rest of backward; POST_BACKWARD waits, PRE_STEP clips on the shards,
POST_STEP all-gathers the updated slices back into the data buffer (reference ``runtime/plugins/zero1.py:98-299``).

Stage 2 keeps no full gradient buffer between micro-steps: a pooled buffer lives for one backward, its reduce-scatter
runs every micro-step and the result is *added* to the shard gradient (reference ``runtime/plugins/zero2.py:183-397``).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.runtime.buffer_allocator import BufferPolicy, acquire_buffer, release_buffer
from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.plugin import PluginId
from maltos_b200.runtime.types import ParamRole, RuntimePhase, SetupPhase
from maltos_b200.utils.distributed import all_gather_single, reduce_scatter_single
from maltos_b200.utils.profiling import span

from .zero_common import ChainedWork, CompletedWork, GroupContext, LocalCopyWork, ZeroPluginBase, padded_len


@dataclass
class FlatBucket:
    index: int
    role: ParamRole
    params: list[nn.Parameter]
    group_context: GroupContext
    data: torch.Tensor                   # flat padded parameter values (model dtype)
    offsets: list[int]
    total: int
    local_param: nn.Parameter = None     # this rank's slice, owned by the optimizer
    grad: torch.Tensor | None = None     # flat padded gradient buffer (stage 1: persistent, stage 2: per backward)
    grad_handle: object = None
    logical_names: list[str] = field(default_factory=list)
    pending: int = 0
    fired: bool = False
    work: ChainedWork | None = None
    shard_scratch: torch.Tensor | None = None

    @property
    def shard_numel(self) -> int:
        return self.data.numel() // self.group_context.world_size

    @property
    def shard_start(self) -> int:
        return self.group_context.rank * self.shard_numel

    @property
    def shard_end(self) -> int:
        return self.shard_start + self.shard_numel

    @property
    def param_shapes(self):
        return [tuple(p.shape) for p in self.params]

    @property
    def param_numels(self):
        return [p.numel() for p in self.params]


class Zero1Plugin(ZeroPluginBase):
    accumulate_on_shard = False     # stage 2 flips this

    def __init__(self, bucket_mb_size: int = 25, *, _id: PluginId = PluginId.ZERO1, _name: str = "zero1") -> None:
        super().__init__(id=_id, name=_name, owns_optimizer=True, bucket_mb_size=bucket_mb_size,
                         runs_after={PluginId.TP, PluginId.TP_SP, PluginId.PP, PluginId.EP, PluginId.CP})

    # ------------------------------------------------------------------ setup
    def bind(self, runtime) -> None:
        super().bind(runtime)
        self.dp_group = runtime.get_group(MeshAxis.DP)
        if runtime.mesh.dp * runtime.mesh.cp <= 1 and runtime.get_group(MeshAxis.EREP) is None:
            raise ValueError(f"{self.name} requires a data-parallel (dp x cp) group larger than 1")
        if self.dp_group is not None:
            self.world_size, self.rank = dist.get_world_size(self.dp_group), dist.get_rank(self.dp_group)

    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        if phase is SetupPhase.MATERIALIZE:
            self._build_buckets(model)
            locals_ = [b.local_param for b in self.buckets]
            self.optimizer = self.runtime.create_optimizer(locals_)
            self.scheduler = self.runtime.create_scheduler(self.optimizer)
        elif phase is SetupPhase.FINALIZE:
            names = {id(p): n for n, p in model.named_parameters()}
            for b in self.buckets:
                b.logical_names = [names[id(p)] for p in b.params]
                for p in b.params:
                    p.register_post_accumulate_grad_hook(self._make_hook(b))
        return model

    def _build_buckets(self, model: nn.Module) -> None:
        self.buckets = []
        for role in (ParamRole.SHARED, ParamRole.EXPERT):
            params = self._role_params(model, role)
            if not params:
                continue
            gc = self._group_context_for_role(role)
            for group in self._build_param_buckets(params):
                total = sum(p.numel() for p in group)
                padded = padded_len(total, gc.world_size)
                data = torch.zeros(padded, dtype=group[0].dtype, device=group[0].device)
                offsets, at = [], 0
                with torch.no_grad():
                    for p in group:
                        offsets.append(at)
                        data[at:at + p.numel()].copy_(p.data.reshape(-1))
                        p.data = data[at:at + p.numel()].view(p.shape)
                        at += p.numel()
                bucket = FlatBucket(index=len(self.buckets), role=role, params=group, group_context=gc, data=data, offsets=offsets, total=total)
                bucket.local_param = nn.Parameter(data[bucket.shard_start:bucket.shard_end].detach().clone())
                if not self.accumulate_on_shard:
                    bucket.grad = torch.zeros_like(data)
                self.buckets.append(bucket)

    # ------------------------------------------------------------------ backward
    def _attach_grad_views(self, b: FlatBucket) -> None:
        base = b.grad.data_ptr()
        esz = b.grad.element_size()
        for p, at in zip(b.params, b.offsets):
            if p.grad is None or p.grad.data_ptr() != base + at * esz:
                p.grad = b.grad[at:at + p.numel()].view(p.shape)

    def _make_hook(self, b: FlatBucket):
        def hook(_param) -> None:
            b.pending -= 1
            if b.pending == 0:
                self._fire(b)

        return hook

    def _reduce_chain(self, b: FlatBucket) -> ChainedWork:
        gc = b.group_context
        if b.shard_scratch is None or b.shard_scratch.numel() != b.shard_numel:
            b.shard_scratch = torch.empty(b.shard_numel, dtype=b.grad.dtype, device=b.grad.device)
        dst = b.shard_scratch

        def reduce():
            if gc.group is None or gc.world_size == 1:
                if gc.correction != 1.0:
                    b.grad.mul_(gc.correction)
                return LocalCopyWork(b.grad[b.shard_start:b.shard_end], dst)
            if gc.correction != 1.0:
                b.grad.mul_(gc.correction)
            w = reduce_scatter_single(dst, b.grad, op=dist.ReduceOp.AVG, group=gc.group, async_op=True)
            return w if w is not None else CompletedWork()

        chain = ChainedWork(None, reduce, blocks_by_stream=gc.supports_async_overlap)
        return self._apply_chained_work_wrappers(chain, dst, b.role)

    def _fire(self, b: FlatBucket) -> None:
        b.work = self._reduce_chain(b)
        b.work.fire()
        b.fired = True

    def _finish(self, b: FlatBucket) -> None:
        if not b.fired:
            self._fire(b)   # a rank whose hooks did not all run still joins the collective
        b.work.wait()
        lp = b.local_param
        if lp.grad is None:
            lp.grad = b.shard_scratch.detach().clone()
        elif self.accumulate_on_shard:
            lp.grad.add_(b.shard_scratch)
        else:
            lp.grad.copy_(b.shard_scratch)
        b.work, b.fired = None, False

    def on_step_phase(self, phase: RuntimePhase) -> None:
        ctx = self.runtime.state.step_context
        if phase is RuntimePhase.PRE_BACKWARD:
            self._pre_backward(ctx)
        elif phase is RuntimePhase.POST_BACKWARD:
            self._post_backward(ctx)
        elif phase is RuntimePhase.PRE_STEP:
            self._maybe_clip_local_shards()
        elif phase is RuntimePhase.POST_STEP:
            self._gather_updated_params()
        elif phase is RuntimePhase.POST_LOAD:
            self._resync_from_buffers()

    def _pre_backward(self, ctx) -> None:
        for b in self.buckets:
            if ctx.accum_start:
                b.grad.zero_()
            self._attach_grad_views(b)
            # only the backward that closes the accumulation window may count down to zero
            b.pending = len(b.params) if ctx.is_step_boundary else 0
            b.fired = False

    def _post_backward(self, ctx) -> None:
        if not ctx.is_step_boundary:
            return
        with span("maltos::zero.grad_sync.wait"):
            for b in self.buckets:
                self._finish(b)

    def _gather_updated_params(self) -> None:
        works = []
        with torch.no_grad():
            for b in self.buckets:
                gc = b.group_context
                src = b.local_param.detach().contiguous()
                if gc.group is None or gc.world_size == 1:
                    b.data[b.shard_start:b.shard_end].copy_(src)
                else:
                    w = all_gather_single(b.data, src, group=gc.group, async_op=True)
                    if w is not None:
                        works.append(w)
            for w in works:
                w.wait()

    def _resync_from_buffers(self) -> None:
        with torch.no_grad():
            for b in self.buckets:
                b.local_param.data.copy_(b.data[b.shard_start:b.shard_end])
        sync = getattr(self.optimizer, "sync_master_params_from_model", None)
        if callable(sync):
            sync()

    # ------------------------------------------------------------------ clipping
    def _bucket_local_sq(self, b: FlatBucket) -> torch.Tensor:
        g = b.local_param.grad
        out = torch.zeros((), dtype=torch.float64, device=b.local_param.device)
        if g is None:
            return out
        lo, hi = b.shard_start, b.shard_end
        for p, at in zip(b.params, b.offsets):
            s, e = max(at, lo), min(at + p.numel(), hi)
            if s < e:
                out.add_(g[s - lo:e - lo].detach().double().pow(2).sum() / float(self.runtime.grad_norm_replica_factor(p)))
        return out


class Zero2Plugin(Zero1Plugin):
    accumulate_on_shard = True

    def __init__(self, bucket_mb_size: int = 25) -> None:
        super().__init__(bucket_mb_size, _id=PluginId.ZERO2, _name="zero2")

    def _pre_backward(self, ctx) -> None:
        for b in self.buckets:
            if ctx.accum_start and b.local_param.grad is not None:
                b.local_param.grad.zero_()
            if b.grad is None:
                b.grad_handle = acquire_buffer(shape=(b.data.numel(),), dtype=b.data.dtype, device=b.data.device, policy=BufferPolicy.TEMPORARY)
                b.grad = b.grad_handle.tensor
            b.grad.zero_()
            self._attach_grad_views(b)
            b.pending = len(b.params)
            b.fired = False

    def _post_backward(self, ctx) -> None:
        with span("maltos::zero.grad_sync.wait"):
            for b in self.buckets:
                self._finish(b)
                for p in b.params:
                    p.grad = None
                if b.grad_handle is not None:
                    release_buffer(b.grad_handle)
                b.grad, b.grad_handle = None, None

    def export_plugin_state(self):
        ctx = self.runtime.state.step_context
        if ctx.microbatch_idx == 0:
            return {}
        return {"bucket_local_grads": [None if b.local_param.grad is None else b.local_param.grad.detach().cpu().clone() for b in self.buckets]}

    def import_plugin_state(self, state) -> None:
        grads = state.get("bucket_local_grads")
        if not isinstance(grads, list):
            return
        for b, g in zip(self.buckets, grads):
            if g is not None:
                b.local_param.grad = g.to(device=b.local_param.device, dtype=b.local_param.dtype)

"""Data parallelism without sharding: per-parameter all-reduce (sync or async) and bucketed all-reduce.

* ``DataParallelPlugin``: at POST_BACKWARD of the window-closing micro-step, ``grad = AVG_dp(grad)`` per non-expert
  parameter (``async_op`` issues all then waits).
* ``BucketDataParallelPlugin``: parameters (reverse order) are packed into flat gradient buffers of >= ``bucket_mb_size``
  MiB, ``param.grad`` are views; a bucket's all-reduce starts from the gradient hook of its last parameter, overlapped
  with the rest of backward, and is waited at POST_BACKWARD; buffers are zeroed when a window opens.
(reference ``runtime/plugins/ddp.py:20-203``)
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.runtime.buffer_allocator import BufferPolicy, acquire_buffer
from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import ParamRole, RuntimePhase, SetupPhase
from maltos_b200.utils.distributed import all_reduce_tensor

from .zero_common import build_param_buckets, rearm_bucket_pending


class _DdpBase(RuntimePlugin):
    def __init__(self, name: str) -> None:
        super().__init__(id=PluginId.DP, name=name, runs_after={PluginId.TP, PluginId.TP_SP, PluginId.PP, PluginId.EP})

    @property
    def dp_group(self):
        return self.runtime.get_group(MeshAxis.DP)

    def _shared_params(self, model: nn.Module) -> list[nn.Parameter]:
        seen: set[int] = set()
        out = []
        for p in model.parameters():
            if p.requires_grad and id(p) not in seen and self.runtime.get_param_role(p) != ParamRole.EXPERT:
                seen.add(id(p))
                out.append(p)
        return out

    def annotate_param_metadata(self) -> None:
        if self.runtime.mesh.dp <= 1:
            return
        sm = self.runtime.state_manager
        for name, entry in sm.params.items():
            if self.runtime.get_param_role(entry.param) != ParamRole.EXPERT:
                sm.update_model_state(name, replicated_axes=entry.attrs.replicated_axes | {MeshAxis.DP})


class DataParallelPlugin(_DdpBase):
    def __init__(self, async_op: bool = False) -> None:
        super().__init__("data_parallel_async" if async_op else "data_parallel")
        self.async_op = async_op

    def on_step_phase(self, phase: RuntimePhase) -> None:
        if phase is not RuntimePhase.POST_BACKWARD or self.dp_group is None:
            return
        if not self.runtime.state.step_context.is_step_boundary:
            return
        works = []
        for p in self._shared_params(self.runtime.model):
            if p.grad is None:
                continue
            w = all_reduce_tensor(p.grad, op=dist.ReduceOp.AVG, group=self.dp_group, async_op=self.async_op)
            if w is not None:
                works.append(w)
        for w in works:
            w.wait()


@dataclass
class _GradBucket:
    params: list[nn.Parameter]
    buffer: torch.Tensor
    pending: int = 0
    work: object = None
    fired: bool = False
    offsets: list[int] = field(default_factory=list)


class BucketDataParallelPlugin(_DdpBase):
    def __init__(self, bucket_mb_size: int = 25) -> None:
        super().__init__("data_parallel_bucket")
        self.bucket_byte_size = bucket_mb_size * 1024 * 1024
        self.buckets: list[_GradBucket] = []

    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        if phase is SetupPhase.FINALIZE and self.dp_group is not None:
            self._build(model)
        return model

    def _build(self, model: nn.Module) -> None:
        params = self._shared_params(model)[::-1]
        for i, group in enumerate(build_param_buckets(params, self.bucket_byte_size)):
            total = sum(p.numel() for p in group)
            buf = acquire_buffer(shape=(total,), dtype=group[0].dtype, device=group[0].device, policy=BufferPolicy.PINNED,
                                 key=f"ddp.bucket{i}.grad").tensor
            buf.zero_()
            bucket = _GradBucket(params=group, buffer=buf)
            at = 0
            for p in group:
                bucket.offsets.append(at)
                p.grad = buf[at:at + p.numel()].view_as(p)
                at += p.numel()
                p.register_post_accumulate_grad_hook(self._make_hook(bucket))
            self.buckets.append(bucket)

    def _make_hook(self, bucket: _GradBucket):
        def hook(param: nn.Parameter) -> None:
            bucket.pending -= 1
            if bucket.pending == 0:
                self._fire(bucket)

        return hook

    def _fire(self, bucket: _GradBucket) -> None:
        bucket.work = all_reduce_tensor(bucket.buffer, op=dist.ReduceOp.AVG, group=self.dp_group, async_op=True)
        bucket.fired = True

    def _reattach(self, bucket: _GradBucket) -> None:
        # optimizer.zero_grad(set_to_none=True) dropped the views: point .grad back into the flat buffer
        for p, at in zip(bucket.params, bucket.offsets):
            if p.grad is None or p.grad.data_ptr() != bucket.buffer.data_ptr() + at * bucket.buffer.element_size():
                p.grad = bucket.buffer[at:at + p.numel()].view_as(p)

    def on_step_phase(self, phase: RuntimePhase) -> None:
        if self.dp_group is None:
            return
        ctx = self.runtime.state.step_context
        if phase is RuntimePhase.PRE_BACKWARD:
            for b in self.buckets:
                if ctx.accum_start:
                    b.buffer.zero_()
                self._reattach(b)
                b.pending = rearm_bucket_pending(len(b.params), grad_accum_end=ctx.is_step_boundary)
                b.fired = False
        elif phase is RuntimePhase.POST_BACKWARD and ctx.is_step_boundary:
            for b in self.buckets:
                if not b.fired:     # some parameter of the bucket got no gradient on this rank: keep ranks in lockstep
                    self._fire(b)
                if b.work is not None:
                    b.work.wait()
                    b.work = None

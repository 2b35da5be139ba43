"""Data parallelism without sharding: per-parameter all-reduce (sync or async) and bucketed all-reduce.

* ``DataParallelPlugin``: at POST_BACKWARD of the window-closing micro-step, ``grad = AVG_dp(grad)`` per non-expert
  parameter (``async_op`` issues all then waits).
* ``BucketDataParallelPlugin``: parameters (reverse order) are packed into flat gradient buffers of >= ``bucket_mb_size``
  MiB, ``param.grad`` are views; a bucket's all-reduce starts from the gradient hook of its last parameter, overlapped
  with the rest of backward, and is waited at POST_BACKWARD; buffers are zeroed when a window opens.
(reference ``runtime/plugins/ddp.py:20-203``)
"""
from __future__ import annotations

import os

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
                # a parameter this rank did not use in the window (an expert without tokens) may have been used elsewhere: every
                # rank must issue the same collectives, so it contributes zeros (what the flat-buffer modes do anyway)
                p.grad = torch.zeros_like(p)
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
    peer_ptrs: list[int] | None = None    # peer-memory mode: address of this bucket in every rank's gradient buffer


class BucketDataParallelPlugin(_DdpBase):
    def __init__(self, bucket_mb_size: int = 25, *, peer_memory: bool | None = None) -> None:
        super().__init__("data_parallel_bucket")
        self.bucket_byte_size = bucket_mb_size * 1024 * 1024
        self.buckets: list[_GradBucket] = []
        #: peer-memory mode (``MALTOS_B200_DDP_PEER=1``): the flat gradient buffers live in CUDA-IPC symmetric memory and
        #: each rank all-reduces its slice of every bucket in place over NVLink with one kernel per bucket
        #: (``ops/zero_fused.peer_all_reduce``) after backward, between two stream-ordered group barriers
        self.peer_memory = (os.environ.get("MALTOS_B200_DDP_PEER", "0") == "1") if peer_memory is None else bool(peer_memory)
        self._token = None

    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        if phase is SetupPhase.FINALIZE and self.dp_group is not None:
            self._build(model)
        return model

    def _build(self, model: nn.Module) -> None:
        params = self._shared_params(model)[::-1]
        groups = build_param_buckets(params, self.bucket_byte_size)
        peer = self._peer_buffers(groups)
        for i, group in enumerate(groups):
            total = sum(p.numel() for p in group)
            if peer is not None:
                buf, ptrs = peer[i]
            else:
                buf, ptrs = acquire_buffer(shape=(total,), dtype=group[0].dtype, device=group[0].device, policy=BufferPolicy.PINNED,
                                           key=f"ddp.bucket{i}.grad").tensor, None
            buf.zero_()
            bucket = _GradBucket(params=group, buffer=buf, peer_ptrs=ptrs)
            at = 0
            for p in group:
                bucket.offsets.append(at)
                p.grad = buf[at:at + p.numel()].view_as(p)
                at += p.numel()
                p.register_post_accumulate_grad_hook(self._make_hook(bucket))
            self.buckets.append(bucket)

    def _peer_buffers(self, groups):
        """Peer-memory mode: per bucket ``(flat gradient view, its address on every rank)`` inside one symmetric
        allocation; None when the mode is off or cannot be used (CPU, gloo, mixed dtypes, more than 16 ranks)."""
        if not self.peer_memory or not groups:
            return None
        first = groups[0][0]
        dtypes = {p.dtype for g in groups for p in g}
        if not first.is_cuda or len(dtypes) != 1 or first.dtype not in (torch.bfloat16, torch.float32):
            return None
        if dist.get_world_size(self.dp_group) > 16:
            return None
        from maltos_b200.ops import comm

        ctx = comm.context_for(self.dp_group)
        if ctx is None:
            return None
        esz = first.element_size()
        starts, at = [], 0
        for g in groups:
            starts.append(at)
            at += (sum(p.numel() for p in g) * esz + 255) // 256 * 256
        sb = ctx.ensure_buffer("ddp.grad", at)
        whole = sb.local_tensor(torch.uint8, at, first.device)
        out = []
        for g, s0 in zip(groups, starts):
            n = sum(p.numel() for p in g)
            out.append((whole[s0:s0 + n * esz].view(first.dtype), [p + s0 for p in sb.peer_ptrs]))
        return out

    def _barrier(self) -> None:
        if self._token is None:
            self._token = torch.zeros(1, dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
        dist.all_reduce(self._token, group=self.dp_group)

    def _peer_all_reduce(self) -> None:
        """Every rank reduces its 1/world slice of every bucket into all ranks' buffers; barriers before (all gradients are
        complete) and after (all results have landed)."""
        from maltos_b200.ops.zero_fused import peer_all_reduce

        world, rank = dist.get_world_size(self.dp_group), dist.get_rank(self.dp_group)
        self._barrier()
        for b in self.buckets:
            n, esz = b.buffer.numel(), b.buffer.element_size()
            per = ((n + world - 1) // world + 15) // 16 * 16          # slices start on 16-byte boundaries for both dtypes
            start = rank * per
            count = min(per, n - start)
            if count > 0:
                peer_all_reduce([p + start * esz for p in b.peer_ptrs], count, b.buffer.dtype, 1.0 / world)
        self._barrier()

    def _make_hook(self, bucket: _GradBucket):
        def hook(param: nn.Parameter) -> None:
            bucket.pending -= 1
            if bucket.pending == 0:
                self._fire(bucket)

        return hook

    def _fire(self, bucket: _GradBucket) -> None:
        if bucket.peer_ptrs is not None:
            return          # peer-memory mode reduces after backward, once every rank's gradients are complete
        bucket.work = all_reduce_tensor(bucket.buffer, op=dist.ReduceOp.AVG, group=self.dp_group, async_op=True)
        bucket.fired = True

    def _reattach(self, bucket: _GradBucket, *, keep_values: bool = False) -> None:
        # optimizer.zero_grad(set_to_none=True) dropped the views: point .grad back into the flat buffer. A gradient that
        # lives elsewhere inside an accumulation window (restored from a checkpoint) is moved into the buffer first.
        for p, at in zip(bucket.params, bucket.offsets):
            if p.grad is None or p.grad.data_ptr() != bucket.buffer.data_ptr() + at * bucket.buffer.element_size():
                view = bucket.buffer[at:at + p.numel()].view_as(p)
                if keep_values and p.grad is not None:
                    view.copy_(p.grad)
                p.grad = view

    def on_step_phase(self, phase: RuntimePhase) -> None:
        if self.dp_group is None:
            return
        ctx = self.runtime.state.step_context
        if phase is RuntimePhase.PRE_BACKWARD:
            for b in self.buckets:
                if ctx.accum_start:
                    b.buffer.zero_()
                self._reattach(b, keep_values=not ctx.accum_start)
                b.pending = rearm_bucket_pending(len(b.params), grad_accum_end=ctx.is_step_boundary)
                b.fired = False
        elif phase is RuntimePhase.POST_BACKWARD and ctx.is_step_boundary:
            if self.buckets and self.buckets[0].peer_ptrs is not None:
                self._peer_all_reduce()
                return
            for b in self.buckets:
                if not b.fired:     # some parameter of the bucket got no gradient on this rank: keep ranks in lockstep
                    self._fire(b)
                if b.work is not None:
                    b.work.wait()
                    b.work = None

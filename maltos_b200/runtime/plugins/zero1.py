"""ZeRO stage 1 and 2: optimizer state (and, for stage 2, gradients) sharded over the data-parallel group.

Parameters of one role (shared / expert), in reverse order, are packed into flat buckets padded to the shard-group
size; ``param.data`` become views of the flat data buffer and the optimizer owns one parameter per bucket = this
rank's ``1/N`` slice. When the last gradient of a bucket arrives on the window-closing micro-step its
reduce-scatter(AVG) starts, overlapped with the rest of backward; POST_BACKWARD waits, PRE_STEP clips on the shards,
POST_STEP all-gathers the updated slices back into the data buffer (reference ``runtime/plugins/zero1.py:98-299``).

Stage 2 keeps no full gradient buffer between micro-steps: a pooled buffer lives for one backward, its reduce-scatter
runs every micro-step and the result is *added* to the shard gradient (reference ``runtime/plugins/zero2.py:183-397``).

Peer-memory mode (``peer_memory=True`` or ``MALTOS_B200_ZERO_PEER=1``; bf16 parameters, NCCL group on one node): the flat
parameter and gradient buffers live in CUDA-IPC symmetric memory. After backward each owner reads its gradient slice
from all ranks' buffers and reduces, scales, accumulates and norms it in one kernel, and the AdamW kernel stores the
updated bf16 slice into every rank's parameter buffer, so neither a reduce-scatter nor an all-gather is launched
(``ops/zero_fused.py``). The kernels never wait on a peer; one-element all-reduces before and after each phase order them
across ranks. Stage 2 keeps its gradient buffer for the whole run in this mode.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn

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
    peer_data_ptrs: list[int] | None = None   # peer-memory mode: device address of this bucket in every rank's data buffer
    peer_grad_ptrs: list[int] | None = None   # ... and in every rank's gradient buffer
    direct: bool = False                      # the reduce kernel wrote the shard gradient itself
    fused_sq: torch.Tensor | None = None      # ||shard gradient||^2 from the reduce kernel (fp64 device scalar)

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

    def __init__(self, bucket_mb_size: int = 25, *, peer_memory: bool | None = None, _id: PluginId = PluginId.ZERO1,
                 _name: str = "zero1") -> None:
        super().__init__(id=_id, name=_name, owns_optimizer=True, bucket_mb_size=bucket_mb_size,
                         runs_after={PluginId.TP, PluginId.TP_SP, PluginId.PP, PluginId.EP, PluginId.CP})
        self.peer_memory = (os.environ.get("MALTOS_B200_ZERO_PEER", "0") == "1") if peer_memory is None else bool(peer_memory)
        self._barrier_tokens: dict[int, torch.Tensor] = {}
        self._pushes = False

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
            self._register_push_destinations()
            self.scheduler = self.runtime.create_scheduler(self.optimizer)
        elif phase is SetupPhase.FINALIZE:
            names = {id(p): n for n, p in model.named_parameters()}
            for b in self.buckets:
                b.logical_names = [names[id(p)] for p in b.params]
                for p in b.params:
                    p.register_post_accumulate_grad_hook(self._make_hook(b))
        return model

    def annotate_param_metadata(self) -> None:
        """Stages 1 and 2 shard optimizer state and gradients, not the weights: every data-parallel rank holds the same
        non-expert parameters, so ONE of them writes each into a checkpoint (the reference leaves the axis unmarked under
        ZeRO-1/2 and every data-parallel replica writes its own copy: dp times the bytes, and an offline conversion that
        joins tensor-parallel pieces sees each piece dp times). Experts are marked by the expert-parallel plugin."""
        if self.runtime.mesh.dp <= 1:
            return
        sm = self.runtime.state_manager
        for name, entry in sm.params.items():
            if self.runtime.get_param_role(entry.param) != ParamRole.EXPERT:
                sm.update_model_state(name, replicated_axes=entry.attrs.replicated_axes | {MeshAxis.DP})

    def _build_buckets(self, model: nn.Module) -> None:
        self.buckets = []
        for role in (ParamRole.SHARED, ParamRole.EXPERT):
            params = self._role_params(model, role)
            if not params:
                continue
            first_of_role = len(self.buckets)
            gc = self._group_context_for_role(role)
            groups = self._build_param_buckets(params)
            peer_slices = self._peer_buffers(role, gc, groups)
            for group in groups:
                total = sum(p.numel() for p in group)
                padded = padded_len(total, gc.world_size)
                peer = None if peer_slices is None else peer_slices[len(self.buckets) - first_of_role]
                data = torch.zeros(padded, dtype=group[0].dtype, device=group[0].device) if peer is None else peer[0]
                offsets, at = [], 0
                with torch.no_grad():
                    for p in group:
                        offsets.append(at)
                        data[at:at + p.numel()].copy_(p.data.reshape(-1))
                        p.data = data[at:at + p.numel()].view(p.shape)
                        at += p.numel()
                bucket = FlatBucket(index=len(self.buckets), role=role, params=group, group_context=gc, data=data, offsets=offsets, total=total)
                bucket.local_param = nn.Parameter(data[bucket.shard_start:bucket.shard_end].detach().clone())
                if peer is not None:
                    bucket.grad, bucket.peer_data_ptrs, bucket.peer_grad_ptrs = peer[1], peer[2], peer[3]
                elif not self.accumulate_on_shard:
                    bucket.grad = torch.zeros_like(data)
                self.buckets.append(bucket)

    def _peer_buffers(self, role: ParamRole, gc: GroupContext, groups):
        """Peer-memory mode: per bucket ``(data, grad, data addresses per rank, grad addresses per rank)`` carved out of two
        symmetric allocations of the role's shard group; None when the mode is off or cannot be used for this role."""
        if not self.peer_memory or not groups or gc.group is None or gc.world_size <= 1 or gc.world_size > 16:
            return None
        first = groups[0][0]
        if not first.is_cuda or any(p.dtype != torch.bfloat16 for g in groups for p in g):
            return None
        from maltos_b200.ops import comm

        ctx = comm.context_for(gc.group)
        if ctx is None:
            return None
        sizes = [padded_len(sum(p.numel() for p in g), gc.world_size) for g in groups]
        starts, at = [], 0
        for n in sizes:
            starts.append(at)
            at += (n + 127) // 128 * 128         # every bucket starts on a 256-byte boundary
        data_sb = ctx.ensure_buffer(f"{self.name}.{role.name}.data", at * 2)
        grad_sb = ctx.ensure_buffer(f"{self.name}.{role.name}.grad", at * 2)
        data_all = data_sb.local_tensor(torch.bfloat16, at, first.device).zero_()
        grad_all = grad_sb.local_tensor(torch.bfloat16, at, first.device).zero_()
        self._barrier(gc.group)   # nobody reads a peer's buffer before it is zeroed
        return [(data_all[s:s + n], grad_all[s:s + n], [p + 2 * s for p in data_sb.peer_ptrs], [p + 2 * s for p in grad_sb.peer_ptrs])
                for s, n in zip(starts, sizes)]

    def _barrier(self, group) -> None:
        """Stream-ordered barrier of ``group``: everything queued before it on any rank completes before anything queued
        after it on any rank starts."""
        tok = self._barrier_tokens.get(id(group))
        if tok is None:
            tok = self._barrier_tokens[id(group)] = torch.zeros(1, dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
        dist.all_reduce(tok, group=group)

    def _peer_groups(self):
        seen = {}
        for b in self.buckets:
            if b.peer_grad_ptrs is not None:
                seen[id(b.group_context.group)] = b.group_context.group
        return list(seen.values())

    def _register_push_destinations(self) -> None:
        """When the optimizer is the fused AdamW over fp32 masters, let its kernel store every updated slice into all
        ranks' parameter buffers (and into the local slice parameter) instead of all-gathering afterwards."""
        from maltos_b200.ops.zero_fused import ring_order
        from maltos_b200.runtime.optim import FusedAdamW, MasterWeightsOptimizer

        opt = self.optimizer
        if not isinstance(opt, MasterWeightsOptimizer) or not isinstance(opt.inner, FusedAdamW):
            return
        master_of = {id(p): m for p, m in zip(opt.model_params, opt.master_params)}
        for b in self.buckets:
            master = master_of.get(id(b.local_param))
            if b.peer_data_ptrs is None or master is None:
                continue
            shard_bytes = b.shard_start * 2
            ring = ring_order([p + shard_bytes for p in b.peer_data_ptrs], b.group_context.rank)
            opt.inner.push_destinations[id(master)] = lambda ring=ring, b=b: ring + [b.local_param.data_ptr()]
            opt.inner.low_precision_params.pop(id(master), None)
            self._pushes = True

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

        b.direct = False
        if b.peer_grad_ptrs is not None:
            return self._peer_reduce_chain(b, dst)

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

    def _peer_reduce_chain(self, b: FlatBucket, dst: torch.Tensor) -> ChainedWork:
        """Owner-side pull of the shard from every rank's gradient buffer. Without further reduction links for the role
        the kernel writes (stage 1) or accumulates into (stage 2) the shard gradient itself and produces its squared norm."""
        from maltos_b200.ops.zero_fused import peer_reduce_shard

        gc = b.group_context
        lp = b.local_param
        has_links = any(only is None or only == b.role for _, only in self._chained_work_wrappers)
        existed = lp.grad is not None
        if not has_links and not existed:
            lp.grad = torch.empty(b.shard_numel, dtype=b.grad.dtype, device=b.grad.device)
        b.direct = not has_links and lp.grad.dtype == b.grad.dtype and lp.grad.is_contiguous() and lp.grad.numel() == b.shard_numel
        accumulate = b.direct and existed and self.accumulate_on_shard
        out = lp.grad if b.direct else dst
        plain_norm = all(float(self._shard_replica_factor(p)) == 1.0 for p in b.params)
        if b.direct and plain_norm:
            b.fused_sq = torch.zeros((), dtype=torch.float64, device=dst.device) if b.fused_sq is None else b.fused_sq.zero_()
        else:
            b.fused_sq = None
        srcs = [p + 2 * b.shard_start for p in b.peer_grad_ptrs]

        def reduce():
            peer_reduce_shard(srcs, gc.rank, b.shard_numel, gc.correction / gc.world_size, out,
                              accumulate=accumulate, sumsq=b.fused_sq)
            return CompletedWork()

        chain = ChainedWork(None, reduce, blocks_by_stream=True)
        return self._apply_chained_work_wrappers(chain, dst, b.role)

    def _fire(self, b: FlatBucket) -> None:
        if b.peer_grad_ptrs is not None and not self._peers_ready:
            return              # the peers' gradients are complete only after the barrier in POST_BACKWARD
        b.work = self._reduce_chain(b)
        b.work.fire()
        b.fired = True

    def _finish(self, b: FlatBucket) -> None:
        if not b.fired:
            self._fire(b)   # a rank whose hooks did not all run still joins the collective
        b.work.wait()
        lp = b.local_param
        if b.direct:
            pass
        elif lp.grad is None:
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
            # with a restored optimizer state the fp32 masters came from the checkpoint; only a weights-only load re-derives them
            self._resync_from_buffers(sync_masters=not self.runtime.state.metadata.get("optimizer_state_restored", False))

    def _pre_backward(self, ctx) -> None:
        for b in self.buckets:
            if ctx.accum_start:
                b.grad.zero_()
            self._attach_grad_views(b)
            # only the backward that closes the accumulation window may count down to zero
            b.pending = len(b.params) if ctx.is_step_boundary else 0
            b.fired = False

    _peers_ready = False

    def _peer_phase(self, begin: bool) -> None:
        """Brackets the owner-side reductions: all ranks' gradients are complete before the first read, and every read is
        done before any rank touches its gradient buffer again."""
        for g in self._peer_groups():
            self._barrier(g)
        self._peers_ready = begin

    def _post_backward(self, ctx) -> None:
        if not ctx.is_step_boundary:
            return
        with span("maltos::zero.grad_sync.wait"):
            self._peer_phase(True)
            for b in self.buckets:
                self._finish(b)
            self._peer_phase(False)

    def _gather_updated_params(self) -> None:
        works = []
        with torch.no_grad():
            for b in self.buckets:
                gc = b.group_context
                if self._pushes and b.peer_data_ptrs is not None:
                    continue            # the optimizer kernel stored the slice into every rank's buffer
                src = b.local_param.detach().contiguous()
                if gc.group is None or gc.world_size == 1:
                    b.data[b.shard_start:b.shard_end].copy_(src)
                else:
                    w = all_gather_single(b.data, src, group=gc.group, async_op=True)
                    if w is not None:
                        works.append(w)
            for w in works:
                w.wait()
            if self._pushes:
                for g in self._peer_groups():
                    self._barrier(g)    # all peers' stores have landed before the next forward reads the parameters

    # ------------------------------------------------------------------ checkpoint inside an accumulation window
    def export_plugin_state(self):
        """The flat gradient buffers hold the micro-steps done so far when a checkpoint is taken inside an accumulation
        window; at a step boundary there is nothing to keep."""
        if self.runtime.state.step_context.microbatch_idx == 0:
            return {}
        return {"bucket_grads": [None if b.grad is None else b.grad.detach().to("cpu").clone() for b in self.buckets]}

    def import_plugin_state(self, state) -> None:
        grads = state.get("bucket_grads")
        if not isinstance(grads, list):
            return
        for b, g in zip(self.buckets, grads):
            if g is not None and b.grad is not None:
                b.grad.copy_(g.to(device=b.grad.device, dtype=b.grad.dtype))

    def _resync_from_buffers(self, *, sync_masters: bool = True) -> None:
        with torch.no_grad():
            for b in self.buckets:
                b.local_param.data.copy_(b.data[b.shard_start:b.shard_end])
        sync = getattr(self.optimizer, "sync_master_params_from_model", None)
        if sync_masters and callable(sync):
            sync()

    # ------------------------------------------------------------------ clipping
    def _bucket_local_sq(self, b: FlatBucket) -> torch.Tensor:
        g = b.local_param.grad
        out = torch.zeros((), dtype=torch.float64, device=b.local_param.device)
        if g is None:
            return out
        if b.direct and b.fused_sq is not None:
            return b.fused_sq.clone()
        lo, hi = b.shard_start, b.shard_end
        for p, at in zip(b.params, b.offsets):
            s, e = max(at, lo), min(at + p.numel(), hi)
            if s < e:
                out.add_(g[s - lo:e - lo].detach().double().pow(2).sum() / float(self._shard_replica_factor(p)))
        return out


def __getattr__(name: str):
    # `zero1.Zero2Plugin` keeps working for callers that imported it from here; the class lives in zero2.py
    if name == "Zero2Plugin":
        from .zero2 import Zero2Plugin

        return Zero2Plugin
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

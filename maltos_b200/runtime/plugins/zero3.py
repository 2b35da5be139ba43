"""ZeRO stage 3: parameters, gradients and optimizer state sharded; full parameters exist only around their use.

Buckets (this order is part of the checkpoint format, reference ``runtime/plugins/zero3.py:181-240``):
  1. parameter groups announced by other plugins through ``param_materialization_groups()`` (q/k/v and gate/up of the
     TP+SP plugin, fused scopes), in plugin order;
  2. every module of a ``wrap_cls`` type in ``named_modules()`` order with its direct, not yet covered parameters.
Each bucket is a flat padded buffer whose ``1/N`` slice is this rank's ``local_param`` (what the optimizer updates and
what ``zero3_bucket_{i}`` stores in a checkpoint).

Execution: a forward-pre hook of the bucket's module waits for the (asynchronous) all-gather of the slices into a
pooled buffer, binds the parameters to views of it and starts the gather of the NEXT bucket in execution order, so that
the transfer runs under this bucket's compute; the forward hook releases the parameters. A backward-pre hook does the
same in reverse (prefetching the PREVIOUS bucket). The execution order is observed during the first forward. When the
last gradient of a bucket has been produced the flat gradient is reduce-scattered asynchronously (AVG x correction); the
results are added to the slice gradients at POST_BACKWARD, after the whole backward pass has been queued. Gradients
accumulate on the slices, so the reduce-scatter runs every micro-step. Recompute under activation checkpointing
re-enters the same hooks. Reference: ``runtime/plugins/zero3.py:384-450`` (prefetch), ``:452-490`` (asynchronous gather),
``:505-544`` (asynchronous reduce-scatter). ``MALTOS_B200_ZERO3_PREFETCH=0`` makes every collective synchronous.
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.runtime.buffer_allocator import BufferPolicy, acquire_buffer, release_buffer
from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.plugin import ParamMaterializationGroupProvider, PluginId
from maltos_b200.runtime.types import ParamRole, RuntimePhase, SetupPhase
from maltos_b200.state.state import ModelStateMeta
from maltos_b200.utils.distributed import all_gather_single, reduce_scatter_single
from maltos_b200.utils.profiling import span

from .zero_common import GroupContext, ZeroPluginBase, padded_len


@dataclass
class ShardedBucket:
    index: int
    module: nn.Module
    params: list[nn.Parameter]
    role: ParamRole
    group_context: GroupContext
    param_shapes: list[tuple[int, ...]]
    param_numels: list[int]
    offsets: list[int]
    total: int
    padded: int
    local_param: nn.Parameter = None
    logical_names: list[str] = field(default_factory=list)
    full_tensor: torch.Tensor | None = None   # flat gathered parameters; its storage has zero bytes while released
    is_materialized: bool = False
    grad_flat: torch.Tensor | None = None
    grad_handle: object = None
    grads_pending: int = 0
    users: int = 0                  # nested materialisations (recompute inside backward)
    hook_module: nn.Module = None   # module whose forward/backward brackets the use of these parameters
    peer_shard_ptrs: list[int] | None = None   # peer-memory mode: address of every rank's shard of this bucket
    gather_work: object = None      # handle of the all-gather in flight into full_handle (None once bound)
    prefetched: bool = False        # gathered ahead of use and not yet claimed by a hook

    @property
    def shard_numel(self) -> int:
        return self.padded // self.group_context.world_size

    @property
    def materialized(self) -> bool:
        return self.is_materialized


class Zero3Plugin(ZeroPluginBase):
    def __init__(self, wrap_cls: set[type] | None = None, bucket_mb_size: int = 25, *, peer_memory: bool | None = None) -> None:
        super().__init__(id=PluginId.ZERO3, name="zero3", owns_optimizer=True, owns_model_state=True, bucket_mb_size=bucket_mb_size,
                         runs_after={PluginId.TP, PluginId.TP_SP, PluginId.PP, PluginId.EP, PluginId.CP, PluginId.COMPILE})
        self.wrap_cls = set(wrap_cls) if wrap_cls is not None else {nn.Linear}
        #: peer-memory mode: the shards live in CUDA-IPC symmetric memory and a gather is a one-sided pull from the
        #: peers' shards (one kernel, no rendezvous); barriers bracket only the optimizer step, when the shards change
        self.peer_memory = (os.environ.get("MALTOS_B200_ZERO_PEER", "0") == "1") if peer_memory is None else bool(peer_memory)
        self._peer_groups: dict[int, object] = {}
        self._barrier_tokens: dict[int, torch.Tensor] = {}
        self._by_param: dict[int, ShardedBucket] = {}
        self._placeholder: dict[int, torch.Tensor] = {}
        self.prefetch = os.environ.get("MALTOS_B200_ZERO3_PREFETCH", "1") != "0"
        self._order: list[int] = []            # bucket indices in the order the first forward used them
        self._order_pos: dict[int, int] = {}
        self._order_final = False
        self._unclaimed: list[ShardedBucket] = []     # prefetched buckets nobody has used yet (oldest first)
        self._reduces: list[tuple] = []        # (bucket, work, piece, grad handle) of reduce-scatters in flight

    # ------------------------------------------------------------------ setup
    def bind(self, runtime) -> None:
        super().bind(runtime)
        self.dp_group = runtime.get_group(MeshAxis.DP)
        if self.dp_group is not None:
            self.world_size, self.rank = dist.get_world_size(self.dp_group), dist.get_rank(self.dp_group)

    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        if phase is SetupPhase.MATERIALIZE:
            self._materialize(model)
        elif phase is SetupPhase.FINALIZE:
            self._register_hooks(model)
        return model

    def _wrap_types(self) -> tuple[type, ...]:
        types = set(self.wrap_cls)
        for t in list(types):
            types |= set(self.runtime.get_module_replacements(t))
        return tuple(types)

    def _collect_groups(self, model: nn.Module) -> list[tuple[nn.Module, list[nn.Parameter]]]:
        covered: set[int] = set()
        groups: list[tuple[nn.Module, list[nn.Parameter]]] = []

        def add(module, params):
            fresh = [p for p in params if p.requires_grad and id(p) not in covered]
            if fresh:
                covered.update(id(p) for p in fresh)
                groups.append((module, fresh))

        for plugin in self.runtime.plugins:
            if plugin is not self and isinstance(plugin, ParamMaterializationGroupProvider):
                for module, params in plugin.param_materialization_groups():
                    add(module, list(params))
        wrap = self._wrap_types()
        for _, module in model.named_modules():
            if isinstance(module, wrap):
                add(module, list(module.parameters(recurse=False)))
        missing = [n for n, p in model.named_parameters() if p.requires_grad and id(p) not in covered]
        if missing:
            raise ValueError(f"Zero3Plugin: parameters not covered by wrap_cls / materialization groups: {missing[:8]}")
        return groups

    def _materialize(self, model: nn.Module) -> None:
        rt = self.runtime
        device = torch.device(rt.device)
        dtype = rt.dtype
        # this plugin owns the model state: the core did not move the model. Buffers (RoPE tables...) move here.
        for mod in model.modules():
            for name, buf in list(mod._buffers.items()):
                if buf is not None:
                    mod._buffers[name] = buf.to(device)
        names = {id(p): n for n, p in model.named_parameters()}
        self.buckets = []
        self._by_param.clear()
        for module, params in self._collect_groups(model):
            role = rt.get_param_role(params[0])
            gc = self._group_context_for_role(role)
            numels = [p.numel() for p in params]
            total = sum(numels)
            padded = padded_len(total, max(gc.world_size, 1))
            offsets, at = [], 0
            for n in numels:
                offsets.append(at)
                at += n
            b = ShardedBucket(index=len(self.buckets), module=module, params=params, role=role, group_context=gc,
                              param_shapes=[tuple(p.shape) for p in params], param_numels=numels, offsets=offsets, total=total,
                              padded=padded, logical_names=[names[id(p)] for p in params])
            want = dtype if (dtype is not None and params[0].is_floating_point()) else params[0].dtype
            flat = torch.zeros(padded, dtype=want, device=device)
            with torch.no_grad():
                for p, off, n in zip(params, offsets, numels):
                    flat[off:off + n].copy_(p.data.reshape(-1))
            lo = gc.rank * b.shard_numel
            shard = flat[lo:lo + b.shard_numel]
            b.local_param = nn.Parameter(self._peer_shard(b, shard) if self._peer_ok(b, want, device) else shard.clone())
            for p in params:
                self._by_param[id(p)] = b
                ph = torch.empty(0, dtype=want, device=device)
                self._placeholder[id(p)] = ph
                p.data = ph
            del flat
            self.buckets.append(b)
        self._peer_barrier()     # every rank's shards are in place before anyone pulls them
        self.optimizer = rt.create_optimizer([b.local_param for b in self.buckets])
        self.scheduler = rt.create_scheduler(self.optimizer)

    # ------------------------------------------------------------------ peer-memory mode
    def _peer_ok(self, b: ShardedBucket, dtype, device) -> bool:
        gc = b.group_context
        return (self.peer_memory and device.type == "cuda" and dtype == torch.bfloat16 and gc.group is not None
                and 1 < gc.world_size <= 16 and (b.shard_numel * 2) % 16 == 0 and self._peer_context(gc) is not None)

    def _peer_context(self, gc: GroupContext):
        from maltos_b200.ops import comm

        ctx = comm.context_for(gc.group)
        if ctx is not None:
            self._peer_groups[id(gc.group)] = gc.group
        return ctx

    def _peer_shard(self, b: ShardedBucket, shard: torch.Tensor) -> torch.Tensor:
        """Collective: this bucket's shard in its own symmetric allocation (values copied), addresses of all ranks' shards."""
        ctx = self._peer_context(b.group_context)
        sb = ctx.ensure_buffer(f"zero3.shard.{b.index}", b.shard_numel * 2)
        local = sb.local_tensor(torch.bfloat16, b.shard_numel, shard.device)
        local.copy_(shard)
        b.peer_shard_ptrs = list(sb.peer_ptrs)
        return local

    def _peer_barrier(self) -> None:
        """Stream-ordered barrier of every shard group in peer-memory mode (no-op otherwise)."""
        for key, group in self._peer_groups.items():
            tok = self._barrier_tokens.get(key)
            if tok is None:
                tok = self._barrier_tokens[key] = torch.zeros(1, dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
            dist.all_reduce(tok, group=group)

    # ------------------------------------------------------------------ gather / release
    def _start_gather(self, b: ShardedBucket) -> None:
        """Launch the all-gather of the bucket into a pooled buffer without waiting for it."""
        if b.materialized:
            return
        gc = b.group_context
        lp = b.local_param
        # The gathered parameters of a bucket always live in the SAME storage object, grown to full size here and shrunk
        # to zero bytes on release: autograd may have saved a view of a weight (``weight.t()`` of a decomposed linear) in
        # the forward pass, and such a view must see the re-gathered values in the backward pass wherever the allocator
        # places them.
        if b.full_tensor is None:
            b.full_tensor = torch.empty(b.padded, dtype=lp.dtype, device=lp.device)
        else:
            b.full_tensor.untyped_storage().resize_(b.padded * lp.element_size())
        b.is_materialized = True
        full = b.full_tensor
        with torch.no_grad():
            if gc.group is None or gc.world_size == 1:
                full.copy_(lp.data)
            elif b.peer_shard_ptrs is not None:
                from maltos_b200.ops.zero_fused import peer_gather

                peer_gather(full, b.peer_shard_ptrs, b.shard_numel * 2)
            else:
                b.gather_work = all_gather_single(full, lp.data.contiguous(), group=gc.group, async_op=self.prefetch)

    def _finish_gather(self, b: ShardedBucket) -> None:
        """Wait for the gather in flight (the current stream waits, not the host, on NCCL) and bind the parameter views."""
        if b.gather_work is not None:
            b.gather_work.wait()
            b.gather_work = None
        full = b.full_tensor
        for p, off, n, shape in zip(b.params, b.offsets, b.param_numels, b.param_shapes):
            p.data = full[off:off + n].view(shape)

    def _gather(self, b: ShardedBucket) -> None:
        b.users += 1
        if b.prefetched:
            b.prefetched = False
            if b in self._unclaimed:
                self._unclaimed.remove(b)
        if b.materialized and b.gather_work is None and b.params[0].data.numel() > 0:
            return
        self._start_gather(b)
        self._finish_gather(b)

    def _prefetch(self, b: ShardedBucket | None) -> None:
        """Start gathering a bucket that the execution order says comes next. A prefetched bucket that is never claimed
        (the order ran past the end of a recomputed block) is dropped once two newer ones are waiting."""
        if b is None or not self.prefetch or b.materialized:
            return
        self._start_gather(b)
        b.prefetched = True
        self._unclaimed.append(b)
        while len(self._unclaimed) > 2:
            stale = self._unclaimed.pop(0)
            if stale.users == 0 and stale.prefetched:
                stale.prefetched = False
                self._release(stale, force=True)

    def _neighbour(self, b: ShardedBucket, step: int):
        if not self._order_final:
            return None
        pos = self._order_pos.get(b.index)
        if pos is None or not (0 <= pos + step < len(self._order)):
            return None
        return self.buckets[self._order[pos + step]]

    def _release(self, b: ShardedBucket, *, force: bool = False) -> None:
        b.users = 0 if force else max(b.users - 1, 0)
        if b.users > 0 or not b.materialized:
            return
        if b.gather_work is not None:      # never hand a buffer back while a collective still writes it
            b.gather_work.wait()
            b.gather_work = None
        b.prefetched = False
        if b in self._unclaimed:
            self._unclaimed.remove(b)
        for p in b.params:
            p.data = self._placeholder[id(p)]
        b.full_tensor.untyped_storage().resize_(0)
        b.is_materialized = False

    def materialize_model(self) -> None:
        """Gather every bucket (tests / export). Pair with :meth:`reshard_model`."""
        for b in self.buckets:
            self._gather(b)

    def reshard_model(self) -> None:
        for b in self.buckets:
            self._release(b, force=True)

    # ------------------------------------------------------------------ hooks
    def _register_hooks(self, model: nn.Module) -> None:
        # Projection groups (q/k/v, gate/up) are consumed by their parent block in one fused op, not through the
        # member modules' own forward: their buckets are bracketed by the parent's forward / backward instead.
        group_owner: dict[int, nn.Module] = {}
        for m in model.modules():
            groups = getattr(m, "parameter_fusion_groups", None)
            if callable(groups):
                for params in groups():
                    for p in params:
                        group_owner[id(p)] = m
        for b in self.buckets:
            owners = {id(group_owner.get(id(p))) for p in b.params}
            first = group_owner.get(id(b.params[0]))
            b.hook_module = first if (first is not None and len(owners) == 1) else b.module
            b.hook_module.register_forward_pre_hook(self._pre_forward(b), prepend=True)
            b.hook_module.register_forward_hook(self._post_forward(b), always_call=True)
            b.hook_module.register_full_backward_pre_hook(self._pre_backward(b))
            for p in b.params:
                p.register_post_accumulate_grad_hook(self._grad_ready(b))

    def _pre_forward(self, b: ShardedBucket):
        def hook(module, args):
            with span("maltos::zero3.materialize.forward"):
                if not self._order_final and b.index not in self._order_pos:
                    self._order_pos[b.index] = len(self._order)
                    self._order.append(b.index)
                self._gather(b)
                self._prefetch(self._neighbour(b, +1))

        return hook

    def _post_forward(self, b: ShardedBucket):
        def hook(module, args, output):
            self._release(b)

        return hook

    def _pre_backward(self, b: ShardedBucket):
        def hook(module, grad_output):
            with span("maltos::zero3.materialize.backward"):
                if not b.materialized or b.prefetched or b.gather_work is not None:
                    self._gather(b)
                self._prefetch(self._neighbour(b, -1))
                if b.grads_pending <= 0:
                    b.grads_pending = sum(1 for p in b.params if p.requires_grad)

        return hook

    def _grad_ready(self, b: ShardedBucket):
        def hook(param: nn.Parameter) -> None:
            if b.grad_flat is None:
                lp = b.local_param
                b.grad_handle = acquire_buffer(shape=(b.padded,), dtype=lp.dtype, device=lp.device, policy=BufferPolicy.TEMPORARY)
                b.grad_flat = b.grad_handle.tensor
                b.grad_flat.zero_()
            i = next(k for k, p in enumerate(b.params) if p is param)
            off, n = b.offsets[i], b.param_numels[i]
            b.grad_flat[off:off + n].add_(param.grad.reshape(-1).to(b.grad_flat.dtype))
            param.grad = None
            if b.grads_pending <= 0:   # backward entered without the module-level hook (e.g. inputs need no grad)
                b.grads_pending = sum(1 for p in b.params if p.requires_grad)
            b.grads_pending -= 1
            if b.grads_pending == 0:
                self._reduce(b)
                self._release(b, force=True)

        return hook

    def _reduce(self, b: ShardedBucket) -> None:
        """Launch the reduce-scatter of the bucket's flat gradient; :meth:`_finish_reduces` adds the result to the slice."""
        gc = b.group_context
        flat = b.grad_flat
        if gc.correction != 1.0:
            flat.mul_(gc.correction)
        if gc.group is None or gc.world_size == 1:
            self._reduces.append((b, None, flat[: b.shard_numel], b.grad_handle))
        else:
            piece = torch.empty(b.shard_numel, dtype=flat.dtype, device=flat.device)
            work = reduce_scatter_single(piece, flat, op=dist.ReduceOp.AVG, group=gc.group, async_op=self.prefetch)
            self._reduces.append((b, work, piece, b.grad_handle))
        b.grad_flat, b.grad_handle = None, None
        if not self.prefetch:
            self._finish_reduces()

    def _finish_reduces(self) -> None:
        for b, work, piece, handle in self._reduces:
            if work is not None:
                work.wait()
            lp = b.local_param
            if lp.grad is None:
                lp.grad = piece.detach().clone()
            else:
                lp.grad.add_(piece)
            release_buffer(handle)
        self._reduces.clear()

    def on_step_phase(self, phase: RuntimePhase) -> None:
        if phase is RuntimePhase.POST_FORWARD:
            if not self._order_final and self._order:
                self._order_final = True        # observed once; prefetching starts with the next pass
        elif phase is RuntimePhase.POST_BACKWARD:
            with span("maltos::zero3.grad_sync.wait"):
                for b in self.buckets:
                    if b.grad_flat is not None:      # some parameter produced no gradient: reduce what arrived
                        b.grads_pending = 0
                        self._reduce(b)
                    if b.materialized:
                        self._release(b, force=True)
                self._finish_reduces()
        elif phase is RuntimePhase.PRE_STEP:
            self._maybe_clip_local_shards()
            self._peer_barrier()     # every pull of the old shards is done before any optimizer overwrites them
        elif phase is RuntimePhase.POST_STEP:
            self._peer_barrier()     # every shard is updated before the next forward pulls it
        elif phase is RuntimePhase.POST_LOAD:
            # with a restored optimizer state the fp32 masters came from the checkpoint; only a weights-only load re-derives them
            sync = getattr(self.optimizer, "sync_master_params_from_model", None)
            if callable(sync) and not self.runtime.state.metadata.get("optimizer_state_restored", False):
                sync()
            self._peer_barrier()

    # ------------------------------------------------------------------ clipping
    def _bucket_local_sq(self, b: ShardedBucket) -> torch.Tensor:
        g = b.local_param.grad
        out = torch.zeros((), dtype=torch.float64, device=b.local_param.device)
        if g is None:
            return out
        lo = b.group_context.rank * b.shard_numel
        hi = lo + b.shard_numel
        sm = self.runtime.state_manager
        for name, off, n in zip(b.logical_names, b.offsets, b.param_numels):
            s, e = max(off, lo), min(off + n, hi)
            if s < e:
                factor = self._replica_factor(name)
                out.add_(g[s - lo:e - lo].detach().double().pow(2).sum() / float(factor))
        del sm
        return out

    def _replica_factor(self, name: str) -> int:
        entry = self.runtime.state_manager.params.get(name)
        if entry is None:
            return 1
        return self._shard_replica_factor(entry.param)

    # ------------------------------------------------------------------ metadata & model state
    def annotate_param_metadata(self) -> None:
        return

    def bucket_checkpoint_names(self, bucket: ShardedBucket) -> list[str]:
        """Names under which the tensors of ``bucket`` go into a checkpoint: the logical name another plugin has recorded for a
        parameter (expert parallelism: ``local_experts.{i}`` of this rank -> ``experts.{global id}``), else the runtime name.
        Without this the expert buckets of different expert-parallel ranks would carry the same names."""
        params = self.runtime.state_manager.params
        out = []
        for name in bucket.logical_names:
            entry = params.get(name)
            logical = list(entry.meta.logical_names) if entry is not None else []
            out.append(logical[0] if len(logical) == 1 else name)
        return out

    def export_model_state(self, state_manager):
        rank = dist.get_rank() if dist.is_initialized() else 0
        tensors: dict[str, torch.Tensor] = {}
        metas: list[ModelStateMeta] = []
        for b in self.buckets:
            key = f"zero3_bucket_{b.index}"
            tensors[key] = b.local_param.detach().cpu().clone()
            metas.append(ModelStateMeta(state_key=key, logical_names=self.bucket_checkpoint_names(b), logical_shapes=[tuple(s) for s in b.param_shapes],
                                        physical_shape=(b.shard_numel,), dtype=str(b.local_param.dtype), source_rank=rank))
        for name, entry in state_manager.buffers.items():
            tensors[name] = entry.tensor.detach().cpu().clone()
            meta = entry.meta
            metas.append(ModelStateMeta(meta.state_key, list(meta.logical_names), list(meta.logical_shapes), tuple(meta.physical_shape), meta.dtype, rank))
        return tensors, metas

    def import_model_state(self, state_manager, model_state) -> None:
        by_key = {f"zero3_bucket_{b.index}": b for b in self.buckets}
        for key, value in model_state.items():
            if key in by_key:
                lp = by_key[key].local_param
                if value.numel() != lp.numel():
                    raise ValueError(f"{key}: shard size mismatch checkpoint={value.numel()} runtime={lp.numel()}")
                lp.data.copy_(value.to(device=lp.device, dtype=lp.dtype).reshape(-1))
            elif key in state_manager.buffers:
                dst = state_manager.buffers[key].tensor
                dst.copy_(value.to(device=dst.device, dtype=dst.dtype))
            else:
                raise KeyError(f"model state not found: {key}")

    def export_plugin_state(self):
        if self.runtime.state.step_context.microbatch_idx == 0:
            return {}
        return {"bucket_local_grads": [None if b.local_param.grad is None else b.local_param.grad.detach().cpu().clone() for b in self.buckets]}

    def import_plugin_state(self, state) -> None:
        grads = state.get("bucket_local_grads")
        if isinstance(grads, list):
            for b, g in zip(self.buckets, grads):
                if g is not None:
                    b.local_param.grad = g.to(device=b.local_param.device, dtype=b.local_param.dtype)

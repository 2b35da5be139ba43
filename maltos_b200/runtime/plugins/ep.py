"""Expert parallelism.

TRANSFORM: every block named by ``model.expert_parallel_spec()`` becomes an ``ExpertParallelMoE`` that keeps
``num_experts / ep`` contiguous experts; parameters are tagged EXPERT or SHARED so the data-parallel plugins pick the
right reduction group. Gradient synchronisation: with a ZeRO plugin present it is delegated (experts shard over EREP);
otherwise expert gradients live in flat buckets of <= ``bucket_mb_size`` MiB whose persistent chain all-reduces
(AVG x correction) over the expert-replica group when the bucket's last gradient arrives on the closing micro-step,
and shared gradients are averaged over DP unless a DP/ZeRO plugin does it. Checkpoint names map
``local_experts.{i}`` to the logical ``experts.{global}`` (reference ``runtime/plugins/ep.py:100-342``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.parallel.protocols import ExpertParallelizableModule
from maltos_b200.runtime.buffer_allocator import BufferPolicy, acquire_buffer
from maltos_b200.runtime.layers.moe import ExpertParallelMoE
from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import ParamRole, RuntimePhase, SetupPhase
from maltos_b200.utils.distributed import all_reduce_tensor

from .tp import set_submodule
from .zero_common import (ChainedWork, CompletedWork, build_param_buckets, expert_data_shards, expert_erep_correction, expert_token_copies,
                          rearm_bucket_pending)

_ZERO = {PluginId.ZERO1, PluginId.ZERO2, PluginId.ZERO3}


@dataclass
class _GradBucket:
    params: list[nn.Parameter]
    grad_buffer: torch.Tensor
    pending: int = 0
    fired: bool = False
    work: ChainedWork | None = None


class ExpertParallelPlugin(RuntimePlugin):
    def __init__(self, bucket_mb_size: int = 25) -> None:
        super().__init__(id=PluginId.EP, name="expert_parallel", runs_after={PluginId.PP, PluginId.TP, PluginId.TP_SP})
        self.bucket_byte_size = bucket_mb_size * 1024 * 1024
        self._expert_param_ids: set[int] = set()
        self._grad_buckets: list[_GradBucket] = []
        self._delegate_shared_dp_sync = False
        self._delegate_expert_sync = False

    @property
    def ep_group(self):
        return self.runtime.get_group(MeshAxis.EP)

    @property
    def edp_group(self):
        return self.runtime.get_group(MeshAxis.EREP)

    @property
    def dp_group(self):
        return self.runtime.get_group(MeshAxis.DP)

    def bind(self, runtime) -> None:
        super().bind(runtime)
        if runtime.mesh.ep <= 1:
            raise ValueError("ExpertParallelPlugin requires mesh.ep > 1")
        active = {p.id for p in runtime.plugins if p is not self}
        self._delegate_shared_dp_sync = bool(({PluginId.DP} | _ZERO) & active)
        self._delegate_expert_sync = bool(_ZERO & active)

    # ------------------------------------------------------------------ setup
    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        if phase is SetupPhase.TRANSFORM:
            return self._transform(model)
        if phase is SetupPhase.MATERIALIZE and not self._delegate_expert_sync:
            self._prepare_grad_buckets(model)
        if phase is SetupPhase.FINALIZE and not self._delegate_expert_sync:
            for b in self._grad_buckets:
                for p in b.params:
                    p.register_post_accumulate_grad_hook(self._make_hook(b))
        return model

    def _transform(self, model: nn.Module) -> nn.Module:
        if not isinstance(model, ExpertParallelizableModule):
            raise TypeError(f"ExpertParallelPlugin requires model.expert_parallel_spec(), got {type(model).__name__}")
        for path in model.expert_parallel_spec().moe_paths:
            if self.runtime.is_module_path_omitted(path):
                continue
            module = model.get_submodule(path)
            # (a Protocol isinstance check would miss sub-modules: nn.Module keeps them outside the instance dict)
            if not all(hasattr(module, a) for a in ("router", "experts", "num_experts", "dim", "hidden_size")):
                raise TypeError("ExpertParallelPlugin requires MoE modules to satisfy ExpertParallelMoEModule, "
                                f"got module type={type(module).__name__}")
            set_submodule(model, path, ExpertParallelMoE.from_moe(module, self.ep_group))
        self._expert_param_ids = {id(p) for m in model.modules() if isinstance(m, ExpertParallelMoE) for p in m.local_experts.parameters()}
        for p in model.parameters():
            if p.requires_grad:
                self.runtime.set_param_role(p, ParamRole.EXPERT if id(p) in self._expert_param_ids else ParamRole.SHARED)
        return model

    def is_expert_param(self, param: nn.Parameter) -> bool:
        return self.runtime.get_param_role(param) == ParamRole.EXPERT

    def _attach(self, bucket: _GradBucket) -> None:
        at = 0
        for p in bucket.params:
            p.grad = bucket.grad_buffer[at:at + p.numel()].view_as(p)
            at += p.numel()

    def _prepare_grad_buckets(self, model: nn.Module) -> None:
        experts = [p for p in model.parameters() if p.requires_grad and id(p) in self._expert_param_ids]
        if not experts:
            return
        group = self.edp_group
        by_stream = group is None or dist.get_backend(group) != "gloo"
        for i, params in enumerate(build_param_buckets(experts, self.bucket_byte_size)):
            buf = acquire_buffer(shape=(sum(p.numel() for p in params),), dtype=params[0].dtype, device=params[0].device,
                                 policy=BufferPolicy.PINNED, key=f"ep.bucket.{i}.grad_buffer").tensor
            buf.zero_()
            bucket = _GradBucket(params=params, grad_buffer=buf)
            self._attach(bucket)
            bucket.work = ChainedWork(None, self._erep_functor(bucket, group), blocks_by_stream=by_stream)
            self._grad_buckets.append(bucket)

    def _erep_functor(self, bucket: _GradBucket, group):
        def functor():
            mesh, plan = self.runtime.mesh, self.runtime.plan
            kw = dict(tp=mesh.tp, cp=mesh.cp, ep=mesh.ep, reuse_tp=plan.reuse_tp_for_ep, reuse_cp=plan.reuse_cp_for_ep)
            shards = expert_data_shards(**kw) * expert_token_copies(self.runtime)
            if group is None or dist.get_world_size(group) <= 1:
                if shards != 1:
                    bucket.grad_buffer.div_(shards)
                return CompletedWork()
            corr = expert_erep_correction(**kw) / shards
            if corr != 1.0:
                bucket.grad_buffer.mul_(corr)
            w = all_reduce_tensor(bucket.grad_buffer, op=dist.ReduceOp.AVG, group=group, async_op=True)
            return w if w is not None else CompletedWork()

        return functor

    def _make_hook(self, bucket: _GradBucket):
        def hook(_p) -> None:
            bucket.pending -= 1
            if bucket.pending == 0:
                bucket.work.fire()
                bucket.fired = True

        return hook

    # ------------------------------------------------------------------ step phases
    def on_step_phase(self, phase: RuntimePhase) -> None:
        rt = self.runtime
        ctx = rt.state.step_context
        if phase is RuntimePhase.PRE_BACKWARD:
            for b in self._grad_buckets:
                if ctx.accum_start:
                    b.grad_buffer.zero_()
                if ctx.accum_start or any(p.grad is None for p in b.params):
                    self._attach(b)
                b.pending = rearm_bucket_pending(len(b.params), grad_accum_end=ctx.is_step_boundary)
                b.fired = False
            return
        if phase is not RuntimePhase.POST_BACKWARD or not ctx.is_step_boundary:
            return
        for b in self._grad_buckets:          # every replica fires the same collectives, hooks or not
            if not b.fired:
                b.work.fire()
                b.fired = True
            b.work.wait()
        if self._delegate_shared_dp_sync or self.dp_group is None or dist.get_world_size(self.dp_group) <= 1:
            return
        works = []
        for p in rt.model.parameters():
            if p.requires_grad and id(p) not in self._expert_param_ids:
                if p.grad is None:      # unused here, maybe used on another rank: same collectives everywhere
                    p.grad = torch.zeros_like(p)
                w = all_reduce_tensor(p.grad, op=dist.ReduceOp.AVG, group=self.dp_group, async_op=True)
                if w is not None:
                    works.append(w)
        for w in works:
            w.wait()

    # ------------------------------------------------------------------ metadata
    def _runtime_to_logical(self) -> dict[str, str]:
        sm = self.runtime.state_manager
        names = list(sm.params) + list(sm.buffers)
        out: dict[str, str] = {}
        for path, module in self.runtime.model.named_modules():
            if not isinstance(module, ExpertParallelMoE):
                continue
            prefix = f"{path}." if path else ""
            for local, glob in enumerate(module.local_expert_ids):
                src, dst = f"{prefix}local_experts.{local}.", f"{prefix}experts.{glob}."
                for n in names:
                    if n.startswith(src):
                        out[n] = dst + n[len(src):]
        return out

    def annotate_param_metadata(self) -> None:
        sm = self.runtime.state_manager
        for name, logical in self._runtime_to_logical().items():
            t = sm.get_model_tensor(name)
            sm.update_model_state(name, logical_names=[logical], logical_shapes=[tuple(t.shape)], physical_shape=tuple(t.shape), dtype=str(t.dtype))
        group = self.edp_group
        if group is not None and dist.get_world_size(group) > 1:
            for name, entry in sm.params.items():
                if id(entry.param) in self._expert_param_ids:
                    sm.update_model_state(name, replicated_axes=entry.attrs.replicated_axes | {MeshAxis.EREP})

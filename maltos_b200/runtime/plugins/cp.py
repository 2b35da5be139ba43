"""Context parallelism: the sequence is split over the CP axis.

* TRANSFORM: every attention block named by ``model.context_parallel_spec()`` gets its ``attn_core`` replaced by the
  all-gather-KV core or the ring core (``plan.cp_attn_core``).
* PRE_STEP_RUNNER: unless the loader already produced CP-local batches (``plan.batch_data_cp_aware``), the canonical
  batch is cut with the plan's token planner (contiguous for all-gather-KV, zigzag for ring by default); the local loss
  is weighted by ``local_targets / global_targets`` so that the SUM over CP ranks is the global mean.
* gradients of non-expert parameters are summed over the CP group: ZeRO plugins already reduce over DP x CP (their
  shard group), otherwise this plugin all-reduces at the window-closing POST_BACKWARD and waits at PRE_STEP.
Reference: ``runtime/plugins/cp.py:56-238``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.parallel.context_batch import ContextParallelBatchSharder
from maltos_b200.parallel.context_interfaces import ContextParallelAttentionCoreType
from maltos_b200.parallel.context_token_planner import ContextTokenPlannerType, build_context_token_planner
from maltos_b200.parallel.protocols import ContextParallelizableModule
from maltos_b200.runtime.layers.all_gather_attention import AllGatherKvAttentionCore
from maltos_b200.runtime.layers.ring_attention import RingAttentionCore
from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import ParamRole, RuntimePhase, SetupPhase
from maltos_b200.utils.distributed import all_reduce_tensor

_ZERO = (PluginId.ZERO1, PluginId.ZERO2, PluginId.ZERO3)


class ContextParallelPlugin(RuntimePlugin):
    def __init__(self) -> None:
        # after the data-parallel plugins: their reductions of the same gradient tensors (blocking or bucketed) are complete
        # when this plugin adds the sum over the context-parallel group - two collectives in flight on one tensor would race
        super().__init__(id=PluginId.CP, name="context_parallel", runs_after={PluginId.PP, PluginId.TP, PluginId.TP_SP, PluginId.DP, PluginId.EP})
        self._sharder: ContextParallelBatchSharder | None = None
        self._pending: list = []

    @property
    def cp_group(self):
        return self.runtime.get_group(MeshAxis.CP)

    def bind(self, runtime) -> None:
        super().bind(runtime)
        if runtime.mesh.cp <= 1:
            raise ValueError("ContextParallelPlugin requires mesh.cp > 1")
        if runtime.has_plugin(PluginId.HDP):
            raise ValueError("ContextParallelPlugin and ByteScaleHdpPlugin are mutually exclusive")

    def planner_type(self) -> ContextTokenPlannerType:
        plan = self.runtime.plan
        if plan.cp_token_planner is not None:
            return ContextTokenPlannerType(plan.cp_token_planner)
        ring = ContextParallelAttentionCoreType(plan.cp_attn_core) is ContextParallelAttentionCoreType.RING
        return ContextTokenPlannerType.FIXED_ZIGZAG if ring else ContextTokenPlannerType.FIXED_CONTIGUOUS

    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        if phase is SetupPhase.TRANSFORM:
            if not isinstance(model, ContextParallelizableModule):
                raise TypeError(f"ContextParallelPlugin requires model.context_parallel_spec(), got {type(model).__name__}")
            kind = ContextParallelAttentionCoreType(self.runtime.plan.cp_attn_core)
            for path in model.context_parallel_spec().attention_paths:
                if self.runtime.is_module_path_omitted(path):
                    continue
                try:
                    block = model.get_submodule(path)
                except AttributeError:
                    continue
                if block is None or not hasattr(block, "attn_core"):
                    continue
                backend = getattr(block.attn_core, "attention_backend", "eager")
                if kind is ContextParallelAttentionCoreType.RING:
                    core = RingAttentionCore(self.cp_group, backend)
                    core.bind_step_context(self.runtime.state.step_context)
                else:
                    core = AllGatherKvAttentionCore(self.cp_group, backend)
                block.attn_core = core
            self._sharder = ContextParallelBatchSharder(build_context_token_planner(self.planner_type()), self.runtime.mesh.cp)
        return model

    def annotate_param_metadata(self) -> None:
        sm = self.runtime.state_manager
        for name, entry in sm.params.items():
            if self.runtime.get_param_role(entry.param) != ParamRole.EXPERT or self.runtime.plan.reuse_cp_for_ep is False:
                sm.update_model_state(name, replicated_axes=entry.attrs.replicated_axes | {MeshAxis.CP})

    def _needs_own_grad_sync(self) -> bool:
        return not any(self.runtime.has_plugin(z) for z in _ZERO)

    def on_step_phase(self, phase: RuntimePhase) -> None:
        rt = self.runtime
        if phase is RuntimePhase.PRE_STEP_RUNNER:
            if not rt.plan.batch_data_cp_aware:
                rt.state.batch = self._sharder.shard(rt.state.batch, rank=dist.get_rank(self.cp_group))
            elif isinstance(rt.state.metadata.get("tokens_micro"), int):
                # the loader handed over this rank's share only: count the whole rows, as in the other arrangement
                rt.state.metadata["tokens_micro"] *= rt.mesh.cp
        elif phase is RuntimePhase.POST_BACKWARD:
            if self._needs_own_grad_sync() and rt.state.step_context.is_step_boundary:
                for p in rt.model.parameters():
                    if not p.requires_grad:
                        continue
                    if rt.get_param_role(p) == ParamRole.EXPERT and rt.plan.reuse_cp_for_ep:
                        continue
                    if p.grad is None:      # unused here, maybe used on another rank: same collectives everywhere
                        p.grad = torch.zeros_like(p)
                    w = all_reduce_tensor(p.grad, op=dist.ReduceOp.SUM, group=self.cp_group, async_op=True)
                    if w is not None:
                        self._pending.append(w)
                # all of them are in flight together, and all are finished before any later plugin (sequence-parallel partial
                # gradients at PRE_STEP, clipping) reads or reduces the same tensors
                for w in self._pending:
                    w.wait()
                self._pending.clear()

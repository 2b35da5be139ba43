"""Tensor + sequence parallelism.

Same sharding as TP, and between blocks activations are ``[B, S/T, H]``:

* ``embed`` (``SEQUENCE`` + ``scatter``): an ``nn.Embedding`` looks up only this rank's ``S/T`` token ids; any other
  module has its output narrowed.
* ``attn`` / ``mlp`` (``SEQUENCE`` + ``all_gather``): modules that declare ``handles_sequence_parallel_input`` call
  ``project_group`` themselves, which runs the ONE all-gather shared by q/k/v (gate/up) fused with the GEMMs
  (``sequence_parallel_grouped_linear``); other modules get a forward-pre hook that all-gathers their input.
  Row-parallel linears finish with GEMM -> reduce-scatter along the sequence.
* loss head: models that declare ``handles_sequence_parallel_loss`` keep the head sequence-parallel (each rank scores
  its own ``S/T`` tokens against the full vocabulary and the scalar loss is all-reduced) instead of all-gathering
  the hidden states and replicating the ``[B*S, V]`` logits on every rank as the reference does
  (``runtime/plugins/tp_sp.py:243-254``, ``models/llama.py:366-368``).

Parameters that stay TP-replicated but only see a sequence slice (norm weights, embeddings, the sequence-parallel
head, row-parallel biases) get partial gradients; their sum over the TP group is taken ONCE per optimizer step at
PRE_STEP when the runtime owns the optimizer, or per micro-step through gradient hooks when a ZeRO plugin consumes
gradients during backward.

``native_comm_overlap`` (reference ``tp_sp.py:108-119``): on CUDA the fused sm_100a all-gather->GEMM / GEMM->reduce-scatter
kernels are always the path when the TP group has peer access; the flag moves the creation of the group's symmetric-memory
context - and, with ``native_comm_overlap_workspace_bytes``, of its transfer buffers - from the first step to setup.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.parallel.protocols import TpSpParallelizableModule
from maltos_b200.parallel.specs import TpSpComm, TpSpShardAxis
from maltos_b200.runtime.layers.functional import all_gather, prewarm_native_comm_overlap_workspace
from maltos_b200.runtime.layers.linear import ColumnParallelLinear, RowParallelLinear
from maltos_b200.runtime.plugin import PluginId
from maltos_b200.runtime.types import ParamRole, RuntimePhase, SetupPhase
from maltos_b200.utils.distributed import all_reduce_tensor

from .tp import TensorParallelTransformPlugin

_ZERO = (PluginId.ZERO1, PluginId.ZERO2, PluginId.ZERO3)


@dataclass(frozen=True)
class _ProjectionGroup:
    module_path: str
    module: nn.Module
    linears: tuple[ColumnParallelLinear, ...]


class TpSpPlugin(TensorParallelTransformPlugin):
    sequence_parallel = True

    def __init__(self, *, native_comm_overlap: bool = False, native_comm_overlap_workspace_bytes: int | None = None) -> None:
        super().__init__(plugin_id=PluginId.TP_SP, name="tensor_sequence_parallel")
        self.native_comm_overlap = native_comm_overlap
        self.native_comm_overlap_workspace_bytes = native_comm_overlap_workspace_bytes
        self.native_comm_overlap_workspace_prewarmed = False
        self._projection_groups: list[_ProjectionGroup] = []
        self._gathered_paths: list[str] = []      # modules whose input covers the full sequence
        self._partial_params: list[nn.Parameter] = []
        self._hooked = False

    @property
    def sp_group(self):
        g = self.tp_group
        if g is None:
            raise ValueError("TpSpPlugin requires a TP process group")
        return g

    @property
    def rank(self) -> int:
        return dist.get_rank(self.sp_group)

    @property
    def world_size(self) -> int:
        return dist.get_world_size(self.sp_group)

    # ------------------------------------------------------------------ setup
    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        model = super().on_setup_phase(phase, model)
        if self.tp_group is None:
            return model
        if phase is SetupPhase.TRANSFORM:
            self._find_projection_groups(model)
        elif phase is SetupPhase.FINALIZE:
            if self.native_comm_overlap:
                if self.native_comm_overlap_workspace_bytes:
                    self.native_comm_overlap_workspace_prewarmed = prewarm_native_comm_overlap_workspace(
                        self.sp_group, min_workspace_bytes=int(self.native_comm_overlap_workspace_bytes))
                else:           # context (rendezvous, signal pad) only; the transfer buffers grow on first use
                    from maltos_b200.ops import comm

                    self.native_comm_overlap_workspace_prewarmed = comm.context_for(self.sp_group) is not None
            self._wire_sequence_rules(model)
            self._collect_partial_params(model)
        return model

    def _sequence_rules(self, model):
        if not isinstance(model, TpSpParallelizableModule):
            return
        for rule in model.tpsp_parallelize_spec().rules:
            if rule.shard_axis is TpSpShardAxis.SEQUENCE and not self.runtime.is_module_path_omitted(rule.module_path):
                try:
                    module = model.get_submodule(rule.module_path)
                except AttributeError:
                    continue
                if module is not None:
                    yield rule, module

    def _find_projection_groups(self, model: nn.Module) -> None:
        self._projection_groups.clear()
        for rule, module in self._sequence_rules(model):
            if rule.pre_comm is not TpSpComm.ALL_GATHER:
                continue
            cols = tuple(c for c in module.children() if isinstance(c, ColumnParallelLinear))
            if cols:
                self._projection_groups.append(_ProjectionGroup(rule.module_path, module, cols))

    def param_materialization_groups(self):
        """q/k/v (gate/up) weights are consumed by one fused op, so ZeRO-3 must gather them as one bucket."""
        return tuple((g.module, tuple(p for lin in g.linears for p in lin.parameters())) for g in self._projection_groups)

    def _wire_sequence_rules(self, model: nn.Module) -> None:
        self._gathered_paths.clear()
        grouped = {g.module: g for g in self._projection_groups}
        for rule, module in self._sequence_rules(model):
            if rule.pre_comm is TpSpComm.ALL_GATHER:
                if getattr(module, "handles_sequence_parallel_input", False):
                    self._gathered_paths.append(rule.module_path)
                    continue
                is_head = isinstance(module, nn.Linear) and getattr(model, "handles_sequence_parallel_loss", False)
                if is_head:
                    module.sp_loss_group = self.sp_group      # the model keeps the head sequence-parallel
                    continue
                self._gathered_paths.append(rule.module_path)
                has_group = module in grouped
                module.register_forward_pre_hook(self._gather_input_hook(rule.comm_dim, has_group))
            elif rule.post_comm is TpSpComm.SCATTER:
                if isinstance(module, nn.Embedding):
                    module.register_forward_pre_hook(self._narrow_ids_hook(rule.comm_dim))
                else:
                    module.register_forward_hook(self._narrow_output_hook(rule.comm_dim))
            else:
                raise NotImplementedError("TpSpPlugin supports sequence rules with pre_comm='all_gather' or post_comm='scatter', "
                                          f"got pre_comm={rule.pre_comm!r}, post_comm={rule.post_comm!r}")

    def _gather_input_hook(self, dim: int, reduce_in_backward: bool):
        def hook(module, args):
            x, *rest = args
            x = all_gather(x, self.sp_group, dim, backward_reduce=dist.ReduceOp.SUM if reduce_in_backward else None)
            return (x, *rest)

        return hook

    def _check_divisible(self, size: int, dim: int) -> None:
        if size % self.world_size:        # a floor division would silently drop the last tokens of every row
            raise ValueError(f"sequence parallelism needs dim {dim} (size {size}) divisible by the tensor-parallel size {self.world_size}")

    def _narrow_ids_hook(self, dim: int):
        def hook(module, args):
            ids, *rest = args
            self._check_divisible(ids.size(dim), dim)
            per = ids.size(dim) // self.world_size
            return (ids.narrow(dim, self.rank * per, per), *rest)

        return hook

    def _narrow_output_hook(self, dim: int):
        def hook(module, args, output):
            self._check_divisible(output.size(dim), dim)
            per = output.size(dim) // self.world_size
            return output.narrow(dim, self.rank * per, per)

        return hook

    # ------------------------------------------------------------------ partial gradients of replicated params
    def _collect_partial_params(self, model: nn.Module) -> None:
        self._partial_params = []
        by_id = {id(p): n for n, p in model.named_parameters()}
        row_bias = {id(m.bias) for m in model.modules() if isinstance(m, RowParallelLinear) and m.bias is not None}
        seen: set[int] = set()
        for name, p in model.named_parameters():
            if not p.requires_grad or id(p) in seen:
                continue
            seen.add(id(p))
            if self.is_tp_sharded(name):
                continue
            if self.runtime.get_param_role(p) == ParamRole.EXPERT and self.runtime.plan.reuse_tp_for_ep and self.runtime.mesh.ep > 1:
                # the expert group reuses the tensor-parallel ranks: each of them holds DIFFERENT experts (or a replica that the
                # expert plugin reduces itself over the expert-replica group) - summing them over the TP group would mix experts
                continue
            full_input = any(name == g or name.startswith(g + ".") for g in self._gathered_paths)
            if full_input and id(p) not in row_bias:
                continue  # its input covers the whole sequence: the gradient is already complete on every rank
            self._partial_params.append(p)
        del by_id
        if self._partial_params and any(self.runtime.has_plugin(z) for z in _ZERO) and not self._hooked:
            for p in self._partial_params:
                p.register_hook(self._sum_over_tp)
            self._hooked = True

    def _sum_over_tp(self, grad: torch.Tensor) -> torch.Tensor:
        g = grad.contiguous().clone()
        all_reduce_tensor(g, op=dist.ReduceOp.SUM, group=self.sp_group)
        return g

    def on_step_phase(self, phase: RuntimePhase) -> None:
        if phase is not RuntimePhase.PRE_STEP or self._hooked or self.tp_group is None:
            return
        works = []
        for p in self._partial_params:
            if p.grad is None:          # unused here, maybe used on another rank: same collectives everywhere
                p.grad = torch.zeros_like(p)
            works.append(all_reduce_tensor(p.grad, op=dist.ReduceOp.SUM, group=self.sp_group, async_op=True))
        for w in works:
            if w is not None:
                w.wait()

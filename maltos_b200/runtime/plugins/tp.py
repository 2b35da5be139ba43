"""Tensor parallelism (Megatron style).

TRANSFORM walks the model's ``tpsp_parallelize_spec()``: ``nn.Linear`` with ``PARAM_OUT`` becomes a
``ColumnParallelLinear`` holding rows ``[rank*out/T, (rank+1)*out/T)``, ``PARAM_IN`` a ``RowParallelLinear`` holding
the matching input columns (all-reduce / reduce-scatter / nothing afterwards, bias replicated and added after the
communication); a ``DistributedRMSNorm`` with ``PARAM_OUT`` keeps a weight slice and all-reduces its statistic.
Shards are cut from the full tensors at once, so the full copies die with the replaced modules. Parameter metadata
records logical vs physical shapes and the TP-sharded / TP-replicated axes (reference ``runtime/plugins/tp.py:53-236``).
"""
from __future__ import annotations

import torch.distributed as dist
import torch.nn as nn

from maltos_b200.parallel.protocols import TpSpParallelizableModule
from maltos_b200.parallel.specs import TpSpComm, TpSpShardAxis, TpSpShardRule
from maltos_b200.runtime.layers.distributed_rmsnorm import DistributedRMSNorm
from maltos_b200.runtime.layers.linear import ColumnParallelLinear, RowParallelLinear
from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import ParamRole, SetupPhase


def set_submodule(root: nn.Module, path: str, new: nn.Module) -> None:
    parent_path, _, leaf = path.rpartition(".")
    parent = root.get_submodule(parent_path) if parent_path else root
    if isinstance(parent, (nn.ModuleList, nn.Sequential)) and leaf.isdigit():
        parent[int(leaf)] = new
    else:
        setattr(parent, leaf, new)


class TensorParallelTransformPlugin(RuntimePlugin):
    """Sharding transform shared by the TP and TP+SP plugins."""

    sequence_parallel = False

    def __init__(self, *, plugin_id: PluginId, name: str) -> None:
        super().__init__(id=plugin_id, name=name)
        self._sharded: dict[str, TpSpShardAxis] = {}          # param name -> axis it is cut along
        self._logical_shapes: dict[str, tuple[int, ...]] = {}  # param name -> unsharded shape
        self._replicated_extra: set[str] = set()               # row-parallel biases

    @property
    def tp_group(self):
        return self.runtime.get_group(MeshAxis.TP)

    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        if phase is SetupPhase.TRANSFORM:
            return self._shard_model(model)
        return model

    # ------------------------------------------------------------------ transform
    def _shard_model(self, model: nn.Module) -> nn.Module:
        if not isinstance(model, TpSpParallelizableModule) or self.tp_group is None:
            return model
        rt = self.runtime
        for rule in model.tpsp_parallelize_spec().rules:
            if rt.is_module_path_omitted(rule.module_path):
                continue
            try:
                module = model.get_submodule(rule.module_path)
            except AttributeError:
                continue
            if module is None:
                continue
            if isinstance(module, nn.Linear) and rule.shard_axis is not TpSpShardAxis.SEQUENCE:
                self._note_linear(rule.module_path, module, rule.shard_axis)
                set_submodule(model, rule.module_path, self._make_linear(module, rule))
            elif isinstance(module, DistributedRMSNorm) and rule.shard_axis is not TpSpShardAxis.SEQUENCE:
                if rule.shard_axis is not TpSpShardAxis.PARAM_OUT:
                    raise ValueError(f"DistributedRMSNorm only supports PARAM_OUT sharding, got {rule.shard_axis} for {rule.module_path}")
                name = f"{rule.module_path}.weight"
                self._sharded[name] = rule.shard_axis
                self._logical_shapes[name] = (module.logical_hidden_size,)
                world, rank = dist.get_world_size(self.tp_group), dist.get_rank(self.tp_group)
                set_submodule(model, rule.module_path, DistributedRMSNorm.from_norm(module, self.tp_group, rank, world))
        rt.add_module_replacement(nn.Linear, ColumnParallelLinear)
        rt.add_module_replacement(nn.Linear, RowParallelLinear)
        rt.add_module_replacement(DistributedRMSNorm, DistributedRMSNorm)
        return model

    def _make_linear(self, module: nn.Linear, rule: TpSpShardRule) -> nn.Module:
        if rule.shard_axis is TpSpShardAxis.PARAM_OUT:
            new = ColumnParallelLinear.from_linear(module, self.tp_group, gather_output=(rule.post_comm is TpSpComm.ALL_GATHER),
                                                   input_is_replicated=not self.sequence_parallel)
            new.sequence_parallel = self.sequence_parallel
            return new
        comm_dim = rule.comm_dim
        if rule.post_comm is TpSpComm.REDUCE_SCATTER and comm_dim in (-1, 0):
            comm_dim = 1  # activations are [batch, sequence, hidden]: the scatter runs along the sequence
        new = RowParallelLinear.from_linear(module, self.tp_group, rule.post_comm.value, comm_dim)
        new.sequence_parallel = self.sequence_parallel
        return new

    def _note_linear(self, path: str, module: nn.Linear, axis: TpSpShardAxis) -> None:
        w = f"{path}.weight"
        self._sharded[w] = axis
        self._logical_shapes[w] = tuple(module.weight.shape)
        if module.bias is not None:
            b = f"{path}.bias"
            self._logical_shapes[b] = tuple(module.bias.shape)
            if axis is TpSpShardAxis.PARAM_OUT:
                self._sharded[b] = axis
            else:
                self._replicated_extra.add(b)

    # ------------------------------------------------------------------ metadata
    def annotate_param_metadata(self) -> None:
        sm = self.runtime.state_manager
        for name, shape in self._logical_shapes.items():
            if name not in sm.params:
                continue
            p = sm.get_model_tensor(name)
            sm.update_model_state(name, logical_names=[name], logical_shapes=[shape], physical_shape=tuple(p.shape), dtype=str(p.dtype))
        if self.runtime.mesh.tp <= 1:
            return
        for name in self._sharded:
            if name in sm.params:
                sm.update_model_state(name, sharded_axes=sm.params[name].attrs.sharded_axes | {MeshAxis.TP})
        for name, entry in sm.params.items():
            if name in self._sharded:
                continue
            if name not in self._replicated_extra and self.runtime.get_param_role(entry.param) is not ParamRole.SHARED:
                continue
            sm.update_model_state(name, replicated_axes=entry.attrs.replicated_axes | {MeshAxis.TP})

    def is_tp_sharded(self, param_name: str) -> bool:
        return param_name in self._sharded


class TensorParallelPlugin(TensorParallelTransformPlugin):
    def __init__(self) -> None:
        super().__init__(plugin_id=PluginId.TP, name="tensor_parallel")

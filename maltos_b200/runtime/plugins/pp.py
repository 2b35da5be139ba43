"""Pipeline parallelism: contiguous, balanced split of the model's ``pipe_layers`` over the PP axis, head layers kept
on the first stage and tail layers on the last; removed modules become ``None`` (their paths are marked omitted so later
plugins skip them) and out-of-stage blocks are replaced by identity layers so indices keep their meaning.
Owns the step runner (AFAB or 1F1B over point-to-point). Reference: ``runtime/plugins/pp.py:19-158``."""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.parallel.protocols import PipelineParallelizableModule
from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.step_runners.pipeline import PipelineScheduleKind, PipelineStepRunner
from maltos_b200.runtime.types import SetupPhase

from .tp import set_submodule


class _IdentityPipeLayer(nn.Module):
    """Stands in for a block that lives on another stage."""

    def forward(self, *args, **kwargs):
        if not args:
            raise ValueError("identity pipe layer expects at least one positional argument")
        return args[0]


def stage_layer_range(num_layers: int, stage: int, stages: int) -> tuple[int, int]:
    base, extra = divmod(num_layers, stages)
    start = stage * base + min(stage, extra)
    return start, start + base + (1 if stage < extra else 0)


_layer_range = stage_layer_range


class PipelineParallelPlugin(RuntimePlugin):
    def __init__(self, schedule: str = "afab") -> None:
        super().__init__(id=PluginId.PP, name="pipeline_parallel", owns_step_runner=True,
                         runs_before={PluginId.DP, PluginId.ZERO1, PluginId.ZERO2, PluginId.ZERO3, PluginId.TP, PluginId.TP_SP,
                                      PluginId.EP, PluginId.FP16})
        self.schedule = PipelineScheduleKind(schedule)
        self.stage_index, self.stage_count = 0, 1
        self.prev_global_rank: int | None = None
        self.next_global_rank: int | None = None
        self.last_global_rank = 0
        self.hidden_size = 0
        self.pp_group = None
        self.sequence_parallel_enabled = False
        self.sequence_parallel_world_size = 1

    def bind(self, runtime) -> None:
        super().bind(runtime)
        self.sequence_parallel_enabled = runtime.has_plugin(PluginId.TP_SP)
        self.sequence_parallel_world_size = runtime.mesh.tp if self.sequence_parallel_enabled else 1

    def build_step_runner(self):
        return PipelineStepRunner(self)

    def _rank_of_stage(self, stage: int) -> int:
        mesh = self.runtime.mesh
        dp, _, cp, tp = mesh.rank_coordinates(dist.get_rank())
        return mesh.rank_id(dp=dp, pp=stage, cp=cp, tp=tp)

    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        if phase is not SetupPhase.TRANSFORM:
            return model
        rt = self.runtime
        if rt.mesh.pp <= 1:
            raise ValueError("PipelineParallelPlugin requires mesh.pp > 1")
        if not dist.is_initialized():
            raise ValueError("PipelineParallelPlugin requires torch.distributed to be initialized")
        if not isinstance(model, PipelineParallelizableModule):
            raise TypeError(f"PipelineParallelPlugin requires model.pipeline_parallel_spec(), got {type(model).__name__}")
        self.pp_group = rt.get_group(MeshAxis.PP)
        _, stage, _, _ = rt.mesh.rank_coordinates(dist.get_rank())
        self.stage_index, self.stage_count = stage, rt.mesh.pp
        self.prev_global_rank = self._rank_of_stage(stage - 1) if stage > 0 else None
        self.next_global_rank = self._rank_of_stage(stage + 1) if stage + 1 < self.stage_count else None
        self.last_global_rank = self._rank_of_stage(self.stage_count - 1)
        spec = model.pipeline_parallel_spec()
        self.hidden_size = _infer_hidden_size(model, spec)
        for path in spec.head_layers:
            if stage != 0:
                rt.mark_module_path_omitted(path)
                set_submodule(model, path, None)
        for path in spec.tail_layers:
            if stage != self.stage_count - 1:
                rt.mark_module_path_omitted(path)
                set_submodule(model, path, None)
        for path in spec.pipe_layers:
            blocks = model.get_submodule(path)
            if not isinstance(blocks, nn.ModuleList):
                raise TypeError(f"PipelineParallelPlugin expects pipe layer path={path!r} to be nn.ModuleList, got {type(blocks).__name__}")
            lo, hi = stage_layer_range(len(blocks), stage, self.stage_count)
            kept = []
            for i, block in enumerate(blocks):
                if lo <= i < hi:
                    kept.append(block)
                else:
                    rt.mark_module_path_omitted(f"{path}.{i}")
                    kept.append(_IdentityPipeLayer())
            set_submodule(model, path, nn.ModuleList(kept))
        return model

    def annotate_param_metadata(self) -> None:
        return


def _infer_hidden_size(model: nn.Module, spec) -> int:
    for path in spec.head_layers:
        m = model.get_submodule(path)
        if isinstance(m, nn.Embedding):
            return int(m.embedding_dim)
    for path in spec.tail_layers:
        w = getattr(model.get_submodule(path), "weight", None)
        if torch.is_tensor(w) and w.ndim >= 1:
            return int(w.shape[0])
    raise ValueError("unable to infer PP hidden size from model/spec")

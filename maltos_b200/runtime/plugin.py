"""Plugin contract of the runtime core.

A plugin is a dataclass with an id, ordering constraints (``requires`` / ``runs_after`` / ``runs_before``) and
optional ownership of the optimizer, the step runner or the model state. The core calls ``bind`` once, then
``on_setup_phase`` for TRANSFORM / MATERIALIZE / FINALIZE, ``annotate_param_metadata``, and ``on_step_phase``
around every forward/backward/optimizer step (reference ``runtime/plugin.py:26-163``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import TYPE_CHECKING, Protocol, runtime_checkable

import torch
import torch.nn as nn

from maltos_b200.parallel.protocols import (ContextParallelizableModule, ExpertParallelizableModule,  # noqa: F401
                                            FlopsEstimatableModule, PipelineParallelizableModule,
                                            TpSpParallelizableModule)

from .types import MetricValue, RuntimePhase, SetupPhase

if TYPE_CHECKING:
    from maltos_b200.state.state import ModelStateMeta, StateManager

    from .core import RuntimeCore
    from .step_runners import StepRunner


class PluginId(str, Enum):
    FP16 = "fp16"
    GRAD_CLIP = "grad_clip"
    TP = "tp"
    TP_SP = "tp_sp"
    DP = "dp"
    PP = "pp"
    CP = "cp"
    HDP = "hdp"
    EP = "ep"
    ZERO1 = "zero1"
    ZERO2 = "zero2"
    ZERO3 = "zero3"
    CHECKPOINT = "checkpoint"
    METRICS = "metrics"
    TORCH_PROFILER = "torch_profiler"
    COMPILE = "compile"
    CUDA_GRAPH = "cuda_graph"     # not in the reference: micro-step recorded into a CUDA graph
    TOKEN_WEIGHTED_LOSS = "token_weighted_loss"     # not in the reference: loss averaged over targets across data-parallel ranks


@runtime_checkable
class OptimizerOwner(Protocol):
    def get_optimizer_and_scheduler(self): ...

    def optimizer_state_source_rank(self, rank_id: int) -> int: ...


@runtime_checkable
class StepRunnerOwner(Protocol):
    def build_step_runner(self): ...


@runtime_checkable
class ModelStateOwner(Protocol):
    def export_model_state(self, state_manager): ...

    def import_model_state(self, state_manager, model_state) -> None: ...


@runtime_checkable
class ParamMaterializationGroupProvider(Protocol):
    """Lets a plugin tell ZeRO-3 which parameters must be gathered together (e.g. q/k/v of one attention)."""

    def param_materialization_groups(self) -> tuple[tuple[nn.Module, tuple[nn.Parameter, ...]], ...]: ...


_OWNERSHIP = (
    ("owns_optimizer", OptimizerOwner, "OptimizerOwner"),
    ("owns_step_runner", StepRunnerOwner, "StepRunnerOwner"),
    ("owns_model_state", ModelStateOwner, "ModelStateOwner"),
)


@dataclass
class RuntimePlugin:
    id: PluginId
    name: str | None = None
    requires: set[PluginId] = field(default_factory=set)
    runs_after: set[PluginId] = field(default_factory=set)
    runs_before: set[PluginId] = field(default_factory=set)
    owns_optimizer: bool = False
    owns_step_runner: bool = False
    owns_model_state: bool = False
    runtime: "RuntimeCore | None" = field(default=None, init=False, repr=False)

    def __post_init__(self) -> None:
        self.name = self.name or self.id.value
        for flag, proto, label in _OWNERSHIP:
            if getattr(self, flag) and not isinstance(self, proto):
                raise ValueError(f"plugin={self.id.value} {flag}=True must satisfy {label}")

    # ---- lifecycle
    def bind(self, runtime: "RuntimeCore") -> None:
        self.runtime = runtime

    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        return model

    def annotate_param_metadata(self) -> None:
        """Record sharded/replicated axes and logical shapes of parameters after all transforms ran."""

    def on_step_phase(self, phase: RuntimePhase) -> None:
        return None

    def close(self) -> None:
        return None

    # ---- ownership hooks
    def build_step_runner(self) -> "StepRunner | None":
        return None

    def get_optimizer_and_scheduler(self):
        return getattr(self, "optimizer", None), getattr(self, "scheduler", None)

    def optimizer_state_source_rank(self, rank_id: int) -> int:
        raise NotImplementedError(f"plugin={self.id.value} owns_optimizer={self.owns_optimizer} must implement optimizer_state_source_rank()")

    def export_model_state(self, state_manager: "StateManager") -> "tuple[dict[str, torch.Tensor], list[ModelStateMeta]]":
        raise NotImplementedError(f"plugin={self.id.value} owns_model_state={self.owns_model_state} must implement export_model_state()")

    def import_model_state(self, state_manager: "StateManager", model_state: dict[str, torch.Tensor]) -> None:
        raise NotImplementedError(f"plugin={self.id.value} owns_model_state={self.owns_model_state} must implement import_model_state()")

    # ---- checkpointable plugin state & metrics
    def export_plugin_state(self) -> dict[str, object]:
        return {}

    def import_plugin_state(self, state: dict[str, object]) -> None:
        return None

    def collect_metrics(self) -> dict[str, MetricValue]:
        return {}

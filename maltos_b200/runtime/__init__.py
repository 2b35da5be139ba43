"""Runtime core: execution engine, mesh, plugin contract, step runners, buffer pool (lazy re-exports)."""
from __future__ import annotations

from importlib import import_module

_WHERE = {
    "buffer_allocator": ("BufferHandle", "BufferPolicy", "BufferPool", "acquire_buffer", "clear_buffer_pool",
                         "global_buffer_pool", "release_buffer"),
    "core": ("RuntimeCore",),
    "mesh": ("MeshAxis", "MeshConfig", "ProcessGroupManager"),
    "optim": ("FusedAdamW", "MasterWeightsOptimizer"),
    "plugin": ("ContextParallelizableModule", "ExpertParallelizableModule", "PipelineParallelizableModule",
               "PluginId", "RuntimePlugin", "TpSpParallelizableModule"),
    "step_runners": ("DefaultStepRunner", "PipelineScheduleKind", "PipelineStepRunner", "StepRunner"),
    "types": ("LossOutput", "MetricValue", "ParamRole", "PipelineOutput", "PpStatus", "RuntimePhase", "RuntimeState",
              "SetupPhase", "StepContext"),
}
_EXPORTS = {name: mod for mod, names in _WHERE.items() for name in names}
__all__ = sorted(_EXPORTS)


def __getattr__(name: str):
    mod = _EXPORTS.get(name)
    if mod is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(import_module(f"{__name__}.{mod}"), name)
    globals()[name] = value
    return value

"""Checkpointable state: the state index, sharded runtime checkpoints and logical (safetensors) checkpoints."""
from .checkpoint import (CheckpointArtifact, CheckpointManifest, RankCheckpointMetadata, load_checkpoint_manifest,
                         load_runtime_spec, load_sharded_checkpoint, save_runtime_spec, save_sharded_checkpoint,
                         save_sharded_checkpoint_from_model_state)
from .state import (BufferEntry, ModelStateMeta, OptimizerState, ParamEntry, RngState, RuntimeParamAttrs, StateManager,
                    TrainerState)

__all__ = [
    "BufferEntry", "CheckpointArtifact", "CheckpointManifest", "ModelStateMeta", "OptimizerState", "ParamEntry",
    "RankCheckpointMetadata", "RngState", "RuntimeParamAttrs", "StateManager", "TrainerState",
    "load_checkpoint_manifest", "load_runtime_spec", "load_sharded_checkpoint", "save_runtime_spec",
    "save_sharded_checkpoint", "save_sharded_checkpoint_from_model_state",
]


def __getattr__(name: str):
    # logical-checkpoint helpers pull in safetensors; import them on first use
    if name in {"save_logical_checkpoint", "load_logical_checkpoint", "load_logical_tensor",
                "iter_logical_checkpoint_tensors", "iter_logical_tensors_from_runtime_checkpoint",
                "LogicalCheckpointTensorReader"}:
        from . import logical_checkpoint

        return getattr(logical_checkpoint, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

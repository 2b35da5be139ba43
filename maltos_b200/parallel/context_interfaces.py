"""Contract of an attention core that a context-parallel plugin installs into a model."""
from __future__ import annotations

from enum import Enum
from typing import Protocol, runtime_checkable

import torch


class ContextParallelAttentionCoreType(str, Enum):
    ALL_GATHER_KV = "all_gather_kv"
    RING = "ring"


@runtime_checkable
class ContextParallelAttentionCore(Protocol):
    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, position_offset: int,
                 position_ids: torch.Tensor | None = None, sequence_ids: torch.Tensor | None = None) -> torch.Tensor: ...

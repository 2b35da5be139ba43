from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ContextParallelSpec:
    """Module paths of attention blocks whose ``attn_core`` a context-parallel plugin may replace."""

    attention_paths: list[str]

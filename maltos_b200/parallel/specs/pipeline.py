from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class PipelineParallelSpec:
    """``head_layers`` live on the first stage, ``tail_layers`` on the last, ``pipe_layers`` are ModuleLists
    that are split into contiguous, balanced chunks over the stages."""

    head_layers: list[str]
    pipe_layers: list[str]
    tail_layers: list[str]

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ExpertParallelSpec:
    """Module paths of mixture-of-experts blocks that can be expert-parallelised."""

    moe_paths: list[str]

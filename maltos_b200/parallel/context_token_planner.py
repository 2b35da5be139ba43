"""Which CP rank owns which canonical sequence position.

Two fixed layouts (reference ``parallel/context_token_planner.py:56-103``): contiguous equal chunks
(``S % C == 0``) and the zigzag split used by ring attention (``S % 2C == 0``; rank r owns chunks r and
2C-1-r so that causal work is balanced).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Protocol, Sequence

import torch


class ContextTokenPlannerType(str, Enum):
    FIXED_CONTIGUOUS = "fixed_contiguous"
    FIXED_ZIGZAG = "fixed_zigzag"

    @property
    def planner_class(self):
        return {
            ContextTokenPlannerType.FIXED_CONTIGUOUS: FixedContiguousTokenPlanner,
            ContextTokenPlannerType.FIXED_ZIGZAG: FixedZigzagTokenPlanner,
        }[self]


@dataclass(frozen=True)
class ContextTokenPlan:
    """``owner_ranks[p]`` = CP rank that holds canonical position ``p`` (same for every batch row)."""

    owner_ranks: torch.Tensor

    def local_positions(self, rank: int) -> torch.Tensor:
        if self.owner_ranks.dim() != 1:
            raise ValueError(f"fixed CP layouts carry one owner per position, got shape {tuple(self.owner_ranks.shape)}")
        return (self.owner_ranks == rank).nonzero(as_tuple=False).flatten()


class ContextTokenPlanner(Protocol):
    planner_type: ContextTokenPlannerType

    def plan(self, *, sequence_lengths: Sequence[int], world_size: int, device: torch.device | None = None) -> ContextTokenPlan: ...


def _common_length(sequence_lengths: Sequence[int]) -> int:
    lengths = [int(x) for x in sequence_lengths]
    if not lengths:
        raise ValueError("Context token planning requires at least one sequence length")
    if min(lengths) < 1:
        raise ValueError(f"Context token lengths must be >= 1, got {tuple(lengths)}")
    if len(set(lengths)) != 1:
        raise ValueError(f"fixed CP token planners require a rectangular batch with equal sequence lengths, got {tuple(lengths)}")
    return lengths[0]


class FixedContiguousTokenPlanner:
    planner_type = ContextTokenPlannerType.FIXED_CONTIGUOUS

    def plan(self, *, sequence_lengths, world_size, device=None) -> ContextTokenPlan:
        n = _common_length(sequence_lengths)
        if n % world_size:
            raise ValueError(f"fixed contiguous layout requires sequence length divisible by cp world size, got seq_len={n}, cp={world_size}")
        per = n // world_size
        return ContextTokenPlan(torch.arange(n, dtype=torch.long, device=device).div(per, rounding_mode="floor"))


class FixedZigzagTokenPlanner:
    planner_type = ContextTokenPlannerType.FIXED_ZIGZAG

    def plan(self, *, sequence_lengths, world_size, device=None) -> ContextTokenPlan:
        n = _common_length(sequence_lengths)
        if n % (2 * world_size):
            raise ValueError(f"CP ring zigzag requires sequence length divisible by 2 * cp world size, got seq_len={n}, cp={world_size}")
        half = n // (2 * world_size)
        chunk = torch.arange(n, dtype=torch.long, device=device).div(half, rounding_mode="floor")
        owners = torch.where(chunk < world_size, chunk, 2 * world_size - 1 - chunk)
        return ContextTokenPlan(owners)


def build_context_token_planner(planner_type: ContextTokenPlannerType | str) -> ContextTokenPlanner:
    return ContextTokenPlannerType(planner_type).planner_class()

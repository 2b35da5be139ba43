"""Canonical batch -> this CP rank's local batch (usable by a CP-aware loader or by the CP plugin after H2D).

Selects the owned positions of ``input_ids / labels / hidden_states / position_ids / sequence_ids``, makes
``position_ids`` explicit, and records ``position_offset`` and ``loss_weight = local_targets / global_targets``
(reference ``parallel/context_batch.py:39-79,146-153``), plus the per-row counts behind that weight, so that a pipeline
runner can weight each of its micro-batches exactly (rows of a packed batch do not split their targets evenly).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from maltos_b200.utils.constants import (AUX_LOSS_WEIGHT_KEY, HIDDEN_STATES_KEY, IGNORE_INDEX, INPUT_IDS_KEY, LABELS_KEY, LOSS_TARGET_COUNTS_KEY,
                                         LOSS_WEIGHT_KEY, POSITION_IDS_KEY, POSITION_OFFSET_KEY, SEQUENCE_IDS_KEY)

from .context_token_planner import ContextTokenPlanner

_SEQ_KEYS = (INPUT_IDS_KEY, LABELS_KEY, HIDDEN_STATES_KEY, POSITION_IDS_KEY, SEQUENCE_IDS_KEY)


def _first_2d(values) -> torch.Tensor | None:
    for v in values:
        if torch.is_tensor(v) and v.dim() >= 2:
            return v
    return None


def _take(value: Any, positions: torch.Tensor, seq_len: int) -> Any:
    if not torch.is_tensor(value):
        return value
    idx = positions.to(value.device)
    if value.dim() >= 2 and value.size(1) == seq_len:
        return value.index_select(1, idx).contiguous()
    if value.dim() == 1 and value.size(0) == seq_len:
        return value.index_select(0, idx).contiguous()
    return value


def _target_counts(full_labels: Any, local_labels: Any) -> torch.Tensor | None:
    """Host tensor ``[rows, 2]``: targets of each row owned by this rank, and in the whole row (one device read)."""
    if not (torch.is_tensor(full_labels) and torch.is_tensor(local_labels)) or full_labels.dim() != 2 or local_labels.dim() != 2:
        return None
    return torch.stack([(local_labels != IGNORE_INDEX).sum(1), (full_labels != IGNORE_INDEX).sum(1)], dim=1).to("cpu", torch.float64)


def target_fraction(counts: torch.Tensor | None) -> float | None:
    """``local targets / global targets`` over the rows of ``counts``; None when there is no target at all."""
    if counts is None:
        return None
    local, total = counts.sum(0).tolist()
    return local / total if total else None


@dataclass(frozen=True)
class ContextParallelBatchSharder:
    planner: ContextTokenPlanner
    world_size: int

    def __post_init__(self) -> None:
        if self.world_size < 1:
            raise ValueError(f"CP world_size must be >= 1, got {self.world_size}")

    def shard(self, batch: Any, *, rank: int) -> Any:
        if not 0 <= rank < self.world_size:
            raise ValueError(f"CP rank must be in [0, {self.world_size}), got {rank}")
        if self.world_size == 1:
            return batch
        if isinstance(batch, dict):
            items = dict(batch)
        elif isinstance(batch, (tuple, list)):
            items = {INPUT_IDS_KEY: batch[0] if len(batch) > 0 else None, LABELS_KEY: batch[1] if len(batch) > 1 else None}
        else:
            raise TypeError(f"ContextParallelBatchSharder does not support batch type={type(batch).__name__}")
        ref = _first_2d(items.get(k) for k in (INPUT_IDS_KEY, LABELS_KEY, HIDDEN_STATES_KEY, SEQUENCE_IDS_KEY))
        if ref is not None:
            seq_len, rows = int(ref.size(1)), int(ref.size(0))
        else:
            pos = items.get(POSITION_IDS_KEY)
            if not torch.is_tensor(pos):
                raise TypeError("ContextParallelBatchSharder could not infer sequence length from batch")
            seq_len, rows = int(pos.size(-1)), int(pos.size(0)) if pos.dim() >= 2 else 1
        plan = self.planner.plan(sequence_lengths=[seq_len] * rows, world_size=self.world_size)
        mine = plan.local_positions(rank)
        full_labels = items.get(LABELS_KEY)
        out = dict(items)
        for key in _SEQ_KEYS:
            out[key] = _take(items.get(key), mine, seq_len)
        local_ref = _first_2d(out.get(k) for k in (INPUT_IDS_KEY, LABELS_KEY, HIDDEN_STATES_KEY, SEQUENCE_IDS_KEY))
        pos_ids = out.get(POSITION_IDS_KEY)
        if torch.is_tensor(pos_ids):
            pos_ids = pos_ids.to(dtype=torch.long)
            if local_ref is not None:
                pos_ids = pos_ids.to(local_ref.device)
        elif local_ref is not None:
            pos_ids = mine.to(local_ref.device).unsqueeze(0).expand(local_ref.size(0), -1).contiguous()
        else:
            pos_ids = mine.clone()
        out[POSITION_IDS_KEY] = pos_ids
        out[POSITION_OFFSET_KEY] = int(mine[0])
        counts = _target_counts(full_labels, out.get(LABELS_KEY))
        out[LOSS_WEIGHT_KEY] = target_fraction(counts)
        if counts is not None:
            out[LOSS_TARGET_COUNTS_KEY] = counts
        out[AUX_LOSS_WEIGHT_KEY] = 1.0 / self.world_size      # every rank holds the same number of tokens
        if not isinstance(batch, dict):
            out = {k: out[k] for k in (INPUT_IDS_KEY, LABELS_KEY, POSITION_IDS_KEY, POSITION_OFFSET_KEY, LOSS_WEIGHT_KEY, AUX_LOSS_WEIGHT_KEY)}
        return out

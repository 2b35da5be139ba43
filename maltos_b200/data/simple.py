"""Deterministic tensor batcher with a checkpointable cursor, for tests (reference ``data/simple.py:17-73``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch


@dataclass(frozen=True)
class SimpleDataLoaderState:
    cursor: int
    epoch: int
    consumed_tokens: int


class SimpleTensorDataLoader:
    def __init__(self, data: torch.Tensor, batch_size: int, *, drop_last: bool = True, cp_batch_sharder=None) -> None:
        n = data.size(0)
        if n <= 0:
            raise ValueError("data must have a non-empty leading batch dimension")
        if batch_size < 1:
            raise ValueError(f"batch_size must be >= 1, got {batch_size}")
        if drop_last and batch_size > n:
            raise ValueError(f"batch_size={batch_size} exceeds dataset size={n}")
        self.data, self.batch_size, self.drop_last = data, batch_size, drop_last
        self.cursor = self.epoch = self.consumed_tokens = 0
        self._cp_batch_sharder = cp_batch_sharder

    def next_batch(self, cp_rank: int | None = None):
        n = self.data.size(0)
        if self.cursor + self.batch_size > n:      # not enough rows left for a full batch: start the next epoch
            self.epoch += 1
            self.cursor = 0
        end = min(self.cursor + self.batch_size, n)
        batch = self.data[self.cursor:end].contiguous()
        self.cursor = end
        self.consumed_tokens += batch.numel()
        if cp_rank is None:
            return batch
        if self._cp_batch_sharder is None:
            raise RuntimeError("CP-local next_batch(cp_rank) requires constructor cp_batch_sharder")
        return self._cp_batch_sharder.shard((batch,), rank=cp_rank)

    def state_dict(self) -> SimpleDataLoaderState:
        return SimpleDataLoaderState(self.cursor, self.epoch, self.consumed_tokens)

    def load_state_dict(self, state: dict[str, Any]) -> None:
        st = SimpleDataLoaderState(**state)
        if not 0 <= st.cursor <= self.data.size(0):
            raise ValueError(f"invalid dataloader cursor={st.cursor}")
        self.cursor, self.epoch, self.consumed_tokens = st.cursor, st.epoch, st.consumed_tokens

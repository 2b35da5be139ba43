"""Token-shard pretraining data: raw ``.bin`` token files are memory-mapped and read as one endless stream.

A sample is ``seq_len + 1`` consecutive tokens (inputs = first ``seq_len``, labels = last ``seq_len``). DP rank ``r``
starts ``r`` samples into the stream and, after each sample, skips the ``dp_world - 1`` samples of its peers, so ranks
never overlap and need no communication. The cursor ``(shard_idx, token_offset)`` plus ``consumed_tokens`` is the
whole resumable state (field names as in the reference's ``data/pretrain.py:12-18``, they are stored in checkpoints).
Cursor moves are computed arithmetically - skipped tokens are never read.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Iterable

import numpy as np
import torch

from maltos_b200.utils.constants import INPUT_IDS_KEY, LABELS_KEY


@dataclass(frozen=True)
class PretrainingDataState:
    shard_idx: int
    token_offset: int
    consumed_tokens: int
    seed: int


class TokenShardDataset:
    def __init__(self, paths: Iterable[str | Path], *, dtype=np.uint32) -> None:
        self.paths = [Path(p) for p in paths]
        if not self.paths:
            raise ValueError("TokenShardDataset requires at least one token shard")
        self.dtype = np.dtype(dtype)
        self.shards = [np.memmap(p, mode="r", dtype=self.dtype) for p in self.paths]
        for p, s in zip(self.paths, self.shards):
            if s.size == 0:
                raise ValueError(f"token shard is empty: {p}")
        self.sizes = [int(s.size) for s in self.shards]

    def __len__(self) -> int:
        return sum(self.sizes)

    def read(self, shard_idx: int, token_offset: int, length: int) -> tuple[np.ndarray, int, int]:
        """``length`` tokens starting at the cursor, streaming across shard boundaries. Returns (tokens, new cursor)."""
        if length < 1:
            raise ValueError(f"length must be >= 1, got {length}")
        out = np.empty(length, dtype=self.dtype)
        done = 0
        shard_idx %= len(self.shards)
        token_offset = int(token_offset)
        while done < length:
            size = self.sizes[shard_idx]
            if token_offset >= size:
                shard_idx, token_offset = (shard_idx + 1) % len(self.shards), 0
                continue
            take = min(length - done, size - token_offset)
            out[done:done + take] = self.shards[shard_idx][token_offset:token_offset + take]
            done += take
            token_offset += take
            if token_offset >= size and done < length:
                shard_idx, token_offset = (shard_idx + 1) % len(self.shards), 0
        return out, shard_idx, token_offset


class PretrainingDataLoader:
    def __init__(self, dataset: TokenShardDataset, *, seq_len: int, micro_batch_size: int, dp_rank: int = 0, dp_world_size: int = 1,
                 seed: int = 1234, start_state: PretrainingDataState | None = None, cp_batch_sharder=None) -> None:
        if seq_len < 1:
            raise ValueError(f"seq_len must be >= 1, got {seq_len}")
        if micro_batch_size < 1:
            raise ValueError(f"micro_batch_size must be >= 1, got {micro_batch_size}")
        if dp_world_size < 1:
            raise ValueError(f"dp_world_size must be >= 1, got {dp_world_size}")
        if not 0 <= dp_rank < dp_world_size:
            raise ValueError(f"dp_rank must be in [0, {dp_world_size}), got {dp_rank}")
        self.dataset = dataset
        self.seq_len, self.micro_batch_size = seq_len, micro_batch_size
        self.dp_rank, self.dp_world_size = dp_rank, dp_world_size
        self.seed = seed
        self._sample = seq_len + 1
        self.shard_idx = 0
        self.token_offset = dp_rank * self._sample
        self.consumed_tokens = 0
        self._cp_batch_sharder = cp_batch_sharder
        if start_state is not None:
            self.load_state_dict(asdict(start_state))

    def next_batch(self, cp_rank: int | None = None) -> dict[str, torch.Tensor]:
        rows = np.empty((self.micro_batch_size, self._sample), dtype=np.int64)
        skip = (self.dp_world_size - 1) * self._sample
        for i in range(self.micro_batch_size):
            toks, self.shard_idx, self.token_offset = self.dataset.read(self.shard_idx, self.token_offset, self._sample)
            rows[i] = toks
            if skip:
                self.shard_idx, self.token_offset = self._skip(skip)
        t = torch.from_numpy(rows)
        self.consumed_tokens += self.micro_batch_size * self.seq_len
        batch = {INPUT_IDS_KEY: t[:, :-1].contiguous(), LABELS_KEY: t[:, 1:].contiguous()}
        if cp_rank is None:
            return batch
        if self._cp_batch_sharder is None:
            raise RuntimeError("CP-local next_batch(cp_rank) requires constructor cp_batch_sharder")
        return self._cp_batch_sharder.shard(batch, rank=cp_rank)

    def _skip(self, count: int) -> tuple[int, int]:
        # same end position as reading `count` tokens and discarding them
        _, s, o = self._probe(count)
        return s, o

    def _probe(self, count: int):
        s, o = self.shard_idx, self.token_offset
        sizes = self.dataset.sizes
        n = len(sizes)
        remaining = count
        while remaining > 0:
            if o >= sizes[s]:
                s, o = (s + 1) % n, 0
                continue
            take = min(remaining, sizes[s] - o)
            o += take
            remaining -= take
            if o >= sizes[s] and remaining > 0:
                s, o = (s + 1) % n, 0
        return None, s, o

    def state_dict(self) -> PretrainingDataState:
        return PretrainingDataState(self.shard_idx, self.token_offset, self.consumed_tokens, self.seed)

    def load_state_dict(self, state: dict[str, Any]) -> None:
        st = PretrainingDataState(**state)
        if not 0 <= st.shard_idx < len(self.dataset.shards):
            raise ValueError(f"invalid shard_idx={st.shard_idx}")
        if not 0 <= st.token_offset <= self.dataset.sizes[st.shard_idx]:
            raise ValueError(f"invalid token_offset={st.token_offset}")
        self.shard_idx, self.token_offset = st.shard_idx, st.token_offset
        self.consumed_tokens, self.seed = st.consumed_tokens, st.seed

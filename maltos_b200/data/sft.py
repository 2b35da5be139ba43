"""Packed SFT data: ``meta.json`` (``format = "maltos_sft_packed"``) lists shard files and, per field, the dtype, byte
offset and ``[rows, seq_len]`` shape of a memory-mapped array (input_ids, labels, position_ids, sequence_ids). Rows are
dealt to DP ranks round-robin; the resumable state is ``(shard_idx, row_offset, consumed_tokens, consumed_sequences,
seed)`` (reference ``data/sft.py:41-245``)."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any

import numpy as np
import torch

from maltos_b200.utils.constants import SFT_BATCH_KEYS


@dataclass(frozen=True)
class SFTDataState:
    shard_idx: int
    row_offset: int
    consumed_tokens: int
    consumed_sequences: int
    seed: int


@dataclass(frozen=True)
class _Shard:
    path: Path
    sequences: int
    fields: dict[str, np.memmap]


def _meta_path(root_or_meta) -> Path:
    p = Path(root_or_meta)
    if p.is_dir():
        p = p / "meta.json"
    if not p.is_file():
        raise ValueError(f"SFT dataset meta.json not found at {p}")
    return p


def _open_field(path: Path, spec: Any) -> np.memmap:
    if not isinstance(spec, dict):
        raise ValueError(f"invalid SFT field spec: {spec!r}")
    shape = tuple(int(x) for x in spec["shape"])
    if len(shape) != 2:
        raise ValueError(f"SFT field shape must be [rows, seq_len], got {shape}")
    return np.memmap(path, mode="r", dtype=np.dtype(str(spec["dtype"])), offset=int(spec["offset"]), shape=shape)


class PackedSFTDataset:
    def __init__(self, root_or_meta) -> None:
        self.meta_path = _meta_path(root_or_meta)
        self.root = self.meta_path.parent
        meta = json.loads(self.meta_path.read_text(encoding="utf-8"))
        if meta.get("format") != "maltos_sft_packed":
            raise ValueError(f"unsupported SFT dataset format={meta.get('format')!r}")
        packing = meta.get("packing")
        if isinstance(packing, dict):
            layout, shard_list = packing.get("layout") or {}, packing.get("shards") or []
        else:
            layout, shard_list = meta, meta.get("shards") or []
        if not isinstance(shard_list, list) or not shard_list:
            raise ValueError(f"SFT dataset meta must define non-empty shards, got {type(shard_list)!r}")
        self.seq_len = int(layout.get("seq_len", meta.get("seq_len", 0)))
        if self.seq_len < 1:
            raise ValueError(f"SFT dataset seq_len must be >= 1, got {self.seq_len}")
        self.shards: list[_Shard] = []
        for item in shard_list:
            path = self.root / str(item["path"])
            fields = item.get("fields")
            if not isinstance(fields, dict):
                raise ValueError(f"invalid shard fields for {path}: {type(fields)!r}")
            self.shards.append(_Shard(path, int(item["sequences"]), {k: _open_field(path, fields.get(k)) for k in SFT_BATCH_KEYS}))
        self.shard_paths = [s.path for s in self.shards]
        self.total_sequences = sum(s.sequences for s in self.shards)
        if self.total_sequences < 1:
            raise ValueError("SFT dataset must contain at least one packed sequence")

    def __len__(self) -> int:
        return self.total_sequences

    def advance(self, shard_idx: int, row_offset: int, rows: int) -> tuple[int, int]:
        if rows < 0:
            raise ValueError(f"rows must be >= 0, got {rows}")
        shard_idx %= len(self.shards)
        left = rows % self.total_sequences if rows >= self.total_sequences else rows
        if rows and not left and rows >= self.total_sequences:
            left = 0
        while left > 0:
            size = self.shards[shard_idx].sequences
            if row_offset >= size:
                shard_idx, row_offset = (shard_idx + 1) % len(self.shards), 0
                continue
            room = size - row_offset
            if left < room:
                row_offset += left
                break
            left -= room
            shard_idx, row_offset = (shard_idx + 1) % len(self.shards), 0
        return shard_idx, row_offset

    def read_rows(self, shard_idx: int, row_offset: int, rows: int) -> tuple[dict[str, np.ndarray], int, int]:
        if rows < 1:
            raise ValueError(f"rows must be >= 1, got {rows}")
        out = {k: np.empty((rows, self.seq_len), dtype=self.shards[0].fields[k].dtype) for k in SFT_BATCH_KEYS}
        done = 0
        shard_idx %= len(self.shards)
        while done < rows:
            shard = self.shards[shard_idx]
            if row_offset >= shard.sequences:
                shard_idx, row_offset = (shard_idx + 1) % len(self.shards), 0
                continue
            take = min(rows - done, shard.sequences - row_offset)
            for k in SFT_BATCH_KEYS:
                out[k][done:done + take] = shard.fields[k][row_offset:row_offset + take]
            done += take
            row_offset += take
            if row_offset >= shard.sequences and done < rows:
                shard_idx, row_offset = (shard_idx + 1) % len(self.shards), 0
        return out, shard_idx, row_offset


class SFTDataLoader:
    def __init__(self, dataset: PackedSFTDataset, *, micro_batch_size: int, dp_rank: int = 0, dp_world_size: int = 1, seed: int = 1234,
                 start_state: SFTDataState | None = None, cp_batch_sharder=None) -> None:
        if micro_batch_size < 1:
            raise ValueError(f"micro_batch_size must be >= 1, got {micro_batch_size}")
        if dp_world_size < 1:
            raise ValueError(f"dp_world_size must be >= 1, got {dp_world_size}")
        if not 0 <= dp_rank < dp_world_size:
            raise ValueError(f"dp_rank must be in [0, {dp_world_size}), got {dp_rank}")
        self.dataset = dataset
        self.micro_batch_size, self.dp_rank, self.dp_world_size, self.seed = micro_batch_size, dp_rank, dp_world_size, seed
        self.shard_idx, self.row_offset = dataset.advance(0, 0, dp_rank)
        self.consumed_sequences = self.consumed_tokens = 0
        self._cp_batch_sharder = cp_batch_sharder
        if start_state is not None:
            self.load_state_dict(asdict(start_state))

    def next_batch(self, cp_rank: int | None = None) -> dict[str, torch.Tensor]:
        rows = {k: [] for k in SFT_BATCH_KEYS}
        for _ in range(self.micro_batch_size):
            sample, self.shard_idx, self.row_offset = self.dataset.read_rows(self.shard_idx, self.row_offset, 1)
            for k in SFT_BATCH_KEYS:
                rows[k].append(sample[k][0])
            self.shard_idx, self.row_offset = self.dataset.advance(self.shard_idx, self.row_offset, self.dp_world_size - 1)
        batch = {k: torch.from_numpy(np.stack(v).astype(np.int64, copy=False)).contiguous() for k, v in rows.items()}
        self.consumed_sequences += self.micro_batch_size
        self.consumed_tokens += self.micro_batch_size * self.dataset.seq_len
        if cp_rank is None:
            return batch
        if self._cp_batch_sharder is None:
            raise RuntimeError("CP-local next_batch(cp_rank) requires constructor cp_batch_sharder")
        return self._cp_batch_sharder.shard(batch, rank=cp_rank)

    def state_dict(self) -> SFTDataState:
        return SFTDataState(self.shard_idx, self.row_offset, self.consumed_tokens, self.consumed_sequences, self.seed)

    def load_state_dict(self, state: dict[str, Any]) -> None:
        st = SFTDataState(**state)
        if not 0 <= st.shard_idx < len(self.dataset.shards):
            raise ValueError(f"invalid shard_idx={st.shard_idx}")
        if not 0 <= st.row_offset <= self.dataset.shards[st.shard_idx].sequences:
            raise ValueError(f"invalid row_offset={st.row_offset}")
        self.shard_idx, self.row_offset = st.shard_idx, st.row_offset
        self.consumed_tokens, self.consumed_sequences, self.seed = st.consumed_tokens, st.consumed_sequences, st.seed

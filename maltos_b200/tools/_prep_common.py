"""Shared pieces of the data-preparation tools: row sources, tokenizer loading, progress lines."""
from __future__ import annotations

import csv
import json
import time
from pathlib import Path
from typing import Any, Iterable, Iterator

LOCAL_FILE_LOADERS = {".json": "json", ".jsonl": "json", ".parquet": "parquet", ".csv": "csv"}


def format_duration(seconds: float) -> str:
    s = int(seconds)
    h, s = divmod(s, 3600)
    m, s = divmod(s, 60)
    if h:
        return f"{h}h{m:02d}m{s:02d}s"
    return f"{m}m{s:02d}s" if m else f"{s}s"


class Progress:
    """Prints a line each time a counter crosses the next multiple of ``every``."""

    def __init__(self, every: int) -> None:
        self.every = every
        self.next_at = every
        self.start = time.perf_counter()

    def elapsed(self) -> float:
        return max(time.perf_counter() - self.start, 1e-9)

    def due(self, count: int) -> bool:
        if count < self.next_at:
            return False
        while count >= self.next_at:
            self.next_at += self.every
        return True


def load_tokenizer(name_or_path: str, expected_vocab_size: int | None):
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(name_or_path, use_fast=True)
    if expected_vocab_size is not None and len(tok) != expected_vocab_size:
        raise ValueError(f"tokenizer vocab size mismatch: tokenizer={name_or_path} vocab={len(tok)}, expected={expected_vocab_size}")
    return tok


def _read_local_file(path: Path) -> Iterator[dict[str, Any]]:
    """Rows of a local json / jsonl / csv / parquet file without needing the ``datasets`` package."""
    suffix = path.suffix.lower()
    if suffix == ".jsonl":
        with path.open(encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    yield json.loads(line)
    elif suffix == ".json":
        data = json.loads(path.read_text(encoding="utf-8"))
        rows = data if isinstance(data, list) else data.get("data", [])
        yield from rows
    elif suffix == ".csv":
        with path.open(encoding="utf-8", newline="") as f:
            yield from csv.DictReader(f)
    elif suffix == ".parquet":
        import pyarrow.parquet as pq

        for batch in pq.ParquetFile(str(path)).iter_batches():
            yield from batch.to_pylist()
    else:
        raise ValueError(f"unsupported local dataset file suffix={suffix!r}")


def open_rows(dataset: str, *, config: str | None, split: str, streaming: bool, seed: int, shuffle_buffer_size: int) -> Iterable[dict]:
    """Rows of a HF dataset id, a ``save_to_disk`` directory, or a single local data file.

    Local files are read directly (offline machines have no hub); everything else goes through ``datasets``. A streaming
    source is shuffled through a bounded buffer, like the reference tools do (``tools/prepare_token_shards.py:57-59``).
    """
    path = Path(dataset)
    if path.is_file():
        if path.suffix.lower() not in LOCAL_FILE_LOADERS:
            raise ValueError(f"unsupported local dataset file suffix={path.suffix.lower()!r}")
        try:
            from datasets import load_dataset
        except ImportError:
            return _read_local_file(path)
        ds = load_dataset(LOCAL_FILE_LOADERS[path.suffix.lower()], data_files=str(path), split=split, streaming=streaming)
    elif path.exists():
        from datasets import DatasetDict, load_from_disk

        if streaming:
            raise ValueError("streaming is not supported for local load_from_disk datasets")
        ds = load_from_disk(str(path))
        if isinstance(ds, DatasetDict):
            if split not in ds:
                raise ValueError(f"split={split!r} not found in local dataset; available={sorted(ds.keys())}")
            ds = ds[split]
        elif split != "train":
            raise ValueError("split selection for local on-disk Dataset is only supported when it is a DatasetDict")
    else:
        from datasets import load_dataset

        ds = load_dataset(dataset, name=config, split=split, streaming=streaming)
    if streaming:
        ds = ds.shuffle(seed=seed, buffer_size=shuffle_buffer_size)
    return ds

"""One-batch background prefetch with pinned host memory.

The wrapped loader runs one batch ahead on a worker thread; ``state_dict`` reports the cursor as it was BEFORE the
in-flight read, so a checkpoint taken now resumes with the batch the trainer has not consumed yet
(reference ``data/prefetch.py:10-75``). Pinned buffers let ``RuntimeCore.run_step`` overlap the H2D copy with compute.
"""
from __future__ import annotations

from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import asdict, is_dataclass
from typing import Any

import torch


def _as_dict(state: Any) -> dict[str, Any]:
    if is_dataclass(state) and not isinstance(state, type):
        return asdict(state)
    if isinstance(state, dict):
        return dict(state)
    raise TypeError(f"dataloader state must be a dataclass or dict, got {type(state)!r}")


def pin_batch(value: Any) -> Any:
    if not torch.cuda.is_available():
        return value
    if torch.is_tensor(value):
        return value.pin_memory() if value.device.type == "cpu" and not value.is_pinned() else value
    if isinstance(value, dict):
        return {k: pin_batch(v) for k, v in value.items()}
    if isinstance(value, (tuple, list)):
        return type(value)(pin_batch(v) for v in value)
    return value


class PrefetchDataLoader:
    def __init__(self, loader) -> None:
        self.loader = loader
        self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="maltos-data")
        self._inflight: Future | None = None
        self._state_before: dict[str, Any] | None = None

    def _fetch(self, cp_rank):
        return pin_batch(self.loader.next_batch(cp_rank))

    def next_batch(self, cp_rank: int | None = None) -> Any:
        if self._inflight is None:
            batch = self._fetch(cp_rank)
        else:
            batch = self._inflight.result()
            self._inflight, self._state_before = None, None
        self._state_before = _as_dict(self.loader.state_dict())
        self._inflight = self._pool.submit(self._fetch, cp_rank)
        return batch

    def state_dict(self):
        if self._state_before is not None:
            return dict(self._state_before)
        return self.loader.state_dict()

    def _drop_inflight(self) -> None:
        if self._inflight is not None:
            if not self._inflight.cancel():
                try:
                    self._inflight.result()
                except Exception:
                    pass
            self._inflight = None
        self._state_before = None

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self._drop_inflight()
        self.loader.load_state_dict(state)

    @property
    def consumed_tokens(self):
        return getattr(self.loader, "consumed_tokens", None)

    def close(self) -> None:
        self._drop_inflight()
        self._pool.shutdown(wait=True, cancel_futures=True)
        inner = getattr(self.loader, "close", None)
        if callable(inner):
            inner()

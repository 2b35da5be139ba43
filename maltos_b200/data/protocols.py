"""Contract of a resumable data loader (reference ``data/protocols.py:10-15``)."""
from __future__ import annotations

from typing import Any, Protocol, runtime_checkable


@runtime_checkable
class StatefulDataLoaderProtocol(Protocol):
    def next_batch(self, cp_rank: int | None = None) -> Any: ...

    def state_dict(self) -> Any: ...

    def load_state_dict(self, state: dict[str, Any]) -> None: ...

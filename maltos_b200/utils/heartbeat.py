"""Host-side liveness of the other ranks, checked between steps (the reference has no counterpart).

A rank that died leaves the survivors in their next collective until the process group's timeout - or, with the one-sided
kernels, in a bounded device wait that ends with ``CommTimeoutError``. Both are late and say little. Here every rank bumps
a counter in the job's key-value store from a background thread, and the same thread watches the counters of the others;
``check()``, called by the trainer before it launches a step, raises ``PeerLostError`` naming the ranks whose counter
has not moved for ``timeout`` seconds. Nothing touches a GPU, and the training thread never waits on the store: it only
reads what the thread has cached.

Ages are measured on the observer's monotonic clock from the moment IT saw a counter change, so clocks of different hosts
need not agree. A rank that finishes normally calls ``stop()``, which marks it as "left on purpose": the others do not
report it.
"""
from __future__ import annotations

import threading
import time

import torch.distributed as dist


class PeerLostError(RuntimeError):
    def __init__(self, ranks: list[int], silent_for: float) -> None:
        super().__init__(f"no heartbeat from rank(s) {ranks} for {silent_for:.1f} s; stopping before the next collective")
        self.ranks = ranks


class HeartbeatMonitor:
    def __init__(self, store, rank: int, world: int, *, interval: float = 1.0, timeout: float = 15.0, prefix: str = "maltos_b200/hb") -> None:
        if timeout <= 2 * interval:
            raise ValueError(f"timeout={timeout} must exceed two beat intervals ({interval} s each)")
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix = float(interval), float(timeout), prefix
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._lock = threading.Lock()
        self._seen: dict[int, tuple[int, float]] = {}          # peer -> (last counter value, monotonic time it changed)
        self._left: set[int] = set()
        self._error: str | None = None

    @classmethod
    def for_default_group(cls, **kw) -> "HeartbeatMonitor":
        from torch.distributed.distributed_c10d import _get_default_store

        return cls(_get_default_store(), dist.get_rank(), dist.get_world_size(), **kw)

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> "HeartbeatMonitor":
        now = time.monotonic()
        self._seen = {r: (-1, now) for r in range(self.world) if r != self.rank}
        self.store.add(f"{self.prefix}/{self.rank}", 1)
        self._thread = threading.Thread(target=self._run, name="maltos-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        """Normal end of this rank: tell the others not to miss it, then end the thread."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1.0)
            self._thread = None
        try:
            self.store.set(f"{self.prefix}/left/{self.rank}", "1")
        except Exception:  # noqa: BLE001 - the store's host may be gone already at shutdown
            pass

    # ------------------------------------------------------------------ background thread
    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self.store.add(f"{self.prefix}/{self.rank}", 1)
                now = time.monotonic()
                for peer in list(self._seen):
                    value = int(self.store.add(f"{self.prefix}/{peer}", 0))
                    left = self.store.check([f"{self.prefix}/left/{peer}"])
                    with self._lock:
                        if left:
                            self._left.add(peer)
                        if value != self._seen[peer][0]:
                            self._seen[peer] = (value, now)
            except Exception as exc:  # noqa: BLE001 - the store itself is unreachable: rank 0's host is gone
                with self._lock:
                    self._error = f"{type(exc).__name__}: {exc}"
                return

    # ------------------------------------------------------------------ queries (never block on the store)
    def silent_peers(self) -> dict[int, float]:
        now = time.monotonic()
        with self._lock:
            return {p: now - t for p, (_, t) in self._seen.items() if p not in self._left and now - t > self.timeout}

    def check(self) -> None:
        with self._lock:
            error = self._error
        if error is not None:
            raise PeerLostError([0], self.timeout) from RuntimeError(f"key-value store unreachable: {error}")
        silent = self.silent_peers()
        if silent:
            raise PeerLostError(sorted(silent), max(silent.values()))


__all__ = ["HeartbeatMonitor", "PeerLostError"]

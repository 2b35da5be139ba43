"""Semantic profiler spans. Span names keep the reference's ``maltos::`` prefix so traces are comparable
(reference ``utils/profiling.py:17-34``)."""
from __future__ import annotations

import functools
from typing import Callable

import torch

SPAN_PREFIX = "maltos::"


def span(name: str):
    """Context manager for one named profiler range."""
    return torch.profiler.record_function(name)


def profiled(name):
    """Decorator: run the function inside a span. ``name`` is a string or a callable of the call arguments."""

    def wrap(fn: Callable):
        @functools.wraps(fn)
        def inner(*args, **kwargs):
            label = name(*args, **kwargs) if callable(name) else name
            with torch.profiler.record_function(label):
                return fn(*args, **kwargs)

        return inner

    return wrap


# ------------------------------------------------------------------------------------------------ exposed communication
#: substrings that mark a device kernel as communication: NCCL's kernels and this library's one-sided collectives
COMM_KERNEL_MARKERS = ("nccl", "pull_reduce_scatter", "pull_all_gather", "peer_rows", "peer_copy", "peer_gather",
                       "peer_reduce_shard", "peer_all_reduce", "rs_reduce", "Memcpy PtoP")


def is_comm_kernel(name: str) -> bool:
    low = name.lower()
    return any(m.lower() in low for m in COMM_KERNEL_MARKERS)


def _union(intervals: list[tuple[float, float]]) -> list[tuple[float, float]]:
    out: list[tuple[float, float]] = []
    for s, e in sorted(intervals):
        if out and s <= out[-1][1]:
            if e > out[-1][1]:
                out[-1] = (out[-1][0], e)
        else:
            out.append((s, e))
    return out


def exposed_comm_us(kernels) -> tuple[float, float, float]:
    """``kernels``: iterable of ``(name, start_us, duration_us)`` of one rank's device kernels over some window.
    Returns ``(exposed, comm_total, busy)`` in microseconds: the time covered by communication kernels but by no
    compute kernel (communication the step actually waits for), the union of all communication intervals, and the
    union of all kernel intervals. A fused kernel that moves data while it computes counts as compute."""
    comm, comp = [], []
    for name, start, dur in kernels:
        (comm if is_comm_kernel(name) else comp).append((float(start), float(start) + float(dur)))
    comm_u, comp_u = _union(comm), _union(comp)
    exposed, j = 0.0, 0
    for s, e in comm_u:
        cur = s
        while j < len(comp_u) and comp_u[j][1] <= cur:
            j += 1
        k = j
        while k < len(comp_u) and comp_u[k][0] < e:
            cs, ce = comp_u[k]
            if cs > cur:
                exposed += cs - cur
            cur = max(cur, ce)
            if cur >= e:
                break
            k += 1
        if cur < e:
            exposed += e - cur
    total = sum(e - s for s, e in comm_u)
    busy = sum(e - s for s, e in _union(comm + comp))
    return exposed, total, busy


def kernels_of_profile(prof) -> list[tuple[str, float, float]]:
    """Device kernels ``(name, start_us, duration_us)`` recorded by a ``torch.profiler.profile``."""
    out = []
    for ev in prof.events():
        if getattr(ev, "device_type", None) is not None and "cuda" in str(ev.device_type).lower():
            rng = ev.time_range
            out.append((ev.name, float(rng.start), float(rng.end - rng.start)))
    return out


def kernels_of_chrome_trace(path) -> list[tuple[str, float, float]]:
    """Device kernels of a Chrome trace exported by ``torch.profiler`` (events of category ``kernel`` / ``gpu_memcpy``)."""
    import json

    with open(path) as fh:
        data = json.load(fh)
    events = data["traceEvents"] if isinstance(data, dict) else data
    return [(e.get("name", ""), float(e["ts"]), float(e.get("dur", 0.0))) for e in events
            if e.get("ph") == "X" and str(e.get("cat", "")).lower() in ("kernel", "gpu_memcpy")]

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

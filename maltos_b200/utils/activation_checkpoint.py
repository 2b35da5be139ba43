"""Tells code running under ``torch.utils.checkpoint`` whether it is the original forward or the recompute
(ZeRO-3 and the fused TP ops key their staging buffers on it). Reference: ``utils/activation_checkpoint.py:26-32``."""
from __future__ import annotations

import contextlib
from contextvars import ContextVar

_recomputing: ContextVar[bool] = ContextVar("maltos_b200_recomputing", default=False)


@contextlib.contextmanager
def _recompute_scope():
    token = _recomputing.set(True)
    try:
        yield
    finally:
        _recomputing.reset(token)


def activation_checkpoint_context_fn():
    """``context_fn`` for non-reentrant ``checkpoint``: (forward context, recompute context)."""
    return contextlib.nullcontext(), _recompute_scope()


def is_activation_checkpoint_recompute() -> bool:
    return _recomputing.get()

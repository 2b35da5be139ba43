"""Tells code running under ``torch.utils.checkpoint`` whether it is the original forward or the recompute
(ZeRO-3 and the fused TP ops key their staging buffers on it). Reference: ``utils/activation_checkpoint.py:26-32``.

It also carries a small per-checkpoint-call stash between the two passes: an op whose result is needed again by its
own backward (flash attention: output and log-sum-exp) records it in the original forward and replays it in the
recompute, so the recompute does not launch that op a second time. The stash lives exactly as long as the checkpointed
call's autograd frame. ``MALTOS_B200_CKPT_STASH=0`` turns it off (the op is then recomputed like everything else)."""
from __future__ import annotations

import contextlib
import os
from contextvars import ContextVar

_recomputing: ContextVar[bool] = ContextVar("maltos_b200_recomputing", default=False)
_stash: ContextVar[object] = ContextVar("maltos_b200_ckpt_stash", default=None)


class CheckpointStash:
    """Results recorded in the original forward of ONE checkpointed call, replayed in order by its recompute."""

    def __init__(self) -> None:
        self.items: list = []
        self.cursor = 0
        self.replaying = False

    def record(self, value) -> None:
        self.items.append(value)

    def replay(self):
        """Next recorded value, or None when the original forward recorded fewer (then the caller computes it)."""
        if self.cursor >= len(self.items):
            return None
        value = self.items[self.cursor]
        self.items[self.cursor] = None      # the autograd graph of the recompute owns it from here on
        self.cursor += 1
        return value


@contextlib.contextmanager
def _forward_scope(stash):
    token = _stash.set(stash)
    try:
        yield
    finally:
        _stash.reset(token)


@contextlib.contextmanager
def _recompute_scope(stash=None):
    token = _recomputing.set(True)
    if stash is not None:
        stash.replaying = True
    stoken = _stash.set(stash)
    try:
        yield
    finally:
        _stash.reset(stoken)
        _recomputing.reset(token)


def activation_checkpoint_context_fn():
    """``context_fn`` for non-reentrant ``checkpoint``: (forward context, recompute context)."""
    stash = CheckpointStash() if os.environ.get("MALTOS_B200_CKPT_STASH", "1") != "0" else None
    return _forward_scope(stash), _recompute_scope(stash)


def is_activation_checkpoint_recompute() -> bool:
    return _recomputing.get()


def current_checkpoint_stash():
    """The stash of the checkpointed call being run (original forward or recompute), or None outside of one."""
    return _stash.get()

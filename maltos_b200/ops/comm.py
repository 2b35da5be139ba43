"""Fused compute + collective ops over NVLink peer memory (sm_100a).

``context_for(group)`` returns the symmetric-memory context of a process group (peer-mapped staging buffers and signal
pads, created on first use with CUDA IPC handles exchanged through ``torch.distributed``) or ``None`` when the fused
path does not apply: CPU tensors, a group of size 1, ranks without peer access, or ``MALTOS_B200_FUSED_COMM=0``. Callers
fall back to ``torch.distributed`` collectives around the local GEMMs in that case (same semantics).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

_contexts: dict[int, object] = {}
_disabled_reason: dict[int, str] = {}


def fused_comm_enabled() -> bool:
    return os.environ.get("MALTOS_B200_FUSED_COMM", "1") != "0"


def context_for(group):
    """Symmetric-memory context for ``group`` or None (see module docstring)."""
    if group is None or not dist.is_initialized() or not torch.cuda.is_available() or not fused_comm_enabled():
        return None
    if dist.get_world_size(group) <= 1 or dist.get_backend(group) != "nccl":
        return None
    key = id(group)
    if key in _contexts:
        return _contexts[key][1]
    if key in _disabled_reason:
        return None
    try:
        from .symm import SymmetricContext

        ctx = SymmetricContext.create(group)
    except Exception as exc:  # noqa: BLE001 - any failure means "no peer path", the NCCL path is always valid
        _disabled_reason[key] = f"{type(exc).__name__}: {exc}"
        return None
    _contexts[key] = (group, ctx)     # holding the group keeps its id from being reused by a later group
    return ctx


def release_context(group) -> None:
    """Collective over ``group``: unmap and free its symmetric memory (call before the group is destroyed)."""
    entry = _contexts.pop(id(group), None)
    _disabled_reason.pop(id(group), None)
    if entry is not None:
        entry[1].close()


def disabled_reason(group) -> str | None:
    return _disabled_reason.get(id(group))


def all_gather_grouped_linear(x_local, weights, ctx, *, seq_dim: int = 1):
    from .fused_tp import all_gather_grouped_linear as impl

    return impl(x_local, weights, ctx, seq_dim=seq_dim)


def linear_reduce_scatter(x, weight, ctx, *, seq_dim: int = 1):
    from .fused_tp import linear_reduce_scatter as impl

    return impl(x, weight, ctx, seq_dim=seq_dim)

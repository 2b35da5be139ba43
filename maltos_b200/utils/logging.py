"""Rank-0 debug logging (reference ``utils/logging.py:5-11`` uses absl ``vlog``; plain ``logging`` here)."""
from __future__ import annotations

import logging
import os

import torch.distributed as dist

_logger = logging.getLogger("maltos_b200")
_VERBOSITY = int(os.environ.get("MALTOS_VLOG", "0"))


def is_rank0() -> bool:
    return not dist.is_initialized() or dist.get_rank() == 0


def vlog(level: int, msg: str, *args) -> None:
    """Log ``msg % args`` on rank 0 when ``MALTOS_VLOG`` >= ``level``."""
    if level <= _VERBOSITY and is_rank0():
        _logger.info(msg, *args)


def rank0_print(*args, **kwargs) -> None:
    if is_rank0():
        print(*args, **kwargs, flush=True)

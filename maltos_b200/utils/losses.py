"""Training losses. ``causal_cross_entropy`` = sum of token CE over non-ignored labels / max(#targets, 1), finite
(0 with zero grads) when a packed micro-batch has no targets (reference ``utils/losses.py:9-15``)."""
from __future__ import annotations

import torch

from .constants import IGNORE_INDEX


def causal_cross_entropy(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Mean CE over targets of already-shifted ``labels``; CUDA bf16/fp32 logits use the fused sm_100a kernel."""
    from maltos_b200.ops.cross_entropy import cross_entropy_mean

    return cross_entropy_mean(logits.reshape(-1, logits.size(-1)), labels.reshape(-1), ignore_index=IGNORE_INDEX)

"""Check that local positions follow the zigzag layout ring attention balances on: rank r of C owns chunks r and
2C-1-r of the sequence cut into 2C equal chunks (reference ``runtime/layers/ring_layout.py:6-43``)."""
from __future__ import annotations

import torch


def zigzag_positions(seq_len: int, rank: int, world: int, device=None) -> torch.Tensor:
    half = seq_len // (2 * world)
    front = torch.arange(rank * half, (rank + 1) * half, device=device)
    back = torch.arange((2 * world - 1 - rank) * half, (2 * world - rank) * half, device=device)
    return torch.cat([front, back])


def is_dense_zigzag_layout(q_positions: torch.Tensor, rank: int, world: int) -> bool:
    if q_positions.dim() != 2 or q_positions.size(1) % 2:
        return False
    local = q_positions.size(1)
    expected = zigzag_positions(local * world, rank, world, device=q_positions.device)
    return bool((q_positions == expected.unsqueeze(0)).all())

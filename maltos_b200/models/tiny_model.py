"""Smallest trainable module used by plumbing tests: ``Linear -> ReLU -> Linear(->1)``, loss ``mean(out^2)``
(reference ``models/tiny_model.py:7-18``; same parameter names)."""
from __future__ import annotations

import torch
import torch.nn as nn


class TinyModel(nn.Module):
    def __init__(self, hidden_size: int = 32) -> None:
        super().__init__()
        self.net = nn.Sequential(nn.Linear(hidden_size, hidden_size), nn.ReLU(), nn.Linear(hidden_size, 1))

    def forward(self, batch: torch.Tensor) -> torch.Tensor:
        return self.net(batch).pow(2).mean()

"""RMSNorm whose normalised dimension may be sharded over the TP group (OLMo-2 QK-norm over the whole
``heads*head_dim`` vector). Local sum of squares in fp32, all-reduced in forward and backward, divided by the
logical width (reference ``runtime/layers/distributed_rmsnorm.py:8-81``). Unsharded, it is the fused RMSNorm kernel."""
from __future__ import annotations

import torch
import torch.nn as nn

from maltos_b200.ops.norm import rms_norm

from .functional import all_reduce_fwd_bwd


class DistributedRMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, *, tp_group=None, logical_hidden_size: int | None = None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps
        self.tp_group = tp_group
        self.logical_hidden_size = logical_hidden_size or hidden_size

    @classmethod
    def from_norm(cls, module: "DistributedRMSNorm", tp_group, rank: int, world: int) -> "DistributedRMSNorm":
        full = module.weight.shape[0]
        if full % world:
            raise ValueError("DistributedRMSNorm width must be divisible by TP world size")
        per = full // world
        new = cls(per, module.eps, tp_group=tp_group, logical_hidden_size=full).to(module.weight.device, dtype=module.weight.dtype)
        with torch.no_grad():
            new.weight.copy_(module.weight[rank * per:(rank + 1) * per])
        return new

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_group is None or self.logical_hidden_size == self.weight.shape[0]:
            return rms_norm(x, self.weight, self.eps)
        ss = x.float().pow(2).sum(dim=-1, keepdim=True)
        ss = all_reduce_fwd_bwd(ss, self.tp_group)
        inv = torch.rsqrt(ss / float(self.logical_hidden_size) + self.eps)
        return self.weight * (x.float() * inv).to(x.dtype)

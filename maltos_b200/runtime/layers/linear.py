"""Megatron-style tensor-parallel linear layers (reference ``runtime/layers/linear.py:13-143``).

``ColumnParallelLinear`` holds ``weight[out/T, in]`` (optionally all-gathers its output), ``RowParallelLinear`` holds
``weight[out, in/T]`` and finishes with all-reduce / reduce-scatter / nothing; its bias is added after the
communication. GEMMs go through ``maltos_b200.ops.gemm.linear`` (tcgen05 on CUDA bf16).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.ops.gemm import linear

from .functional import all_gather, all_reduce, copy_to_group, row_parallel_reduce_scatter


def _init_like_linear(weight: torch.Tensor, bias: torch.Tensor | None, fan_in: int) -> None:
    nn.init.kaiming_uniform_(weight, a=math.sqrt(5))
    if bias is not None:
        bound = 1 / math.sqrt(fan_in)
        nn.init.uniform_(bias, -bound, bound)


class ColumnParallelLinear(nn.Module):
    def __init__(self, in_features, out_features, tp_group, bias=True, gather_output=True, init=True, input_is_replicated=False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.tp_group = tp_group
        self.gather_output = gather_output
        #: True in plain TP (no SP): the input is identical on all ranks, so its gradient must be summed over TP
        self.input_is_replicated = input_is_replicated
        self.rank = dist.get_rank(tp_group)
        self.world_size = dist.get_world_size(tp_group)
        if out_features % self.world_size:
            raise ValueError("out_features must be divisible by TP world size")
        self.out_features_per_shard = out_features // self.world_size
        self.weight = nn.Parameter(torch.empty(self.out_features_per_shard, in_features))
        if bias:
            self.bias = nn.Parameter(torch.empty(self.out_features_per_shard))
        else:
            self.register_parameter("bias", None)
        if init:
            _init_like_linear(self.weight, self.bias, in_features)

    @classmethod
    def from_linear(cls, module: nn.Linear, tp_group, gather_output=True, **kw) -> "ColumnParallelLinear":
        new = cls(module.in_features, module.out_features, tp_group, bias=module.bias is not None,
                  gather_output=gather_output, init=False, **kw).to(module.weight.device, dtype=module.weight.dtype)
        lo = new.rank * new.out_features_per_shard
        with torch.no_grad():
            new.weight.copy_(module.weight[lo:lo + new.out_features_per_shard])
            if module.bias is not None:
                new.bias.copy_(module.bias[lo:lo + new.out_features_per_shard])
        return new

    def forward(self, x):
        if self.input_is_replicated and self.world_size > 1:
            x = copy_to_group(x, self.tp_group)
        y = linear(x, self.weight, self.bias)
        if self.gather_output and self.world_size > 1:
            y = all_gather(y, self.tp_group, -1)
        return y


class RowParallelLinear(nn.Module):
    def __init__(self, in_features, out_features, tp_group, comm="none", comm_dim=0, bias=True, init=True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.tp_group, self.comm, self.comm_dim = tp_group, comm, comm_dim
        self.rank = dist.get_rank(tp_group)
        self.world_size = dist.get_world_size(tp_group)
        if in_features % self.world_size:
            raise ValueError("in_features must be divisible by TP world size")
        self.in_features_per_shard = in_features // self.world_size
        self.weight = nn.Parameter(torch.empty(out_features, self.in_features_per_shard))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        if init:
            _init_like_linear(self.weight, self.bias, in_features)

    @classmethod
    def from_linear(cls, module: nn.Linear, tp_group, comm, comm_dim=0) -> "RowParallelLinear":
        new = cls(module.in_features, module.out_features, tp_group, comm, comm_dim, bias=module.bias is not None,
                  init=False).to(module.weight.device, dtype=module.weight.dtype)
        lo = new.rank * new.in_features_per_shard
        with torch.no_grad():
            new.weight.copy_(module.weight[:, lo:lo + new.in_features_per_shard])
            if module.bias is not None:
                new.bias.copy_(module.bias)
        return new

    def forward(self, x):
        if self.comm == "reduce_scatter" and self.world_size > 1:
            return row_parallel_reduce_scatter(x, self.weight, self.bias, self.tp_group, seq_dim=self.comm_dim)
        y = linear(x, self.weight)
        if self.comm == "all_reduce" and self.world_size > 1:
            y = all_reduce(y, self.tp_group, dist.ReduceOp.SUM)
        return y if self.bias is None else y + self.bias

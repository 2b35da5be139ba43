"""Differentiable collectives and the fused tensor/sequence-parallel linear ops.

Two implementations sit behind every op here:

* CUDA with a symmetric-memory context for the group (``maltos_b200.ops.comm``): ONE sm_100a kernel per op that
  moves peer data over NVLink from inside the GEMM (all-gather -> GEMM, GEMM -> reduce-scatter).
* anything else (CPU/gloo tests, groups without peer access): ``torch.distributed`` collectives around the local
  GEMMs. This path defines the semantics and is the oracle of the fused kernels' tests.

Semantics follow the reference's ``runtime/layers/functional.py`` (autograd collectives ``:163-270,489-616``,
grouped SP linear ``:369-486``, row-parallel reduce-scatter ``:273-366``).
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from maltos_b200.ops import gemm as _gemm_ops
from maltos_b200.ops.grouped import grouped_linear
from maltos_b200.utils.distributed import (all_gather_single, all_reduce_tensor, group_rank, group_size,
                                           pairwise_send_recv_async, reduce_scatter_single)


def native_comm_overlap_workspace_bytes(*, micro_batch_size: int, seq_len: int, hidden_size: int, tp_size: int, dtype: torch.dtype) -> int:
    """Size of the largest symmetric transfer buffer the fused tensor / sequence-parallel ops need for one micro-batch:
    two copies (alternating by call, so that a peer may still read call ``n`` while call ``n + 1`` is written) of the
    FULL-sequence hidden states. The reference's estimate (``runtime/layers/functional.py:85-114``) is two copies of the
    LOCAL shard, because its library op keeps only the local output in symmetric memory; here the gathered operand
    (all-gather -> GEMM) and the un-reduced partial (GEMM -> reduce-scatter) live there, which is ``tp_size`` times that."""
    for name, value in (("micro_batch_size", micro_batch_size), ("seq_len", seq_len), ("hidden_size", hidden_size), ("tp_size", tp_size)):
        if value < 1:
            raise ValueError(f"{name} must be >= 1, got {value}")
    if seq_len % tp_size:
        raise ValueError(f"seq_len={seq_len} must be divisible by tp_size={tp_size}")
    return 2 * micro_batch_size * seq_len * hidden_size * torch.empty((), dtype=dtype).element_size()


def prewarm_native_comm_overlap_workspace(group, *, min_workspace_bytes: int) -> bool:
    """Creates the group's symmetric-memory context and its transfer buffers before the first step (reference
    ``runtime/layers/functional.py:117-160``). False where the fused path does not exist: no CUDA, a backend other than
    NCCL, no peer access inside the group."""
    if group is None or not torch.cuda.is_available() or dist.get_backend(group) != "nccl":
        return False
    from maltos_b200.ops import comm, fused_tp

    symm = comm.context_for(group)
    if symm is None:
        return False
    fused_tp.prewarm_workspace(symm, int(min_workspace_bytes))
    torch.cuda.synchronize()
    return True


def _move_dim0(t: torch.Tensor, dim: int) -> torch.Tensor:
    return t if dim == 0 else t.transpose(0, dim)


def _gather_along(t: torch.Tensor, group, dim: int) -> torch.Tensor:
    world = group_size(group)
    if world == 1:
        return t
    src = _move_dim0(t, dim).contiguous()
    out = torch.empty((world * src.shape[0], *src.shape[1:]), dtype=t.dtype, device=t.device)
    all_gather_single(out, src, group=group)
    return _move_dim0(out, dim).contiguous() if dim != 0 else out


def _reduce_scatter_along(t: torch.Tensor, group, dim: int, op=dist.ReduceOp.SUM) -> torch.Tensor:
    world = group_size(group)
    if world == 1:
        return t
    src = _move_dim0(t, dim).contiguous()
    if src.shape[0] % world:
        raise ValueError(f"reduce_scatter: dim {dim} of size {src.shape[0]} is not divisible by group size {world}")
    out = torch.empty((src.shape[0] // world, *src.shape[1:]), dtype=t.dtype, device=t.device)
    reduce_scatter_single(out, src, op=op, group=group)
    return _move_dim0(out, dim).contiguous() if dim != 0 else out


def _narrow_mine(t: torch.Tensor, group, dim: int) -> torch.Tensor:
    world, rank = group_size(group), group_rank(group)
    if world == 1:
        return t
    if t.shape[dim] % world:      # a floor division here would silently drop the last tokens of every row
        raise ValueError(f"sequence-parallel split: dim {dim} of size {t.shape[dim]} is not divisible by group size {world}")
    per = t.shape[dim] // world
    return t.narrow(dim, rank * per, per).contiguous()


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim, backward_reduce):
        ctx.group, ctx.dim, ctx.backward_reduce = group, dim % x.dim(), backward_reduce
        return _gather_along(x, group, ctx.dim)

    @staticmethod
    def backward(ctx, dy):
        if ctx.backward_reduce is None:
            return _narrow_mine(dy, ctx.group, ctx.dim), None, None, None
        return _reduce_scatter_along(dy.contiguous(), ctx.group, ctx.dim, ctx.backward_reduce), None, None, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim, op):
        ctx.group, ctx.dim = group, dim % x.dim()
        return _reduce_scatter_along(x, group, ctx.dim, op)

    @staticmethod
    def backward(ctx, dy):
        return _gather_along(dy.contiguous(), ctx.group, ctx.dim), None, None, None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, op):
        if group_size(group) == 1:
            return x
        y = x.contiguous().clone()
        all_reduce_tensor(y, op=op, group=group)
        return y

    @staticmethod
    def backward(ctx, dy):
        return dy, None, None


class _AllReduceBoth(torch.autograd.Function):
    """All-reduce in forward AND backward (a sum whose every term is used on every rank)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        if group_size(group) == 1:
            return x
        y = x.contiguous().clone()
        all_reduce_tensor(y, op=dist.ReduceOp.SUM, group=group)
        return y

    @staticmethod
    def backward(ctx, dy):
        if group_size(ctx.group) == 1:
            return dy, None
        g = dy.contiguous().clone()
        all_reduce_tensor(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


class _CopyToGroup(torch.autograd.Function):
    """Identity forward, all-reduce(SUM) backward: entry of a tensor-parallel region fed by replicated input."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, dy):
        if group_size(ctx.group) == 1:
            return dy, None
        g = dy.contiguous().clone()
        all_reduce_tensor(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


def ring_exchange(t: torch.Tensor, group, shift: int = 1) -> torch.Tensor:
    """Every rank sends ``t`` to ``rank + shift`` and returns what it received from ``rank - shift``."""
    world, rank = group_size(group), group_rank(group)
    if world == 1:
        return t
    ranks = dist.get_process_group_ranks(group)
    out = torch.empty_like(t)
    works = pairwise_send_recv_async(t.contiguous(), out, send_rank=ranks[(rank + shift) % world],
                                     recv_rank=ranks[(rank - shift) % world], group=group)
    for w in works:
        w.wait()
    return out


class _RingShift(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, shift):
        ctx.group, ctx.shift = group, shift
        return ring_exchange(x, group, shift)

    @staticmethod
    def backward(ctx, dy):
        return ring_exchange(dy.contiguous(), ctx.group, -ctx.shift), None, None


def all_gather(x, group, dim: int = 0, *, backward_reduce=None, alloc_key: str | None = None):
    """Concatenate over ranks along ``dim``. Backward: this rank's slice, or reduce-scatter(op) if given."""
    return _AllGather.apply(x, group, dim, backward_reduce)


def reduce_scatter(x, group, dim: int = 0, op=dist.ReduceOp.SUM, *, alloc_key: str | None = None):
    return _ReduceScatter.apply(x, group, dim, op)


def all_reduce(x, group, op=dist.ReduceOp.SUM, *, alloc_key: str | None = None):
    return _AllReduce.apply(x, group, op)


def all_reduce_fwd_bwd(x, group):
    return _AllReduceBoth.apply(x, group)


def copy_to_group(x, group):
    return _CopyToGroup.apply(x, group)


def ring_shift(x, group, shift: int = 1):
    return _RingShift.apply(x, group, shift)


# ------------------------------------------------------------------------------------------------ SP fused ops
def _fused_ctx(group, *tensors):
    """Symmetric-memory context of ``group`` if the fused sm_100a path applies to these tensors, else None."""
    if not all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors):
        return None
    from maltos_b200.ops import comm

    return comm.context_for(group)


def sequence_parallel_grouped_linear(x_local: torch.Tensor, weights: Sequence[torch.Tensor], group, *, seq_dim: int = 1):
    """SP entry of a column-parallel projection group.

    ``x_local [B, S/T, H]`` is all-gathered along the sequence ONCE and multiplied by every weight shard
    (q/k/v or gate/up). Returns ``(packed [B, S, sum(out_i/T)], offsets)``. Backward: dgrad summed over members,
    reduce-scattered (SUM) back to ``[B, S/T, H]``; wgrads use the re-gathered input.
    """
    ctx = _fused_ctx(group, x_local, *weights)
    if ctx is not None:
        from maltos_b200.ops import comm

        return comm.all_gather_grouped_linear(x_local, list(weights), ctx, seq_dim=seq_dim)
    x_full = all_gather(x_local, group, seq_dim, backward_reduce=dist.ReduceOp.SUM)
    return grouped_linear(x_full, weights)


def row_parallel_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, bias, group, *, seq_dim: int = 1):
    """SP exit of a row-parallel linear: ``reduce_scatter_seq(x @ W_shard^T) (+ bias)`` -> ``[B, S/T, out]``."""
    ctx = _fused_ctx(group, x, weight)
    if ctx is not None:
        from maltos_b200.ops import comm

        y = comm.linear_reduce_scatter(x, weight, ctx, seq_dim=seq_dim)
    else:
        y = reduce_scatter(_gemm_ops.linear(x, weight), group, seq_dim)
    return y if bias is None else y + bias


row_parallel_reduce_scatter_async = row_parallel_reduce_scatter

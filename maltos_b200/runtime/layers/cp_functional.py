"""Context-parallel building blocks over an ordered SUBSET of a process group (dynamic per-document rings of HDP).

All ranks of the HDP group share one process group; a document names the members that hold its tokens and only those
exchange its K/V, point to point, in the order of the member tuple. No ``dist.new_group`` per document: creating groups
for every variable-length batch would be slow and fragile (reference ``runtime/layers/cp_functional.py:1-364``,
``runtime/layers/hdp_attention.py:3-10``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from maltos_b200.utils.distributed import pairwise_send_recv_async

from .ring_attention import _RingComm, flash_ring_attention


def _shift_once(t: torch.Tensor, comm: _RingComm, *, backward: bool = False) -> torch.Tensor:
    recv = torch.empty_like(t)
    send_to, recv_from = (comm.prev_rank, comm.next_rank) if backward else (comm.next_rank, comm.prev_rank)
    for w in pairwise_send_recv_async(t.contiguous(), recv, send_rank=send_to, recv_rank=recv_from, group=comm.group):
        w.wait()
    return recv


class _SubsetRingShift(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, participant_ranks):
        ctx.group, ctx.participants = group, participant_ranks
        return _shift_once(x, _RingComm(group, participant_ranks))

    @staticmethod
    def backward(ctx, dy):
        return _shift_once(dy, _RingComm(ctx.group, ctx.participants), backward=True), None, None


def subset_ring_shift(x: torch.Tensor, *, group, participant_ranks) -> torch.Tensor:
    """Differentiable: every member sends ``x`` to its successor in ``participant_ranks`` and returns what its
    predecessor sent; gradients travel the other way."""
    if len(participant_ranks) <= 1:
        return x
    return _SubsetRingShift.apply(x, group, tuple(participant_ranks))


def subset_ring_exchange_metadata(t: torch.Tensor, *, group, participant_ranks) -> torch.Tensor:
    """The same shift for integer side information (positions, sequence ids); no gradient."""
    if len(participant_ranks) <= 1:
        return t
    with torch.no_grad():
        return _shift_once(t, _RingComm(group, tuple(participant_ranks)))


def dynamic_flash_ring_attention(q, k, v, *, positions, sequence_ids, group, participant_ranks, module_id=None,
                                 partition_tokens: int | None = None, metadata_cache=None, metadata_cache_key=None, scale=None):
    """Ring attention of one document's local ``[1, L, h, D]`` block over the document's member ranks.

    K/V keep their native GQA head count on the wire; the flash block kernels (CUDA bf16) or the fp32 block primitives
    do the per-step work, blocks that lie entirely in the future of the local queries are skipped, and partial results
    are merged by log-sum-exp - the same machinery as fixed context parallelism, on a subset ring.
    """
    return flash_ring_attention(q, k, v, group, q_positions=positions, q_sequence_ids=sequence_ids, scale=scale,
                                module_id=module_id, participant_ranks=tuple(participant_ranks))


__all__ = ["subset_ring_shift", "subset_ring_exchange_metadata", "dynamic_flash_ring_attention"]

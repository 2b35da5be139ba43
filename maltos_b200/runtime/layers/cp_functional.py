"""Context-parallel building blocks over an ordered SUBSET of a process group (dynamic per-document rings of HDP).

All ranks of the HDP group share one process group; a document names the members that hold its tokens and only those
exchange its K/V, point to point, in the order of the member tuple. No ``dist.new_group`` per document: creating groups
for every variable-length batch would be slow and fragile (reference ``runtime/layers/cp_functional.py:1-364``,
``runtime/layers/hdp_attention.py:3-10``).
"""
from __future__ import annotations

import torch

from maltos_b200.utils.distributed import pairwise_send_recv_async

from .ring_attention import RingPlan, _RingComm, flash_ring_attention


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


def document_ring_plan(*, sequence_length: int, padded_length: int, local_length: int, ring_size: int) -> RingPlan:
    """What the host knows about one document's ring WITHOUT any communication (subset rings may not issue collectives).

    The loader lays a document out zigzag over its ring (member ``i`` holds chunks ``i`` and ``2R-1-i`` of the document
    padded to a multiple of ``2R``), so every block is visible. The half-block schedule with unmasked kernels applies when
    the tail padding is confined to the LAST chunk: that chunk is the second half of member 0, whose keys are only ever
    read by member 0's own (masked) diagonal block - blocks of earlier members are read through their first half, and no
    member comes before member 0. Padding QUERIES of member 0 then attend to real keys; their rows carry no loss, receive a
    zero output gradient and are never read as keys, so nothing real depends on them.
    """
    visible = (True,) * ring_size
    if ring_size < 2 or padded_length % (2 * ring_size):
        return RingPlan(False, visible)
    chunk = padded_length // (2 * ring_size)
    confined = 0 <= padded_length - sequence_length <= chunk
    return RingPlan(bool(confined and local_length == 2 * chunk), visible)


def dynamic_flash_ring_attention(q, k, v, *, positions, sequence_ids, group, participant_ranks, module_id=None,
                                 partition_tokens: int | None = None, metadata_cache=None, metadata_cache_key=None, scale=None,
                                 plan: RingPlan | None = None):
    """Ring attention of one document's local ``[1, L, h, D]`` block over the document's member ranks.

    K/V keep their native GQA head count on the wire; the flash block kernels (CUDA bf16) or the fp32 block primitives
    do the per-step work and partial results are merged by log-sum-exp - the same machinery as fixed context parallelism,
    on a subset ring. ``plan`` (see :func:`document_ring_plan`) is kept in ``metadata_cache`` under ``metadata_cache_key`` so
    that all layers of a wave share it; without one every block runs through the masked kernel.
    """
    if plan is None and metadata_cache is not None and metadata_cache_key is not None:
        plan = metadata_cache.get(metadata_cache_key)
    elif plan is not None and metadata_cache is not None and metadata_cache_key is not None:
        metadata_cache[metadata_cache_key] = plan
    return flash_ring_attention(q, k, v, group, q_positions=positions, q_sequence_ids=sequence_ids, scale=scale,
                                module_id=module_id, participant_ranks=tuple(participant_ranks), plan=plan)


__all__ = ["subset_ring_shift", "subset_ring_exchange_metadata", "dynamic_flash_ring_attention", "document_ring_plan"]

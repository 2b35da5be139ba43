"""Ring attention over the context-parallel group.

K/V (with their positions and sequence ids) travel ``rank -> rank+1``; at every step the local queries attend to the
block in hand and partial results are merged by log-sum-exp, so no rank ever holds more than one remote block. The
next block is requested before the current one is computed. With the zigzag token layout every rank has the same
amount of visible work. Backward re-circulates K/V together with an fp32 ``dK/dV`` accumulator that arrives back at
its owner after a full turn (reference ``runtime/layers/ring_attention.py:36-258`` and
``runtime/layers/functional.py:619-1166``). Visibility comes from positions/sequence ids, so dense, zigzag and
packed-document batches share one code path; blocks that are entirely invisible are skipped.

On CUDA bf16 the per-block work is the tcgen05 flash kernel (``maltos_b200.ops.flash_attn``); elsewhere the fp32 block
primitives of ``maltos_b200.ops.attention``. Between GPUs of one node the exchange itself goes over peer memory by default
(``MALTOS_B200_RING_PEER=0`` turns that off)
(``maltos_b200.ops.peer_ring``): blocks are pulled from their owners on a copy stream, dK/dV contributions are pushed
once to the owner's slots; the point-to-point ring below is the NCCL / gloo implementation and the oracle.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.ops.attention import attention, attention_block_backward, attention_block_forward, merge_attention_blocks
from maltos_b200.utils.constants import PAD_SEQUENCE_ID
from maltos_b200.utils.distributed import pairwise_send_recv_async
from maltos_b200.utils.profiling import span

from .attn_masking_utils import canonical_position_ids, canonical_sequence_ids


class _RingComm:
    """Shift tensors one place forward along a ring; requests are posted early and waited late. The ring is the whole
    group, or - for per-document dynamic context parallelism - an ordered subset of its ranks (no sub-group is ever
    created: members talk point to point inside the parent group)."""

    def __init__(self, group, participant_ranks=None) -> None:
        self.group = group
        members = list(participant_ranks) if participant_ranks is not None else list(range(dist.get_world_size(group)))
        me = dist.get_rank(group)
        if me not in members:
            raise ValueError(f"rank {me} is not a member of ring {members}")
        self.world = len(members)
        self.rank = members.index(me)
        to_global = dist.get_process_group_ranks(group)
        self.next_rank = to_global[members[(self.rank + 1) % self.world]]
        self.prev_rank = to_global[members[(self.rank - 1) % self.world]]

    def start(self, tensors: list[torch.Tensor]):
        outs, works = [], []
        for t in tensors:
            recv = torch.empty_like(t)
            works += pairwise_send_recv_async(t.contiguous(), recv, send_rank=self.next_rank, recv_rank=self.prev_rank, group=self.group)
            outs.append(recv)
        return outs, works

    @staticmethod
    def finish(works) -> None:
        for w in works:
            w.wait()


def _block_visible(q_pos, k_pos) -> bool:
    """False when no key of the block can be visible to any local query (all keys lie in the future)."""
    return bool(k_pos.min() <= q_pos.max())


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, q_pos, q_seq, group, scale, participants=None):
        from maltos_b200.ops.peer_ring import peer_ring_for

        B, S, hq, D = q.shape
        out = torch.zeros((B, S, hq, D), dtype=torch.float32, device=q.device)
        lse = torch.full((B, hq, S), float("-inf"), dtype=torch.float32, device=q.device)
        seq_or_zero = q_seq if q_seq is not None else torch.zeros_like(q_pos)
        cur = [k, v, q_pos, seq_or_zero]
        ring = peer_ring_for(group, q, participants)
        if ring is not None:
            layout, _ = ring.publish(cur)
            main = torch.cuda.current_stream()
            nxt = ring.pull(layout, (ring.rank - 1) % ring.world) if ring.world > 1 else None
            for step in range(ring.world):
                k_b, v_b, kp_b, ks_b = cur
                upcoming = nxt
                nxt = ring.pull(layout, (ring.rank - step - 2) % ring.world) if step + 2 < ring.world else None
                if _block_visible(q_pos, kp_b):
                    o_b, l_b = attention_block_forward(q, k_b, v_b, q_positions=q_pos, k_positions=kp_b, q_sequence_ids=q_seq,
                                                       k_sequence_ids=ks_b if q_seq is not None else None, scale=scale)
                    out, lse = merge_attention_blocks(out, lse, o_b.float(), l_b.float())
                if upcoming is not None:
                    main.wait_event(upcoming[1])
                    cur = upcoming[0]
            result = out.to(q.dtype)
            ctx.save_for_backward(q, k, v, result, lse, q_pos, seq_or_zero)
            ctx.group, ctx.scale, ctx.has_seq, ctx.participants = group, scale, q_seq is not None, participants
            return result
        comm = _RingComm(group, participants)
        for step in range(comm.world):
            nxt, works = (comm.start(cur) if step + 1 < comm.world else (None, []))
            k_b, v_b, kp_b, ks_b = cur
            if _block_visible(q_pos, kp_b):
                o_b, l_b = attention_block_forward(q, k_b, v_b, q_positions=q_pos, k_positions=kp_b,
                                                   q_sequence_ids=q_seq, k_sequence_ids=ks_b if q_seq is not None else None, scale=scale)
                out, lse = merge_attention_blocks(out, lse, o_b.float(), l_b.float())
            comm.finish(works)
            if nxt is not None:
                cur = nxt
        result = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, result, lse, q_pos, seq_or_zero)
        ctx.group, ctx.scale, ctx.has_seq, ctx.participants = group, scale, q_seq is not None, participants
        return result

    @staticmethod
    def backward(ctx, dout):
        from maltos_b200.ops.peer_ring import peer_ring_for

        q, k, v, out, lse, q_pos, seq_ids = ctx.saved_tensors
        q_seq = seq_ids if ctx.has_seq else None
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        dout = dout.contiguous()
        ring = peer_ring_for(ctx.group, q, ctx.participants)
        if ring is not None:
            cur = [k, v, q_pos, seq_ids]
            layout, slots = ring.publish(cur, grad_slots_like=[k, v])
            main = torch.cuda.current_stream()
            nxt = ring.pull(layout, (ring.rank - 1) % ring.world) if ring.world > 1 else None
            for step in range(ring.world):
                k_b, v_b, kp_b, ks_b = cur
                upcoming = nxt
                nxt = ring.pull(layout, (ring.rank - step - 2) % ring.world) if step + 2 < ring.world else None
                if _block_visible(q_pos, kp_b):
                    dq_b, dk_b, dv_b = attention_block_backward(q, k_b, v_b, out, lse, dout, q_positions=q_pos, k_positions=kp_b,
                                                                q_sequence_ids=q_seq, k_sequence_ids=ks_b if ctx.has_seq else None,
                                                                scale=ctx.scale)
                    dq += dq_b
                    ring.push_grads(slots, (ring.rank - step) % ring.world, [dk_b, dv_b])
                if upcoming is not None:
                    main.wait_event(upcoming[1])
                    cur = upcoming[0]
            dk, dv = ring.reduce_grads(slots, [k.shape, v.shape])
            return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None, None, None
        comm = _RingComm(ctx.group, ctx.participants)
        dk_acc = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
        dv_acc = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
        cur = [k, v, q_pos, seq_ids]
        for step in range(comm.world):
            k_b, v_b, kp_b, ks_b = cur
            nxt, works = (comm.start(cur) if step + 1 < comm.world else (None, []))
            if _block_visible(q_pos, kp_b):
                dq_b, dk_b, dv_b = attention_block_backward(q, k_b, v_b, out, lse, dout, q_positions=q_pos, k_positions=kp_b,
                                                            q_sequence_ids=q_seq, k_sequence_ids=ks_b if ctx.has_seq else None,
                                                            scale=ctx.scale)
                dq += dq_b
                dk_acc += dk_b
                dv_acc += dv_b
            comm.finish(works)
            # the accumulator follows its block: after `world` shifts it is back at the owner with every contribution
            (dk_acc, dv_acc), gworks = comm.start([dk_acc, dv_acc])
            comm.finish(gworks)
            if nxt is not None:
                cur = nxt
        return dq.to(q.dtype), dk_acc.to(k.dtype), dv_acc.to(v.dtype), None, None, None, None, None


def flash_ring_attention(q, k, v, group, *, q_positions, q_sequence_ids=None, scale=None, module_id=None, mb_idx: int = 0,
                         participant_ranks=None):
    """Ring attention of ``[B, S, h, D]`` blocks over ``group`` or over the ordered subset ``participant_ranks`` of it."""
    with span("maltos::cp.ring.flash" if q.is_cuda else "maltos::cp.ring.eager"):
        return _RingAttention.apply(q, k, v, q_positions, q_sequence_ids, group, scale,
                                    tuple(participant_ranks) if participant_ranks is not None else None)


class RingAttentionCore(nn.Module):
    preserves_native_gqa = True
    layout = "bshd"

    def __init__(self, group, attention_backend: str = "eager") -> None:
        super().__init__()
        self.group = group
        self.attention_backend = attention_backend
        self._step_context = None

    def bind_step_context(self, step_context) -> None:
        self._step_context = step_context

    def forward(self, q, k, v, position_offset: int = 0, position_ids=None, sequence_ids=None):
        B, S = q.shape[:2]
        q_pos = canonical_position_ids(position_ids, batch_size=B, seq_len=S, position_offset=position_offset, device=q.device)
        q_seq = canonical_sequence_ids(sequence_ids, batch_size=B, seq_len=S, device=q.device)
        if self.group is None or dist.get_world_size(self.group) == 1:
            with span("maltos::cp.ring.single_rank"):
                return attention(q, k, v, q_positions=q_pos, k_positions=q_pos, q_sequence_ids=q_seq, k_sequence_ids=q_seq)
        if q_seq is not None:
            # padding keys must never be visible, also to padding queries of another rank
            q_seq = q_seq.clone()
        return flash_ring_attention(q, k, v, self.group, q_positions=q_pos, q_sequence_ids=q_seq)


__all__ = ["RingAttentionCore", "flash_ring_attention", "PAD_SEQUENCE_ID"]

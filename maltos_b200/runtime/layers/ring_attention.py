"""Ring attention over the context-parallel group.

K/V (with their positions and sequence ids) travel ``rank -> rank+1``; at every step the local queries attend to the
block in hand and partial results are merged by log-sum-exp, so no rank ever holds more than one remote block. The
next block is requested before the current one is computed. With the zigzag token layout every rank has the same
amount of visible work. Backward re-circulates K/V together with an fp32 ``dK/dV`` accumulator that arrives back at
its owner after a full turn (reference ``runtime/layers/ring_attention.py:36-258`` and
``runtime/layers/functional.py:619-1166``). Visibility comes from positions/sequence ids, so dense, zigzag and
packed-document batches share one code path. What can be decided before launching - which blocks are invisible, and
whether the dense zigzag layout allows the unmasked half-block schedule - is read ONCE per micro-batch
(:class:`RingPlan`), not per ring step and not per layer.

On CUDA bf16 the per-block work is the tcgen05 flash kernel (``maltos_b200.ops.flash_attn``); elsewhere the fp32 block
primitives of ``maltos_b200.ops.attention``. Between GPUs of one node the exchange itself goes over peer memory by default
(``MALTOS_B200_RING_PEER=0`` turns that off)
(``maltos_b200.ops.peer_ring``): blocks are pulled from their owners on a copy stream, dK/dV contributions are pushed
once to the owner's slots; the point-to-point ring below is the NCCL / gloo implementation and the oracle.
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.ops.attention import attention, attention_block_backward, attention_block_forward, merge_attention_blocks
from maltos_b200.utils.constants import PAD_SEQUENCE_ID
from maltos_b200.utils.distributed import pairwise_send_recv_async
from maltos_b200.utils.profiling import span

from .attn_masking_utils import canonical_position_ids, canonical_sequence_ids
from .ring_layout import zigzag_positions


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


@dataclass(frozen=True)
class RingPlan:
    """What the host knows about one micro-batch's ring before any block is launched.

    ``visible[o]``: some key owned by ring member ``o`` can be seen by some local query (blocks that lie entirely in the
    future are never launched). ``zigzag``: every member holds the dense zigzag layout (chunks ``r`` and ``2C-1-r``) and
    there are no sequence ids, so the half-block schedule applies: a block from an earlier member is attended by all
    queries through its FIRST half only, a block from a later member by the SECOND half of the queries only, both without
    any mask; only the member's own block needs the masked kernel (reference ``runtime/layers/functional.py:1012-1065``).
    """
    zigzag: bool
    visible: tuple


_PLAN_CACHE: dict = {}
plan_builds = 0   # number of plans computed (each costs one small all-gather and ONE host read); tests read it


def _ring_members(group, participants):
    members = list(participants) if participants is not None else list(range(dist.get_world_size(group)))
    return members, members.index(dist.get_rank(group))


def build_ring_plan(q_pos: torch.Tensor, q_seq, group, participants=None) -> RingPlan:
    """One tiny all-gather of ``(min position, max position, is-zigzag)`` and one host read for the whole micro-batch -
    instead of a host read per ring step. Subset rings (dynamic context parallelism: members talk point to point, no
    collective may be issued for them) launch every block; their layout is zigzag by construction."""
    global plan_builds
    members, me = _ring_members(group, participants)
    world = len(members)
    if participants is not None:
        return RingPlan(False, (True,) * world)
    plan_builds += 1
    S = q_pos.shape[1]
    if q_seq is None and S % 2 == 0:
        zz = (q_pos == zigzag_positions(S * world, me, world, device=q_pos.device).unsqueeze(0)).all().to(torch.int64)
    else:
        zz = torch.zeros((), dtype=torch.int64, device=q_pos.device)
    mine = torch.stack([q_pos.min().to(torch.int64), q_pos.max().to(torch.int64), zz])
    everyone = torch.empty((world, 3), dtype=torch.int64, device=q_pos.device)
    dist.all_gather_into_tensor(everyone, mine.unsqueeze(0), group=group)
    rows = everyone.tolist()                                               # the one host read
    q_max = rows[me][1]
    return RingPlan(all(r[2] == 1 for r in rows), tuple(r[0] <= q_max for r in rows))


def ring_plan_for(key_pos, key_seq, q_pos, q_seq, group, participants=None) -> RingPlan:
    """The plan of this micro-batch, computed once and reused by every layer: cached on the identity (and version counter)
    of the position / sequence-id tensors the model hands down, which are the same objects for all layers of a step."""
    if participants is not None or key_pos is None:
        return build_ring_plan(q_pos, q_seq, group, participants)
    slot = (id(group), id(key_pos))
    hit = _PLAN_CACHE.get(slot)
    if hit is not None:
        pos_ref, pos_ver, seq_ref, seq_ver, plan = hit
        same_seq = (key_seq is None and seq_ref is None) or (seq_ref is not None and seq_ref() is key_seq and key_seq._version == seq_ver)
        if pos_ref() is key_pos and key_pos._version == pos_ver and same_seq:
            return plan
    plan = build_ring_plan(q_pos, q_seq, group, participants)
    for dead in [k for k, v in _PLAN_CACHE.items() if v[0]() is None]:
        del _PLAN_CACHE[dead]
    _PLAN_CACHE[slot] = (weakref.ref(key_pos), key_pos._version, None if key_seq is None else weakref.ref(key_seq),
                         0 if key_seq is None else key_seq._version, plan)
    return plan


def _merge_rows(out, lse, o_b, l_b, rows=None):
    """Merge a block result into the running ``(out, lse)``; ``rows`` restricts it to a slice of the local queries."""
    if rows is None:
        return merge_attention_blocks(out, lse, o_b.float(), l_b.float())
    o, l = merge_attention_blocks(out[:, rows], lse[:, :, rows], o_b.float(), l_b.float())
    out[:, rows] = o
    lse[:, :, rows] = l
    return out, lse


def _block_forward(plan, me, owner, q, blk, q_pos, q_seq, scale, out, lse):
    """Attend the local queries to the block of ring member ``owner`` and merge; returns the new ``(out, lse)``."""
    k_b, v_b, kp_b, ks_b = blk
    if not plan.visible[owner]:
        return out, lse
    if plan.zigzag and owner != me:
        half = q.shape[1] // 2
        if owner < me:                                    # earlier member: its first chunk is in everyone's past
            o_b, l_b = attention_block_forward(q, k_b[:, :half], v_b[:, :half], q_positions=None, k_positions=None, scale=scale)
            return _merge_rows(out, lse, o_b, l_b)
        rows = slice(half, None)                          # later member: only my second chunk lies after both of its chunks
        o_b, l_b = attention_block_forward(q[:, rows], k_b, v_b, q_positions=None, k_positions=None, scale=scale)
        return _merge_rows(out, lse, o_b, l_b, rows)
    o_b, l_b = attention_block_forward(q, k_b, v_b, q_positions=q_pos, k_positions=kp_b, q_sequence_ids=q_seq,
                                       k_sequence_ids=ks_b if q_seq is not None else None, scale=scale)
    return _merge_rows(out, lse, o_b, l_b)


def _block_backward(plan, me, owner, q, blk, out, lse, dout, q_pos, q_seq, scale, dq):
    """Backward of one block: adds the query gradient into ``dq`` and returns ``(dk_b, dv_b, key_rows)`` in fp32 - the
    gradient of the block's keys / values and the slice of the block they cover (None: the whole block) - or None when the
    block is invisible."""
    k_b, v_b, kp_b, ks_b = blk
    if not plan.visible[owner]:
        return None
    if plan.zigzag and owner != me:
        half = q.shape[1] // 2
        if owner < me:
            keys = slice(0, half)
            dq_b, dk_b, dv_b = attention_block_backward(q, k_b[:, keys], v_b[:, keys], out, lse, dout, q_positions=None,
                                                        k_positions=None, scale=scale)
            dq += dq_b
            return dk_b, dv_b, keys
        rows = slice(half, None)
        dq_b, dk_b, dv_b = attention_block_backward(q[:, rows], k_b, v_b, out[:, rows], lse[:, :, rows], dout[:, rows],
                                                    q_positions=None, k_positions=None, scale=scale)
        dq[:, rows] += dq_b
        return dk_b, dv_b, None
    dq_b, dk_b, dv_b = attention_block_backward(q, k_b, v_b, out, lse, dout, q_positions=q_pos, k_positions=kp_b,
                                                q_sequence_ids=q_seq, k_sequence_ids=ks_b if q_seq is not None else None,
                                                scale=scale)
    dq += dq_b
    return dk_b, dv_b, None


def _whole_block(grad, keys, like):
    """The gradient of a key slice placed into a zero tensor of the whole block's shape (fp32)."""
    if keys is None:
        return grad
    full = torch.zeros(like.shape, dtype=torch.float32, device=like.device)
    full[:, keys] = grad
    return full


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, q_pos, q_seq, group, scale, participants=None, plan=None):
        from maltos_b200.ops.peer_ring import peer_ring_for

        B, S, hq, D = q.shape
        if plan is None:
            plan = build_ring_plan(q_pos, q_seq, group, participants)
        out = torch.zeros((B, S, hq, D), dtype=torch.float32, device=q.device)
        lse = torch.full((B, hq, S), float("-inf"), dtype=torch.float32, device=q.device)
        seq_or_zero = q_seq if q_seq is not None else torch.zeros_like(q_pos)
        cur = [k, v, q_pos, seq_or_zero]
        ring = peer_ring_for(group, q, participants)
        if ring is not None:
            layout, _ = ring.publish(cur)
            main = torch.cuda.current_stream()
            # invisible blocks are neither fetched nor computed: the list of owners to visit is known on the host
            owners = [o for o in ((ring.rank - s) % ring.world for s in range(1, ring.world)) if plan.visible[o]]
            nxt = ring.pull(layout, owners[0]) if owners else None
            out, lse = _block_forward(plan, ring.rank, ring.rank, q, cur, q_pos, q_seq, scale, out, lse)
            for i, owner in enumerate(owners):
                main.wait_event(nxt[1])
                blk = nxt[0]
                nxt = ring.pull(layout, owners[i + 1]) if i + 1 < len(owners) else None
                out, lse = _block_forward(plan, ring.rank, owner, q, blk, q_pos, q_seq, scale, out, lse)
        else:
            comm = _RingComm(group, participants)
            for step in range(comm.world):
                nxt, works = (comm.start(cur) if step + 1 < comm.world else (None, []))
                out, lse = _block_forward(plan, comm.rank, (comm.rank - step) % comm.world, q, cur, q_pos, q_seq, scale, out, lse)
                comm.finish(works)
                if nxt is not None:
                    cur = nxt
        result = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, result, lse, q_pos, seq_or_zero)
        ctx.group, ctx.scale, ctx.has_seq, ctx.participants, ctx.plan = group, scale, q_seq is not None, participants, plan
        return result

    @staticmethod
    def backward(ctx, dout):
        from maltos_b200.ops.peer_ring import peer_ring_for

        q, k, v, out, lse, q_pos, seq_ids = ctx.saved_tensors
        plan = ctx.plan
        q_seq = seq_ids if ctx.has_seq else None
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        dout = dout.contiguous()
        cur = [k, v, q_pos, seq_ids]
        ring = peer_ring_for(ctx.group, q, ctx.participants)
        if ring is not None:
            layout, slots = ring.publish(cur, grad_slots_like=[k, v])
            main = torch.cuda.current_stream()
            owners = [o for o in ((ring.rank - s) % ring.world for s in range(1, ring.world)) if plan.visible[o]]
            nxt = ring.pull(layout, owners[0]) if owners else None
            blk = cur
            for i, owner in enumerate([ring.rank] + owners):
                if i > 0:
                    main.wait_event(nxt[1])
                    blk = nxt[0]
                    nxt = ring.pull(layout, owners[i]) if i < len(owners) else None
                res = _block_backward(plan, ring.rank, owner, q, blk, out, lse, dout, q_pos, q_seq, ctx.scale, dq)
                if res is not None:
                    ring.push_grads(slots, owner, [_whole_block(res[0], res[2], k), _whole_block(res[1], res[2], v)])
            dk, dv = ring.reduce_grads(slots, [k.shape, v.shape])
            return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None, None, None, None
        comm = _RingComm(ctx.group, ctx.participants)
        dk_acc = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
        dv_acc = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
        for step in range(comm.world):
            nxt, works = (comm.start(cur) if step + 1 < comm.world else (None, []))
            res = _block_backward(plan, comm.rank, (comm.rank - step) % comm.world, q, cur, out, lse, dout, q_pos, q_seq, ctx.scale, dq)
            if res is not None:
                keys = res[2] if res[2] is not None else slice(None)
                dk_acc[:, keys] += res[0]
                dv_acc[:, keys] += res[1]
            comm.finish(works)
            # the accumulator follows its block: after `world` shifts it is back at the owner with every contribution
            (dk_acc, dv_acc), gworks = comm.start([dk_acc, dv_acc])
            comm.finish(gworks)
            if nxt is not None:
                cur = nxt
        return dq.to(q.dtype), dk_acc.to(k.dtype), dv_acc.to(v.dtype), None, None, None, None, None, None


def flash_ring_attention(q, k, v, group, *, q_positions, q_sequence_ids=None, scale=None, module_id=None, mb_idx: int = 0,
                         participant_ranks=None, plan: RingPlan | None = None):
    """Ring attention of ``[B, S, h, D]`` blocks over ``group`` or over the ordered subset ``participant_ranks`` of it.
    ``plan``: the micro-batch's :class:`RingPlan` when the caller has it already (it is computed here otherwise)."""
    with span("maltos::cp.ring.flash" if q.is_cuda else "maltos::cp.ring.eager"):
        return _RingAttention.apply(q, k, v, q_positions, q_sequence_ids, group, scale,
                                    tuple(participant_ranks) if participant_ranks is not None else None, plan)


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
        plan = ring_plan_for(position_ids, sequence_ids, q_pos, q_seq, self.group)
        return flash_ring_attention(q, k, v, self.group, q_positions=q_pos, q_sequence_ids=q_seq, plan=plan)


__all__ = ["RingAttentionCore", "flash_ring_attention", "PAD_SEQUENCE_ID"]

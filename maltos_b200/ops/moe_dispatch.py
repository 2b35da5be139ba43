"""Expert-parallel token dispatch / combine over peer memory (``csrc/moe_dispatch.cu``).

Every rank all-gathers its per-expert assignment counts (one small collective and the only host read), from which each
source computes the exact row of every routed token in the destination rank's expert-major buffer. Dispatch then is a
one-sided row push into the peers' symmetric buffers, combine a one-sided row pull from them, and the gradients are the
opposite transfers. Gates and expert ids never travel: rows arrive sorted by expert, the gate is applied by the source.
This replaces the four variable-split all-to-alls of the reference layer (``runtime/layers/moe.py:112-150``).

The row kernels never wait on a peer. Each transfer is ``[local write or push] -> group barrier -> [local read or
pull]``; with the two buffers used alternately (pushes land in "a", pulls read "b") two consecutive transfers never touch
the same buffer without a barrier between them, in forward, backward and recomputation order alike.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _lib, comm


def enabled() -> bool:
    return os.environ.get("MALTOS_B200_MOE_PEER", "1") == "1"


def peer_context(group, x: torch.Tensor):
    """Symmetric-memory context of the expert-parallel group when the peer path can carry ``x``'s rows, else None."""
    if not enabled() or not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        return None
    if (x.shape[-1] * x.element_size()) % 16:
        return None
    return comm.context_for(group)


@dataclass
class DispatchPlan:
    ctx: object                      # SymmetricContext
    group: object
    hidden: int
    dtype: torch.dtype
    order: torch.Tensor              # [M] assignment indices sorted by expert (stable)
    peer_rank: torch.Tensor          # [M] int32 destination rank of sorted assignment j
    peer_row: torch.Tensor           # [M] int64 row in the destination's buffer
    recv_rows: int                   # rows this rank receives
    capacity: int                    # rows of the symmetric buffers (same on every rank)
    local_counts: list[int] | None   # received rows per local expert, expert order (host copy; None for a static plan)
    recv_counts: torch.Tensor | None = None   # static plan: int32 device tensor, valid rows of every local expert's slot
    slot_rows: int = 0               # static plan: rows of one local expert's slot

    @property
    def row_bytes(self) -> int:
        return self.hidden * torch.empty((), dtype=self.dtype).element_size()

    def buffer(self, name: str):
        sb = self.ctx.ensure_buffer(f"moe_{name}", self.capacity * self.row_bytes)
        if not getattr(sb, "_cleared", False):
            # a fresh allocation may hold any bit pattern; rows nobody writes must at least be finite numbers
            sb.local_tensor(torch.uint8, sb.nbytes, self.order.device).zero_()
            torch.cuda.current_stream().synchronize()
            dist.barrier(group=self.group)
            sb._cleared = True
        return sb

    def local_rows(self, name: str) -> torch.Tensor:
        sb = self.buffer(name)
        rows = sb.nbytes // self.row_bytes
        return sb.local_tensor(self.dtype, rows * self.hidden, self.order.device).view(rows, self.hidden)[:self.recv_rows]

    def barrier(self) -> None:
        tok = getattr(self.ctx, "_barrier_token", None)
        if tok is None:
            tok = self.ctx._barrier_token = torch.zeros(1, dtype=torch.float32, device=self.order.device)
        dist.all_reduce(tok, group=self.group)

    def _transfer(self, fn, local: torch.Tensor, local_row: torch.Tensor | None, name: str) -> None:
        sb = self.buffer(name)
        if local.stride(-1) != 1 and local.shape[-1] != 1:
            raise ValueError("peer row transfer needs rows that are contiguous in memory")
        esz = local.element_size()
        _lib.check(fn(_lib.ptr(local), _lib.c_ll(local.stride(0) * esz), _lib.ptr(local_row), _lib.c_ll(local.shape[0]),
                      _lib.ptr(sb.table), _lib.c_ll(0), _lib.c_ll(self.row_bytes), _lib.c_ll(sb.nbytes // self.row_bytes),
                      _lib.ptr(self.peer_rank), _lib.ptr(self.peer_row), _lib.c_ll(self.peer_row.numel()), _lib.c_int(self.row_bytes),
                      _lib.c_int(self.ctx.world), _lib.stream_ptr()), "peer row transfer")

    def push(self, local: torch.Tensor, local_row: torch.Tensor | None, name: str) -> None:
        self._transfer(_lib.lib().mb_peer_push_rows, local, local_row, name)

    def pull(self, name: str) -> torch.Tensor:
        out = torch.empty(self.peer_row.numel(), self.hidden, dtype=self.dtype, device=self.order.device)
        self._transfer(_lib.lib().mb_peer_pull_rows, out, None, name)
        return out


def plan_rows(all_counts: torch.Tensor, rank: int, experts_per_rank: int):
    """From the ``[world, experts]`` count matrix (host tensor): for every global expert the first row of THIS rank's tokens
    in the owner's buffer, the rows every rank receives, and the rows per local expert of this rank. Rows of one owner are
    ordered by local expert, then by source rank, then by the source's own order."""
    world, experts = all_counts.shape
    total = all_counts.sum(0)                                        # [E]
    by_owner = total.view(world, experts_per_rank)
    base = (by_owner.cumsum(1) - by_owner).reshape(-1)               # first row of expert e at its owner
    my_start = base + all_counts[:rank].sum(0)
    return my_start, by_owner.sum(1), by_owner[rank]


def build_plan(ctx, group, expert_of_assignment: torch.Tensor, num_experts: int, hidden: int, dtype: torch.dtype) -> DispatchPlan:
    """Collective over ``group`` (one all-gather of ``num_experts`` counts, one device->host read)."""
    rank, world = ctx.rank, ctx.world
    per = num_experts // world
    dev = expert_of_assignment.device
    counts = torch.bincount(expert_of_assignment, minlength=num_experts)
    all_counts = torch.empty(world, num_experts, dtype=counts.dtype, device=dev)
    dist.all_gather_into_tensor(all_counts.view(-1), counts, group=group)
    host = all_counts.cpu()
    my_start, recv_rows, local_counts = plan_rows(host, rank, per)
    order = torch.argsort(expert_of_assignment, stable=True)
    sorted_e = expert_of_assignment[order]
    group_start = counts.cumsum(0) - counts
    pos = torch.arange(sorted_e.numel(), device=dev) - group_start[sorted_e]
    peer_row = (my_start.to(dev)[sorted_e] + pos).to(torch.int64)
    peer_rank = torch.div(sorted_e, per, rounding_mode="floor").to(torch.int32)
    need = max(1, int(recv_rows.max()))
    capacity = max(1024, 1 << (need - 1).bit_length())               # grows in powers of two: few collective re-allocations
    return DispatchPlan(ctx=ctx, group=group, hidden=hidden, dtype=dtype, order=order, peer_rank=peer_rank, peer_row=peer_row,
                        recv_rows=int(recv_rows[rank]), capacity=capacity, local_counts=[int(c) for c in local_counts])


def static_slot_rows(world: int, per_source_capacity: int) -> int:
    """Rows of one local expert's slot when every source sends at most ``per_source_capacity`` rows to it."""
    return (world * per_source_capacity + 127) // 128 * 128


def build_static_plan(ctx, group, expert_of_assignment: torch.Tensor, num_experts: int, hidden: int, dtype: torch.dtype,
                      per_source_capacity: int) -> DispatchPlan:
    """Plan with STATIC shapes and no host read. ``expert_of_assignment [M]`` holds the expert of every (token, choice) or
    ``num_experts`` for an assignment the capacity limit dropped; every source sends at most ``per_source_capacity`` rows
    to one expert, so a local expert's slot of ``static_slot_rows`` rows always suffices. Collective over ``group`` (one
    all-gather of the counts, which stay on the device); the valid rows per local expert come back as a device tensor
    for the grouped expert GEMM."""
    rank, world = ctx.rank, ctx.world
    per = num_experts // world
    dev = expert_of_assignment.device
    slot = static_slot_rows(world, per_source_capacity)
    counts = torch.bincount(expert_of_assignment, minlength=num_experts + 1)              # [E + 1], last = dropped
    all_counts = torch.empty(world, num_experts + 1, dtype=counts.dtype, device=dev)
    dist.all_gather_into_tensor(all_counts.view(-1), counts, group=group)
    order = torch.argsort(expert_of_assignment, stable=True)
    sorted_e = expert_of_assignment[order]
    group_start = counts.cumsum(0) - counts
    pos = torch.arange(sorted_e.numel(), device=dev) - group_start[sorted_e]
    before_me = all_counts[:rank].sum(0) if rank > 0 else torch.zeros_like(counts)       # rows of lower ranks per expert
    valid = sorted_e < num_experts
    local_e = torch.remainder(sorted_e, per)
    peer_row = torch.where(valid, local_e * slot + before_me[sorted_e] + pos, torch.zeros_like(pos)).to(torch.int64)
    peer_rank = torch.where(valid, torch.div(sorted_e, per, rounding_mode="floor"), torch.full_like(sorted_e, -1)).to(torch.int32)
    recv_counts = all_counts[:, rank * per:(rank + 1) * per].sum(0).to(torch.int32)
    return DispatchPlan(ctx=ctx, group=group, hidden=hidden, dtype=dtype, order=order, peer_rank=peer_rank, peer_row=peer_row,
                        recv_rows=per * slot, capacity=per * slot, local_counts=None, recv_counts=recv_counts, slot_rows=slot)


class _PeerDispatch(torch.autograd.Function):
    """``flat[token_of_row]`` rows -> the owners' expert-major buffers; returns this rank's received rows."""

    @staticmethod
    def forward(ctx, flat, token_of_row, plan: DispatchPlan):
        flat = flat.contiguous()
        plan.push(flat, token_of_row, "a")
        plan.barrier()
        ctx.plan, ctx.token_of_row, ctx.n_tokens = plan, token_of_row, flat.shape[0]
        return plan.local_rows("a").clone()

    @staticmethod
    def backward(ctx, d_recv):
        plan = ctx.plan
        plan.local_rows("b").copy_(d_recv)
        plan.barrier()
        d_rows = plan.pull("b")
        d_flat = torch.zeros(ctx.n_tokens, plan.hidden, dtype=d_rows.dtype, device=d_rows.device).index_add_(0, ctx.token_of_row, d_rows)
        return d_flat, None, None


class _PeerCombine(torch.autograd.Function):
    """This rank's processed rows (expert-major) -> every source pulls its rows back, in its sorted assignment order."""

    @staticmethod
    def forward(ctx, processed, plan: DispatchPlan):
        plan.local_rows("b").copy_(processed)
        plan.barrier()
        ctx.plan = plan
        return plan.pull("b")

    @staticmethod
    def backward(ctx, d_back):
        plan = ctx.plan
        plan.push(d_back.contiguous(), None, "a")
        plan.barrier()
        return plan.local_rows("a").clone(), None


def dispatch(flat: torch.Tensor, token_of_row: torch.Tensor, plan: DispatchPlan) -> torch.Tensor:
    return _PeerDispatch.apply(flat, token_of_row, plan)


def combine(processed: torch.Tensor, plan: DispatchPlan) -> torch.Tensor:
    return _PeerCombine.apply(processed, plan)

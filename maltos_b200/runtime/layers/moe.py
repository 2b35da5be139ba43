"""Expert-parallel mixture of experts.

Each rank of the EP group keeps ``num_experts / ep`` contiguous experts. Tokens are routed (softmax router, top-k,
optional capacity limit), sorted by destination rank, exchanged with a variable-split all-to-all together with their
gate weights and local expert ids, run through the local experts in expert order, and returned to their source rank
where the gated outputs are summed per token. Every local expert is called even with zero tokens so that all replicas
execute the same module sequence (ZeRO-3 hooks depend on it). The Switch-style load-balance loss is computed from the
local tokens. With the defaults (top-1, no capacity) this is the reference layer (``runtime/layers/moe.py:19-163``).

On CUDA with peer access (default; ``MALTOS_B200_MOE_PEER=0`` turns it off) dispatch and combine are one-sided row
transfers over NVLink into /
out of the peers' expert-major buffers (``maltos_b200.ops.moe_dispatch``): one count all-gather instead of the count
exchange, no gate / expert-id traffic, two row kernels instead of four all-to-alls. The ``all_to_all_single`` path below
is the NCCL / gloo implementation and the oracle.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.parallel.expert_interfaces import ExpertParallelMoEModule


def _all_to_all_v(out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits, group) -> None:
    """Variable-split all-to-all along dim 0; gloo goes through fp32 for 16-bit floats."""
    low = inp.dtype in (torch.bfloat16, torch.float16) and dist.get_backend(group) == "gloo"
    if low:
        o32 = torch.empty(out.shape, dtype=torch.float32, device=out.device)
        dist.all_to_all_single(o32, inp.float().contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        out.copy_(o32)
    else:
        dist.all_to_all_single(out, inp.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.out_splits, ctx.in_splits, ctx.group = out_splits, in_splits, group
        out = torch.empty((sum(out_splits), *x.shape[1:]), dtype=x.dtype, device=x.device)
        _all_to_all_v(out, x, out_splits, in_splits, group)
        return out

    @staticmethod
    def backward(ctx, dy):
        dx = torch.empty((sum(ctx.in_splits), *dy.shape[1:]), dtype=dy.dtype, device=dy.device)
        _all_to_all_v(dx, dy.contiguous(), ctx.in_splits, ctx.out_splits, ctx.group)
        return dx, None, None, None


def exchange_counts(send_counts: torch.Tensor, group) -> torch.Tensor:
    recv = torch.empty_like(send_counts)
    ones = [1] * send_counts.numel()
    dist.all_to_all_single(recv, send_counts.contiguous(), output_split_sizes=ones, input_split_sizes=ones, group=group)
    return recv


class ExpertParallelMoE(nn.Module):
    def __init__(self, *, router: nn.Module, local_experts: nn.ModuleList, local_expert_ids: list[int], dim: int,
                 num_experts: int, ep_group, top_k: int = 1, capacity_factor: float | None = None) -> None:
        super().__init__()
        self.router = router
        self.local_experts = local_experts
        self.local_expert_ids = tuple(local_expert_ids)
        self.hidden_size = dim
        self.num_experts = num_experts
        self.ep_group = ep_group
        self.ep_rank = dist.get_rank(ep_group)
        self.ep_world_size = dist.get_world_size(ep_group)
        self.top_k = top_k
        self.capacity_factor = capacity_factor
        if num_experts % self.ep_world_size:
            raise ValueError(f"ExpertParallelPlugin requires num_experts divisible by ep size, got num_experts={num_experts}, ep={self.ep_world_size}")
        if len(self.local_expert_ids) * self.ep_world_size != num_experts:
            raise ValueError("ExpertParallelPlugin expected evenly sharded local experts")

    @classmethod
    def from_moe(cls, moe: ExpertParallelMoEModule, ep_group) -> "ExpertParallelMoE":
        n = int(moe.num_experts)
        if len(moe.experts) != n:
            raise ValueError(f"ExpertParallelPlugin expected len(experts)==num_experts, got {len(moe.experts)} vs {n}")
        if int(moe.dim) <= 0 or int(moe.hidden_size) <= 0:
            raise ValueError("ExpertParallelPlugin requires positive moe.dim and moe.hidden_size")
        rank, world = dist.get_rank(ep_group), dist.get_world_size(ep_group)
        per = n // world
        ids = list(range(rank * per, (rank + 1) * per))
        return cls(router=moe.router, local_experts=nn.ModuleList([moe.experts[i] for i in ids]), local_expert_ids=ids,
                   dim=int(moe.dim), num_experts=n, ep_group=ep_group, top_k=int(getattr(moe, "top_k", 1)),
                   capacity_factor=getattr(moe, "capacity_factor", None))

    def forward(self, x: torch.Tensor, *, return_aux_loss: bool = False):
        from maltos_b200.models.tiny_moe_transformer import capacity_keep_mask, route_and_balance

        B, S, H = x.shape
        flat = x.reshape(-1, H)
        N = flat.shape[0]
        logits = self.router(flat)
        idx, gate, aux = route_and_balance(logits, self.top_k, need_aux=return_aux_loss)   # [N,k]
        if self.capacity_factor is not None:
            cap = max(1, int(self.capacity_factor * N * self.top_k / self.num_experts + 0.999999))
            keep = capacity_keep_mask(idx, self.num_experts, cap)
        else:
            keep = None
        per = len(self.local_expert_ids)
        a_expert = idx.reshape(-1)
        a_gate = gate.reshape(-1)
        a_token = torch.arange(N, device=x.device).repeat_interleave(self.top_k)
        from maltos_b200.ops import moe_dispatch
        from maltos_b200.ops.moe import swiglu_expert_weights

        peer = moe_dispatch.peer_context(self.ep_group, flat)
        weights = swiglu_expert_weights(self.local_experts, flat) if (peer is not None and keep is not None) else None
        if weights is not None:
            # capacity-bounded product path: static shapes end to end, counts stay on the device (no host read)
            out = self._forward_peer_static(peer, flat, a_expert, a_gate, a_token, keep.reshape(-1), cap, weights).view(B, S, H)
            return (out, aux) if return_aux_loss else out
        if keep is not None:                                              # dropped assignments are not sent at all
            sel = keep.reshape(-1).nonzero(as_tuple=False).flatten()
            a_expert, a_gate, a_token = a_expert[sel], a_gate[sel], a_token[sel]
        if peer is not None:
            out = self._forward_peer(peer, flat, a_expert, a_gate, a_token).view(B, S, H)
            return (out, aux) if return_aux_loss else out
        dest = torch.div(a_expert, per, rounding_mode="floor")
        order = torch.argsort(dest, stable=True)
        send_tok = flat.index_select(0, a_token[order])
        send_gate = a_gate[order]
        send_local = (a_expert - dest * per)[order].to(torch.int64)
        send_counts = torch.bincount(dest, minlength=self.ep_world_size).to(torch.int64)
        recv_counts = exchange_counts(send_counts, self.ep_group)
        in_splits, out_splits = send_counts.tolist(), recv_counts.tolist()
        recv_tok = _AllToAll.apply(send_tok, out_splits, in_splits, self.ep_group)
        recv_gate = _AllToAll.apply(send_gate.unsqueeze(1), out_splits, in_splits, self.ep_group).squeeze(1)
        recv_local = torch.empty(sum(out_splits), dtype=torch.int64, device=x.device)
        dist.all_to_all_single(recv_local, send_local.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=self.ep_group)
        # run the local experts on contiguous slices (sorted by expert), always entering every expert
        by_expert = torch.argsort(recv_local, stable=True)
        counts = torch.bincount(recv_local, minlength=per).tolist()
        grouped = recv_tok.index_select(0, by_expert)
        g_gate = recv_gate.index_select(0, by_expert).unsqueeze(1).to(grouped.dtype)
        outs, at = [], 0
        for e, n in enumerate(counts):
            piece = self.local_experts[e](grouped[at:at + n])
            outs.append(piece * g_gate[at:at + n])
            at += n
        processed = torch.cat(outs, dim=0) if outs else grouped
        recv_out = torch.zeros_like(recv_tok).index_copy(0, by_expert, processed.to(recv_tok.dtype))
        back = _AllToAll.apply(recv_out, in_splits, out_splits, self.ep_group)
        out = torch.zeros_like(flat).index_add(0, a_token[order], back)
        out = out.view(B, S, H)
        if not return_aux_loss:
            return out
        return out, aux

    def _forward_peer_static(self, peer, flat, a_expert, a_gate, a_token, keep, cap, weights):
        """Capacity-limited routing with static shapes: dropped assignments keep their place in the (token, choice) list
        with the sentinel expert ``num_experts``; rows travel one-sided into fixed expert slots of the owners' symmetric
        buffers; ALL local experts run in one grouped tcgen05 GEMM launch per projection that reads the valid row counts
        from device memory. Nothing in this path waits for the host."""
        from maltos_b200.ops import moe_dispatch
        from maltos_b200.ops.moe import grouped_swiglu_experts

        a_expert = torch.where(keep, a_expert, torch.full_like(a_expert, self.num_experts))
        plan = moe_dispatch.build_static_plan(peer, self.ep_group, a_expert, self.num_experts, flat.shape[1], flat.dtype, cap)
        token_of_row = a_token[plan.order]
        received = moe_dispatch.dispatch(flat, token_of_row, plan)          # [experts_here * slot_rows, H]
        gates, ups, downs = weights
        processed = grouped_swiglu_experts(received, plan.recv_counts, plan.slot_rows, gates, ups, downs)
        back = moe_dispatch.combine(processed, plan)                        # [N * k, H]; zeros for dropped assignments
        gated = back * a_gate[plan.order].unsqueeze(1).to(back.dtype)
        return torch.zeros_like(flat).index_add(0, token_of_row, gated)

    def _forward_peer(self, peer, flat, a_expert, a_gate, a_token):
        """Dispatch / combine as one-sided row transfers through the peers' symmetric buffers."""
        from maltos_b200.ops import moe_dispatch

        plan = moe_dispatch.build_plan(peer, self.ep_group, a_expert, self.num_experts, flat.shape[1], flat.dtype)
        token_of_row = a_token[plan.order]
        received = moe_dispatch.dispatch(flat, token_of_row, plan)          # [rows, H], sorted by local expert
        outs, at = [], 0
        for e, n in enumerate(plan.local_counts):                           # every expert is entered, also with zero rows
            outs.append(self.local_experts[e](received[at:at + n]))
            at += n
        processed = torch.cat(outs, dim=0).to(flat.dtype) if outs else received
        back = moe_dispatch.combine(processed, plan)                        # [assignments, H] in dispatch order
        gated = back * a_gate[plan.order].unsqueeze(1).to(back.dtype)
        return torch.zeros_like(flat).index_add(0, token_of_row, gated)

"""Fused MoE router: softmax, top-k (optionally renormalised), assignment counts and mean router probabilities in one
kernel pass (``csrc/moe_router.cu``), with a matching backward; eager PyTorch elsewhere.

``route(logits, top_k, renormalize) -> (expert_idx [N,k] int64, gate [N,k], mean_prob [E] fp32, counts [E] int64)``.
``gate`` and ``mean_prob`` are differentiable with respect to ``logits``; the Switch-style load-balance loss is
``E * sum_e counts_e / (N k) * mean_prob_e``.
"""
from __future__ import annotations

import torch

from . import _lib


def route_reference(logits: torch.Tensor, top_k: int, renormalize: bool = True):
    probs = logits.float().softmax(dim=-1)
    gate, idx = probs.topk(top_k, dim=-1)
    if top_k > 1 and renormalize:
        gate = gate / gate.sum(dim=-1, keepdim=True)
    counts = torch.bincount(idx.reshape(-1), minlength=logits.shape[-1])
    return idx, gate.to(logits.dtype), probs.mean(dim=0), counts


class _Route(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, top_k, renormalize):
        N, E = logits.shape
        dev = logits.device
        idx = torch.empty((N, top_k), dtype=torch.int64, device=dev)
        gate = torch.empty((N, top_k), dtype=torch.float32, device=dev)
        rowmax = torch.empty(N, dtype=torch.float32, device=dev)
        rowsum = torch.empty(N, dtype=torch.float32, device=dev)
        prob_sum = torch.zeros(E, dtype=torch.float32, device=dev)
        counts = torch.zeros(E, dtype=torch.int32, device=dev)
        x = logits.contiguous()
        _lib.check(_lib.lib().mb_moe_router_fwd(_lib.ptr(x), _lib.c_int(1 if x.dtype == torch.bfloat16 else 0), _lib.c_ll(N), _lib.c_int(E),
                                                _lib.c_int(top_k), _lib.c_int(1 if renormalize else 0), _lib.ptr(idx), _lib.ptr(gate),
                                                _lib.ptr(rowmax), _lib.ptr(rowsum), _lib.ptr(prob_sum), _lib.ptr(counts), _lib.stream_ptr()),
                   "mb_moe_router_fwd")
        ctx.save_for_backward(x, idx, gate, rowmax, rowsum)
        ctx.top_k, ctx.renormalize = top_k, renormalize
        ctx.mark_non_differentiable(idx, counts)
        return idx, gate, prob_sum / max(N, 1), counts.to(torch.int64)

    @staticmethod
    def backward(ctx, _didx, dgate, dmean, _dcounts):
        x, idx, gate, rowmax, rowsum = ctx.saved_tensors
        N, E = x.shape
        dgate = torch.zeros_like(gate) if dgate is None else dgate.float().contiguous()
        aux_w = None if dmean is None else (dmean.float() / max(N, 1)).contiguous()
        dlogits = torch.empty_like(x)
        _lib.check(_lib.lib().mb_moe_router_bwd(_lib.ptr(x), _lib.c_int(1 if x.dtype == torch.bfloat16 else 0), _lib.c_ll(N), _lib.c_int(E),
                                                _lib.c_int(ctx.top_k), _lib.c_int(1 if ctx.renormalize else 0), _lib.ptr(idx), _lib.ptr(gate),
                                                _lib.ptr(dgate), _lib.ptr(rowmax), _lib.ptr(rowsum), _lib.ptr(aux_w), _lib.ptr(dlogits),
                                                _lib.stream_ptr()), "mb_moe_router_bwd")
        return dlogits, None, None


def _kernel_ok(logits: torch.Tensor, top_k: int) -> bool:
    return (logits.is_cuda and logits.dim() == 2 and logits.dtype in (torch.float32, torch.bfloat16) and logits.shape[1] <= 1024
            and 1 <= top_k <= min(8, logits.shape[1]))


def route(logits: torch.Tensor, top_k: int = 1, renormalize: bool = True):
    """See module docstring. ``gate`` comes back in the dtype of ``logits``."""
    if _kernel_ok(logits, top_k):
        idx, gate, mean_prob, counts = _Route.apply(logits, top_k, renormalize)
        return idx, gate.to(logits.dtype), mean_prob, counts
    return route_reference(logits, top_k, renormalize)


def load_balance_loss_from_stats(mean_prob: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    total = counts.sum().clamp_min(1).to(mean_prob.dtype)
    return mean_prob.shape[0] * (counts.to(mean_prob.dtype) / total * mean_prob).sum()

"""Cross-entropy and the fused linear + cross-entropy head (``csrc/loss_optim.cu`` + ``csrc/gemm.cu``).

``cross_entropy_mean(logits, labels)`` is the reference's ``causal_cross_entropy`` (``utils/losses.py:9-15``):
``sum(CE over labels != ignore) / max(#targets, 1)``.

``linear_cross_entropy(h, weight, labels)`` computes the same loss for ``logits = h @ weight.T`` without keeping
the logits: tokens are processed in chunks; for each chunk the logits GEMM, the softmax statistics, the in-place
``d logits`` and the two backward GEMMs (``dh`` and the accumulation into ``dW``) run back to back while the chunk
is hot, and only ``dh``/``dW`` survive. The target count stays on the device (no host sync). This replaces the
replicated ``[B*S, V]`` logits + ATen CE of the reference head (``models/llama.py:366-368``).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import gemm

DEFAULT_CHUNK_TOKENS = 8192


def _ce_launch(logits, labels, loss_rows, lse, grad_out, grad_scale, ignore_index) -> None:
    rows, V = logits.shape
    _lib.check(_lib.lib().mb_cross_entropy(_lib.ptr(logits), _lib.c_int(int(logits.dtype == torch.float32)), _lib.c_ll(logits.stride(0)),
                                           _lib.ptr(labels), _lib.ptr(loss_rows), _lib.ptr(lse), _lib.ptr(grad_out), _lib.ptr(grad_scale),
                                           _lib.c_ll(rows), _lib.c_int(V), _lib.c_ll(ignore_index), _lib.stream_ptr()), "mb_cross_entropy")


class _CrossEntropyMean(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index):
        rows = logits.shape[0]
        loss_rows = torch.empty(rows, device=logits.device, dtype=torch.float32)
        _ce_launch(logits, labels, loss_rows, None, None, None, ignore_index)
        inv = 1.0 / (labels != ignore_index).sum().clamp_min(1).to(torch.float32)
        ctx.save_for_backward(logits, labels, inv)
        ctx.ignore_index = ignore_index
        return (loss_rows.sum() * inv).to(torch.float32)

    @staticmethod
    def backward(ctx, dloss):
        logits, labels, inv = ctx.saved_tensors
        scale = (dloss.float() * inv).reshape(1).contiguous()
        grad = torch.empty_like(logits)
        scratch = torch.empty(logits.shape[0], device=logits.device, dtype=torch.float32)
        _ce_launch(logits, labels, scratch, None, grad, scale, ctx.ignore_index)
        return grad, None, None


def cross_entropy_mean(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """``logits [N, V]``, ``labels [N]`` (already shifted). Returns an fp32 scalar."""
    if _lib.use_kernels(logits) and logits.dtype in (torch.bfloat16, torch.float32):
        lg = logits if logits.stride(-1) == 1 else logits.contiguous()
        return _CrossEntropyMean.apply(lg, labels.contiguous().to(torch.long), ignore_index)
    total = F.cross_entropy(logits.float(), labels, ignore_index=ignore_index, reduction="sum")
    return total / (labels != ignore_index).sum().clamp_min(1)


class _LinearCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, weight, labels, ignore_index, chunk_tokens, group):
        N, H = h.shape
        V = weight.shape[0]
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        count = _global_count(labels, ignore_index, group)
        inv = (1.0 / count.clamp_min(1).to(torch.float32)).reshape(1)
        loss_rows = torch.empty(N, device=h.device, dtype=torch.float32)
        dh = torch.empty_like(h) if need_dh else None
        # several token chunks add into dW: the running sum stays in fp32 and is rounded to the weight's dtype once
        n_chunks = (N + chunk_tokens - 1) // chunk_tokens
        dw = None
        if need_dw:
            dw = torch.zeros(weight.shape, device=weight.device, dtype=torch.float32 if n_chunks > 1 else weight.dtype)
        want_grad = need_dh or need_dw
        logits_buf = torch.empty((min(chunk_tokens, N), V), device=h.device, dtype=h.dtype)
        for start in range(0, N, chunk_tokens):
            n = min(chunk_tokens, N - start)
            hc = h[start:start + n]
            lg = logits_buf[:n]
            gemm(hc, weight, out=lg)
            _ce_launch(lg, labels[start:start + n], loss_rows[start:start + n], None, lg if want_grad else None, inv, ignore_index)
            if need_dh:
                gemm(lg, weight, b_mn=True, out=dh[start:start + n])          # dlogits[n,V] @ W[V,H]
            if need_dw:
                gemm(lg, hc, a_mn=True, b_mn=True, out=dw, accumulate=True)   # dlogits^T[V,n] @ h[n,H]
        if dw is not None and dw.dtype != weight.dtype:
            dw = dw.to(weight.dtype)
        ctx.save_for_backward(dh, dw)
        return _sum_over_group(loss_rows.sum() * inv.squeeze(0), group)

    @staticmethod
    def backward(ctx, dloss):
        dh, dw = ctx.saved_tensors
        g = dloss.to(torch.float32)
        if dh is not None:
            dh = dh * g.to(dh.dtype)
        if dw is not None:
            dw = dw * g.to(dw.dtype)
        return dh, dw, None, None, None, None


def _global_count(labels: torch.Tensor, ignore_index: int, group) -> torch.Tensor:
    count = (labels != ignore_index).sum()
    if group is not None:
        import torch.distributed as dist

        count = count.to(torch.float32 if labels.is_cuda else torch.float64)
        dist.all_reduce(count, op=dist.ReduceOp.SUM, group=group)
    return count


def _sum_over_group(value: torch.Tensor, group) -> torch.Tensor:
    if group is None:
        return value
    import torch.distributed as dist

    out = value.detach().clone()
    dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
    return out


class _GroupSum(torch.autograd.Function):
    """Forward: sum of the per-rank scalars over the group. Backward: identity (each rank differentiates its term)."""

    @staticmethod
    def forward(ctx, value, group):
        return _sum_over_group(value, group)

    @staticmethod
    def backward(ctx, grad):
        return grad, None


def linear_cross_entropy(h: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                         chunk_tokens: int = DEFAULT_CHUNK_TOKENS, group=None) -> torch.Tensor:
    """Mean CE of ``h @ weight.T`` against ``labels`` without materialising all logits. ``h [N,H]``, ``weight [V,H]``.

    With ``group`` the tokens are split over the ranks of the group (sequence-parallel head): the mean is taken over
    the targets of all ranks and the returned scalar is the same on every rank."""
    h2 = h.reshape(-1, h.shape[-1])
    lab = labels.reshape(-1)
    if _lib.use_kernels(h2, weight) and h2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        return _LinearCrossEntropy.apply(h2.contiguous(), weight, lab.contiguous().to(torch.long), ignore_index, chunk_tokens, group)
    if group is None:
        return cross_entropy_mean(F.linear(h2, weight), lab, ignore_index)
    total = F.cross_entropy(F.linear(h2, weight).float(), lab, ignore_index=ignore_index, reduction="sum")
    count = _global_count(lab, ignore_index, group).clamp_min(1)
    return _GroupSum.apply(total / count.to(total.dtype), group)

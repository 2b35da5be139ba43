"""Several linear layers that consume the same input, run as ONE GEMM (q/k/v, gate/up).

If the weights sit back to back in one storage (see :func:`fuse_parameters`) the fused weight is a zero-copy view and
forward / dgrad / wgrad are one tcgen05 GEMM each; the per-layer weight gradients are views of the fused result.
Otherwise every member gets its own GEMM writing into its column slice of the packed output. The packed layout is
returned as ``offsets`` (column offset of each member) so consumers (RoPE split, SwiGLU) can index it.

This is the single-device counterpart of the reference's grouped projection
(``runtime/layers/functional.py:369-486``), which also shares one input (there: one all-gather) across members.
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import _lib
from .gemm import gemm


def _memory_order(weights: Sequence[torch.Tensor]) -> list[int] | None:
    """Indices of ``weights`` in address order if they tile one contiguous region, else None."""
    if any((not w.is_contiguous()) or w.dim() != 2 for w in weights):
        return None
    k = weights[0].shape[1]
    if any(w.shape[1] != k or w.dtype != weights[0].dtype or w.device != weights[0].device for w in weights):
        return None
    try:
        base = weights[0].untyped_storage().data_ptr()
        if any(w.untyped_storage().data_ptr() != base for w in weights):
            return None
    except RuntimeError:
        return None
    order = sorted(range(len(weights)), key=lambda i: weights[i].data_ptr())
    for a, b in zip(order, order[1:]):
        wa = weights[a]
        if wa.data_ptr() + wa.numel() * wa.element_size() != weights[b].data_ptr():
            return None
    return order


def _fused_view(weights: Sequence[torch.Tensor], order: list[int]) -> torch.Tensor:
    first = weights[order[0]]
    rows = sum(w.shape[0] for w in weights)
    return torch.as_strided(first, (rows, first.shape[1]), (first.shape[1], 1), first.storage_offset())


def fuse_parameters(params: Sequence[torch.nn.Parameter]) -> torch.Tensor:
    """Re-point ``param.data`` of 2-D parameters with equal inner size at consecutive slices of one new buffer
    (values preserved, in the given order). Returns the fused ``[sum(rows), K]`` buffer."""
    k = params[0].shape[1]
    if any(p.dim() != 2 or p.shape[1] != k for p in params):
        raise ValueError("fuse_parameters: all parameters must be 2-D with the same inner size")
    rows = [p.shape[0] for p in params]
    buf = torch.empty((sum(rows), k), dtype=params[0].dtype, device=params[0].device)
    at = 0
    with torch.no_grad():
        for p, r in zip(params, rows):
            buf[at:at + r].copy_(p.data)
            p.data = buf[at:at + r]
            at += r
    return buf


class _GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, *weights):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        order = _memory_order(weights)
        M = x2.shape[0]
        n_total = sum(w.shape[0] for w in weights)
        out = torch.empty((M, n_total), device=x.device, dtype=x.dtype)
        if order is not None:
            gemm(x2, _fused_view(weights, order), out=out)
            layout = order
        else:
            layout = list(range(len(weights)))
            at = 0
            for i in layout:
                n = weights[i].shape[0]
                gemm(x2, weights[i], out=out[:, at:at + n])
                at += n
        ctx.save_for_backward(x2, *weights)
        ctx.fused = order is not None
        ctx.layout = layout
        ctx.xshape = x.shape
        return out.view(*x.shape[:-1], n_total)

    @staticmethod
    def backward(ctx, dout):
        x2, *weights = ctx.saved_tensors
        layout = ctx.layout
        n_total = dout.shape[-1]
        d2 = dout.reshape(-1, n_total)
        if d2.stride(1) != 1 or d2.stride(0) % 8:
            d2 = d2.contiguous()
        need_x = ctx.needs_input_grad[0]
        need_w = any(ctx.needs_input_grad[1:])
        dx = None
        dws: list = [None] * len(weights)
        if ctx.fused:
            # the members may have been re-materialised elsewhere since the forward (sharded parameters): the zero-copy
            # view is only valid if they still tile one region in the same order, otherwise pack a copy
            fused = _fused_view(weights, layout) if _memory_order(weights) == layout else torch.cat([weights[i] for i in layout], dim=0)
            if need_x:
                dx = gemm(d2, fused, b_mn=True).view(ctx.xshape)
            if need_w:
                dwf = gemm(d2, x2, a_mn=True, b_mn=True)
                at = 0
                for i in layout:
                    n = weights[i].shape[0]
                    dws[i] = dwf[at:at + n]
                    at += n
        else:
            at = 0
            first = True
            if need_x:
                dx2 = torch.empty_like(x2)
            for i in layout:
                n = weights[i].shape[0]
                piece = d2[:, at:at + n]
                if need_x:
                    gemm(piece, weights[i], b_mn=True, out=dx2, accumulate=not first)
                if ctx.needs_input_grad[1 + i]:
                    dws[i] = gemm(piece, x2, a_mn=True, b_mn=True)
                first = False
                at += n
            if need_x:
                dx = dx2.view(ctx.xshape)
        return (dx, *dws)


def packed_offsets(weights: Sequence[torch.Tensor]) -> list[int]:
    """Column offset of every member inside the packed output of :func:`grouped_linear`."""
    order = _memory_order(weights) if _lib.use_kernels(*weights) else None
    layout = order if order is not None else list(range(len(weights)))
    offs = [0] * len(weights)
    at = 0
    for i in layout:
        offs[i] = at
        at += weights[i].shape[0]
    return offs


def grouped_linear(x: torch.Tensor, weights: Sequence[torch.Tensor]) -> tuple[torch.Tensor, list[int]]:
    """``[x @ w_i.T for w_i in weights]`` packed along the last dim. Returns ``(packed, offsets)``."""
    weights = list(weights)
    if _lib.use_kernels(x, *weights) and x.dtype == torch.bfloat16 and all(w.dtype == torch.bfloat16 for w in weights):
        offs = packed_offsets(weights)
        return _GroupedLinear.apply(x, *weights), offs
    offs, at = [], 0
    for w in weights:
        offs.append(at)
        at += w.shape[0]
    return torch.nn.functional.linear(x, torch.cat(weights, dim=0)), offs

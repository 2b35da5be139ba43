"""Multi-tensor optimizer kernels (``csrc/loss_optim.cu``): AdamW over fp32 masters with optional bf16 write-back and
a device-resident gradient scale, sum of squares over many tensors, and in-place scaling by a device scalar.
One launch per call regardless of the number of tensors; replaces ATen's multi-tensor fused Adam + cast kernels
used by the reference (``runtime/optim.py:43-71`` with ``torch.optim.AdamW(fused=True)``)."""
from __future__ import annotations

import math
import struct

import torch

from . import _lib

_CHUNK = None


def _chunk() -> int:
    global _CHUNK
    if _CHUNK is None:
        _CHUNK = int(_lib.lib().mb_mt_chunk())
    return _CHUNK


def _nchunks(n: int) -> int:
    return max(1, (n + _chunk() - 1) // _chunk())


def _adamw_reference(p, g, m, v, lowp, step, lr, beta1, beta2, eps, weight_decay, grad_scale) -> None:
    g = g.to(torch.float32)
    if grad_scale is not None:
        g = g * grad_scale.to(g.device)
    p.mul_(1 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
    if lowp is not None:
        lowp.copy_(p)


def adamw_multi_tensor(items, *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
                       grad_scale: torch.Tensor | None = None) -> None:
    """``items``: list of ``(param_fp32, grad, exp_avg, exp_avg_sq, low_precision_param_or_None, step)``."""
    if not items:
        return
    if not items[0][0].is_cuda:
        for p, g, m, v, lowp, step in items:
            _adamw_reference(p.data, g, m, v, lowp.data if lowp is not None else None, step, lr, beta1, beta2, eps, weight_decay, grad_scale)
        return
    device = items[0][0].device
    rows, corr, keep = [], [], []
    first = 0
    for p, g, m, v, lowp, step in items:
        if p.dtype != torch.float32 or m.dtype != torch.float32 or v.dtype != torch.float32:
            raise TypeError("adamw_multi_tensor: params and moments must be fp32")
        if g.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"adamw_multi_tensor: unsupported grad dtype {g.dtype}")
        if not (p.is_contiguous() and m.is_contiguous() and v.is_contiguous()):
            raise ValueError("adamw_multi_tensor: params and moments must be contiguous")
        if not g.is_contiguous():
            # the copy's address goes into the table: it must stay allocated until the launch below has been queued,
            # otherwise the next temporary of this loop could reuse its block and two rows would alias
            g = g.contiguous()
            keep.append(g)
        if lowp is not None and (lowp.dtype != torch.bfloat16 or not lowp.is_contiguous()):
            raise TypeError("adamw_multi_tensor: low-precision params must be contiguous bf16")
        n = p.numel()
        rows.append((p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), lowp.data_ptr() if lowp is not None else 0,
                     n, int(g.dtype == torch.bfloat16), first))
        first += _nchunks(n)
        corr += [1 - beta1 ** step, math.sqrt(1 - beta2 ** step)]
    table = torch.tensor(rows, dtype=torch.int64).to(device, non_blocking=False)
    bias = torch.tensor(corr, dtype=torch.float32).to(device, non_blocking=False)
    _lib.check(_lib.lib().mb_adamw_multi_tensor(_lib.ptr(table), _lib.ptr(bias), _lib.c_int(len(rows)), _lib.c_ll(first),
                                                _lib.c_float(lr), _lib.c_float(beta1), _lib.c_float(beta2), _lib.c_float(eps),
                                                _lib.c_float(weight_decay), _lib.ptr(grad_scale), _lib.stream_ptr()), "mb_adamw_multi_tensor")
    # the launch is asynchronous: keep the tables alive until the stream has consumed them
    table.record_stream(torch.cuda.current_stream())
    bias.record_stream(torch.cuda.current_stream())
    for t in keep:
        t.record_stream(torch.cuda.current_stream())


def _vec_table(tensors, weights, device):
    rows = []
    first = 0
    for t, w in zip(tensors, weights):
        if t.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"multi-tensor op: unsupported dtype {t.dtype}")
        if not t.is_contiguous():
            raise ValueError("multi-tensor op: tensors must be contiguous")
        wbits = struct.unpack("<q", struct.pack("<d", float(w)))[0]
        rows.append((t.data_ptr(), t.numel(), int(t.dtype == torch.bfloat16), first, wbits, 0, 0, 0))
        first += _nchunks(t.numel())
    return torch.tensor(rows, dtype=torch.int64).to(device), first


def sum_of_squares(tensors, weights=None) -> torch.Tensor:
    """Device fp64 scalar ``sum_t w_t * ||x_t||^2`` (one launch on CUDA). ``weights`` default to 1."""
    tensors = [t for t in tensors if t is not None and t.numel() > 0]
    weights = [1.0] * len(tensors) if weights is None else list(weights)
    if not tensors:
        return torch.zeros((), dtype=torch.float64)
    device = tensors[0].device
    if not tensors[0].is_cuda:
        acc = torch.zeros((), dtype=torch.float64, device=device)
        for t, w in zip(tensors, weights):
            acc += t.detach().double().pow(2).sum() * w
        return acc
    out = torch.zeros((), dtype=torch.float64, device=device)
    table, total = _vec_table(tensors, weights, device)
    _lib.check(_lib.lib().mb_sumsq_multi_tensor(_lib.ptr(table), _lib.c_int(len(tensors)), _lib.c_ll(total), _lib.ptr(out),
                                                _lib.stream_ptr()), "mb_sumsq_multi_tensor")
    table.record_stream(torch.cuda.current_stream())
    return out


def scale_tensors_(tensors, scale: torch.Tensor) -> None:
    """In place ``x_t *= scale`` for all tensors; ``scale`` is a one-element fp32 tensor on the same device."""
    tensors = [t for t in tensors if t is not None and t.numel() > 0]
    if not tensors:
        return
    if not tensors[0].is_cuda:
        for t in tensors:
            t.mul_(scale.to(t.dtype))
        return
    table, total = _vec_table(tensors, [1.0] * len(tensors), tensors[0].device)
    sc = scale.reshape(1).to(torch.float32)
    _lib.check(_lib.lib().mb_scale_multi_tensor(_lib.ptr(table), _lib.c_int(len(tensors)), _lib.c_ll(total), _lib.ptr(sc),
                                                _lib.stream_ptr()), "mb_scale_multi_tensor")
    table.record_stream(torch.cuda.current_stream())


def clip_coefficient(sumsq: torch.Tensor, max_norm: float) -> tuple[torch.Tensor, torch.Tensor]:
    """``(coef, norm)`` as one-element fp32 device tensors: ``coef = min(1, max_norm / (sqrt(sumsq) + 1e-6))``."""
    if not sumsq.is_cuda:
        norm = sumsq.double().sqrt()
        coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm and max_norm > 0 else torch.ones_like(norm)
        return coef.float().reshape(1), norm.float().reshape(1)
    coef = torch.empty(1, device=sumsq.device, dtype=torch.float32)
    norm = torch.empty(1, device=sumsq.device, dtype=torch.float32)
    sq = sumsq.reshape(1).to(torch.float64)
    _lib.check(_lib.lib().mb_clip_coef(_lib.ptr(sq), _lib.c_float(float(max_norm or 0.0)), _lib.ptr(coef), _lib.ptr(norm),
                                       _lib.stream_ptr()), "mb_clip_coef")
    return coef, norm

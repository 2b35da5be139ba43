"""RMSNorm with an optional fused residual add (``csrc/norm_rope_act.cu``).

``rms_norm(x, w, eps)`` = ``w * x * rsqrt(mean(x^2) + eps)`` with the statistics in fp32, replacing the un-fused
eager ops of the reference (``models/llama.py:55-57``). ``add_rms_norm(x, residual, w, eps)`` returns
``(norm(x + residual), x + residual)`` from a single pass over memory; its backward also folds the gradient of
the residual stream into ``dx``.
"""
from __future__ import annotations

import torch

from . import _lib


def rms_norm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def _kernel_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return _lib.use_kernels(x) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps):
        H = x.shape[-1]
        x2 = x.reshape(-1, H).contiguous()
        rows = x2.shape[0]
        r2 = residual.reshape(-1, H).contiguous() if residual is not None else None
        y = torch.empty_like(x2)
        h = torch.empty_like(x2) if r2 is not None else None
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        w = weight.contiguous()
        _lib.check(_lib.lib().mb_rmsnorm_fwd(_lib.ptr(x2), _lib.ptr(r2), _lib.ptr(w), _lib.ptr(y), _lib.ptr(h), _lib.ptr(rstd),
                                             _lib.c_ll(rows), _lib.c_int(H), _lib.c_float(eps), _lib.stream_ptr()), "mb_rmsnorm_fwd")
        ctx.save_for_backward(h if h is not None else x2, w, rstd)
        ctx.shape = x.shape
        ctx.fused = r2 is not None
        if ctx.fused:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        h, w, rstd = ctx.saved_tensors
        H = h.shape[-1]
        rows = h.shape[0]
        dy2 = dy.reshape(-1, H).contiguous()
        dres = dh.reshape(-1, H).contiguous() if (ctx.fused and dh is not None) else None
        L = _lib.lib()
        nblk = L.mb_rmsnorm_bwd_blocks(_lib.c_ll(rows))
        partial = torch.empty((nblk, H), device=h.device, dtype=torch.float32)
        dx = torch.empty_like(h)
        dw = torch.empty_like(w)
        _lib.check(L.mb_rmsnorm_bwd(_lib.ptr(dy2), _lib.ptr(h), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres), _lib.ptr(dx),
                                    _lib.ptr(partial), _lib.ptr(dw), _lib.c_void_p(0), _lib.c_int(0), _lib.c_ll(rows),
                                    _lib.c_int(H), _lib.stream_ptr()), "mb_rmsnorm_bwd")
        dx = dx.view(ctx.shape)
        if ctx.fused:
            return dx, dx, dw, None
        return dx, None, dw, None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if _kernel_ok(x, weight):
        return _RmsNorm.apply(x, None, weight, eps)
    return rms_norm_reference(x, weight, eps)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """Returns ``(rms_norm(x + residual), x + residual)``."""
    if _kernel_ok(x, weight) and residual.dtype == torch.bfloat16:
        return _RmsNorm.apply(x, residual, weight, eps)
    h = x + residual
    return rms_norm_reference(h, weight, eps), h

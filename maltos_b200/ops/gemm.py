"""bf16 GEMM on the tcgen05 tensor cores and the linear layer built on it.

``gemm`` is the raw entry (``csrc/gemm.cu``); ``linear`` is the differentiable ``y = x W^T (+ b)`` whose
forward, dgrad and wgrad are three calls of the same kernel with different operand layouts, so no
transposed copy of an activation or a weight is ever made. This replaces the ``F.linear`` calls of the
reference (cuBLAS through ATen, e.g. its ``models/llama.py:115-127,196-206``).

On CPU tensors the functions compute the same thing with PyTorch matmuls (test oracle / gloo runs).
"""
from __future__ import annotations

import torch

from . import _lib


def _as_2d(t: torch.Tensor) -> torch.Tensor:
    return t.reshape(-1, t.shape[-1])


def _row_major_2d(t: torch.Tensor) -> torch.Tensor:
    """Return a 2-D view usable by TMA: unit inner stride, 16-byte aligned rows (else a packed copy)."""
    if t.dim() != 2:
        t = _as_2d(t)
    if t.stride(1) != 1 or (t.stride(0) % 8) != 0 or (t.data_ptr() % 16) != 0 or t.stride(0) < t.shape[1]:
        t = t.contiguous()
        if (t.stride(0) % 8) != 0:
            raise ValueError(f"bf16 GEMM operands need a row length that is a multiple of 8, got {tuple(t.shape)}")
    return t


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    accumulate: bool = False,
    bias: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    block_n: int = 0,
) -> torch.Tensor:
    """``C[M,N] (+)= op(A) @ op(B) (+ bias)`` with fp32 accumulation.

    ``a`` is ``[M,K]`` (``a_mn=False``) or stored transposed as ``[K,M]`` (``a_mn=True``);
    ``b`` is ``[N,K]`` (``b_mn=False``) or stored as ``[K,N]`` (``b_mn=True``). ``out`` may be bf16 or fp32.
    """
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"gemm: contraction mismatch {K} vs {Kb}")
    if out is None:
        if accumulate:
            raise ValueError("gemm: accumulate=True needs an `out`")
        out = torch.empty((M, N), device=a.device, dtype=out_dtype or a.dtype)
    if out.shape != (M, N) or out.stride(1) != 1:
        raise ValueError(f"gemm: out must be [{M},{N}] with unit inner stride, got {tuple(out.shape)}")

    if not _lib.use_kernels(a, b):
        af = a.float().t() if a_mn else a.float()
        bf = b.float() if b_mn else b.float().t()
        res = af @ bf
        if bias is not None:
            res = res + bias.float()
        if accumulate:
            res = res + out.float()
        out.copy_(res.to(out.dtype))
        return out

    if M == 0 or N == 0:
        return out                      # nothing to compute (an expert without tokens, an empty shard)
    if K == 0:                          # empty contraction: the product is zero
        if not accumulate:
            out.zero_()
            if bias is not None:
                out += bias.to(out.dtype)
        return out
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError(f"gemm kernel takes bf16 operands, got {a.dtype} / {b.dtype}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"gemm kernel writes bf16 or fp32, got {out.dtype}")
    a2 = _row_major_2d(a)
    b2 = _row_major_2d(b)
    if bias is not None:
        bias = bias.contiguous()
        if bias.dtype != torch.bfloat16:
            bias = bias.to(torch.bfloat16)
    rc = _lib.lib().mb_gemm_bf16(
        _lib.ptr(a2), _lib.c_int(int(a_mn)), _lib.c_ll(a2.stride(0)),
        _lib.ptr(b2), _lib.c_int(int(b_mn)), _lib.c_ll(b2.stride(0)),
        _lib.ptr(out), _lib.c_ll(out.stride(0)),
        _lib.c_int(M), _lib.c_int(N), _lib.c_int(K),
        _lib.c_int(int(out.dtype == torch.float32)), _lib.c_int(int(accumulate)),
        _lib.ptr(bias), _lib.c_int(block_n), _lib.stream_ptr(),
    )
    _lib.check(rc, "mb_gemm_bf16")
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        x2 = _as_2d(x)
        y = gemm(x2, weight, bias=bias)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = _as_2d(dy)
        x2 = _as_2d(x)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view_as(x)  # dy[M,N] @ W[N,K]
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True)  # dy^T[N,M] @ x[M,K]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """Differentiable ``x @ weight.T (+ bias)``; tcgen05 GEMMs on CUDA bf16, ``F.linear`` otherwise."""
    if _lib.use_kernels(x, weight) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        return _Linear.apply(x, weight, bias)
    return torch.nn.functional.linear(x, weight, bias)

"""Attention dispatch on CUDA bf16.

* ``flash_forward`` / ``flash_block_forward``: this library's tcgen05 flash-attention FORWARD kernel
  (``csrc/flash_attn.cu``): full, causal and general position / sequence-id masks, native GQA, returns the log-sum-exp.
  It serves the blocks of ring and HDP attention and, with ``MALTOS_B200_ATTENTION=own``, forward-only dense calls.
* There is no tcgen05 backward kernel yet, so differentiable dense causal attention goes through a LIBRARY path
  (same role as cuBLAS for plain GEMMs): cuDNN's fused attention via torch SDPA with native GQA - on B200 about 3.5x
  the throughput of flash-attn 2 in both directions - then flash-attn 2, then the eager restatement.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from . import _lib


def flash_attention(q, k, v, *, q_positions=None, k_positions=None, q_sequence_ids=None, k_sequence_ids=None,
                    causal=True, scale=None, return_lse=False):
    from .attention import attention_reference

    dense = q_positions is None and q_sequence_ids is None
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v))
    if dense and not needs_grad and os.environ.get("MALTOS_B200_ATTENTION") == "own":
        out, lse = flash_forward(q, k, v, mode=1 if causal else 0, scale=scale)
        return (out, lse) if return_lse else out
    if dense and not return_lse:
        out = _sdpa_cudnn(q, k, v, causal, scale)
        if out is not None:
            return out
        try:
            from flash_attn import flash_attn_func

            return flash_attn_func(q, k, v, causal=causal, softmax_scale=scale)
        except ImportError:
            pass
    return attention_reference(q, k, v, q_positions=q_positions, k_positions=k_positions, q_sequence_ids=q_sequence_ids,
                               k_sequence_ids=k_sequence_ids, causal=causal, scale=scale, return_lse=return_lse)


_CUDNN_SDPA_OK: bool | None = None


def _sdpa_cudnn(q, k, v, causal, scale):
    """``[B,S,h,D]`` attention through torch SDPA pinned to the cuDNN backend; None when that backend is unavailable."""
    global _CUDNN_SDPA_OK
    if _CUDNN_SDPA_OK is False or (causal and q.shape[1] != k.shape[1]):
        return None
    try:
        import torch.nn.functional as F
        from torch.nn.attention import SDPBackend, sdpa_kernel

        with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
            out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal,
                                                 scale=scale, enable_gqa=q.shape[2] != k.shape[2])
        _CUDNN_SDPA_OK = True
        return out.transpose(1, 2)
    except (RuntimeError, ImportError):
        if _CUDNN_SDPA_OK is None:
            _CUDNN_SDPA_OK = False
        return None


def _as_bshd(t: torch.Tensor) -> torch.Tensor:
    """A view the kernel can address: heads contiguous inside a token, token / batch strides multiples of 8 elements."""
    D = t.shape[-1]
    if t.stride(3) != 1 or t.stride(2) != D or t.stride(1) % 8 or t.stride(0) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def flash_forward(q, k, v, *, mode: int, q_positions=None, k_positions=None, q_sequence_ids=None, k_sequence_ids=None, scale=None):
    """tcgen05 flash-attention forward (``csrc/flash_attn.cu``): ``(out [B,Sq,hq,D] bf16, lse [B,hq,Sq] fp32)``.

    ``mode`` 0: all keys visible; 1: causal with offset ``Sk - Sq``; 2: general rule on positions / sequence ids.
    """
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    q, k, v = _as_bshd(q), _as_bshd(k), _as_bshd(v)
    if k.stride() != v.stride():
        v = v.contiguous()
        k = k.contiguous()
    out = torch.empty((B, Sq, Hq, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    to_i32 = lambda t: None if t is None else t.to(torch.int32).contiguous()   # noqa: E731
    qp, kp, qs, ks = (to_i32(t) for t in (q_positions, k_positions, q_sequence_ids, k_sequence_ids))
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    rc = _lib.lib().mb_flash_attn_fwd(
        _lib.ptr(q), _lib.c_ll(q.stride(1)), _lib.c_ll(q.stride(0)), _lib.ptr(k), _lib.ptr(v), _lib.c_ll(k.stride(1)), _lib.c_ll(k.stride(0)),
        _lib.ptr(out), _lib.c_ll(out.stride(1)), _lib.ptr(lse), _lib.ptr(qp), _lib.ptr(kp), _lib.ptr(qs), _lib.ptr(ks),
        _lib.c_int(B), _lib.c_int(Sq), _lib.c_int(Sk), _lib.c_int(Hq), _lib.c_int(Hkv), _lib.c_int(D), _lib.c_int(mode),
        ctypes.c_float(scale), _lib.stream_ptr())
    _lib.check(rc, "mb_flash_attn_fwd")
    return out, lse


def flash_block_forward(q, k, v, q_positions, k_positions, q_sequence_ids, k_sequence_ids, scale):
    """Kernel block forward returning ``(out, lse)`` for the general visibility rule; None when the kernel does not cover
    the case (then the caller uses the fp32 block primitive)."""
    if os.environ.get("MALTOS_B200_FLASH_BLOCKS", "1") == "0":
        return None
    if q.dtype != torch.bfloat16 or q.shape[-1] not in (64, 128) or q.shape[2] % k.shape[2]:
        return None
    if (q_sequence_ids is None) != (k_sequence_ids is None):
        return None
    return flash_forward(q, k, v, mode=2, q_positions=q_positions, k_positions=k_positions, q_sequence_ids=q_sequence_ids,
                         k_sequence_ids=k_sequence_ids, scale=scale)


def flash_block_backward(q, k, v, out, lse, dout, q_positions, k_positions, q_sequence_ids, k_sequence_ids, scale):
    """No tcgen05 backward kernel yet: the caller falls back to the fp32 block primitive."""
    return None

"""Attention on CUDA bf16: this library's tcgen05 flash-attention kernels, forward AND backward.

* ``flash_forward`` / ``flash_backward``: the kernels of ``csrc/flash_attn.cu`` and ``csrc/flash_attn_bwd.cu``: full,
  causal, general position / sequence-id masks and packed documents inside a row, native GQA, head_dim 64 / 128; the
  forward returns the log-sum-exp, the backward takes it (flash formulation: nothing of size ``S x S`` is kept).
* ``flash_attention``: the differentiable entry point used by the models and by the context-parallel cores; it is an
  autograd function over the two kernels. ``flash_block_forward`` / ``flash_block_backward`` are the block primitives of
  ring and HDP attention (the backward of a block takes the GLOBAL output and log-sum-exp of its query rows).
* ``MALTOS_B200_ATTENTION=cudnn`` routes dense causal attention through cuDNN's fused attention (a LIBRARY path kept
  for A/B timing only); the default is this library's kernels everywhere.

The reference takes this op from torch SDPA or the flash-attn 2 package (utils/attention_backend.py:42-135,
runtime/layers/flash_utils.py:180-260).
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from . import _lib

MODE_FULL, MODE_CAUSAL, MODE_GENERAL, MODE_PACKED_CAUSAL = 0, 1, 2, 3


class _FlashAttention(torch.autograd.Function):
    """Differentiable attention over the tcgen05 forward and backward kernels."""

    @staticmethod
    def forward(ctx, q, k, v, mode, q_pos, k_pos, q_seq, k_seq, scale):
        # Under activation checkpointing the original forward keeps (out, lse) for the recompute: the backward needs
        # exactly these two and nothing else of the forward, so the recompute pass launches no attention kernel.
        from maltos_b200.utils.activation_checkpoint import current_checkpoint_stash

        stash = current_checkpoint_stash()
        kept = stash.replay() if stash is not None and stash.replaying else None
        if kept is not None and kept[0].shape == q.shape:
            out, lse = kept
        else:
            out, lse = flash_forward(q, k, v, mode=mode, q_positions=q_pos, k_positions=k_pos, q_sequence_ids=q_seq,
                                     k_sequence_ids=k_seq, scale=scale)
            if stash is not None and not stash.replaying:
                stash.record((out, lse))
        ctx.save_for_backward(q, k, v, out, lse, *(t for t in (q_pos, k_pos, q_seq, k_seq) if t is not None))
        ctx.has = tuple(t is not None for t in (q_pos, k_pos, q_seq, k_seq))
        ctx.mode, ctx.scale = mode, scale
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, out, lse, *rest = ctx.saved_tensors
        it = iter(rest)
        q_pos, k_pos, q_seq, k_seq = (next(it) if h else None for h in ctx.has)
        dq, dk, dv = flash_backward(q, k, v, out, lse, dout, mode=ctx.mode, q_positions=q_pos, k_positions=k_pos,
                                    q_sequence_ids=q_seq, k_sequence_ids=k_seq, scale=ctx.scale)
        return dq, dk, dv, None, None, None, None, None, None


def flash_attention(q, k, v, *, q_positions=None, k_positions=None, q_sequence_ids=None, k_sequence_ids=None,
                    causal=True, scale=None, return_lse=False, packed_causal=False):
    """Differentiable attention ``[B,S,h,D]`` on the tcgen05 kernels. ``packed_causal``: the rows hold packed documents
    in order, so visibility is "causal by row index and same sequence id" (key blocks above the diagonal are skipped)."""
    dense = q_positions is None and q_sequence_ids is None
    if dense and causal and not return_lse and os.environ.get("MALTOS_B200_ATTENTION") == "cudnn":
        out = _sdpa_cudnn(q, k, v, causal, scale)
        if out is not None:
            return out
    if dense:
        mode = MODE_CAUSAL if causal else MODE_FULL
    elif packed_causal and q_sequence_ids is not None:
        mode, q_positions, k_positions = MODE_PACKED_CAUSAL, None, None
    else:
        mode = MODE_GENERAL
        if q_positions is None:      # sequence ids only: order inside the row decides causality
            Sq, Sk = q.shape[1], k.shape[1]
            q_positions = torch.arange(Sk - Sq, Sk, device=q.device, dtype=torch.int32).unsqueeze(0).expand(q.shape[0], Sq)
            k_positions = torch.arange(Sk, device=q.device, dtype=torch.int32).unsqueeze(0).expand(q.shape[0], Sk)
    to_i32 = lambda t: None if t is None else t.to(torch.int32).contiguous()   # noqa: E731
    out, lse = _FlashAttention.apply(q, k, v, mode, to_i32(q_positions), to_i32(k_positions), to_i32(q_sequence_ids),
                                     to_i32(k_sequence_ids), scale)
    return (out, lse) if return_lse else out


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
    if q_positions is None:                                     # every key visible: the unmasked kernel
        return flash_forward(q, k, v, mode=MODE_FULL, scale=scale)
    return flash_forward(q, k, v, mode=MODE_GENERAL, q_positions=q_positions, k_positions=k_positions, q_sequence_ids=q_sequence_ids,
                         k_sequence_ids=k_sequence_ids, scale=scale)


def flash_backward(q, k, v, out, lse, dout, *, mode: int, q_positions=None, k_positions=None, q_sequence_ids=None,
                   k_sequence_ids=None, scale=None, fp32_out: bool = False, accumulate_into=None):
    """tcgen05 flash-attention backward (``csrc/flash_attn_bwd.cu``): ``(dq [B,Sq,hq,D], dk, dv [B,Sk,hkv,D])`` in bf16, or
    in fp32 with ``fp32_out``; ``accumulate_into=(dq, dk, dv)`` (fp32, contiguous) adds the gradients to those tensors.
    ``out`` / ``lse`` are the forward's results for the query rows (for a block of ring attention: the merged ones)."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    q, k, v, out, dout = _as_bshd(q), _as_bshd(k), _as_bshd(v), _as_bshd(out), _as_bshd(dout)
    if dout.dtype != torch.bfloat16:
        dout = dout.to(torch.bfloat16)
    if out.dtype != torch.bfloat16:
        out = out.to(torch.bfloat16)
    if k.stride() != v.stride():
        v = v.contiguous()
        k = k.contiguous()
    lse = lse.float().contiguous()
    if accumulate_into is not None:
        dq, dk, dv = accumulate_into
        fp32_out = True
        for t in (dq, dk, dv):
            assert t.dtype == torch.float32 and t.is_contiguous()
    else:
        dt = torch.float32 if fp32_out else torch.bfloat16
        dq = torch.empty((B, Sq, Hq, D), dtype=dt, device=q.device)
        dk = torch.empty((B, Sk, Hkv, D), dtype=dt, device=q.device)
        dv = torch.empty((B, Sk, Hkv, D), dtype=dt, device=q.device)
    L = _lib.lib()
    L.mb_flash_attn_bwd_scratch_words.restype = ctypes.c_longlong
    words = int(L.mb_flash_attn_bwd_scratch_words(_lib.c_int(B), _lib.c_int(Sq), _lib.c_int(Sk), _lib.c_int(Hq), _lib.c_int(Hkv), _lib.c_int(D)))
    scratch = torch.empty((words,), dtype=torch.float32, device=q.device)
    to_i32 = lambda t: None if t is None else t.to(torch.int32).contiguous()   # noqa: E731
    qp, kp, qs, ks = (to_i32(t) for t in (q_positions, k_positions, q_sequence_ids, k_sequence_ids))
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    rc = L.mb_flash_attn_bwd(
        _lib.ptr(q), _lib.c_ll(q.stride(1)), _lib.c_ll(q.stride(0)), _lib.ptr(k), _lib.ptr(v), _lib.c_ll(k.stride(1)),
        _lib.c_ll(k.stride(0)), _lib.ptr(out), _lib.c_ll(out.stride(1)), _lib.c_ll(out.stride(0)), _lib.ptr(dout),
        _lib.c_ll(dout.stride(1)), _lib.c_ll(dout.stride(0)), _lib.ptr(lse), _lib.ptr(dq), _lib.c_ll(dq.stride(1)), _lib.ptr(dk),
        _lib.ptr(dv), _lib.c_ll(dk.stride(1)), _lib.ptr(qp), _lib.ptr(kp), _lib.ptr(qs), _lib.ptr(ks), _lib.ptr(scratch),
        _lib.c_int(B), _lib.c_int(Sq), _lib.c_int(Sk), _lib.c_int(Hq), _lib.c_int(Hkv), _lib.c_int(D), _lib.c_int(mode),
        ctypes.c_float(scale), _lib.c_int(1 if fp32_out else 0), _lib.c_int(1 if accumulate_into is not None else 0),
        _lib.stream_ptr())
    _lib.check(rc, "mb_flash_attn_bwd")
    return dq, dk, dv


def flash_block_backward(q, k, v, out, lse, dout, q_positions, k_positions, q_sequence_ids, k_sequence_ids, scale):
    """Kernel block backward for the general visibility rule: fp32 ``(dq, dk, dv)``; None when the kernel does not cover
    the case (then the caller uses the fp32 block primitive)."""
    if os.environ.get("MALTOS_B200_FLASH_BLOCKS", "1") == "0":
        return None
    if q.dtype != torch.bfloat16 or q.shape[-1] not in (64, 128) or q.shape[2] % k.shape[2]:
        return None
    if (q_sequence_ids is None) != (k_sequence_ids is None):
        return None
    if q_positions is None:
        return flash_backward(q, k, v, out, lse, dout, mode=MODE_FULL, scale=scale, fp32_out=True)
    return flash_backward(q, k, v, out, lse, dout, mode=MODE_GENERAL, q_positions=q_positions, k_positions=k_positions,
                          q_sequence_ids=q_sequence_ids, k_sequence_ids=k_sequence_ids, scale=scale, fp32_out=True)

"""Rotary position embedding, both conventions of the reference: interleaved pairs ``(2i, 2i+1)``
(``models/llama.py:89-94``) and rotate-half pairs ``(i, i + D/2)`` (``models/olmo.py:91-96``).

``rope_qkv_split`` takes the packed output of a fused q/k/v projection ``[..., (hq + 2*hkv) * D]`` and returns
contiguous ``q [..., hq, D]``, ``k [..., hkv, D]`` (both rotated) and ``v [..., hkv, D]`` in one pass per tensor,
so the split copy and the rotation cost a single read and write. Its backward rotates ``dq``/``dk`` back and
writes all three gradients straight into one packed buffer for the projection's dgrad/wgrad GEMMs.
"""
from __future__ import annotations

import torch

from . import _lib


def build_rope_cache(max_pos: int, head_dim: int, theta: float, device=None) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos``/``sin`` tables of shape ``[max_pos, head_dim // 2]``."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32, device=device), inv)
    return ang.cos().contiguous(), ang.sin().contiguous()


def _positions(T_shape, position_ids, position_offset: int, device) -> torch.Tensor:
    B, S = T_shape
    if position_ids is not None:
        p = position_ids.to(device=device, dtype=torch.long)
        if p.dim() == 1:
            p = p.unsqueeze(0).expand(B, S)
        return p
    return (torch.arange(S, device=device, dtype=torch.long) + position_offset).unsqueeze(0).expand(B, S)


def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, interleaved: bool,
                   inverse: bool = False) -> torch.Tensor:
    """x: [B, S, h, D]; positions: [B, S]. fp32 math."""
    c = cos.to(x.device)[positions].unsqueeze(2)
    s = sin.to(x.device)[positions].unsqueeze(2)
    if inverse:
        s = -s
    xf = x.float()
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2)
    else:
        half = x.shape[-1] // 2
        a, b = xf[..., :half], xf[..., half:]
        out = torch.cat((a * c - b * s, a * s + b * c), dim=-1)
    return out.to(x.dtype)


def _launch(src, src_stride, dst, dst_stride, T, heads, D, pos, cos, sin, interleaved, backward, rotate) -> None:
    _lib.check(_lib.lib().mb_rope(_lib.ptr(src), _lib.c_ll(src_stride), _lib.ptr(dst), _lib.c_ll(dst_stride), _lib.c_ll(T),
                                  _lib.c_int(heads), _lib.c_int(D), _lib.ptr(pos), _lib.c_int(0), _lib.c_int(1),
                                  _lib.ptr(cos), _lib.ptr(sin), _lib.c_int(cos.shape[0]), _lib.c_int(int(interleaved)),
                                  _lib.c_int(int(backward)), _lib.c_int(int(rotate)), _lib.stream_ptr()), "mb_rope")


class _RopeQkvSplit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, positions, hq, hkv, D, interleaved, offsets):
        lead = qkv.shape[:-1]
        W = (hq + 2 * hkv) * D
        packed = qkv.reshape(-1, W)
        if packed.stride(1) != 1:
            packed = packed.contiguous()
        T = packed.shape[0]
        pos = positions.reshape(-1).contiguous()
        q = torch.empty((T, hq, D), device=qkv.device, dtype=qkv.dtype)
        k = torch.empty((T, hkv, D), device=qkv.device, dtype=qkv.dtype)
        v = torch.empty((T, hkv, D), device=qkv.device, dtype=qkv.dtype)
        st = packed.stride(0)
        qo, ko, vo = offsets
        _launch(packed[:, qo:], st, q, hq * D, T, hq, D, pos, cos, sin, interleaved, False, True)
        _launch(packed[:, ko:], st, k, hkv * D, T, hkv, D, pos, cos, sin, interleaved, False, True)
        _launch(packed[:, vo:], st, v, hkv * D, T, hkv, D, pos, cos, sin, interleaved, False, False)
        ctx.save_for_backward(cos, sin, pos)
        ctx.meta = (lead, hq, hkv, D, interleaved, W, offsets)
        return q.view(*lead, hq, D), k.view(*lead, hkv, D), v.view(*lead, hkv, D)

    @staticmethod
    def backward(ctx, dq, dk, dv):
        cos, sin, pos = ctx.saved_tensors
        lead, hq, hkv, D, interleaved, W, (qo, ko, vo) = ctx.meta
        T = pos.numel()
        out = torch.empty((T, W), device=dq.device, dtype=dq.dtype)
        dq2 = dq.reshape(T, hq * D).contiguous()
        dk2 = dk.reshape(T, hkv * D).contiguous()
        dv2 = dv.reshape(T, hkv * D).contiguous()
        _launch(dq2, hq * D, out[:, qo:], W, T, hq, D, pos, cos, sin, interleaved, True, True)
        _launch(dk2, hkv * D, out[:, ko:], W, T, hkv, D, pos, cos, sin, interleaved, True, True)
        _launch(dv2, hkv * D, out[:, vo:], W, T, hkv, D, pos, cos, sin, interleaved, False, False)
        return out.view(*lead, W), None, None, None, None, None, None, None, None


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, positions, interleaved):
        shape = x.shape  # [B, S, h, D]
        h, D = shape[-2], shape[-1]
        x2 = x.reshape(-1, h * D).contiguous()
        T = x2.shape[0]
        pos = positions.reshape(-1).contiguous()
        out = torch.empty_like(x2)
        _launch(x2, h * D, out, h * D, T, h, D, pos, cos, sin, interleaved, False, True)
        ctx.save_for_backward(cos, sin, pos)
        ctx.meta = (shape, interleaved)
        return out.view(shape)

    @staticmethod
    def backward(ctx, dy):
        cos, sin, pos = ctx.saved_tensors
        shape, interleaved = ctx.meta
        h, D = shape[-2], shape[-1]
        d2 = dy.reshape(-1, h * D).contiguous()
        out = torch.empty_like(d2)
        _launch(d2, h * D, out, h * D, d2.shape[0], h, D, pos, cos, sin, interleaved, True, True)
        return out.view(shape), None, None, None, None


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, position_ids=None, position_offset: int = 0,
               interleaved: bool = True) -> torch.Tensor:
    """Rotate ``x [B, S, heads, D]`` by the angles of its positions."""
    positions = _positions(x.shape[:2], position_ids, position_offset, x.device)
    if _lib.use_kernels(x) and x.dtype == torch.bfloat16:
        return _Rope.apply(x, cos, sin, positions, interleaved)
    return rope_reference(x, cos, sin, positions, interleaved)


def rope_qkv_split(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, num_heads: int, num_kv_heads: int,
                   head_dim: int, position_ids=None, position_offset: int = 0, interleaved: bool = True,
                   offsets: tuple[int, int, int] | None = None, rotate: bool = True):
    """Packed ``[B, S, (hq+2hkv)*D]`` -> rotated ``q [B,S,hq,D]``, rotated ``k [B,S,hkv,D]``, ``v [B,S,hkv,D]``."""
    B, S = qkv.shape[:2]
    nq, nk = num_heads * head_dim, num_kv_heads * head_dim
    if offsets is None:
        offsets = (0, nq, nq + nk)
    positions = _positions((B, S), position_ids, position_offset, qkv.device)
    if rotate and _lib.use_kernels(qkv) and qkv.dtype == torch.bfloat16:
        return _RopeQkvSplit.apply(qkv, cos, sin, positions, num_heads, num_kv_heads, head_dim, interleaved, tuple(offsets))
    qo, ko, vo = offsets
    q = qkv[..., qo:qo + nq].reshape(B, S, num_heads, head_dim)
    k = qkv[..., ko:ko + nk].reshape(B, S, num_kv_heads, head_dim)
    v = qkv[..., vo:vo + nk].reshape(B, S, num_kv_heads, head_dim)
    if rotate:
        q = rope_reference(q, cos, sin, positions, interleaved)
        k = rope_reference(k, cos, sin, positions, interleaved)
    return q, k, v

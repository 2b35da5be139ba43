"""SwiGLU gate: ``silu(gate) * up`` (reference ``models/llama.py:205-206`` as eager ops), one fused kernel each way.
``swiglu_packed`` takes the output of a fused gate/up projection ``[..., 2F]`` (gate first) and its backward writes
``[dgate | dup]`` into one packed buffer for the projection's backward GEMMs."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib


class _SwigluPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        two_f = gu.shape[-1]
        f = two_f // 2
        g2 = gu.reshape(-1, two_f)
        if g2.stride(1) != 1:
            g2 = g2.contiguous()
        T = g2.shape[0]
        out = torch.empty((T, f), device=gu.device, dtype=gu.dtype)
        _lib.check(_lib.lib().mb_swiglu_fwd(_lib.ptr(g2), _lib.ptr(g2[:, f:]), _lib.c_ll(g2.stride(0)), _lib.ptr(out), _lib.c_ll(f),
                                            _lib.c_ll(T), _lib.c_int(f), _lib.stream_ptr()), "mb_swiglu_fwd")
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], f)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        two_f = g2.shape[-1]
        f = two_f // 2
        T = g2.shape[0]
        d2 = dout.reshape(T, f).contiguous()
        dgu = torch.empty((T, two_f), device=dout.device, dtype=dout.dtype)
        _lib.check(_lib.lib().mb_swiglu_bwd(_lib.ptr(d2), _lib.c_ll(f), _lib.ptr(g2), _lib.ptr(g2[:, f:]), _lib.c_ll(g2.stride(0)),
                                            _lib.ptr(dgu), _lib.ptr(dgu[:, f:]), _lib.c_ll(two_f), _lib.c_ll(T), _lib.c_int(f),
                                            _lib.stream_ptr()), "mb_swiglu_bwd")
        return dgu.view(ctx.shape)


class _Swiglu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        f = gate.shape[-1]
        g2 = gate.reshape(-1, f).contiguous()
        u2 = up.reshape(-1, f).contiguous()
        T = g2.shape[0]
        out = torch.empty_like(g2)
        # gate and up are separate allocations: pass `up` through its own pointer with the same row stride
        _lib.check(_lib.lib().mb_swiglu_fwd(_lib.ptr(g2), _lib.ptr(u2), _lib.c_ll(f), _lib.ptr(out), _lib.c_ll(f), _lib.c_ll(T),
                                            _lib.c_int(f), _lib.stream_ptr()), "mb_swiglu_fwd")
        ctx.save_for_backward(g2, u2)
        ctx.shape = gate.shape
        return out.view(gate.shape)

    @staticmethod
    def backward(ctx, dout):
        g2, u2 = ctx.saved_tensors
        T, f = g2.shape
        d2 = dout.reshape(T, f).contiguous()
        dg = torch.empty_like(g2)
        du = torch.empty_like(u2)
        _lib.check(_lib.lib().mb_swiglu_bwd(_lib.ptr(d2), _lib.c_ll(f), _lib.ptr(g2), _lib.ptr(u2), _lib.c_ll(f), _lib.ptr(dg),
                                            _lib.ptr(du), _lib.c_ll(f), _lib.c_ll(T), _lib.c_int(f), _lib.stream_ptr()), "mb_swiglu_bwd")
        return dg.view(ctx.shape), du.view(ctx.shape)


def _ok(t: torch.Tensor, f: int) -> bool:
    return _lib.use_kernels(t) and t.dtype == torch.bfloat16 and f % 8 == 0


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if _ok(gate, gate.shape[-1]) and up.dtype == torch.bfloat16:
        return _Swiglu.apply(gate, up)
    return F.silu(gate) * up


def swiglu_packed(gate_up: torch.Tensor) -> torch.Tensor:
    f = gate_up.shape[-1] // 2
    if _ok(gate_up, f):
        return _SwigluPacked.apply(gate_up)
    return F.silu(gate_up[..., :f]) * gate_up[..., f:]

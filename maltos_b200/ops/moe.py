"""Mixture-of-experts token processing on one device.

``moe_experts_forward`` sends every (token, choice) assignment through its expert and sums the gated results:
assignments are sorted by expert once (stable, so capacity order is token order) and each expert runs on a
contiguous slice. The expert count per slice is read on the host (one sync per call) - the expert-parallel layer
uses capacity-bounded buffers instead when a capacity factor is set.
"""
from __future__ import annotations

import torch


def swiglu_expert_weights(experts, like: torch.Tensor):
    """``(gates, ups, downs)`` weight lists when every expert is a bias-free SwiGLU MLP (``gate``/``up``/``down`` linear
    layers) whose bf16 weights are materialised on ``like``'s CUDA device - the case the grouped expert GEMM covers -
    else None."""
    from . import _lib

    if not (_lib.use_kernels(like) and like.dtype == torch.bfloat16 and len(experts) <= 16):
        return None
    gates, ups, downs = [], [], []
    for e in experts:
        parts = [getattr(e, n, None) for n in ("gate", "up", "down")]
        if any(p is None or getattr(p, "bias", None) is not None or not hasattr(p, "weight") for p in parts):
            return None
        ws = [p.weight for p in parts]
        if any(w.dtype != torch.bfloat16 or w.numel() == 0 or w.dim() != 2 or not w.is_cuda or w.shape[1] % 8 for w in ws):
            return None
        gates.append(ws[0]), ups.append(ws[1]), downs.append(ws[2])
    return gates, ups, downs


def _moe_experts_forward_static(flat, expert_idx, gate, keep, weights, capacity: int) -> torch.Tensor:
    """Single-device capacity-limited experts with static shapes: kept assignments are copied into fixed expert slots,
    the experts run as grouped GEMMs with device-side counts, dropped assignments read a row of zeros."""
    N, H = flat.shape
    k = expert_idx.shape[1]
    gates, ups, downs = weights
    E = len(gates)
    slot = (capacity + 127) // 128 * 128
    a_expert = torch.where(keep.reshape(-1), expert_idx.reshape(-1), torch.full_like(expert_idx.reshape(-1), E))
    token_of = torch.arange(N, device=flat.device).repeat_interleave(k)
    order = torch.argsort(a_expert, stable=True)
    sorted_e = a_expert[order]
    counts = torch.bincount(a_expert, minlength=E + 1)
    start = counts.cumsum(0) - counts
    pos = torch.arange(sorted_e.numel(), device=flat.device) - start[sorted_e]
    trash = E * slot                                                # one extra block of rows that nothing reads
    row = torch.where(sorted_e < E, sorted_e * slot + pos, torch.full_like(pos, trash))
    tokens_sorted = token_of[order]
    buf = torch.zeros((E * slot + 64, H), dtype=flat.dtype, device=flat.device).index_copy(0, row, flat.index_select(0, tokens_sorted))
    y = grouped_swiglu_experts(buf[:E * slot], counts[:E].to(torch.int32), slot, gates, ups, downs)
    y = torch.cat([y, y.new_zeros((64, H))], dim=0)
    gated = y.index_select(0, row) * gate.reshape(-1)[order].unsqueeze(1).to(flat.dtype)
    return torch.zeros_like(flat).index_add(0, tokens_sorted, gated)


def _has_module_hooks(expert) -> bool:
    mods = expert.modules() if isinstance(expert, torch.nn.Module) else ()
    return any(m._forward_pre_hooks or m._forward_hooks or m._backward_hooks or m._backward_pre_hooks for m in mods)


def moe_experts_forward(flat: torch.Tensor, expert_idx: torch.Tensor, gate: torch.Tensor, keep: torch.Tensor | None,
                        experts: list, capacity: int | None = None) -> torch.Tensor:
    """``flat [N,H]``, ``expert_idx/gate [N,k]``, ``keep [N,k]`` bool or None, ``experts``: callables ``[n,H]->[n,H]``.
    With a capacity limit on CUDA the grouped, host-sync-free path runs (``capacity`` = rows an expert may take)."""
    if keep is not None and capacity is not None:
        weights = swiglu_expert_weights(experts, flat)
        if weights is not None:
            return _moe_experts_forward_static(flat, expert_idx, gate, keep, weights, capacity)
    N, H = flat.shape
    k = expert_idx.shape[1]
    E = len(experts)
    assign_expert = expert_idx.reshape(-1)
    assign_gate = gate.reshape(-1)
    if keep is not None:
        assign_gate = assign_gate * keep.reshape(-1).to(assign_gate.dtype)
        assign_expert = torch.where(keep.reshape(-1), assign_expert, torch.full_like(assign_expert, E))
    token_of = torch.arange(N, device=flat.device).repeat_interleave(k)
    order = torch.argsort(assign_expert, stable=True)
    sorted_tokens = token_of[order]
    counts = torch.bincount(assign_expert, minlength=E + 1)[:E].tolist()
    gathered = flat.index_select(0, sorted_tokens)
    gates_sorted = assign_gate[order].unsqueeze(1).to(flat.dtype)
    out = torch.zeros_like(flat)
    at = 0
    pieces = []
    for e, n in enumerate(counts):
        # an expert with module hooks is entered also with zero rows: under sharded parameters (ZeRO-3) each call gathers
        # the expert's weights collectively, so all ranks must make the same sequence of calls
        if n == 0 and not _has_module_hooks(experts[e]):
            continue
        pieces.append(experts[e](gathered[at:at + n]) * gates_sorted[at:at + n])
        at += n
    if pieces:
        out = out.index_add(0, sorted_tokens[:at], torch.cat(pieces, dim=0))
    return out


# ------------------------------------------------------------------------------------------------ grouped expert GEMMs
def _ptr_array(tensors):
    import ctypes

    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def grouped_gemm(mode: int, a: torch.Tensor, bs, counts: torch.Tensor, cap: int, *, out_dtype=None):
    """All local experts' GEMMs in ONE launch with the per-expert row counts read on the device (``csrc/grouped_gemm.cu``).

    ``a [G*cap, .]`` holds expert ``g``'s rows at ``[g*cap, g*cap + counts[g])``; ``counts`` is an int32 device tensor.
      mode 0: ``bs[g]`` is ``[N, K]``, returns ``[G*cap, N]`` with ``out[rows of g] = a[rows of g] @ bs[g].T``;
      mode 1: ``bs[g]`` is ``[K, N]``, returns ``[G*cap, N]`` with ``out[rows of g] = a[rows of g] @ bs[g]``;
      mode 2: ``bs = [b]`` with ``b [G*cap, N]``, returns ``[G, M, N]`` with ``out[g] = a[rows of g].T @ b[rows of g]``.
    Rows beyond ``counts[g]`` of the outputs of modes 0/1 are left as they were allocated (zeros). For mode 2 the rows of
    ``a`` between ``counts[g]`` and the next multiple of 64 must be zero. CPU tensors take a plain loop (test oracle)."""
    from . import _lib

    G = counts.numel()
    out_dtype = out_dtype or a.dtype
    if mode == 2:
        M, N = a.shape[1], bs[0].shape[1]
    else:
        N = bs[0].shape[0] if mode == 0 else bs[0].shape[1]
    if not _lib.use_kernels(a):
        cnt = counts.tolist()
        if mode == 2:
            out = torch.zeros((G, M, N), dtype=out_dtype, device=a.device)
            for g, n in enumerate(cnt):
                out[g] = (a[g * cap:g * cap + n].float().t() @ bs[0][g * cap:g * cap + n].float()).to(out_dtype)
            return out
        out = torch.zeros((G * cap, N), dtype=out_dtype, device=a.device)
        for g, n in enumerate(cnt):
            w = bs[g].float()
            out[g * cap:g * cap + n] = (a[g * cap:g * cap + n].float() @ (w.t() if mode == 0 else w)).to(out_dtype)
        return out
    if a.dtype != torch.bfloat16 or any(b.dtype != torch.bfloat16 for b in bs):
        raise TypeError("grouped_gemm kernel takes bf16 operands")
    if cap % 64 or counts.dtype != torch.int32 or not counts.is_cuda:
        raise ValueError("grouped_gemm: cap must be a multiple of 64 and counts an int32 device tensor")
    a = a if (a.stride(1) == 1 and a.stride(0) % 8 == 0) else a.contiguous()
    bs = [b if (b.stride(1) == 1 and b.stride(0) % 8 == 0) else b.contiguous() for b in bs]
    if len({b.stride(0) for b in bs}) != 1:
        raise ValueError("grouped_gemm: all group operands must share one row stride")
    if mode == 2:
        out = torch.empty((G, M, N), dtype=out_dtype, device=a.device)
        c_list = [out[g] for g in range(G)]
        K = cap
    else:
        out = torch.zeros((G * cap, N), dtype=out_dtype, device=a.device)
        c_list = [out]
        M, K = cap, a.shape[1]
    rc = _lib.lib().mb_grouped_gemm_bf16(_lib.c_int(mode), _lib.ptr(a), _lib.c_ll(a.stride(0)), _ptr_array(bs), _lib.c_ll(bs[0].stride(0)),
                                         _ptr_array(c_list), _lib.c_ll(N), _lib.ptr(counts), _lib.c_int(G), _lib.c_int(cap),
                                         _lib.c_int(M), _lib.c_int(N), _lib.c_int(K), _lib.c_int(int(out_dtype == torch.float32)),
                                         _lib.stream_ptr())
    _lib.check(rc, "mb_grouped_gemm_bf16")
    return out


class _GroupedSwiGLUExperts(torch.autograd.Function):
    """``y[rows of g] = down_g(silu(gate_g(x)) * up_g(x))`` for all local experts with device-side row counts: seven grouped
    launches forward + backward per layer instead of nine GEMM calls per expert, and no host read of the counts."""

    @staticmethod
    def forward(ctx, x, counts, cap, n_experts, *weights):
        from .swiglu import swiglu

        gates, ups, downs = weights[:n_experts], weights[n_experts:2 * n_experts], weights[2 * n_experts:]
        with torch.no_grad():
            hg = grouped_gemm(0, x, list(gates), counts, cap)
            hu = grouped_gemm(0, x, list(ups), counts, cap)
            act = swiglu(hg, hu)
            y = grouped_gemm(0, act, list(downs), counts, cap)
        ctx.save_for_backward(x, counts, hg, hu, *weights)
        ctx.cap, ctx.n = cap, n_experts
        return y

    @staticmethod
    def backward(ctx, dy):
        from .swiglu import swiglu

        x, counts, hg, hu, *weights = ctx.saved_tensors
        n, cap = ctx.n, ctx.cap
        gates, ups, downs = weights[:n], weights[n:2 * n], weights[2 * n:]
        # rows beyond an expert's count may hold anything in the incoming gradient buffer: they must be zero for the
        # weight-gradient reductions, which run over whole 64-row blocks
        r = torch.arange(dy.shape[0], device=dy.device)
        valid = torch.remainder(r, cap) < counts.to(torch.long)[torch.div(r, cap, rounding_mode="floor")]
        dy = torch.where(valid.unsqueeze(1), dy, torch.zeros((), dtype=dy.dtype, device=dy.device)).contiguous()
        dact = grouped_gemm(1, dy, list(downs), counts, cap)                    # [rows, F]   (down_g is [H, F] = [K, N])
        with torch.enable_grad():
            g_, u_ = hg.detach().requires_grad_(True), hu.detach().requires_grad_(True)
            act = swiglu(g_, u_)
        dg, du = torch.autograd.grad(act, (g_, u_), dact)
        d_down = grouped_gemm(2, dy, [act.detach()], counts, cap)               # [G, H, F]
        dx = grouped_gemm(1, dg, list(gates), counts, cap)                      # gate_g is [F, H] = [K, N]
        dx = dx + grouped_gemm(1, du, list(ups), counts, cap)
        d_gate = grouped_gemm(2, dg, [x], counts, cap)                          # [G, F, H]
        d_up = grouped_gemm(2, du, [x], counts, cap)
        grads = [d_gate[g] for g in range(n)] + [d_up[g] for g in range(n)] + [d_down[g] for g in range(n)]
        return (dx, None, None, None, *grads)


def grouped_swiglu_experts(x: torch.Tensor, counts: torch.Tensor, cap: int, gates, ups, downs) -> torch.Tensor:
    """SwiGLU expert MLPs over a capacity-bounded, expert-major row buffer ``x [G*cap, H]`` (see :func:`grouped_gemm`).
    Rows beyond ``counts[g]`` must hold finite values (zeros); their outputs are zeros."""
    return _GroupedSwiGLUExperts.apply(x, counts, cap, len(gates), *gates, *ups, *downs)

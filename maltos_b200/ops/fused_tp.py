"""Tensor/sequence-parallel linear ops with the collective inside the GEMM kernel (``csrc/gemm.cu``).

``all_gather_grouped_linear``: the SP all-gather of ``x [B, S/T, H]`` and the q/k/v (gate/up) projection are ONE launch:
push warps in every block of the kernel store this rank's rows into every peer's gathered buffer over NVLink (plain P2P stores into
CUDA-IPC mapped memory, per-source flags), while the tcgen05 GEMM blocks start on the rows that are already local and
reach a peer's rows only after its flag arrived - the transfer hides behind the math tile by tile. Buffers are
double-buffered by call parity and a "consumed" flag keeps a fast rank from overwriting a buffer a slow rank still reads.

``linear_reduce_scatter`` / the input gradient of ``all_gather_grouped_linear``: GEMM and reduce-scatter are one GEMM
launch whose epilogue stores partial tiles into the owner rank's staging slots over NVLink, plus a small reduce kernel
(:func:`gemm_reduce_scatter`).

In groups above four ranks (two for the reduce-scatter) the in-kernel push does not pay: there the collectives are the
one-sided PULL kernels of ``csrc/tp_pull.cu`` (:func:`gemm_reduce_scatter_pull`, :func:`all_gather_pull`): the GEMM
writes its partial result into this rank's symmetric buffer and the owner of a sequence slice reads it from all ranks
with the whole grid's loads in flight; the all-gather publishes the local rows and pulls the peers' rows the same way.
NCCL is only the fallback for ranks without peer access (and ``MALTOS_B200_TP_PULL=0`` for A/B timing).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib
from .gemm import gemm
from .grouped import _fused_view, _memory_order

PUSH_CTAS = 4   # push warps per block


def _nccl_all_gather_rows(x2: torch.Tensor, ctx, B: int, rows: int) -> torch.Tensor:
    """[B*rows, K] local slices -> [B*rows*T, K] in batch-major, rank-minor order (one collective per batch element, each
    landing in place, so no permuting copy of the gathered tensor is needed)."""
    T = ctx.world
    K = x2.shape[1]
    x2 = x2.contiguous()
    out = torch.empty((B, T * rows, K), dtype=x2.dtype, device=x2.device)
    works = [dist.all_gather_into_tensor(out[b].view(T * rows, K), x2[b * rows:(b + 1) * rows], group=ctx.group, async_op=B > 1)
             for b in range(B)]
    for w in works:
        if w is not None:
            w.wait()
    return out.view(B * T * rows, K)


def _nccl_reduce_scatter_rows(y_full: torch.Tensor, ctx, B: int, rows: int) -> torch.Tensor:
    """[B*T*rows, K] (batch-major) -> sum over ranks of this rank's [B*rows, K] slice (one collective per batch element)."""
    T = ctx.world
    K = y_full.shape[1]
    y_full = y_full.contiguous()
    out = torch.empty((B * rows, K), dtype=y_full.dtype, device=y_full.device)
    works = [dist.reduce_scatter_tensor(out[b * rows:(b + 1) * rows], y_full[b * T * rows:(b + 1) * T * rows], op=dist.ReduceOp.SUM,
                                        group=ctx.group, async_op=B > 1) for b in range(B)]
    for w in works:
        if w is not None:
            w.wait()
    return out


def _pull_ok(symm) -> bool:
    return symm is not None and symm.world in (2, 4, 8) and os.environ.get("MALTOS_B200_TP_PULL", "1") != "0"


def _peer_table(ptrs, offset_bytes: int = 0):
    return (ctypes.c_ulonglong * 8)(*([p + offset_bytes for p in ptrs] + [0] * (8 - len(ptrs))))


def gemm_reduce_scatter_pull(x2: torch.Tensor, w: torch.Tensor, symm, B: int, rows: int, *, b_mn: bool) -> torch.Tensor:
    """``reduce_scatter_over_ranks(x2 @ op(w))`` along the sequence: the GEMM writes its bf16 partial ``[B*S, N]`` into this
    rank's symmetric buffer, then ONE kernel (``csrc/tp_pull.cu``) exchanges the "partial complete" flags and lets the
    owner of each sequence slice read it from every rank over NVLink and sum in fp32. Returns ``[B*rows, N]``."""
    T = symm.world
    N = w.shape[1] if b_mn else w.shape[0]
    M = B * rows * T
    stage = symm.ensure_buffer("sp_partial", 2 * M * N * 2)
    half = stage.nbytes // 2 // 256 * 256
    seq = symm.next_seq("pull_scatter")
    off = (seq & 1) * half
    partial = stage.local_tensor(torch.bfloat16, stage.nbytes // 2, x2.device)[off // 2: off // 2 + M * N].view(M, N)
    gemm(x2, w, b_mn=b_mn, out=partial)
    out = torch.empty((B * rows, N), dtype=torch.bfloat16, device=x2.device)
    rc = _lib.lib().mb_pull_reduce_scatter_bf16(_peer_table(stage.peer_ptrs, off), _peer_table(symm.pad.peer_ptrs), _lib.ptr(out),
                                                _lib.c_int(B), _lib.c_ll(rows), _lib.c_ll(N), _lib.c_int(symm.rank), _lib.c_int(T),
                                                ctypes.c_uint(seq & 0xFFFFFFFF), _lib.stream_ptr())
    _lib.check(rc, "mb_pull_reduce_scatter_bf16")
    return out


def all_gather_pull(x2: torch.Tensor, symm, B: int, rows: int) -> torch.Tensor:
    """``[B*rows, K]`` local rows -> ``[B*rows*T, K]`` (batch-major, rank-minor) with ONE kernel: publish the local rows in
    symmetric memory, exchange flags, pull the peers' rows over NVLink. The result is an ordinary tensor."""
    T = symm.world
    K = x2.shape[1]
    x2 = x2.contiguous()
    nbytes = B * rows * K * 2
    pub = symm.ensure_buffer("sp_publish", 2 * nbytes)
    half = pub.nbytes // 2 // 256 * 256
    seq = symm.next_seq("pull_gather")
    off = (seq & 1) * half
    out = torch.empty((B * rows * T, K), dtype=torch.bfloat16, device=x2.device)
    rc = _lib.lib().mb_pull_all_gather_bf16(_lib.ptr(x2), _peer_table(pub.peer_ptrs, off), _peer_table(symm.pad.peer_ptrs), _lib.ptr(out),
                                            _lib.c_int(B), _lib.c_ll(rows), _lib.c_ll(K), _lib.c_int(symm.rank), _lib.c_int(T),
                                            ctypes.c_uint(seq & 0xFFFFFFFF), _lib.stream_ptr())
    _lib.check(rc, "mb_pull_all_gather_bf16")
    return out


def gather_rows(x2: torch.Tensor, symm, B: int, rows: int) -> torch.Tensor:
    """Sequence all-gather of ``[B*rows, K]`` rows: the pull kernel over peer memory, NCCL only without it."""
    if _pull_ok(symm) and x2.dtype == torch.bfloat16 and x2.is_cuda and (rows * x2.shape[1]) % 8 == 0:
        return all_gather_pull(x2, symm, B, rows)
    return _nccl_all_gather_rows(x2, symm, B, rows)


def reduce_scatter_gemm(x2: torch.Tensor, w: torch.Tensor, symm, B: int, rows: int, *, b_mn: bool) -> torch.Tensor:
    """``reduce_scatter(x2 @ op(w))`` by the best path for the group: GEMM epilogue push (two ranks), GEMM + pull kernel
    (larger groups), GEMM + NCCL (no peer memory)."""
    n_out = w.shape[1] if b_mn else w.shape[0]
    if _fused_scatter_ok(symm, x2, n_out):
        return gemm_reduce_scatter(x2, w, symm, B, rows, b_mn=b_mn)
    if _pull_ok(symm) and x2.dtype == torch.bfloat16 and x2.is_cuda and (rows * n_out) % 8 == 0:
        return gemm_reduce_scatter_pull(x2, w, symm, B, rows, b_mn=b_mn)
    return _nccl_reduce_scatter_rows(gemm(x2, w, b_mn=b_mn), symm, B, rows)


def gemm_reduce_scatter(x2: torch.Tensor, w: torch.Tensor, symm, B: int, rows: int, *, b_mn: bool) -> torch.Tensor:
    """``reduce_scatter_over_ranks(x2 @ op(w))`` along the sequence in ONE GEMM launch plus a small reduce kernel.

    ``x2 [B*S, K_local]``; ``op(w) = w[N, K_local]^T`` (``b_mn=False``) or ``w[K_local, N]`` (``b_mn=True``). The GEMM epilogue
    stores each bf16 partial tile straight into the owner rank's staging slot over NVLink (tile by tile, behind the math
    of the following tiles); the owner sums the slots in fp32 once every writer's flag has arrived. Returns this rank's
    ``[B*rows, N]`` rows. Staging is double-buffered by call parity with a "reduced" flag as back-pressure.
    """
    T = symm.world
    K = x2.shape[1]
    N = w.shape[1] if b_mn else w.shape[0]
    if x2.stride(1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    if w.stride(1) != 1 or w.stride(0) % 8:
        w = w.contiguous()
    slot_elems = B * rows * N
    stage = symm.ensure_buffer("sp_scatter", 2 * T * slot_elems * 2)
    seq = symm.next_seq("scatter")
    out = torch.empty((B * rows, N), dtype=x2.dtype, device=x2.device)
    stage_ptrs = (ctypes.c_ulonglong * 8)(*(stage.peer_ptrs + [0] * (8 - T)))
    pads = (ctypes.c_ulonglong * 8)(*(symm.pad.peer_ptrs + [0] * (8 - T)))
    rc = _lib.lib().mb_gemm_rs_bf16(
        _lib.ptr(x2), _lib.c_ll(x2.stride(0)), _lib.ptr(w), _lib.c_int(1 if b_mn else 0), _lib.c_ll(w.stride(0)), _lib.ptr(out),
        _lib.c_int(B), _lib.c_int(rows), _lib.c_int(N), _lib.c_int(K), _lib.c_int(symm.rank), _lib.c_int(T),
        ctypes.c_uint(seq & 0xFFFFFFFF), stage_ptrs, pads, _lib.ptr(symm.pad.table), _lib.stream_ptr())
    _lib.check(rc, "mb_gemm_rs_bf16")
    return out


def set_push_mode(bulk: bool) -> None:
    """How the fused all-gather moves rows to the peers: ``bulk=True`` one thread per block issues 16 KB bulk async copies
    through a shared-memory staging buffer; ``False`` four copy warps per block use 16-byte loads / stores."""
    _lib.lib().mb_gemm_set_push_bulk(ctypes.c_int(1 if bulk else 0))


if os.environ.get("MALTOS_B200_PUSH_BULK", "1") == "1":   # measured faster than the copy warps (243 vs 258 us, qkv at TP=2)
    set_push_mode(True)

_SCATTER_KIND = int(os.environ.get("MALTOS_B200_SCATTER_KIND", "0"))
if _SCATTER_KIND:
    _lib.lib().mb_gemm_set_scatter_kind(ctypes.c_int(_SCATTER_KIND))


def _fused_scatter_ok(symm, x2: torch.Tensor, n_out: int) -> bool:
    # MALTOS_B200_FUSED_SCATTER: "1" always, "0" never, unset = only for groups of two. Measured on B200 at TP=2 the
    # epilogue push beats GEMM + NCCL reduce-scatter (o_proj 214 vs 247 us, down 469 vs 542 us, +2.3 % on the training
    # step); in larger groups GEMM + the owner-side pull kernel is the faster pair (TP=4: 165 vs 171 us, TP=8: 163 vs
    # 267 us for o_proj), which is what reduce_scatter_gemm picks there.
    mode = os.environ.get("MALTOS_B200_FUSED_SCATTER", "auto")
    if mode == "0" or (mode != "1" and symm.world > 2):
        return False
    return getattr(symm, "fused_scatter", True) and x2.dtype == torch.bfloat16 and x2.is_cuda and n_out % 8 == 0


def _fused_gather_ok(symm, M: int, N: int, K: int) -> bool:
    """Whether the all-gather should ride inside the GEMM launch. MALTOS_B200_FUSED_GATHER: "1" always, "0" never, unset =
    measured rule: in groups larger than four a GEMM of less than ~1.5e11 FLOP is shorter than the push of this rank's
    rows to seven peers, so the gather runs as a launch of its own in front of the GEMM (q/k/v at TP=8: pull kernel + GEMM
    231 us vs 257 us with the push inside; gate/up at TP=8 and every shape at TP=2 and TP=4 are faster fused)."""
    mode = os.environ.get("MALTOS_B200_FUSED_GATHER", "auto")
    if mode in ("0", "1"):
        return mode == "1"
    return symm.world <= 4 or 2.0 * M * N * K >= 1.5e11


def workspace_plan(world: int, workspace_bytes: int) -> dict[str, int]:
    """Symmetric transfer buffers the sequence-parallel ops of a group of ``world`` ranks will ask for, with their sizes,
    given ``workspace_bytes`` = two copies (call parities) of one micro-batch of hidden states, ``2 * tokens * hidden *
    itemsize``: every tensor that crosses the group in forward or backward has the hidden width. Follows the automatic path
    selection (``_fused_scatter_ok`` / ``_fused_gather_ok`` without environment overrides): gathered operand of the fused
    all-gather GEMM, published rows of the pull all-gather (one rank's share), and the reduce-scatter staging - per-source
    slots for two ranks, the rank's own partial for larger groups."""
    if world < 2:
        return {}
    plan = {"sp_gather": workspace_bytes, "sp_publish": -(-workspace_bytes // world)}
    plan["sp_scatter" if world <= 2 else "sp_partial"] = workspace_bytes
    return plan


def prewarm_workspace(symm, workspace_bytes: int) -> dict[str, int]:
    """Allocates the buffers of :func:`workspace_plan` now (collective over the group), so that neither the rendezvous nor a
    later growth falls into the first training step, where a sharded optimizer issues collectives on other groups at
    the same time. Returns the sizes actually held."""
    held = {}
    for name, nbytes in workspace_plan(symm.world, int(workspace_bytes)).items():
        held[name] = symm.ensure_buffer(name, nbytes).nbytes
    return held


def all_gather_gemm_unfused(x2: torch.Tensor, w: torch.Tensor, symm, B: int, rows: int, *, b_mn: bool):
    """Same contract as :func:`all_gather_gemm` with the all-gather as a launch of its own (pull kernel over peer memory,
    NCCL without it) in front of a plain GEMM launch; ``gathered`` is an ordinary tensor."""
    x_full = gather_rows(x2, symm, B, rows)
    return gemm(x_full, w, b_mn=b_mn), x_full


def all_gather_gemm(x2: torch.Tensor, w: torch.Tensor, symm, B: int, rows: int, *, b_mn: bool):
    """``(gather_over_ranks(x2) @ op(w), gathered)`` in one launch (see module docstring).

    ``x2 [B*rows, K]`` local rows; ``op(w) = w[N, K]^T`` (``b_mn=False``) or ``w[K, N]`` (``b_mn=True``). ``gathered`` is a view
    ``[B*rows*T, K]`` of this rank's symmetric buffer holding the gathered operand; it stays valid until the second next
    call of this function on the context (peers overwrite a slot only after they have seen this rank start the NEXT call,
    which in stream order is after every kernel launched before it), so a weight-gradient GEMM issued right after may read it.
    """
    T = symm.world
    K = x2.shape[1]
    N = w.shape[1] if b_mn else w.shape[0]
    if not _fused_gather_ok(symm, B * rows * T, N, K):
        return all_gather_gemm_unfused(x2, w, symm, B, rows, b_mn=b_mn)
    if x2.stride(1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    if w.stride(1) != 1 or w.stride(0) % 8:
        w = w.contiguous()
    M = B * rows * T
    buf_elems = M * K
    buf = symm.ensure_buffer("sp_gather", 2 * buf_elems * 2)
    buf_stride = buf.nbytes // 4      # elements per half: the two call parities never share memory, whatever the call sizes
    seq = symm.next_seq("gather")
    out = torch.empty((M, N), dtype=x2.dtype, device=x2.device)
    gathered = (ctypes.c_ulonglong * 8)(*(buf.peer_ptrs + [0] * (8 - T)))
    pads = (ctypes.c_ulonglong * 8)(*(symm.pad.peer_ptrs + [0] * (8 - T)))
    rc = _lib.lib().mb_ag_gemm_bf16(
        _lib.ptr(x2), _lib.c_ll(x2.stride(0)), _lib.c_int(B), _lib.c_int(rows), _lib.ptr(w), _lib.c_int(1 if b_mn else 0),
        _lib.c_ll(w.stride(0)), _lib.ptr(out), _lib.c_ll(out.stride(0)), _lib.c_int(N), _lib.c_int(K), _lib.c_int(symm.rank), _lib.c_int(T),
        ctypes.c_uint(seq & 0xFFFFFFFF), gathered, pads, _lib.c_ll(buf_stride), _lib.c_int(PUSH_CTAS), _lib.stream_ptr())
    _lib.check(rc, "mb_ag_gemm_bf16")
    full = buf.local_tensor(torch.bfloat16, 2 * buf_stride, x2.device)[(seq & 1) * buf_stride:(seq & 1) * buf_stride + buf_elems].view(M, K)
    return out, full


class _AllGatherGroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, symm, *weights):
        B, rows, K = x_local.shape
        T = symm.world
        order = _memory_order(weights)
        fused = _fused_view(weights, order) if order is not None else torch.cat([w for w in weights], dim=0)
        layout = order if order is not None else list(range(len(weights)))
        N = fused.shape[0]
        x2 = x_local.reshape(B * rows, K)
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        out, gathered = all_gather_gemm(x2, fused, symm, B, rows, b_mn=False)
        # The weight gradient needs the gathered input again. A device copy of it (taken while it is still in the
        # symmetric buffer; only when a gradient is wanted, i.e. in the recomputation pass under activation
        # checkpointing) replaces the all-gather the backward would otherwise launch.
        keep = any(ctx.needs_input_grad[2:]) and os.environ.get("MALTOS_B200_KEEP_GATHERED", "1") == "1"
        ctx.kept = keep
        if keep and _fused_gather_ok(symm, B * rows * T, N, K):
            gathered = gathered.clone()          # the symmetric buffer is recycled two calls later
        ctx.save_for_backward(x2, *weights, *([gathered] if keep else []))
        ctx.symm, ctx.layout, ctx.fused_ok = symm, layout, order is not None
        ctx.dims = (B, rows, K, N)
        return out.view(B, rows * T, N)

    @staticmethod
    def backward(ctx, dout):
        x2, *weights = ctx.saved_tensors
        x_kept = weights.pop() if ctx.kept else None
        B, rows, K, N = ctx.dims
        symm = ctx.symm
        d2 = dout.reshape(-1, N)
        if d2.stride(1) != 1 or d2.stride(0) % 8:
            d2 = d2.contiguous()
        # re-checked here: sharded parameters may have been re-materialised at other addresses since the forward
        still_adjacent = ctx.fused_ok and _memory_order(weights) == ctx.layout
        fused = _fused_view(weights, ctx.layout) if still_adjacent else torch.cat([weights[i] for i in ctx.layout], dim=0)
        dx_local = None
        dws = [None] * len(weights)
        if ctx.needs_input_grad[0]:
            dx_local = reduce_scatter_gemm(d2, fused, symm, B, rows, b_mn=True).view(B, rows, K)
        if any(ctx.needs_input_grad[2:]):
            x_full = x_kept if x_kept is not None else gather_rows(x2, symm, B, rows)
            dwf = gemm(d2, x_full, a_mn=True, b_mn=True)               # [N, K]
            at = 0
            for i in ctx.layout:
                n = weights[i].shape[0]
                dws[i] = dwf[at:at + n]
                at += n
        return (dx_local, None, *dws)


def all_gather_grouped_linear(x_local: torch.Tensor, weights, symm, *, seq_dim: int = 1):
    """``x_local [B, S/T, H]`` -> ``(packed [B, S, sum(out_i)], column offsets)``; see module docstring."""
    if seq_dim != 1 or x_local.dim() != 3:
        raise ValueError("all_gather_grouped_linear expects [batch, sequence/T, hidden] with the sequence on dim 1")
    weights = list(weights)
    order = _memory_order(weights)
    layout = order if order is not None else list(range(len(weights)))
    offs = [0] * len(weights)
    at = 0
    for i in layout:
        offs[i] = at
        at += weights[i].shape[0]
    return _AllGatherGroupedLinear.apply(x_local, symm, *weights), offs


class _LinearReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, symm):
        B, S, Kin = x.shape
        T = symm.world
        rows = S // T
        x2 = x.reshape(B * S, Kin)
        y = reduce_scatter_gemm(x2, weight, symm, B, rows, b_mn=False)
        ctx.save_for_backward(x2, weight)
        ctx.symm, ctx.dims = symm, (B, S, rows, Kin)
        return y.view(B, rows, weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        B, S, rows, Kin = ctx.dims
        H = weight.shape[0]
        dy2 = dy.reshape(B * rows, H)
        if (ctx.needs_input_grad[0] and dy2.dtype == torch.bfloat16 and dy2.is_cuda and Kin % 8 == 0
                and os.environ.get("MALTOS_B200_FUSED_DGRAD_GATHER", "1") == "1"):
            # dX = gather(dY) @ W in one launch; the gathered dY stays in the symmetric buffer for the weight gradient
            dx_full, dy_full = all_gather_gemm(dy2, weight, ctx.symm, B, rows, b_mn=True)
            dx = dx_full.view(B, S, Kin)
        else:
            dy_full = gather_rows(dy2, ctx.symm, B, rows)   # [B*S, H]
            dx = gemm(dy_full, weight, b_mn=True).view(B, S, Kin) if ctx.needs_input_grad[0] else None
        dw = gemm(dy_full, x2, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        return dx, dw, None


def linear_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, symm, *, seq_dim: int = 1) -> torch.Tensor:
    """Row-parallel ``x [B, S, in/T] @ W^T`` followed by reduce-scatter along the sequence -> ``[B, S/T, out]``."""
    if seq_dim != 1 or x.dim() != 3:
        raise ValueError("linear_reduce_scatter expects [batch, sequence, in/T] with the sequence on dim 1")
    return _LinearReduceScatter.apply(x, weight, symm)

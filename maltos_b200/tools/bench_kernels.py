"""Micro-benchmarks of the library's sm_100a kernels (CUDA events, warm-up, L2 flushed between timed launches).

    python -m maltos_b200.tools.bench_kernels gemm --m 8192 --n 8192 --k 4096            # all kernel kinds + torch.matmul
    python -m maltos_b200.tools.bench_kernels gemm --m 16384 --n 4096 --k 14336 --kind 1024 --layout nt --iters 3
    python -m maltos_b200.tools.bench_kernels rmsnorm --rows 65536 --hidden 4096
    python -m maltos_b200.tools.bench_kernels swiglu --rows 65536 --hidden 14336
    python -m maltos_b200.tools.bench_kernels adamw --numel 500000000
    python -m maltos_b200.tools.bench_kernels attention --seq 8192 --heads 32 --kv-heads 8

Every line reports the achieved rate and, where ``--peaks MEASURED_PEAKS.json`` is given, the fraction of the measured
copy bandwidth / cuBLAS throughput of the machine. Small ``--iters`` runs are what profiler captures are taken from.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch


def _flush_l2(scratch: torch.Tensor) -> None:
    scratch.zero_()     # 256 MiB write: evicts the 126 MB L2


def _time(fn, iters: int, warmup: int = 3, flush: torch.Tensor | None = None) -> float:
    """Median device time of ``fn`` in milliseconds."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            _flush_l2(flush)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    return sorted(times)[len(times) // 2]


def _peaks(path: str | None) -> dict:
    if path and Path(path).is_file():
        return json.loads(Path(path).read_text())
    return {}


def bench_gemm(args) -> None:
    from maltos_b200.ops import _lib
    from maltos_b200.ops.gemm import gemm

    M, N, K = args.m, args.n, args.k
    a_mn, b_mn = {"nn": (False, False), "nt": (False, True), "tt": (True, True), "tn": (True, False)}[args.layout]
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g).bfloat16()
    out = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    peak = _peaks(args.peaks).get("bf16_tflops")
    kinds = [args.kind] if args.kind is not None else [256, 512, 1024, 0]
    names = {0: "auto", 128: "single-CTA 128x128", 256: "single-CTA 128x256", 512: "CTA pair 256x256", 1024: "CTA pair 256x512"}
    flops = 2.0 * M * N * K
    for kind in kinds:
        ms = _time(lambda: gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, block_n=kind), args.iters, flush=flush)
        tf = flops / ms / 1e9
        print(f"gemm {M}x{N}x{K} {args.layout} {names[kind]:>20}: {ms * 1e3:8.1f} us  {tf:7.1f} TFLOP/s" +
              (f"  {tf / peak:.2f} of measured cuBLAS" if peak else ""))
    if args.kind is None:
        af = a.t() if a_mn else a
        bf = b if b_mn else b.t()
        ms = _time(lambda: torch.matmul(af, bf, out=out), args.iters, flush=flush)
        print(f"gemm {M}x{N}x{K} {args.layout} {'torch.matmul (cuBLAS)':>20}: {ms * 1e3:8.1f} us  {flops / ms / 1e9:7.1f} TFLOP/s")
    _lib.fetch_status()


def _report_bw(name: str, nbytes: float, ms: float, peaks: dict) -> None:
    gbs = nbytes / ms / 1e6
    hbm = peaks.get("hbm_gbs")
    print(f"{name}: {ms * 1e3:8.1f} us  {gbs:8.1f} GB/s" + (f"  {gbs / hbm:.2f} of measured copy bandwidth" if hbm else ""))


def bench_rmsnorm(args) -> None:
    from maltos_b200.ops.norm import add_rms_norm, rms_norm

    rows, H = args.rows, args.hidden
    x = torch.randn(rows, H, device="cuda").bfloat16().requires_grad_()
    r = torch.randn(rows, H, device="cuda").bfloat16()
    w = torch.ones(H, device="cuda").bfloat16().requires_grad_()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    peaks = _peaks(args.peaks)
    with torch.no_grad():
        _report_bw(f"rmsnorm fwd [{rows},{H}]", 2 * rows * H * 2, _time(lambda: rms_norm(x, w, 1e-5), args.iters, flush=flush), peaks)
        _report_bw(f"add+rmsnorm fwd [{rows},{H}]", 4 * rows * H * 2, _time(lambda: add_rms_norm(x, r, w, 1e-5), args.iters, flush=flush), peaks)
    y = rms_norm(x, w, 1e-5)
    dy = torch.randn_like(y)

    def bwd():
        x.grad = w.grad = None
        y.backward(dy, retain_graph=True)

    _report_bw(f"rmsnorm bwd [{rows},{H}]", 3 * rows * H * 2, _time(bwd, args.iters, flush=flush), peaks)


def bench_swiglu(args) -> None:
    from maltos_b200.ops.swiglu import swiglu_packed

    rows, F = args.rows, args.hidden
    gu = torch.randn(rows, 2 * F, device="cuda").bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    with torch.no_grad():
        _report_bw(f"swiglu fwd [{rows},2x{F}]", 3 * rows * F * 2, _time(lambda: swiglu_packed(gu), args.iters, flush=flush), _peaks(args.peaks))


def bench_adamw(args) -> None:
    from maltos_b200.ops.optim import adamw_multi_tensor

    n = args.numel
    chunks = 16
    per = n // chunks
    master = [torch.randn(per, device="cuda") for _ in range(chunks)]
    model = [m.bfloat16() for m in master]
    grads = [torch.randn(per, device="cuda").bfloat16() for _ in range(chunks)]
    m1 = [torch.zeros_like(m) for m in master]
    m2 = [torch.zeros_like(m) for m in master]
    items = [(p_, g_, a_, b_, lp, 1) for p_, g_, a_, b_, lp in zip(master, grads, m1, m2, model)]

    def run():
        adamw_multi_tensor(items, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)

    ms = _time(run, args.iters)
    # per element: read fp32 master + m + v + bf16 grad, write fp32 master + m + v + bf16 weight
    _report_bw(f"adamw multi-tensor {per * chunks:,} params", per * chunks * (12 + 2 + 12 + 2), ms, _peaks(args.peaks))


def bench_shard_paths(args) -> None:
    """The sharded-optimizer kernels with the ranks' buffers emulated as tensors of THIS GPU: what the kernels cost in
    HBM traffic when NVLink is not the limit (the peers' buffers are ordinary device addresses to them)."""
    from maltos_b200.ops.zero_fused import adamw_push, peer_all_reduce, peer_gather, peer_reduce_shard

    world, n = args.world, args.numel // args.world * args.world
    shard = n // world
    peaks = _peaks(args.peaks)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    buckets = [torch.randn(shard, device="cuda").bfloat16() for _ in range(world)]      # this rank's slice in every rank's bucket
    out = torch.empty(shard, device="cuda", dtype=torch.bfloat16)
    sq = torch.zeros((), dtype=torch.float64, device="cuda")
    ptrs = [b.data_ptr() for b in buckets]
    ms = _time(lambda: peer_reduce_shard(ptrs, 0, shard, 1.0 / world, out, sumsq=sq), args.iters, flush=flush)
    _report_bw(f"peer_reduce_shard world={world} shard={shard:,} bf16", shard * 2 * (world + 1), ms, peaks)
    ms = _time(lambda: peer_all_reduce(ptrs, shard, torch.bfloat16, 1.0 / world), args.iters, flush=flush)
    _report_bw(f"peer_all_reduce world={world} slice={shard:,} bf16", shard * 2 * 2 * world, ms, peaks)
    master = torch.randn(shard, device="cuda")
    m1, m2 = torch.zeros_like(master), torch.zeros_like(master)
    ms = _time(lambda: adamw_push(master, out, m1, m2, ptrs, step=1.0, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1),
               args.iters, flush=flush)
    _report_bw(f"adamw_push world={world} shard={shard:,}", shard * (12 + 2 + 12 + 2 * world), ms, peaks)
    full = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: peer_gather(full, ptrs, shard * 2), args.iters, flush=flush)
    _report_bw(f"peer_gather world={world} total={n:,} bf16", n * 2 * 2, ms, peaks)


def bench_attention(args) -> None:
    from maltos_b200.ops import _lib
    from maltos_b200.ops.flash_attn import _sdpa_cudnn, flash_backward, flash_forward

    B, S, Hq, Hkv, D = args.batch, args.seq, args.heads, args.kv_heads, args.head_dim
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(B, S, Hq, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(B, S, Hkv, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda", generator=g).bfloat16()
    dout = torch.randn(B, S, Hq, D, device="cuda", generator=g).bfloat16()
    flops = 4.0 * B * S * S * D * Hq / (2 if args.causal else 1)
    mode = 1 if args.causal else 0
    rows, rows_bwd = [], []
    with torch.no_grad():
        rows.append(("tcgen05 flash forward (this library)", _time(lambda: flash_forward(q, k, v, mode=mode), args.iters)))
        out, lse = flash_forward(q, k, v, mode=mode)
        rows_bwd.append(("tcgen05 flash backward (this library)",
                         _time(lambda: flash_backward(q, k, v, out, lse, dout, mode=mode), args.iters)))
        if _sdpa_cudnn(q, k, v, args.causal, None) is not None:
            rows.append(("cuDNN fused attention (library)", _time(lambda: _sdpa_cudnn(q, k, v, args.causal, None), args.iters)))
    if args.libraries:
        ql, kl, vl = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = _sdpa_cudnn(ql, kl, vl, args.causal, None)
        if o is not None:
            rows_bwd.append(("cuDNN fused attention backward (library)",
                             _time(lambda: torch.autograd.grad(o, (ql, kl, vl), dout, retain_graph=True), args.iters)))
        try:
            from flash_attn import flash_attn_func

            with torch.no_grad():
                rows.append(("flash-attn 2 (library)", _time(lambda: flash_attn_func(q, k, v, causal=args.causal), args.iters)))
            o2 = flash_attn_func(ql, kl, vl, causal=args.causal)
            rows_bwd.append(("flash-attn 2 backward (library)",
                             _time(lambda: torch.autograd.grad(o2, (ql, kl, vl), dout, retain_graph=True), args.iters)))
        except ImportError:
            pass
    tag = f"B{B} S{S} h{Hq}/{Hkv} D{D} {'causal' if args.causal else 'full'}"
    for name, ms in rows:
        print(f"attention fwd {tag} {name:>42}: {ms * 1e3:8.1f} us  {flops / ms / 1e9:7.1f} TFLOP/s")
    for name, ms in rows_bwd:
        print(f"attention bwd {tag} {name:>42}: {ms * 1e3:8.1f} us  {2.5 * flops / ms / 1e9:7.1f} TFLOP/s")
    _lib.fetch_status()


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--peaks", default="MEASURED_PEAKS.json", help="JSON with hbm_gbs / bf16_tflops of this machine")
    p.add_argument("--iters", type=int, default=10)
    sub = p.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192)
    g.add_argument("--n", type=int, default=8192)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--layout", choices=("nn", "nt", "tt", "tn"), default="nn", help="nn: y = x w^T (both K-major); nt: dgrad; tt: wgrad")
    g.add_argument("--kind", type=int, choices=(0, 128, 256, 512, 1024), default=None)
    for name in ("rmsnorm", "swiglu"):
        s = sub.add_parser(name)
        s.add_argument("--rows", type=int, default=65536)
        s.add_argument("--hidden", type=int, default=4096)
    t = sub.add_parser("attention")
    t.add_argument("--batch", type=int, default=2)
    t.add_argument("--seq", type=int, default=8192)
    t.add_argument("--heads", type=int, default=32)
    t.add_argument("--kv-heads", type=int, default=8)
    t.add_argument("--head-dim", type=int, default=128)
    t.add_argument("--causal", action=argparse.BooleanOptionalAction, default=True)
    t.add_argument("--libraries", action=argparse.BooleanOptionalAction, default=True, help="also time the library kernels")
    a = sub.add_parser("adamw")
    a.add_argument("--numel", type=int, default=500_000_000)
    z = sub.add_parser("shard-paths")
    z.add_argument("--numel", type=int, default=400_000_000, help="elements of the whole bucket")
    z.add_argument("--world", type=int, default=8)
    args = p.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("bench_kernels needs a CUDA device")
    {"gemm": bench_gemm, "rmsnorm": bench_rmsnorm, "swiglu": bench_swiglu, "adamw": bench_adamw, "attention": bench_attention,
     "shard-paths": bench_shard_paths}[args.what](args)


if __name__ == "__main__":
    main()

"""Micro-benchmarks of the fused tensor-parallel kernels against their NCCL + GEMM baselines, one process per GPU:

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 -m maltos_b200.tools.bench_fused_tp [--seq 8192 --hidden 4096]

For the column-parallel projections of LLaMA-3 8B (q/k/v and gate/up) it times the all-gather pushed from inside the GEMM
launch, the pull all-gather kernel + GEMM, NCCL all-gather + GEMM, and the GEMM alone; for the row-parallel projections
(o_proj, down) the GEMM whose epilogue pushes the partial tiles, GEMM + pull reduce-scatter kernel, GEMM + NCCL
reduce-scatter and the GEMM alone. The first column of every row is the path the library takes by default. Device time (CUDA events), maximum over ranks, and the roofline target
``max(FLOPs / measured GEMM peak, bytes leaving this GPU / NVLink bandwidth)`` with the achieved fraction.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist


def _time(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) * 1e3    # us


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--qkv", type=int, default=6144)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--peaks", default="MEASURED_PEAKS.json")
    ap.add_argument("--nvlink-gbs", type=float, default=770.0, help="measured peer-copy bandwidth per direction")
    args = ap.parse_args(argv)

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    import maltos_b200  # noqa: F401
    from maltos_b200.ops import _lib, comm
    from maltos_b200.ops.fused_tp import (_nccl_all_gather_rows, _nccl_reduce_scatter_rows, all_gather_gemm, all_gather_pull,
                                          gemm_reduce_scatter, gemm_reduce_scatter_pull, reduce_scatter_gemm)
    from maltos_b200.ops.gemm import gemm

    group = dist.new_group(list(range(world)))
    ctx = comm.context_for(group)
    if ctx is None:
        raise SystemExit(f"no symmetric-memory context: {comm.disabled_reason(group)}")
    peak = 1590.0
    if Path(args.peaks).exists():
        peak = float(json.loads(Path(args.peaks).read_text()).get("bf16_tflops", peak))
    S, H = args.seq, args.hidden
    rows = S // world

    def report(name, flops, link_bytes, results):
        target = max(flops / peak / 1e6, link_bytes / args.nvlink_gbs / 1e3)     # us
        if rank == 0:
            parts = " | ".join(f"{k} {v:.0f} us" for k, v in results.items())
            best = results[next(iter(results))]
            print(f"{name} T={world}: {parts} | roofline target {target:.0f} us, default path achieves {target / best:.2f}", flush=True)

    with torch.no_grad():
        for name, n_full in (("qkv", args.qkv), ("gate_up", 2 * args.ffn)):
            n = n_full // world
            w = torch.nn.Parameter((torch.randn(n, H, device="cuda") * 0.02).bfloat16())
            x = torch.randn(1, rows, H, device="cuda").bfloat16()
            x2 = x.view(-1, H)
            default = _time(lambda: all_gather_gemm(x2, w, ctx, 1, rows, b_mn=False), args.iters)
            os.environ["MALTOS_B200_FUSED_GATHER"] = "1"
            fused = _time(lambda: all_gather_gemm(x2, w, ctx, 1, rows, b_mn=False), args.iters)
            _lib.lib().mb_gemm_set_push_split(1)
            split = _time(lambda: all_gather_gemm(x2, w, ctx, 1, rows, b_mn=False), args.iters)
            _lib.lib().mb_gemm_set_push_split(0)
            os.environ.pop("MALTOS_B200_FUSED_GATHER")
            pull = _time(lambda: gemm(all_gather_pull(x2, ctx, 1, rows), w), args.iters)
            pull_only = _time(lambda: all_gather_pull(x2, ctx, 1, rows), args.iters)
            nccl = _time(lambda: gemm(_nccl_all_gather_rows(x2, ctx, 1, rows), w), args.iters)
            nccl_only = _time(lambda: _nccl_all_gather_rows(x2, ctx, 1, rows), args.iters)
            xf = _nccl_all_gather_rows(x2, ctx, 1, rows)
            alone = _time(lambda: gemm(xf, w), args.iters)
            report(f"all-gather -> GEMM {name} N={n}", 2.0 * S * H * n, (world - 1) * rows * H * 2,
                   {"default": default, "push inside GEMM": fused, "push launch + GEMM": split, "pull kernel + GEMM": pull, "NCCL all-gather + GEMM": nccl,
                    "pull kernel alone": pull_only, "NCCL all-gather alone": nccl_only, "GEMM alone": alone})
        for name, k_full in (("o_proj", H), ("down", args.ffn)):
            k = k_full // world
            w = torch.nn.Parameter((torch.randn(H, k, device="cuda") * 0.02).bfloat16())
            x = torch.randn(S, k, device="cuda").bfloat16()
            default = _time(lambda: reduce_scatter_gemm(x, w, ctx, 1, rows, b_mn=False), args.iters)
            fused = _time(lambda: gemm_reduce_scatter(x, w, ctx, 1, rows, b_mn=False), args.iters)
            pull = _time(lambda: gemm_reduce_scatter_pull(x, w, ctx, 1, rows, b_mn=False), args.iters)
            nccl = _time(lambda: _nccl_reduce_scatter_rows(gemm(x, w), ctx, 1, rows), args.iters)
            alone = _time(lambda: gemm(x, w), args.iters)
            report(f"GEMM -> reduce-scatter {name} K={k}", 2.0 * S * H * k, (world - 1) * rows * H * 2,
                   {"default": default, "push from GEMM epilogue": fused, "GEMM + pull kernel": pull, "GEMM + NCCL reduce-scatter": nccl,
                    "GEMM alone": alone})
    status = _lib.fetch_status(raise_on_error=False)
    if status[0]:
        print(f"rank {rank}: kernel status {status}", flush=True)
    dist.barrier()
    comm.release_context(group)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

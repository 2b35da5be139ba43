"""Bandwidth of SM-issued copies between two GPUs over NVLink (``csrc/peer_copy.cu``), one process per GPU:

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 -m maltos_b200.tools.bench_peer_copy [--mib 256]

Rank 0 times a push (its memory -> the peer's symmetric buffer) and a pull (the peer's buffer -> its memory) with the
plain 16-byte load/store kernel at several grid sizes while rank 1 idles, then both ranks copy at the same time (every
link direction busy). CUDA events, median of ``--iters`` launches. These are the ceilings for the library's one-sided
transfers (fused all-gather pushes, ring K/V pulls, expert dispatch, shard gathers).
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def _time(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    return sorted(times)[len(times) // 2]


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--mib", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    import maltos_b200  # noqa: F401
    from maltos_b200.ops import comm
    from maltos_b200.ops.peer_ring import _copy

    group = dist.new_group(list(range(world)))
    ctx = comm.context_for(group)
    if ctx is None:
        raise SystemExit(f"no symmetric-memory context: {comm.disabled_reason(group)}")
    nbytes = args.mib << 20
    sb = ctx.ensure_buffer("bench_peer_copy", nbytes)
    local = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    peer = sb.peer_ptrs[(rank + 1) % world]
    results = {}
    for both in (False, True):
        for blocks in (0, 64, 32, 8):
            for name, dst, src in (("push", peer, local.data_ptr()), ("pull", local.data_ptr(), peer)):
                dist.barrier(group=group)
                torch.cuda.synchronize()
                if both or rank == 0:
                    ms = _time(lambda: _copy(dst, src, nbytes, blocks), args.iters)
                    results[(both, blocks, name)] = nbytes / ms / 1e6
                dist.barrier(group=group)
    if rank == 0:
        for (both, blocks, name), gbs in results.items():
            who = "both ranks copy" if both else "rank 0 alone"
            grid = "4 blocks per SM" if blocks == 0 else f"{blocks} blocks"
            print(f"{name} {args.mib} MiB, {grid}, {who}: {gbs:7.1f} GB/s", flush=True)
    dist.barrier(group=group)
    comm.release_context(group)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Helpers to run a function on N gloo ranks on this host (CPU), the way the distributed tests do."""
from __future__ import annotations

import io
import os
import socket
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank: int, world: int, port: int, fn, args, queue) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), GLOO_SOCKET_IFNAME="lo", OMP_NUM_THREADS="1")
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    torch.set_num_threads(1)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        # tensors are shipped as bytes: a child may exit before the parent has read the queue
        buf = io.BytesIO()
        torch.save(out, buf)
        queue.put((rank, "ok", buf.getvalue()))
    except BaseException:  # noqa: BLE001
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_distributed(fn, world: int, *args, timeout: float = 240.0) -> list:
    """Run ``fn(rank, world, *args)`` on ``world`` gloo ranks; returns the per-rank results (rank order)."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, queue), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    results: dict[int, object] = {}
    errors = []
    try:
        for _ in range(world):
            rank, status, payload = queue.get(timeout=timeout)
            if status == "ok":
                results[rank] = torch.load(io.BytesIO(payload), weights_only=False)
            else:
                errors.append(f"rank {rank}:\n{payload}")
                break
    finally:
        for p in procs:
            p.join(timeout=5 if not errors else 1)
            if p.is_alive():
                p.kill()  # exact child processes started above
    if errors:
        raise AssertionError("distributed run failed\n" + "\n".join(errors))
    return [results[r] for r in range(world)]

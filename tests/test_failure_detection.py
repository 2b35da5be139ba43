"""Failure detection without faulting a GPU.

* Host side (CPU / gloo): a rank that leaves before a collective makes the survivor's collective fail within the process
  group's timeout; a data loader that raises mid-run propagates out of the trainer after the runtime was closed; a
  truncated checkpoint artifact and a full disk guard are refused with clear errors.
* Device side: a kernel waits (with a short limit) on a flag that nothing ever sets; it must return by itself, report
  "peer flag wait timed out" through the status word, and leave the context usable for the next launch.
"""
import datetime
import json
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.dist_utils import free_port


# ------------------------------------------------------------------------------------------------ host side
def _leaver_worker(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    t = torch.ones(4)
    dist.all_reduce(t)                       # one healthy step
    if rank == 1:
        queue.put((rank, "left"))
        queue.close()
        queue.join_thread()
        os._exit(0)                          # the rank disappears between steps, nothing of its own in flight
    try:
        dist.all_reduce(t)
        queue.put((rank, "no error"))
    except Exception as exc:  # noqa: BLE001 - any backend error type is fine, it must be an error and not a hang
        queue.put((rank, f"error:{type(exc).__name__}"))
    queue.close()
    queue.join_thread()
    os._exit(0)


def test_survivor_sees_an_error_not_a_hang_when_a_rank_leaves():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_leaver_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert got[1] == "left" and got[0].startswith("error:"), got


class _ExplodingLoader:
    consumed_tokens = 0

    def __init__(self, good: int) -> None:
        self.good = good

    def next_batch(self, cp_rank=None):
        if self.good == 0:
            raise OSError("shard vanished")
        self.good -= 1
        g = torch.Generator().manual_seed(self.good)
        ids = torch.randint(0, 64, (2, 16), generator=g)
        return {"input_ids": ids, "labels": ids.roll(-1, 1)}

    def state_dict(self):
        return {}

    def load_state_dict(self, state):
        pass


def test_loader_failure_propagates_and_checkpoint_guards(tmp_path):
    import maltos_b200  # noqa: F401
    from maltos_b200 import models
    from maltos_b200.runtime import RuntimeCore
    from maltos_b200.state.checkpoint import load_sharded_checkpoint, save_sharded_checkpoint
    from maltos_b200.train import Trainer, TrainerConfig

    torch.manual_seed(0)
    rt = RuntimeCore(model=models.TinyTransformer(32, 2, 2, 64, 1e-5, 1, 64, 16), optimizer_factory=lambda ps: torch.optim.AdamW(ps, lr=1e-3))
    trainer = Trainer(runtime=rt, dataloader=_ExplodingLoader(good=3), config=TrainerConfig(max_steps=10, log_every=100))
    trainer.setup()
    with pytest.raises(OSError, match="shard vanished"):
        trainer.fit()
    # a healthy runtime to exercise the checkpoint guards
    rt2 = RuntimeCore(model=models.TinyTransformer(32, 2, 2, 64, 1e-5, 1, 64, 16), optimizer_factory=lambda ps: torch.optim.AdamW(ps, lr=1e-3))
    rt2.setup()
    ckpt = tmp_path / "step_00000001"
    save_sharded_checkpoint(rt2.state_manager, ckpt)
    with pytest.raises((ValueError, FileExistsError)):
        save_sharded_checkpoint(rt2.state_manager, ckpt)                      # never overwrite
    with pytest.raises(RuntimeError, match="insufficient free space"):
        save_sharded_checkpoint(rt2.state_manager, tmp_path / "step_00000002", min_free_gb=1e9)   # disk-space guard
    manifest = json.loads((ckpt / "manifest.json").read_text())
    model_file = next(a["path"] for a in manifest["artifacts"] if a["kind"] == "model")
    data = (ckpt / model_file).read_bytes()
    (ckpt / model_file).write_bytes(data[: len(data) // 3])                   # truncated artifact
    with pytest.raises(Exception):
        load_sharded_checkpoint(rt2.state_manager, ckpt)
    rt2.close()


def _truncated_file_case(rank, world, root):
    """Two data-parallel ranks with ZeRO-3 (every rank reads its own files); rank 1's model file is cut short."""
    import time

    from maltos_b200.state import load_sharded_checkpoint, save_sharded_checkpoint
    from maltos_b200.train import cli, flags as F

    a = F.parse_args_from(["--model", "tiny", "--dim", "32", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "64", "--n-layers", "1", "--vocab-size", "64",
                           "--seq-len", "16", "--dp-size", "2", "--zero-stage", "3", "--precision", "fp32", "--disable-metrics"], require_data=False)
    torch.manual_seed(0)
    core = cli._build_runtime(a, cli._build_model(a), torch.device("cpu"))
    core.setup()
    ckpt = f"{root}/step_00000000"
    save_sharded_checkpoint(core.state_manager, ckpt)
    if rank == 1:
        path = f"{ckpt}/model_rank_1.pt"
        data = open(path, "rb").read()
        open(path, "wb").write(data[: len(data) // 2])
    import torch.distributed as dist

    dist.barrier()
    t0 = time.monotonic()
    try:
        load_sharded_checkpoint(core.state_manager, ckpt)
        outcome = "loaded"
    except Exception as exc:  # noqa: BLE001
        outcome = f"{type(exc).__name__}: {exc}"
    seconds = time.monotonic() - t0
    try:                                   # a second save into the same place: rank 0 refuses, rank 1 must not wait in a barrier
        save_sharded_checkpoint(core.state_manager, ckpt)
        second = "saved"
    except Exception as exc:  # noqa: BLE001
        second = f"{type(exc).__name__}: {exc}"
    core.close()
    return outcome, seconds, second


def test_every_rank_stops_when_one_rank_cannot_read_its_checkpoint_file(tmp_path):
    from tests.dist_utils import run_distributed

    (own, t_own, save_1), (other, t_other, save_0) = reversed(run_distributed(_truncated_file_case, 2, str(tmp_path)))
    assert save_0.startswith("FileExistsError") and save_1.startswith("RuntimeError") and "failed on rank(s) [0]" in save_1, (save_0, save_1)
    assert own.startswith("ValueError") and "model_rank_1.pt cannot be read" in own, own
    assert other.startswith("RuntimeError") and "failed on rank(s) [1]" in other, other      # the healthy rank does not wait for a timeout
    assert max(t_own, t_other) < 20.0


def _graceful_stop_case(rank, world, root):
    """Rank 1 alone is told to stop while step 3 is being prepared (a scheduler's SIGTERM reaches ranks at different
    times); both ranks must leave after the SAME step with a checkpoint of it."""
    from maltos_b200.data import SimpleTensorDataLoader
    from maltos_b200.train import Trainer, TrainerConfig, cli, flags as F

    a = F.parse_args_from(["--model", "tiny", "--dim", "32", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "64", "--n-layers", "1", "--vocab-size", "64",
                           "--seq-len", "16", "--dp-size", "2", "--zero-stage", "1", "--precision", "fp32", "--disable-metrics", "--lr", "1e-2"], require_data=False)

    def run(ckpt_dir, resume, stop_at, max_steps):
        torch.manual_seed(0)
        core = cli._build_runtime(a, cli._build_model(a), torch.device("cpu"))
        g = torch.Generator().manual_seed(5 + rank)
        loader = SimpleTensorDataLoader(torch.randint(0, 64, (64, 17), generator=g), batch_size=2)
        trainer = Trainer(runtime=core, dataloader=loader, runtime_spec={"v": 1},
                          config=TrainerConfig(max_steps=max_steps, log_every=100, checkpoint_every=50, checkpoint_dir=ckpt_dir, resume_from=resume))
        trainer.setup()
        trainer.enable_graceful_stop()
        inner = loader.next_batch
        calls = {"n": 0}

        def next_batch(cp_rank=None):
            calls["n"] += 1
            if stop_at is not None and rank == 1 and calls["n"] == stop_at:
                trainer.request_stop()
            t = inner(cp_rank)
            t = t["input_ids"] if isinstance(t, dict) else t
            return {"input_ids": t[:, :-1].contiguous(), "labels": t[:, 1:].contiguous()}

        loader.next_batch = next_batch
        losses = []
        step_optimizer = core.step_optimizer

        def record():
            step_optimizer()
            losses.append(float(core.collect_metrics()["loss"]))

        core.step_optimizer = record
        trainer.fit()
        return trainer.stopped_early_at, losses

    stopped, first = run(f"{root}/a", None, 3, 8)
    from maltos_b200.train.cli import latest_checkpoint

    newest = latest_checkpoint(f"{root}/a")
    _, rest = run(f"{root}/a", str(newest), None, 8)
    _, straight = run(f"{root}/b", None, None, 8)
    return stopped, newest.name, first, rest, straight


def test_a_stop_request_on_one_rank_ends_all_ranks_after_the_same_step_with_a_checkpoint(tmp_path):
    from tests.dist_utils import run_distributed

    results = run_distributed(_graceful_stop_case, 2, str(tmp_path))
    stops = {r[0] for r in results}
    assert len(stops) == 1 and 3 <= next(iter(stops)) <= 5, stops                  # requested before step 3, effective within two steps
    step = next(iter(stops))
    for stopped, newest, first, rest, straight in results:
        assert newest == f"step_{step:08d}" and len(first) == step
        assert first + rest == pytest.approx(straight, abs=1e-6) and len(straight) == 8      # stop + resume == uninterrupted


def _heartbeat_worker(rank, world, port, queue):
    import time

    from maltos_b200.utils.heartbeat import HeartbeatMonitor, PeerLostError

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    monitor = HeartbeatMonitor.for_default_group(interval=0.3, timeout=3.0).start()
    t = torch.ones(1)
    dist.all_reduce(t)                               # a healthy step with everyone
    if rank == 3:                                    # finishes normally: must not be reported
        monitor.stop()
        queue.put((rank, "left on purpose"))
    elif rank == 2:                                  # disappears between steps, nothing of its own in flight
        queue.put((rank, "vanished"))
        queue.close()
        queue.join_thread()
        os._exit(0)
    else:
        t0 = time.monotonic()
        outcome = "nothing noticed"
        while time.monotonic() - t0 < 20:
            try:
                monitor.check()                      # what the trainer does before every micro-step
            except PeerLostError as exc:
                outcome = f"lost {exc.ranks} after {time.monotonic() - t0:.1f}s"
                break
            time.sleep(0.1)
        monitor.stop()
        queue.put((rank, outcome))
    queue.close()
    queue.join_thread()
    os._exit(0)                                      # no collective shutdown: a peer is gone


def test_heartbeat_names_the_rank_that_vanished_before_the_next_collective():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_heartbeat_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=90) for _ in range(4))
    for p in procs:
        p.join(timeout=30)
    assert got[2] == "vanished" and got[3] == "left on purpose"
    for survivor in (0, 1):
        assert got[survivor].startswith("lost [2] after"), got           # rank 3 ended normally and is not reported
        assert float(got[survivor].split("after ")[1][:-1]) < 15.0, got


# ------------------------------------------------------------------------------------------------ device side
@pytest.mark.gpu
def test_wait_on_a_flag_nobody_sets_times_out_cleanly():
    import ctypes

    from maltos_b200.ops import _lib
    from maltos_b200.ops.gemm import gemm

    dev = torch.device("cuda", 0)
    L = _lib.lib()
    B, rows, K, N, world = 1, 256, 256, 256, 2
    x = torch.randn(B * rows, K, device=dev).bfloat16()
    w = torch.randn(N, K, device=dev).bfloat16()
    out = torch.empty(B * rows * world, N, device=dev, dtype=torch.bfloat16)
    buf_elems = B * rows * world * K
    # a two-rank group of which only rank 0 exists: rank 1's buffers are plain local memory that nothing ever fills,
    # so its "rows have arrived" flag in rank 0's signal pad is never written
    bufs = [torch.zeros(2 * buf_elems, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    pads = [torch.zeros(1024, device=dev, dtype=torch.int32) for _ in range(world)]
    gathered = (ctypes.c_ulonglong * 8)(*([b.data_ptr() for b in bufs] + [0] * 6))
    pad_ptrs = (ctypes.c_ulonglong * 8)(*([p.data_ptr() for p in pads] + [0] * 6))
    _lib.fetch_status(raise_on_error=False)
    _lib.set_wait_timeout_ms(300)
    try:
        rc = L.mb_ag_gemm_bf16(_lib.ptr(x), _lib.c_ll(K), _lib.c_int(B), _lib.c_int(rows), _lib.ptr(w), _lib.c_int(0), _lib.c_ll(K), _lib.ptr(out),
                               _lib.c_ll(N), _lib.c_int(N), _lib.c_int(K), _lib.c_int(0), _lib.c_int(world), ctypes.c_uint(1), gathered, pad_ptrs,
                               _lib.c_ll(buf_elems), _lib.c_int(4), _lib.stream_ptr())
        assert rc == 0
        with pytest.raises(_lib.CommTimeoutError) as err:
            _lib.fetch_status()
        assert err.value.peer == 1
    finally:
        _lib.set_wait_timeout_ms(0)
    # the kernel returned by itself, the status word is clear again and the context still works
    assert _lib.fetch_status(raise_on_error=False)[0] == 0
    a = torch.randn(256, 128, device=dev).bfloat16()
    c = gemm(a, w[:, :128].contiguous())
    ref = a.float() @ w[:, :128].float().t()
    assert ((c.float() - ref).abs().max() / ref.abs().max()).item() < 1e-2
    _lib.fetch_status()
    # the rows that WERE local have been multiplied correctly
    ref0 = x.float() @ w.float().t()
    assert ((out[:rows].float() - ref0).abs().max() / ref0.abs().max()).item() < 1e-2

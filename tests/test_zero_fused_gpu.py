"""Peer-memory paths of the sharded optimizers: the owner-side gradient reduction and the AdamW kernel that stores the
updated slice into every rank's buffer. The kernels are checked on one GPU with the ranks' buffers emulated as local
tensors (they never wait on a peer), the plugin path on 2 GPUs against the NCCL path."""
import os

import pytest
import torch

from tests.dist_utils import free_port

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,n,offset", [(2, 8 * 1024 + 3, 0), (4, 1 << 20, 0), (8, 40_000, 0), (3, 5000, 1), (16, 4096, 0)])
@pytest.mark.parametrize("out_dtype,accumulate", [(torch.bfloat16, False), (torch.bfloat16, True), (torch.float32, False), (torch.float32, True)])
def test_peer_reduce_shard_matches_fp32_sum(world, n, offset, out_dtype, accumulate):
    from maltos_b200.ops import _lib
    from maltos_b200.ops.zero_fused import peer_reduce_shard, peer_reduce_shard_reference

    g = torch.Generator(device="cuda").manual_seed(world * 1000 + n)
    buckets = [torch.randn(n + 16, device="cuda", generator=g).bfloat16() for _ in range(world)]
    shards = [b[offset:offset + n] for b in buckets]         # offset 1 -> 2-byte aligned only: the scalar path
    scale = 0.7 / world
    for rank in (0, world - 1):
        out = torch.randn(n, device="cuda", generator=g).to(out_dtype)
        ref = out.clone()
        sq = torch.zeros((), dtype=torch.float64, device="cuda")
        peer_reduce_shard([s.data_ptr() for s in shards], rank, n, scale, out, accumulate=accumulate, sumsq=sq)
        ref_sq = peer_reduce_shard_reference(shards, scale, ref, accumulate=accumulate)
        torch.cuda.synchronize()
        tol = 1e-2 if out_dtype == torch.bfloat16 else 1e-5
        assert (out.float() - ref.float()).abs().max().item() <= tol * max(1.0, ref.float().abs().max().item())
        assert abs(sq.item() - ref_sq.item()) <= 1e-3 * ref_sq.item()
    assert _lib.fetch_status(raise_on_error=False)[0] == 0


@pytest.mark.parametrize("n,grad_dtype,ndst", [(8 * 2048, torch.bfloat16, 3), (100_003, torch.bfloat16, 5), (4096, torch.float32, 1)])
def test_adamw_push_matches_reference_and_reaches_every_destination(n, grad_dtype, ndst):
    from maltos_b200.ops.optim import _adamw_reference
    from maltos_b200.ops.zero_fused import adamw_push

    g = torch.Generator(device="cuda").manual_seed(n)
    master = torch.randn(n, device="cuda", generator=g)
    m = torch.randn(n, device="cuda", generator=g) * 0.1
    v = torch.rand(n, device="cuda", generator=g) * 0.01
    grad = torch.randn(n, device="cuda", generator=g).to(grad_dtype)
    scale = torch.tensor([0.5], device="cuda")
    ref_p, ref_m, ref_v = master.clone(), m.clone(), v.clone()
    ref_low = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    dsts = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(ndst)]
    kw = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    for step in (1.0, 2.0):
        adamw_push(master, grad, m, v, [d.data_ptr() for d in dsts], step=step, grad_scale=scale, **kw)
        _adamw_reference(ref_p, grad, ref_m, ref_v, ref_low, step, kw["lr"], kw["beta1"], kw["beta2"], kw["eps"], kw["weight_decay"], scale)
    torch.cuda.synchronize()
    assert torch.allclose(master, ref_p, rtol=1e-5, atol=1e-6)
    assert torch.allclose(m, ref_m, rtol=1e-5, atol=1e-7) and torch.allclose(v, ref_v, rtol=1e-5, atol=1e-9)
    for d in dsts:
        assert torch.equal(d, master.bfloat16())


@pytest.mark.parametrize("world,bytes_each", [(2, 16), (4, 4096 + 16), (8, 3 << 20)])
def test_peer_gather_concatenates_the_pieces(world, bytes_each):
    from maltos_b200.ops.zero_fused import peer_gather

    g = torch.Generator(device="cuda").manual_seed(bytes_each)
    pieces = [torch.randint(0, 255, (bytes_each + 64,), dtype=torch.uint8, device="cuda", generator=g) for _ in range(world)]
    out = torch.zeros(world * bytes_each + 32, dtype=torch.uint8, device="cuda")
    peer_gather(out, [p.data_ptr() for p in pieces], bytes_each)
    assert torch.equal(out[:world * bytes_each], torch.cat([p[:bytes_each] for p in pieces]))
    assert int(out[world * bytes_each:].sum()) == 0


@pytest.mark.parametrize("world,n,dtype", [(2, 8 * 1000 + 5, torch.bfloat16), (4, 1 << 18, torch.bfloat16), (8, 4 * 777 + 3, torch.float32), (16, 4096, torch.float32)])
def test_peer_all_reduce_writes_the_scaled_sum_into_every_bucket(world, n, dtype):
    from maltos_b200.ops.zero_fused import peer_all_reduce

    g = torch.Generator(device="cuda").manual_seed(n + world)
    bufs = [torch.randn(n + 32, device="cuda", generator=g).to(dtype) for _ in range(world)]
    want = sum(b[:n].float() for b in bufs) * (1.0 / world)
    tails = [b[n:].clone() for b in bufs]
    peer_all_reduce([b.data_ptr() for b in bufs], n, dtype, 1.0 / world)
    torch.cuda.synchronize()
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-6
    for b, t in zip(bufs, tails):
        assert (b[:n].float() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
        assert torch.equal(b[n:], t)                     # nothing beyond the slice is touched
    assert all(torch.equal(bufs[0][:n], b[:n]) for b in bufs)


# ------------------------------------------------------------------------------------------------ plugin path on 2 GPUs
def _train(rank, world, stage, peer):
    import torch.distributed as dist

    import maltos_b200  # noqa: F401
    from maltos_b200 import models
    from maltos_b200.parallel import ParallelPlan
    from maltos_b200.runtime import MeshConfig, RuntimeCore
    from maltos_b200.runtime.optim import FusedAdamW
    from maltos_b200.runtime.plugins import zero1

    torch.manual_seed(4321)
    model = models.TinyTransformer(128, 4, 2, 256, 1e-5, 2, 96, 32)
    if stage == 0:
        from maltos_b200.runtime.plugins import ddp

        plugin = ddp.BucketDataParallelPlugin(bucket_mb_size=1, peer_memory=peer)
    elif stage == 3:
        import torch.nn as nn

        from maltos_b200.models.tiny_transformer import RmsNorm
        from maltos_b200.runtime.plugins import zero3

        plugin = zero3.Zero3Plugin(wrap_cls={nn.Linear, nn.Embedding, RmsNorm}, peer_memory=peer)
    else:
        cls = zero1.Zero1Plugin if stage == 1 else zero1.Zero2Plugin
        plugin = cls(bucket_mb_size=1, peer_memory=peer)
    rt = RuntimeCore(model=model, mesh=MeshConfig(dp=world), plan=ParallelPlan(), plugins=[plugin], dtype=torch.bfloat16,
                     device=torch.device("cuda", rank), optimizer_factory=lambda ps: FusedAdamW(ps, lr=1e-2, weight_decay=0.01),
                     grad_accum_steps=2, grad_clip_max_norm=None if stage == 0 else 0.5)
    rt.setup()
    if stage == 0:
        assert (plugin.buckets[0].peer_ptrs is not None) == peer
    elif stage == 3:
        assert all((b.peer_shard_ptrs is not None) == peer for b in plugin.buckets)
    else:
        assert (plugin.buckets[0].peer_grad_ptrs is not None) == peer and plugin._pushes == peer
    g = torch.Generator().manual_seed(99)
    losses = []
    for _ in range(3):
        for _ in range(2):
            ids = torch.randint(0, 96, (world * 4, 32), generator=g)
            batch = {"input_ids": ids[rank * 4:(rank + 1) * 4].cuda(), "labels": ids.roll(-1, 1)[rank * 4:(rank + 1) * 4].cuda()}
            loss, _ = rt.run_step(batch)
            if rank == 0:
                print(f"stage {stage} peer {peer}: micro-step loss {float(loss):.4f}", flush=True)
        rt.step_optimizer()
        losses.append(float(rt.collect_metrics()["loss"]))
    if stage == 3:
        plugin.materialize_model()
    params = torch.cat([p.detach().float().reshape(-1) for p in rt.model.parameters()]).cpu()
    norm = rt.state.metadata.get("grad_norm")
    rt.close()
    dist.barrier()
    return losses, params, norm


def _worker(rank, world, port, queue):
    import traceback

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        out = {}
        for stage in (0, 1, 2, 3):      # 0 = bucketed data parallel, 1-3 = ZeRO stages
            for peer in (False, True):
                try:
                    out[(stage, peer)] = _train(rank, world, stage, peer)
                except Exception as exc:  # noqa: BLE001 - name the failing configuration
                    raise RuntimeError(f"stage {stage}, peer_memory={peer} failed") from exc
        from maltos_b200.ops import _lib

        queue.put((rank, "ok", (out, _lib.fetch_status(raise_on_error=False))))
    except BaseException:  # noqa: BLE001
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.multigpu
def test_zero_peer_memory_mode_matches_nccl_mode_two_gpus():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=240)
            assert status == "ok", payload
            got[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    for rank, (out, status) in got.items():
        assert status[0] == 0, f"rank {rank} kernel status {status}"
        for stage in (0, 1, 2, 3):
            (l0, p0, n0), (l1, p1, n1) = out[(stage, False)], out[(stage, True)]
            assert max(abs(a - b) for a, b in zip(l0, l1)) < 2e-2, (stage, l0, l1)
            assert (p0 - p1).abs().max().item() < 2e-2, stage
            if stage:
                assert abs(n0 - n1) < 2e-2 * max(1.0, abs(n0)), (stage, n0, n1)
    # every rank holds the same parameters after the pushes
    assert torch.equal(got[0][0][(1, True)][1], got[1][0][(1, True)][1])

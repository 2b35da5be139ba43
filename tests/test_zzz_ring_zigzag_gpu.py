"""Ring attention with the dense zigzag layout on 2 GPUs: the half-block schedule (unmasked kernels on half of the keys or
half of the queries) against fp32 attention over the gathered sequence, over peer memory and over the point-to-point ring."""
import os

import pytest
import torch

from tests.dist_utils import free_port

pytestmark = pytest.mark.gpu


def _run(rank, world, group, peer):
    import torch.distributed as dist

    from maltos_b200.ops.attention import attention_reference
    from maltos_b200.runtime.layers import ring_attention as ra
    from maltos_b200.runtime.layers.ring_layout import zigzag_positions

    os.environ["MALTOS_B200_RING_PEER"] = "1" if peer else "0"
    B, S, hq, hkv, D = 2, 256, 4, 2, 64
    g = torch.Generator(device="cuda").manual_seed(5 + rank)
    q = (torch.randn(B, S, hq, D, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_()
    k = (torch.randn(B, S, hkv, D, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_()
    v = (torch.randn(B, S, hkv, D, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_()
    w = torch.randn(B, S, hq, D, device="cuda", generator=g).bfloat16()
    pos = zigzag_positions(S * world, rank, world, device="cuda").unsqueeze(0).expand(B, -1).contiguous()
    plan = ra.build_ring_plan(pos, None, group)
    assert plan.zigzag and all(plan.visible)
    o = ra.flash_ring_attention(q, k, v, group, q_positions=pos, plan=plan)
    (o.float() * w.float()).sum().backward()

    def gathered(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous(), group=group)
        return torch.cat(parts, dim=1)

    qa, ka, va = (gathered(t.detach()).float().requires_grad_() for t in (q, k, v))
    pa, wa = gathered(pos), gathered(w).float()
    ref = attention_reference(qa, ka, va, q_positions=pa, k_positions=pa)
    (ref * wa).sum().backward()
    mine = slice(rank * S, (rank + 1) * S)
    errs = {}
    for name, got, want in (("out", o, ref), ("dq", q.grad, qa.grad), ("dk", k.grad, ka.grad), ("dv", v.grad, va.grad)):
        want = want.detach()[:, mine]
        errs[name] = ((got.detach().float() - want).abs().max() / want.abs().max().clamp_min(1e-3)).item()
    return errs


def _worker(rank, world, port, queue):
    import traceback

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import maltos_b200  # noqa: F401
        from maltos_b200.ops import _lib

        group = dist.new_group(list(range(world)))
        res = {peer: _run(rank, world, group, peer) for peer in (False, True)}
        torch.cuda.synchronize()
        dist.barrier(group=group)
        queue.put((rank, "ok", (res, _lib.fetch_status(raise_on_error=False))))
    except BaseException:  # noqa: BLE001
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.multigpu
def test_zigzag_half_block_schedule_matches_whole_sequence_attention_two_gpus():
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
    for rank, (res, status) in got.items():
        assert status[0] == 0, f"rank {rank} kernel status {status}"
        for peer, errs in res.items():
            for name, e in errs.items():
                assert e <= 4e-2, (rank, peer, name, e)

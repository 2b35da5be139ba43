"""Ring attention with the block exchange over peer memory (pulls on a copy stream, gradient slots at the owner)
against the point-to-point ring, on 2 GPUs; and the peer copy kernel on one GPU."""
import os

import pytest
import torch

from tests.dist_utils import free_port

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nbytes", [16, 4096 + 7, 3 * (1 << 20) + 5])
def test_peer_copy_kernel_copies_any_byte_count(nbytes):
    from maltos_b200.ops import _lib
    from maltos_b200.ops.peer_ring import _copy

    src = torch.randint(0, 255, (nbytes + 32,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros_like(src)
    _copy(dst.data_ptr(), src.data_ptr(), nbytes, 4)
    assert torch.equal(dst[:nbytes], src[:nbytes]) and int(dst[nbytes:].sum()) == 0
    _copy(dst.data_ptr(), src.data_ptr(), nbytes)
    assert torch.equal(dst[:nbytes], src[:nbytes])
    assert _lib.fetch_status(raise_on_error=False)[0] == 0


def _run(rank, world, group, peer, packed):
    from maltos_b200.runtime.layers.ring_attention import flash_ring_attention

    os.environ["MALTOS_B200_RING_PEER"] = "1" if peer else "0"
    B, S, hq, hkv, D = 2, 256, 4, 2, 64
    g = torch.Generator(device="cuda").manual_seed(5 + rank)
    outs = []
    for rep in range(2):
        q = (torch.randn(B, S, hq, D, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_()
        k = (torch.randn(B, S, hkv, D, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_()
        v = (torch.randn(B, S, hkv, D, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_()
        pos = (torch.arange(S, device="cuda") + rank * S).unsqueeze(0).expand(B, -1).contiguous()
        seq = None
        if packed:      # two documents per row; the second one spans the rank boundary
            seq = (pos >= S // 2).long()
        o = flash_ring_attention(q, k, v, group, q_positions=pos, q_sequence_ids=seq)
        w = torch.randn(o.shape, device="cuda", generator=g).bfloat16()
        (o.float() * w.float()).sum().backward()
        outs.append([t.detach().float().cpu() for t in (o, q.grad, k.grad, v.grad)])
    return outs


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
        res = {}
        for packed in (False, True):
            res[packed] = (_run(rank, world, group, False, packed), _run(rank, world, group, True, packed))
        torch.cuda.synchronize()
        dist.barrier(group=group)
        queue.put((rank, "ok", (res, _lib.fetch_status(raise_on_error=False))))
    except BaseException:  # noqa: BLE001
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.multigpu
def test_ring_attention_peer_exchange_matches_point_to_point_ring_two_gpus():
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
        for packed, (ref, peer) in res.items():
            for a_rep, b_rep in zip(ref, peer):
                for name, a, b in zip(("out", "dq", "dk", "dv"), a_rep, b_rep):
                    assert (a - b).abs().max().item() <= 2e-2 * max(1e-2, a.abs().max().item()), (rank, packed, name)

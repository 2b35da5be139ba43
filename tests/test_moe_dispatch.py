"""Expert-parallel dispatch / combine over peer memory: the row plan on the host, the row kernels on one GPU with the
ranks' buffers emulated as local tensors, and the layer on 2 GPUs against the all-to-all path."""
import os

import pytest
import torch

from tests.dist_utils import free_port


def test_row_plan_is_a_permutation_sorted_by_expert_then_source():
    from maltos_b200.ops.moe_dispatch import plan_rows

    g = torch.Generator().manual_seed(3)
    world, per = 4, 3
    counts = torch.randint(0, 7, (world, world * per), generator=g)
    counts[:, 5] = 0                                                  # an expert nobody routes to
    rows_of = {d: [] for d in range(world)}                           # owner -> (row, expert, source)
    for rank in range(world):
        my_start, recv_rows, local_counts = plan_rows(counts, rank, per)
        assert recv_rows.tolist() == counts.sum(0).view(world, per).sum(1).tolist()
        assert local_counts.tolist() == counts.sum(0).view(world, per)[rank].tolist()
        for e in range(world * per):
            for j in range(int(counts[rank, e])):
                rows_of[e // per].append((int(my_start[e]) + j, e, rank))
    for d, rows in rows_of.items():
        rows.sort()
        assert [r for r, _, _ in rows] == list(range(len(rows)))      # dense, no collisions
        assert [(e, s) for _, e, s in rows] == sorted((e, s) for _, e, s in rows)


@pytest.mark.gpu
@pytest.mark.parametrize("hidden,dtype", [(64, torch.bfloat16), (1024, torch.bfloat16), (200, torch.float32)])
def test_push_and_pull_rows_between_emulated_ranks(hidden, dtype):
    from maltos_b200.ops import _lib

    lib = _lib.lib()
    world, cap, m, n_tokens = 3, 97, 150, 40
    g = torch.Generator(device="cuda").manual_seed(hidden)
    bufs = [torch.zeros(cap, hidden, device="cuda", dtype=dtype) for _ in range(world)]
    table = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    flat = torch.randn(n_tokens, hidden, device="cuda", generator=g).to(dtype)
    token = torch.randint(0, n_tokens, (m,), device="cuda", generator=g)
    slots = torch.randperm(world * cap, device="cuda", generator=g)[:m]          # distinct (rank, row) targets
    peer_rank, peer_row = (slots // cap).to(torch.int32), (slots % cap).to(torch.int64)
    row_bytes = hidden * flat.element_size()
    args = (_lib.ptr(table), _lib.c_ll(0), _lib.c_ll(row_bytes), _lib.c_ll(cap), _lib.ptr(peer_rank), _lib.ptr(peer_row), _lib.c_ll(m),
            _lib.c_int(row_bytes), _lib.c_int(world), _lib.stream_ptr())
    _lib.check(lib.mb_peer_push_rows(_lib.ptr(flat), _lib.c_ll(row_bytes), _lib.ptr(token), _lib.c_ll(n_tokens), *args), "push")
    ref = [torch.zeros_like(b) for b in bufs]
    for j in range(m):
        ref[int(peer_rank[j])][int(peer_row[j])] = flat[int(token[j])]
    for b, r in zip(bufs, ref):
        assert torch.equal(b, r)
    out = torch.empty(m, hidden, device="cuda", dtype=dtype)
    _lib.check(lib.mb_peer_pull_rows(_lib.ptr(out), _lib.c_ll(row_bytes), None, _lib.c_ll(m), *args), "pull")
    assert torch.equal(out, flat[token])
    assert _lib.fetch_status(raise_on_error=False)[0] == 0
    # an out-of-range row is reported through the status word and skipped
    peer_row[3] = cap + 5
    _lib.check(lib.mb_peer_pull_rows(_lib.ptr(out), _lib.c_ll(row_bytes), None, _lib.c_ll(m), *args), "pull")
    torch.cuda.synchronize()
    assert _lib.fetch_status(raise_on_error=False)[0] & 4


# ------------------------------------------------------------------------------------------------ layer on 2 GPUs
def _layer_run(rank, world, group, peer_mode, top_k, capacity, swiglu=False):
    import torch.distributed as dist
    import torch.nn as nn

    from maltos_b200.runtime.layers.moe import ExpertParallelMoE

    os.environ["MALTOS_B200_MOE_PEER"] = "1" if peer_mode else "0"
    H, E, N = 128, 4, 96
    torch.manual_seed(11)
    router = nn.Linear(H, E, bias=False).cuda().bfloat16()
    if swiglu:   # SwiGLU experts + a capacity limit: the peer path is then the static one with the grouped expert GEMM
        from maltos_b200.models.tiny_transformer import MLP

        experts = nn.ModuleList([MLP(H, 2 * H) for _ in range(E)]).cuda().bfloat16()
    else:
        experts = nn.ModuleList([nn.Sequential(nn.Linear(H, 2 * H, bias=False), nn.GELU(), nn.Linear(2 * H, H, bias=False)) for _ in range(E)]).cuda().bfloat16()
    per = E // world
    ids = list(range(rank * per, (rank + 1) * per))
    layer = ExpertParallelMoE(router=router, local_experts=nn.ModuleList([experts[i] for i in ids]), local_expert_ids=ids, dim=H,
                              num_experts=E, ep_group=group, top_k=top_k, capacity_factor=capacity)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    outs = []
    for _ in range(2):                                    # two calls: buffers are reused
        x = torch.randn(2, N // 2, H, device="cuda", generator=gen).bfloat16().requires_grad_()
        y, aux = layer(x, return_aux_loss=True)
        (y.float().pow(2).mean() + 0.01 * aux.float()).backward()
        grads = [p.grad.detach().float().clone() for p in layer.parameters()]
        outs.append((y.detach().float().cpu(), x.grad.float().cpu(), [g.cpu() for g in grads]))
        for p in layer.parameters():
            p.grad = None
    dist.barrier(group=group)
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
        for top_k, capacity in ((1, None), (2, None), (2, 1.0)):
            res[(top_k, capacity)] = (_layer_run(rank, world, group, False, top_k, capacity), _layer_run(rank, world, group, True, top_k, capacity))
        before = _lib.launch_count()
        res[("swiglu", 2, 1.0)] = (_layer_run(rank, world, group, False, 2, 1.0, True), _layer_run(rank, world, group, True, 2, 1.0, True))
        res[("swiglu", 1, 1.25)] = (_layer_run(rank, world, group, False, 1, 1.25, True), _layer_run(rank, world, group, True, 1, 1.25, True))
        assert _lib.launch_count() > before
        queue.put((rank, "ok", (res, _lib.fetch_status(raise_on_error=False))))
    except BaseException:  # noqa: BLE001
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.multigpu
def test_expert_parallel_layer_peer_path_matches_all_to_all_two_gpus():
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
        for key, (ref, peer) in res.items():
            for (y0, dx0, g0), (y1, dx1, g1) in zip(ref, peer):
                assert (y0 - y1).abs().max().item() <= 2e-2 * max(1.0, y0.abs().max().item()), key
                assert (dx0 - dx1).abs().max().item() <= 2e-2 * max(1e-3, dx0.abs().max().item()), key
                for a, b in zip(g0, g1):
                    assert (a - b).abs().max().item() <= 3e-2 * max(1e-3, a.abs().max().item()), key

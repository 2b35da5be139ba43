"""Fused tensor-parallel collectives over NVLink peer memory (in-GEMM push, GEMM epilogue scatter, and the pull kernels)
against NCCL collectives + fp32 matmul, on 2, 4 and 8 GPUs (the larger groups skip where fewer GPUs are present)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.dist_utils import free_port

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _worker(rank, world, port, queue):
    import io
    import traceback

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MALTOS_B200_FUSED_SCATTER="1", MALTOS_B200_FUSED_DGRAD_GATHER="1")   # the fused GEMM -> reduce-scatter is opt-in
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import maltos_b200  # noqa: F401
        from maltos_b200.ops import _lib, comm
        from maltos_b200.ops.fused_tp import all_gather_grouped_linear
        from maltos_b200.ops.grouped import fuse_parameters

        group = dist.new_group(list(range(world)))
        ctx = comm.context_for(group)
        assert ctx is not None, comm.disabled_reason(group)
        results = []
        torch.manual_seed(7)   # same weights everywhere
        for (B, rows, K, outs) in [(1, 256, 256, (256, 128, 128)), (2, 192, 512, (384, 384)), (1, 1024, 1024, (1024, 256, 256)),
                                   (1, 256, 256, (256, 128, 128))]:
            ws = [torch.nn.Parameter((torch.randn(n, K, device="cuda") * 0.05).bfloat16()) for n in outs]
            fuse_parameters(ws)
            g = torch.Generator(device="cuda").manual_seed(100 + rank)
            for rep in range(8):          # several calls: both buffer parities, the consumed handshake, all push modes
                from maltos_b200.ops.fused_tp import set_push_mode

                set_push_mode(rep >= 2)
                # the last two calls take the NCCL all-gather + GEMM route that large groups use for short GEMMs
                os.environ["MALTOS_B200_FUSED_GATHER"] = "0" if rep in (4, 5) else "1"
                # calls 6 and 7: the push as a launch of its own in front of the GEMM launch
                _lib.lib().mb_gemm_set_push_split(1 if rep >= 6 else 0)
                x = torch.randn(B, rows, K, device="cuda", generator=g).bfloat16().requires_grad_()
                y, offs = all_gather_grouped_linear(x, ws, ctx)
                full = torch.empty(world, B, rows, K, device="cuda", dtype=torch.bfloat16)
                dist.all_gather_into_tensor(full.view(-1, K), x.detach().reshape(-1, K).contiguous(), group=group)
                xf = full.permute(1, 0, 2, 3).reshape(B, world * rows, K).float()
                ref = torch.cat([xf @ w.detach().float().t() for w in ws], dim=-1)
                err = ((y.float() - ref).abs().max() / ref.abs().max()).item()
                dy = torch.randn_like(y)
                y.backward(dy)
                dyf = dy.float()
                dx_full = dyf @ torch.cat([w.detach().float() for w in ws], 0)
                dist.all_reduce(dx_full, group=group)
                dx_ref = dx_full.view(B, world, rows, K)[:, rank]
                gerr = ((x.grad.float() - dx_ref).abs().max() / dx_ref.abs().max()).item()
                dw_ref = dyf.reshape(-1, dyf.shape[-1]).t() @ xf.reshape(-1, K)          # weight gradients from the gathered input
                at = 0
                for w in ws:
                    piece = dw_ref[at:at + w.shape[0]]
                    gerr = max(gerr, ((w.grad.float() - piece).abs().max() / piece.abs().max()).item())
                    at += w.shape[0]
                results.append((B, rows, K, rep, err, gerr))
                for w in ws:
                    w.grad = None
        set_push_mode(False)
        _lib.lib().mb_gemm_set_push_split(0)
        os.environ.pop("MALTOS_B200_FUSED_GATHER", None)
        # the NCCL helpers of the non-fused paths keep the batch-major layout for B > 1 without a permuting copy
        from maltos_b200.ops.fused_tp import _nccl_all_gather_rows, _nccl_reduce_scatter_rows

        B, rows, K = 2, 64, 128
        xs = torch.randn(B * rows, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(300 + rank)).bfloat16()
        got = _nccl_all_gather_rows(xs, ctx, B, rows)
        allx = torch.empty(world, B, rows, K, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(allx.view(-1, K), xs, group=group)
        assert torch.equal(got, allx.permute(1, 0, 2, 3).reshape(B * world * rows, K))
        yf = torch.randn(B * world * rows, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(400 + rank)).bfloat16()
        got = _nccl_reduce_scatter_rows(yf, ctx, B, rows)
        tot = yf.float()
        dist.all_reduce(tot, group=group)
        want = tot.view(B, world, rows, K)[:, rank].reshape(B * rows, K)
        assert (got.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
        # row-parallel GEMM fused with the reduce-scatter (forward) and its backward
        from maltos_b200.ops.fused_tp import linear_reduce_scatter

        import ctypes

        # the last case runs on the 256x512 kernel (forced), whose epilogue writes whole 128-byte lines into the peers' slots
        for (B, S, Kin, H, kind) in [(1, 512, 256, 256, 0), (2, 384, 128, 512, 0), (1, 2048, 512, 1024, 0), (1, 2048, 512, 1024, 1024)]:
            _lib.lib().mb_gemm_set_scatter_kind(ctypes.c_int(kind))
            w = torch.nn.Parameter((torch.randn(H, Kin, device="cuda", generator=torch.Generator(device="cuda").manual_seed(50 + rank)) * 0.05).bfloat16())
            g = torch.Generator(device="cuda").manual_seed(200 + rank)
            rows = S // world
            for rep in range(6):
                # calls 0-2: partial tiles pushed by the GEMM epilogue; calls 3-5: GEMM into symmetric memory + pull kernel
                os.environ["MALTOS_B200_FUSED_SCATTER"] = "1" if rep < 3 else "0"
                x = torch.randn(B, S, Kin, device="cuda", generator=g).bfloat16().requires_grad_()
                y = linear_reduce_scatter(x, w, ctx)
                ref_full = x.detach().float() @ w.detach().float().t()
                dist.all_reduce(ref_full, group=group)
                ref = ref_full.view(B, world, rows, H)[:, rank]
                err = ((y.float() - ref).abs().max() / ref.abs().max()).item()
                dy = torch.randn_like(y)
                y.backward(dy)
                dy_full = torch.empty(world, B, rows, H, device="cuda", dtype=torch.bfloat16)
                dist.all_gather_into_tensor(dy_full.view(-1, H), dy.reshape(-1, H).contiguous(), group=group)
                dyf = dy_full.permute(1, 0, 2, 3).reshape(B, S, H).float()
                dx_ref = dyf @ w.detach().float()
                gerr = ((x.grad.float() - dx_ref).abs().max() / dx_ref.abs().max()).item()
                dw_ref = dyf.reshape(-1, H).t() @ x.detach().float().reshape(-1, Kin)
                gerr = max(gerr, ((w.grad.float() - dw_ref).abs().max() / dw_ref.abs().max()).item())
                results.append((B, S, Kin, 10 + rep, err, gerr))
                w.grad = None
        _lib.lib().mb_gemm_set_scatter_kind(ctypes.c_int(0))
        # the pull kernels called directly, batch-major layout with B > 1, both buffer parities
        from maltos_b200.ops.fused_tp import all_gather_pull, gemm_reduce_scatter_pull

        B, rows, K, N = 2, 96, 256, 384
        for rep in range(4):
            gen = torch.Generator(device="cuda").manual_seed(500 + 10 * rep + rank)
            xs = torch.randn(B * rows, K, device="cuda", generator=gen).bfloat16()
            got = all_gather_pull(xs, ctx, B, rows)
            allx = torch.empty(world, B, rows, K, device="cuda", dtype=torch.bfloat16)
            dist.all_gather_into_tensor(allx.view(-1, K), xs, group=group)
            assert torch.equal(got, allx.permute(1, 0, 2, 3).reshape(B * world * rows, K)), ("all_gather_pull", rep)
            xr = torch.randn(B * world * rows, K, device="cuda", generator=gen).bfloat16()
            wr = (torch.randn(N, K, device="cuda", generator=gen) * 0.05).bfloat16()
            got = gemm_reduce_scatter_pull(xr, wr, ctx, B, rows, b_mn=False)
            tot = xr.float() @ wr.float().t()
            dist.all_reduce(tot, group=group)
            want = tot.view(B, world, rows, N)[:, rank].reshape(B * rows, N)
            assert (got.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item(), ("gemm_reduce_scatter_pull", rep)
        status = _lib.fetch_status(raise_on_error=False)
        queue.put((rank, "ok", (results, status)))
        ctx.close()
    except BaseException:  # noqa: BLE001
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_tensor_parallel_collectives(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=400)
            assert status == "ok", payload
            out[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    for rank, (results, status) in out.items():
        assert status[0] == 0, f"rank {rank} kernel status {status}"
        for B, rows, K, rep, err, gerr in results:
            assert err < 1e-2, (rank, B, rows, K, rep, err)
            assert gerr < 2e-2, (rank, B, rows, K, rep, gerr)

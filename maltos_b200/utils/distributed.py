"""Collective wrappers used by the PyTorch-collective (CPU/gloo and oracle) paths of the runtime.

On CUDA the hot collectives are not issued from here: they are fused into the sm_100a kernels in
``maltos_b200.ops.comm``. These wrappers exist for gloo worlds (tests, CPU runs), the control plane and
pipeline p2p. gloo cannot reduce or move bf16/fp16, so such tensors are staged through fp32 and copied
back when the work is waited on (behaviour of the reference's ``utils/distributed.py:9-153``).
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist

_LOW_PRECISION = (torch.float16, torch.bfloat16)


class CompletedWork:
    """A finished work handle (for code paths that need no communication)."""

    def wait(self) -> None:
        return None

    def block_current_stream(self) -> None:
        return None

    def is_completed(self) -> bool:
        return True


class PostProcessWork:
    """Wraps works plus a callback that must run after they complete (e.g. the fp32 -> bf16 copy-back)."""

    def __init__(self, works: Sequence, *, post_wait: Callable[[], None] | None = None, keepalive=None) -> None:
        self.works = list(works)
        self.post_wait = post_wait
        self.keepalive = list(keepalive or [])
        self._finished = False

    def wait(self) -> None:
        if self._finished:
            return
        for w in self.works:
            w.wait()
        if self.post_wait is not None:
            self.post_wait()
        self._finished = True
        self.keepalive.clear()

    def block_current_stream(self) -> None:
        if self._finished:
            return
        if self.post_wait is not None:
            # The callback touches host-visible state, so it has to be ordered after a real wait.
            self.wait()
            return
        for w in self.works:
            blocker = getattr(w, "block_current_stream", None)
            if blocker is not None:
                blocker()
            else:
                w.wait()

    def is_completed(self) -> bool:
        return self._finished


def backend_of(group: dist.ProcessGroup | None = None) -> str | None:
    if not dist.is_initialized():
        return None
    return dist.get_backend(group) if group is not None else dist.get_backend()


def is_gloo_group(group: dist.ProcessGroup | None = None) -> bool:
    return backend_of(group) == "gloo"


def needs_fp32_comm(tensor: torch.Tensor, group: dist.ProcessGroup | None = None) -> bool:
    return tensor.dtype in _LOW_PRECISION and is_gloo_group(group)


def _cast_into(dst: torch.Tensor, src: torch.Tensor) -> None:
    with torch.no_grad():
        dst.copy_(src)


def _finish(work, async_op: bool):
    if async_op:
        return work
    if work is not None:
        work.wait()
    return None


def all_gather_single(output: torch.Tensor, input: torch.Tensor, *, group=None, async_op: bool = False):
    """``output`` (dim-0 concatenation over ranks) <- all-gather of ``input``."""
    if needs_fp32_comm(input, group):
        staged_out = torch.empty_like(output, dtype=torch.float32)
        staged_in = input.detach().float().contiguous()
        inner = dist.all_gather_into_tensor(staged_out, staged_in, group=group, async_op=True)
        work = PostProcessWork([inner], post_wait=lambda: _cast_into(output, staged_out), keepalive=[staged_in, staged_out])
        return _finish(work, async_op)
    return dist.all_gather_into_tensor(output, input.contiguous(), group=group, async_op=async_op)


def reduce_scatter_single(output: torch.Tensor, input: torch.Tensor, *, op=dist.ReduceOp.SUM, group=None, async_op: bool = False):
    """``output`` <- this rank's dim-0 slice of the reduction of ``input`` over ranks.

    gloo has no reduce-scatter: it is emulated by an all-reduce followed by a narrow, and AVG by SUM / world.
    """
    if is_gloo_group(group):
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        staged = input.detach().float().contiguous() if input.dtype in _LOW_PRECISION else input.detach().clone().contiguous()
        use_avg = op == dist.ReduceOp.AVG
        inner = dist.all_reduce(staged, op=dist.ReduceOp.SUM if use_avg else op, group=group, async_op=True)
        chunk = staged.shape[0] // world

        def _post() -> None:
            piece = staged.narrow(0, rank * chunk, chunk)
            if use_avg:
                piece = piece / world
            _cast_into(output, piece)

        work = PostProcessWork([inner], post_wait=_post, keepalive=[staged])
        return _finish(work, async_op)
    return dist.reduce_scatter_tensor(output, input.contiguous(), op=op, group=group, async_op=async_op)


def all_reduce_tensor(tensor: torch.Tensor, *, op=dist.ReduceOp.SUM, group=None, async_op: bool = False):
    """In-place all-reduce. On gloo, AVG is SUM followed by a division and bf16/fp16 go through fp32."""
    if is_gloo_group(group):
        world = dist.get_world_size(group)
        use_avg = op == dist.ReduceOp.AVG
        low = tensor.dtype in _LOW_PRECISION
        if not low and not use_avg:
            return dist.all_reduce(tensor, op=op, group=group, async_op=async_op)
        staged = tensor.detach().float().contiguous() if low else tensor
        inner = dist.all_reduce(staged, op=dist.ReduceOp.SUM if use_avg else op, group=group, async_op=True)

        def _post() -> None:
            with torch.no_grad():
                if use_avg:
                    staged.div_(world)
                if staged is not tensor:
                    tensor.copy_(staged)

        work = PostProcessWork([inner], post_wait=_post, keepalive=[staged])
        return _finish(work, async_op)
    return dist.all_reduce(tensor, op=op, group=group, async_op=async_op)


def _p2p(ops: list) -> list:
    return list(dist.batch_isend_irecv(ops))


def isend_tensor_async(tensor: torch.Tensor, dst: int, *, group=None):
    """Asynchronous send to global rank ``dst``; returns a waitable."""
    if needs_fp32_comm(tensor, group):
        staged = tensor.detach().float().contiguous()
        return PostProcessWork(_p2p([dist.P2POp(dist.isend, staged, dst, group)]), keepalive=[staged])
    return PostProcessWork(_p2p([dist.P2POp(dist.isend, tensor, dst, group)]), keepalive=[tensor])


def irecv_tensor_async(tensor: torch.Tensor, src: int, *, group=None):
    """Asynchronous receive from global rank ``src`` into ``tensor``; returns a waitable."""
    if needs_fp32_comm(tensor, group):
        staged = torch.empty_like(tensor, dtype=torch.float32)
        return PostProcessWork(
            _p2p([dist.P2POp(dist.irecv, staged, src, group)]),
            post_wait=lambda: _cast_into(tensor, staged),
            keepalive=[staged],
        )
    return PostProcessWork(_p2p([dist.P2POp(dist.irecv, tensor, src, group)]))


def pairwise_send_recv_async(send_tensor, recv_tensor, *, send_rank: int, recv_rank: int, group) -> list:
    """One batched isend+irecv pair (ring exchange step). Returns a list of waitables."""
    if needs_fp32_comm(send_tensor, group) or needs_fp32_comm(recv_tensor, group):
        s = send_tensor.detach().float().contiguous()
        r = torch.empty_like(recv_tensor, dtype=torch.float32)
        works = _p2p([dist.P2POp(dist.isend, s, send_rank, group), dist.P2POp(dist.irecv, r, recv_rank, group)])
        return [PostProcessWork(works, post_wait=lambda: _cast_into(recv_tensor, r), keepalive=[s, r])]
    return _p2p([dist.P2POp(dist.isend, send_tensor, send_rank, group), dist.P2POp(dist.irecv, recv_tensor, recv_rank, group)])


def distributed_barrier() -> None:
    if not dist.is_initialized():
        return
    if dist.get_backend() == "nccl" and torch.cuda.is_available():
        dist.barrier(device_ids=[torch.cuda.current_device()])
    else:
        dist.barrier()


def raise_if_any_rank_failed(error: BaseException | None, what: str) -> None:
    """Collective over the world: every rank reports whether its part of ``what`` worked; if one failed, ALL raise - the
    failing rank its own exception, the others a ``RuntimeError`` that names the ranks - instead of walking into the next
    collective without it and waiting there for the process-group timeout."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        if error is not None:
            raise error
        return
    on_gpu = dist.get_backend() == "nccl" and torch.cuda.is_available()
    flags = torch.zeros(dist.get_world_size(), dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()) if on_gpu else "cpu")
    if error is not None:
        flags[dist.get_rank()] = 1
    dist.all_reduce(flags, op=dist.ReduceOp.MAX)
    failed = [r for r, f in enumerate(flags.tolist()) if f]
    if error is not None:
        raise error
    if failed:
        raise RuntimeError(f"{what} failed on rank(s) {failed}; this rank stops with them")


def group_size(group) -> int:
    if group is None or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None or not dist.is_initialized():
        return 0
    return dist.get_rank(group)

"""Ring attention's block exchange over peer memory.

Instead of forwarding K/V (and, in backward, an fp32 dK/dV accumulator) ``rank -> rank+1`` with point-to-point
collectives for ``world`` steps (reference ``runtime/layers/ring_attention.py:36-258``), every rank publishes its K/V
block, positions and sequence ids once in CUDA-IPC symmetric memory; at step ``s`` a rank pulls the block of rank
``rank - s`` straight from its owner over NVLink (any-to-any through NVSwitch, no dependency chain between steps) on a
copy stream while the previous block is computed. In backward each dK/dV contribution is pushed once into the slot the
owner keeps for the contributing rank, and the owner sums its slots in rank order (deterministic), so the accumulator
never circulates.

The copy kernel never waits on a peer. Barriers (one-element all-reduces, stream-ordered): B after publishing (and
zeroing the gradient slots), C in backward after the pushes. The published block is double-buffered by call parity, which
makes a barrier in front of the publish unnecessary: a rank reaches the publish of call ``n + 2`` only after barrier B of
call ``n + 1``, which every rank enters (in stream order) after its pulls of call ``n``; the gradient slots are recycled
only after barrier C (``utils/flag_protocol.ring_publish`` checks both over every interleaving).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from . import _lib, comm

_ALIGN = 256


def enabled() -> bool:
    return os.environ.get("MALTOS_B200_RING_PEER", "1") == "1"


def peer_ring_for(group, q: torch.Tensor, participants) -> "PeerRing | None":
    if not enabled() or participants is not None or not q.is_cuda:
        return None
    ctx = comm.context_for(group)
    if ctx is None:
        return None
    ring = getattr(ctx, "_peer_ring", None)
    if ring is None:
        ring = ctx._peer_ring = PeerRing(ctx, group)
    return ring


def _copy(dst_ptr: int, src_ptr: int, nbytes: int, max_blocks: int = 0) -> None:
    _lib.check(_lib.lib().mb_peer_copy(_lib.c_void_p(dst_ptr), _lib.c_void_p(src_ptr), _lib.c_ll(nbytes), _lib.c_int(max_blocks),
                                       _lib.stream_ptr()), "mb_peer_copy")


class PeerRing:
    #: blocks of the pull kernel: a fraction of the GPU, so that it shares it with the attention kernel it overlaps; remote
    #: READS need many loads in flight (measured: 32 blocks 243 GB/s, 64 blocks 470 GB/s, 592 blocks 735 GB/s)
    PULL_BLOCKS = 96

    def __init__(self, ctx, group) -> None:
        self.ctx, self.group = ctx, group
        self.rank, self.world = ctx.rank, ctx.world
        self.copy_stream = torch.cuda.Stream(device=ctx.device)
        self._token = torch.zeros(1, dtype=torch.float32, device=ctx.device)
        self._calls = 0          # publishes so far; its parity picks the half of the published buffer (same on every rank)

    def barrier(self) -> None:
        dist.all_reduce(self._token, group=self.group)

    # ------------------------------------------------------------------ layout of the published block
    @staticmethod
    def _layout(tensors):
        offs, at = [], 0
        for t in tensors:
            offs.append(at)
            at += (t.numel() * t.element_size() + _ALIGN - 1) // _ALIGN * _ALIGN
        return offs, at

    def publish(self, tensors, *, grad_slots_like=None):
        """Collective. Copies ``tensors`` (same shapes on every rank) into this rank's published block; with
        ``grad_slots_like`` also zeroes ``world`` fp32 slots shaped like those tensors. Returns the layout."""
        tensors = [t.contiguous() for t in tensors]
        offs, total = self._layout(tensors)
        sb = self.ctx.ensure_buffer("ring_kv", 2 * total)
        half = sb.nbytes // 2 // _ALIGN * _ALIGN           # from the buffer's size: equal on every rank, stable while it lives
        base = (self._calls & 1) * half
        self._calls += 1
        offs = [base + o for o in offs]
        slots = None
        if grad_slots_like is not None:
            sizes = [t.numel() * 4 for t in grad_slots_like]
            g_offs, at = [], 0
            for n in sizes:
                g_offs.append(at)
                at += (n + _ALIGN - 1) // _ALIGN * _ALIGN
            g_total = at
            gsb = self.ctx.ensure_buffer("ring_dkv", g_total * self.world)
            slots = (gsb, g_offs, g_total)
        for t, o in zip(tensors, offs):
            _copy(sb.local_ptr + o, t.data_ptr(), t.numel() * t.element_size())
        if slots is not None:
            gsb, _, g_total = slots
            gsb.local_tensor(torch.uint8, g_total * self.world, self.ctx.device).zero_()
        self.barrier()                                                                    # B
        return (sb, offs, total, [(t.shape, t.dtype) for t in tensors], base), slots

    def pull(self, layout, owner: int):
        """Starts fetching ``owner``'s published block on the copy stream; returns ``(views, event)``."""
        sb, offs, total, metas, base = layout
        main = torch.cuda.current_stream()
        stage = torch.empty(total, dtype=torch.uint8, device=self.ctx.device)
        self.copy_stream.wait_stream(main)               # the staging memory may have been in use on the main stream
        with torch.cuda.stream(self.copy_stream):
            _copy(stage.data_ptr(), sb.peer_ptrs[owner] + base, total, self.PULL_BLOCKS)
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        stage.record_stream(self.copy_stream)
        views = []
        for o, (shape, dtype) in zip((o - base for o in offs), metas):
            n = 1
            for d in shape:
                n *= d
            nbytes = n * torch.empty((), dtype=dtype).element_size()
            views.append(stage[o:o + nbytes].view(dtype).view(shape))
        return views, ev

    def push_grads(self, slots, owner: int, grads) -> None:
        """Stores this rank's fp32 contributions for ``owner``'s block into the slot ``owner`` keeps for this rank."""
        gsb, g_offs, g_total = slots
        base = gsb.peer_ptrs[owner] + self.rank * g_total
        for g, o in zip(grads, g_offs):
            g = g.to(torch.float32).contiguous()
            _copy(base + o, g.data_ptr(), g.numel() * 4)
            g.record_stream(torch.cuda.current_stream())

    def reduce_grads(self, slots, shapes):
        """Collective (barrier C), then the sum of this rank's slots in rank order."""
        gsb, g_offs, g_total = slots
        self.barrier()                                                                    # C
        flat = gsb.local_tensor(torch.float32, g_total * self.world // 4, self.ctx.device).view(self.world, g_total // 4)
        out = []
        for shape, o in zip(shapes, g_offs):
            n = 1
            for d in shape:
                n *= d
            out.append(flat[:, o // 4:o // 4 + n].sum(0).view(shape))
        return out

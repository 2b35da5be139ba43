"""Symmetric-memory context of a process group on one node.

Every rank allocates the same named buffers (``csrc/symm.cu``: ``cudaMalloc`` + CUDA IPC handle), the handles are
exchanged with ``all_gather_object`` over the group, and each rank maps all peers' buffers. A context owns

* a signal pad per rank (zero-initialised ``uint32`` words) that peers write sequence numbers into,
* named data buffers, grown collectively when an op needs more room (all ranks run the same op sequence, so they reach
  the same decision at the same call),
* a call counter used as the sequence number of the flag protocols.

Kernels receive the peers' base addresses as an ``int64`` device tensor. All waits on these flags inside kernels are
bounded; a wait that runs out raises the device status bit "peer flag wait timed out" instead of hanging the GPU.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from . import _lib

PAD_WORDS = 1024   # uint32 words per rank


@dataclass
class SymmetricBuffer:
    name: str
    nbytes: int
    local_ptr: int
    peer_ptrs: list[int]                 # index = rank in group; own entry = local_ptr
    table: torch.Tensor = None           # int64 [world] on device, for kernels
    opened: list[int] = field(default_factory=list)

    def local_tensor(self, dtype: torch.dtype, numel: int, device) -> torch.Tensor:
        """A tensor view of (the head of) the local buffer. The memory is owned by the context, not by torch."""
        itemsize = torch.empty((), dtype=dtype).element_size()
        if numel * itemsize > self.nbytes:
            raise ValueError(f"symmetric buffer {self.name}: view of {numel * itemsize} bytes exceeds {self.nbytes}")
        return _tensor_from_ptr(self.local_ptr, numel, dtype, device)


#: buffers whose every consumed byte is written by a transfer of the same call: safe to poison
_POISONABLE = ("sp_partial", "sp_publish", "sp_scatter", "sp_gather", "ring_kv")


def poison_wanted(name: str) -> bool:
    """``MALTOS_B200_POISON=1`` fills the transfer buffers of the sequence-parallel collectives and of the ring exchange
    with NaN patterns at allocation (race / stale-read detection; off by default). Signal pads, gradient slots that are
    summed, sharded-optimizer buffers and the expert slots (whose unused rows are read and multiplied by zero) are left
    zeroed."""
    import os

    return os.environ.get("MALTOS_B200_POISON", "0") == "1" and name in _POISONABLE


class _CudaArrayInterface:
    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _tensor_from_ptr(ptr: int, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
    itemsize = torch.empty((), dtype=dtype).element_size()
    raw = torch.as_tensor(_CudaArrayInterface(ptr, numel * itemsize), device=device)
    return raw.view(dtype)


class SymmetricContext:
    def __init__(self, group, rank: int, world: int, device: torch.device) -> None:
        self.group, self.rank, self.world, self.device = group, rank, world, device
        self.buffers: dict[str, SymmetricBuffer] = {}
        self.seq: dict[str, int] = {}
        self.pad: SymmetricBuffer | None = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def create(cls, group) -> "SymmetricContext":
        import socket

        rank, world = dist.get_rank(group), dist.get_world_size(group)
        device = torch.device("cuda", torch.cuda.current_device())
        info = [None] * world
        dist.all_gather_object(info, (socket.gethostname(), device.index), group=group)
        if len({h for h, _ in info}) != 1:
            raise RuntimeError("symmetric memory needs all ranks of the group on one node")
        lib = _lib.lib()
        for _, peer_dev in info:
            if peer_dev != device.index and not lib.mb_can_access_peer(ctypes.c_int(device.index), ctypes.c_int(peer_dev)):
                raise RuntimeError(f"no peer access from device {device.index} to device {peer_dev}")
        ctx = cls(group, rank, world, device)
        ctx.pad = ctx._allocate("signal_pad", PAD_WORDS * 4)
        return ctx

    def _allocate(self, name: str, nbytes: int) -> SymmetricBuffer:
        lib = _lib.lib()
        nbytes = (nbytes + 255) // 256 * 256
        ptr = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        _lib.check(lib.mb_symm_alloc(ctypes.c_size_t(nbytes), ctypes.byref(ptr), handle), "mb_symm_alloc")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=self.group)
        peers, opened = [], []
        for r, h in enumerate(handles):
            if r == self.rank:
                peers.append(int(ptr.value))
                continue
            p = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            _lib.check(lib.mb_symm_open(buf, ctypes.byref(p)), "mb_symm_open")
            peers.append(int(p.value))
            opened.append(int(p.value))
        if poison_wanted(name):
            # debug aid: transfer buffers start as 0xFF bytes (NaN as bf16 / fp32), so a read of rows that no peer has
            # written yet shows up as NaN in the result instead of as plausible zeros
            _tensor_from_ptr(int(ptr.value), nbytes, torch.uint8, self.device).fill_(0xFF)
            torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        table = torch.tensor(peers, dtype=torch.int64, device=self.device)
        sb = SymmetricBuffer(name=name, nbytes=nbytes, local_ptr=int(ptr.value), peer_ptrs=peers, table=table, opened=opened)
        self.buffers[name] = sb
        return sb

    def ensure_buffer(self, name: str, nbytes: int) -> SymmetricBuffer:
        """Collective: returns the named buffer with at least ``nbytes`` (every rank must call with the same sizes)."""
        cur = self.buffers.get(name)
        if cur is not None and cur.nbytes >= nbytes:
            return cur
        if cur is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
            self._release(cur)
        return self._allocate(name, nbytes)

    def _release(self, sb: SymmetricBuffer) -> None:
        lib = _lib.lib()
        for p in sb.opened:
            lib.mb_symm_close(ctypes.c_void_p(p))
        lib.mb_symm_free(ctypes.c_void_p(sb.local_ptr))
        self.buffers.pop(sb.name, None)

    def next_seq(self, protocol: str = "gather") -> int:
        """Next call number of one flag protocol (each fused op family counts its own calls, starting at 1)."""
        self.seq[protocol] = self.seq.get(protocol, 0) + 1
        return self.seq[protocol]

    def close(self) -> None:
        if not self.buffers:
            return
        torch.cuda.synchronize(self.device)
        try:
            dist.barrier(group=self.group)
        except Exception:
            pass
        for sb in list(self.buffers.values()):
            self._release(sb)

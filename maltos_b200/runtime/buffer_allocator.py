"""Process-wide pool of communication/staging buffers.

Policies (names follow the reference's ``runtime/buffer_allocator.py:9-256``):
  * ``PINNED``     - one persistent buffer per ``(key, device, shape, dtype)``; "pinned" means *kept*, not page-locked.
  * ``CACHEABLE`` / ``TEMPORARY`` - sub-allocated from byte slabs (4 MiB minimum, 256-byte granularity) with a
    first-fit free list whose neighbours are merged on release.
Slabs are raw byte storages shared by all dtypes of a device, sized for the 180 GB HBM of a B200: large requests
get their own slab, nothing is ever returned to the CUDA allocator until ``clear``.
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass, field
from enum import Enum

import torch

ALIGN_BYTES = 256
MIN_SLAB_BYTES = 4 << 20


class BufferPolicy(str, Enum):
    PINNED = "pinned"
    CACHEABLE = "cacheable"
    TEMPORARY = "temporary"


@dataclass
class BufferHandle:
    tensor: torch.Tensor
    policy: BufferPolicy
    pool_key: tuple | None = None
    slab_index: int | None = None
    start: int = 0          # byte offset inside the slab
    alloc_numel: int = 0    # bytes reserved (multiple of ALIGN_BYTES)
    released: bool = False


class _Slab:
    def __init__(self, nbytes: int, device: torch.device) -> None:
        self.storage = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.free: list[tuple[int, int]] = [(0, nbytes)]  # sorted (offset, length)

    def take(self, nbytes: int) -> int | None:
        for i, (off, length) in enumerate(self.free):
            if length >= nbytes:
                if length == nbytes:
                    self.free.pop(i)
                else:
                    self.free[i] = (off + nbytes, length - nbytes)
                return off
        return None

    def give_back(self, off: int, nbytes: int) -> None:
        i = bisect.bisect_left(self.free, (off, 0))
        self.free.insert(i, (off, nbytes))
        merged: list[tuple[int, int]] = []
        for o, l in self.free:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + l)
            else:
                merged.append((o, l))
        self.free = merged


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


@dataclass
class BufferPool:
    _persistent: dict[tuple, BufferHandle] = field(default_factory=dict)
    _slabs: dict[tuple, list[_Slab]] = field(default_factory=dict)

    def acquire(self, *, shape, dtype: torch.dtype, device, policy, key: str | None = None) -> BufferHandle:
        policy = BufferPolicy(policy)
        device = torch.device(device)
        shape = tuple(int(s) for s in shape)
        if policy is BufferPolicy.PINNED:
            if key is None:
                raise ValueError("pinned buffers require a key")
            ident = (key, device, shape, dtype)
            handle = self._persistent.get(ident)
            if handle is None:
                handle = BufferHandle(tensor=torch.empty(shape, dtype=dtype, device=device), policy=policy)
                self._persistent[ident] = handle
            return handle
        if key is not None:
            raise ValueError(f"{policy.value} buffers do not accept a key")
        itemsize = torch.empty((), dtype=dtype).element_size()
        want = max(_round_up(_numel(shape) * itemsize, ALIGN_BYTES), ALIGN_BYTES)
        pool_key = (policy, device)
        slabs = self._slabs.setdefault(pool_key, [])
        for idx, slab in enumerate(slabs):
            off = slab.take(want)
            if off is not None:
                return self._handle(slab, idx, off, want, shape, dtype, policy, pool_key)
        slab = _Slab(max(want, MIN_SLAB_BYTES), device)
        slabs.append(slab)
        off = slab.take(want)
        return self._handle(slab, len(slabs) - 1, off, want, shape, dtype, policy, pool_key)

    @staticmethod
    def _handle(slab, idx, off, want, shape, dtype, policy, pool_key) -> BufferHandle:
        itemsize = torch.empty((), dtype=dtype).element_size()
        view = slab.storage.narrow(0, off, _numel(shape) * itemsize).view(dtype).view(shape)
        return BufferHandle(tensor=view, policy=policy, pool_key=pool_key, slab_index=idx, start=off, alloc_numel=want)

    def release(self, handle: BufferHandle) -> None:
        if handle.policy is BufferPolicy.PINNED:
            return
        if handle.released:
            raise ValueError("buffer handle has already been released")
        if handle.pool_key is None or handle.slab_index is None:
            raise ValueError("buffer handle is missing slab metadata")
        slabs = self._slabs.get(handle.pool_key)
        if slabs is None or handle.slab_index >= len(slabs):
            raise ValueError("buffer handle refers to an unknown slab")
        slabs[handle.slab_index].give_back(handle.start, handle.alloc_numel)
        handle.released = True

    def clear(self) -> None:
        self._persistent.clear()
        self._slabs.clear()

    def reserved_bytes(self) -> int:
        total = sum(s.storage.numel() for slabs in self._slabs.values() for s in slabs)
        total += sum(h.tensor.numel() * h.tensor.element_size() for h in self._persistent.values())
        return total


_GLOBAL_POOL = BufferPool()


def global_buffer_pool() -> BufferPool:
    return _GLOBAL_POOL


def acquire_buffer(*, shape, dtype, device, policy, key: str | None = None) -> BufferHandle:
    return _GLOBAL_POOL.acquire(shape=shape, dtype=dtype, device=device, policy=policy, key=key)


def release_buffer(handle: BufferHandle) -> None:
    _GLOBAL_POOL.release(handle)


def clear_buffer_pool() -> None:
    _GLOBAL_POOL.clear()

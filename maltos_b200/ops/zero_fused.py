"""Peer-memory data paths of the sharded optimizers (``csrc/zero_fused.cu``).

``peer_reduce_shard``: the owner of a shard reads its slice of the flat bf16 gradient bucket from every rank's buffer
over NVLink, sums in fp32, scales, writes / accumulates the shard gradient and adds the squared norm of the result to
a device scalar - one kernel instead of reduce-scatter + scale + accumulate + norm partial
(reference ``runtime/plugins/zero1.py:183-231``, ``zero2.py:262-330``).

``adamw_push``: AdamW on the fp32 master shard with the bf16 result stored into every rank's flat parameter buffer -
one kernel instead of optimizer step + cast + all-gather (reference ``runtime/optim.py:43-104``, ``zero1.py:264-283``).

Both take raw device addresses because the peers' buffers are CUDA-IPC mappings that no tensor owns. Neither kernel
waits on another GPU; callers bracket them with stream-ordered group barriers. The ``*_reference`` functions are the
plain PyTorch restatements used as oracles.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib

OUT_WRITE, OUT_ACCUMULATE = 0, 1


def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = ctypes.c_void_p(int(p))
    return arr


def peer_reduce_shard(src_ptrs, rank: int, numel: int, scale: float, out: torch.Tensor, *, accumulate: bool = False,
                      sumsq: torch.Tensor | None = None) -> None:
    """``out (+)= scale * sum_r bucket_r[shard]``; ``src_ptrs[r]`` = device address of the shard's first bf16 element in
    rank r's bucket. ``out`` is a contiguous bf16 or fp32 tensor of ``numel`` elements; ``sumsq`` an fp64 device scalar
    that receives ``+= ||out||^2``."""
    if out.dtype not in (torch.bfloat16, torch.float32) or not out.is_contiguous() or out.numel() != numel:
        raise ValueError("peer_reduce_shard: out must be a contiguous bf16/fp32 tensor of numel elements")
    if sumsq is not None and (sumsq.dtype != torch.float64 or sumsq.numel() != 1):
        raise ValueError("peer_reduce_shard: sumsq must be a one-element fp64 tensor")
    mode = (3 if accumulate else 0) if out.dtype == torch.bfloat16 else (2 if accumulate else 1)
    _lib.check(_lib.lib().mb_peer_reduce_shard(_ptr_array(src_ptrs), _lib.c_int(len(src_ptrs)), _lib.c_int(rank), _lib.c_ll(numel),
                                               _lib.c_float(scale), _lib.ptr(out), _lib.c_int(mode), _lib.ptr(sumsq), _lib.stream_ptr()),
               "mb_peer_reduce_shard")


def peer_reduce_shard_reference(shards, scale: float, out: torch.Tensor, *, accumulate: bool = False) -> torch.Tensor:
    """Oracle on tensors: ``shards[r]`` is rank r's slice. Returns ``||out||^2`` (fp64)."""
    acc = torch.zeros(out.shape, dtype=torch.float32, device=out.device)
    for s in shards:
        acc += s.to(torch.float32)
    acc *= scale
    if accumulate:
        acc += out.to(torch.float32)
    out.copy_(acc.to(out.dtype))
    return out.double().pow(2).sum()


def adamw_push(master: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, dst_ptrs, *, step: float,
               lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, grad_scale: torch.Tensor | None = None) -> None:
    """One AdamW step on a contiguous fp32 shard; the updated values are stored as bf16 at every address of
    ``dst_ptrs`` (peers' flat parameter buffers first, own buffers last)."""
    for t in (master, exp_avg, exp_avg_sq):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError("adamw_push: master and moments must be contiguous fp32")
    if grad.dtype not in (torch.float32, torch.bfloat16) or not grad.is_contiguous() or grad.numel() != master.numel():
        raise TypeError("adamw_push: grad must be contiguous fp32/bf16 of the shard's size")
    _lib.check(_lib.lib().mb_adamw_push(_lib.ptr(master), _lib.ptr(grad), _lib.c_int(int(grad.dtype == torch.bfloat16)), _lib.ptr(exp_avg),
                                        _lib.ptr(exp_avg_sq), _lib.c_ll(master.numel()), _ptr_array(dst_ptrs), _lib.c_int(len(dst_ptrs)),
                                        _lib.c_float(lr), _lib.c_float(beta1), _lib.c_float(beta2), _lib.c_float(eps),
                                        _lib.c_float(weight_decay), _lib.c_float(1 - beta1 ** step), _lib.c_float(math.sqrt(1 - beta2 ** step)),
                                        _lib.ptr(grad_scale), _lib.stream_ptr()), "mb_adamw_push")


def ring_order(ptrs, rank: int):
    """Peers starting after ``rank`` and wrapping around, the own entry last."""
    world = len(ptrs)
    return [ptrs[(rank + s) % world] for s in range(1, world + 1)]


def peer_gather(out: torch.Tensor, src_ptrs, bytes_each: int) -> None:
    """``out`` (contiguous) receives ``len(src_ptrs)`` pieces of ``bytes_each`` bytes back to back, piece r read from the
    device address ``src_ptrs[r]`` (this GPU's or a peer's memory): a one-sided all-gather without a rendezvous."""
    if not out.is_contiguous() or out.numel() * out.element_size() < len(src_ptrs) * bytes_each:
        raise ValueError("peer_gather: out must be contiguous and hold all pieces")
    _lib.check(_lib.lib().mb_peer_gather(_lib.ptr(out), _ptr_array(src_ptrs), _lib.c_int(len(src_ptrs)), _lib.c_ll(bytes_each),
                                         _lib.stream_ptr()), "mb_peer_gather")


def peer_all_reduce(slice_ptrs, numel: int, dtype: torch.dtype, scale: float) -> None:
    """In-place all-reduce of THIS rank's slice of a flat bucket that every rank keeps in symmetric memory:
    ``slice_ptrs[r]`` = device address of the slice inside rank r's bucket (16-byte aligned), ``numel`` elements of
    ``dtype`` (bf16 or fp32). The sum over ranks times ``scale`` is stored back into every rank's bucket
    (reference ``runtime/plugins/ddp.py:20-203``: ``all_reduce(AVG)``)."""
    if dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"peer_all_reduce: unsupported dtype {dtype}")
    _lib.check(_lib.lib().mb_peer_all_reduce(_ptr_array(slice_ptrs), _lib.c_int(len(slice_ptrs)), _lib.c_ll(numel),
                                             _lib.c_int(int(dtype == torch.bfloat16)), _lib.c_float(scale), _lib.stream_ptr()),
               "mb_peer_all_reduce")

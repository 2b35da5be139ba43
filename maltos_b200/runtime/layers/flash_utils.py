"""Variable-length (packed-document) attention helpers in the ``[B, S, heads, D]`` layout.

Packed rows hold several documents back to back plus tail padding; attention must stay inside a document. This module
runs it as ONE launch of this library's flash kernel over the padded rows (mask rule "causal by row index and same
sequence id": no compaction, no ``cu_seqlens``, no device->host read), and also offers the flat layout helpers
(valid tokens compacted, ``cu_seqlens`` boundaries) that callers of the reference's interface expect. Also the dense
with-LSE block forward/backward used by ring attention. The reference reaches the same results through the flash-attn
package (``runtime/layers/flash_utils.py:87-135,356-563``); that package is not used here.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from maltos_b200.ops.attention import attention, attention_block_backward, attention_block_forward
from maltos_b200.utils.constants import PAD_SEQUENCE_ID



@dataclass(frozen=True)
class VarlenQkvMetadata:
    """Layout of one packed micro-batch, shared by all attention layers."""

    source_version: int
    token_mask: torch.Tensor        # [B, S] bool: not padding
    flat_indices: torch.Tensor      # [n_valid] long: positions of the valid tokens in the flattened [B*S] order
    cu_seqlens: torch.Tensor        # [n_docs + 1] int32
    max_seqlen: int


@dataclass(frozen=True)
class PackedQkv:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    cu_seqlens: torch.Tensor
    max_seqlen: int
    token_mask: torch.Tensor
    flat_indices: torch.Tensor


@dataclass(frozen=True)
class FlashAttnBlockOutput:
    out: torch.Tensor
    lse: torch.Tensor


# ------------------------------------------------------------------------------------------------ availability
def flash_attn_import_error() -> Exception | None:
    """Kept for callers of the reference's interface: the kernels are part of this library, nothing is imported."""
    return None


def flash_attn_is_available() -> bool:
    return True


def flash_attn_fallback_reason(q: torch.Tensor) -> str | None:
    """None when the tcgen05 flash kernels take ``q``; otherwise why the fp32 restatement runs instead."""
    if not q.is_cuda:
        return "the flash kernels require CUDA tensors"
    if q.dtype != torch.bfloat16:
        return f"the flash kernels require bf16 tensors, got {q.dtype}"
    if q.shape[-1] not in (64, 128):
        return f"the flash kernels cover head_dim 64 and 128, got {q.shape[-1]}"
    return None


def flash_attn_block_fallback_reason(q: torch.Tensor) -> str | None:
    """Block (with-LSE) forward/backward is provided by this library's own primitives on every device: never a reason."""
    return None


flash_attn_dense_block_fallback_reason = flash_attn_block_fallback_reason


def flash_attn_block_is_available() -> bool:
    return True


# ------------------------------------------------------------------------------------------------ varlen layout
def _varlen_qkv_metadata(sequence_ids: torch.Tensor) -> VarlenQkvMetadata:
    """Built once per ``sequence_ids`` tensor (cached on the tensor, guarded by its mutation counter): computing the
    integer ``max_seqlen`` needs a device->host read that would otherwise stall every layer."""
    cached = getattr(sequence_ids, "_maltos_varlen_metadata", None)
    if isinstance(cached, VarlenQkvMetadata) and cached.source_version == sequence_ids._version:
        return cached
    valid = sequence_ids != PAD_SEQUENCE_ID
    flat_valid = valid.reshape(-1)
    flat_indices = torch.nonzero(flat_valid).flatten()
    if flat_indices.numel() == 0:
        meta = VarlenQkvMetadata(sequence_ids._version, valid, flat_indices, torch.zeros(1, dtype=torch.int32, device=sequence_ids.device), 0)
    else:
        prev_ids = torch.roll(sequence_ids, 1, dims=1)
        prev_valid = torch.roll(valid, 1, dims=1)
        prev_valid[:, 0] = False
        starts = valid & (~prev_valid | (sequence_ids != prev_ids))     # first token of every document (rows never join)
        doc_of_token = starts.reshape(-1)[flat_valid].to(torch.int64).cumsum(0) - 1
        lengths = torch.bincount(doc_of_token)
        cu = torch.zeros(lengths.numel() + 1, dtype=torch.int32, device=sequence_ids.device)
        cu[1:] = lengths.cumsum(0).to(torch.int32)
        meta = VarlenQkvMetadata(sequence_ids._version, valid, flat_indices, cu, int(lengths.max().item()))
    try:
        sequence_ids._maltos_varlen_metadata = meta
    except AttributeError:
        pass
    return meta


def pack_varlen_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sequence_ids: torch.Tensor) -> PackedQkv:
    """``[B, S, h, D]`` -> ``[n_valid, h, D]`` with document boundaries."""
    meta = _varlen_qkv_metadata(sequence_ids)
    flat = lambda t: t.reshape(-1, t.shape[2], t.shape[3]).index_select(0, meta.flat_indices)   # noqa: E731
    return PackedQkv(flat(q), flat(k), flat(v), meta.cu_seqlens, meta.max_seqlen, meta.token_mask, meta.flat_indices)


def unpack_varlen_output_by_indices(out: torch.Tensor, flat_indices: torch.Tensor, *, batch_size: int, seq_len: int) -> torch.Tensor:
    """``[n_valid, h, D]`` -> zero-padded ``[B, S, h, D]`` (differentiable)."""
    full = out.new_zeros((batch_size * seq_len, out.shape[1], out.shape[2]))
    return full.index_copy(0, flat_indices, out).view(batch_size, seq_len, out.shape[1], out.shape[2])


def unpack_varlen_output(out: torch.Tensor, token_mask: torch.Tensor) -> torch.Tensor:
    return unpack_varlen_output_by_indices(out, torch.nonzero(token_mask.reshape(-1)).flatten(), batch_size=token_mask.shape[0],
                                           seq_len=token_mask.shape[1])


def flash_attn_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sequence_ids: torch.Tensor) -> torch.Tensor:
    """Causal attention inside every document of a packed ``[B, S, h, D]`` batch; padding rows come back as zeros."""
    out = attention(q, k, v, q_sequence_ids=sequence_ids, k_sequence_ids=sequence_ids, causal=True, packed_causal=True)
    return out * (sequence_ids != PAD_SEQUENCE_ID).unsqueeze(-1).unsqueeze(-1).to(out.dtype)


def flash_attn_varlen_segments(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, token_indices: torch.Tensor, cu_seqlens: torch.Tensor,
                               max_seqlen: int) -> torch.Tensor:
    """Attention over independent contiguous documents given as flattened token indices (``[B*S]`` order) and their
    boundaries - a layout-only interface, so callers can cache both per batch. Runs as one masked launch over the rows."""
    if q.dim() != 4 or k.shape != v.shape or q.shape[:2] != k.shape[:2] or q.shape[3] != k.shape[3] or q.shape[2] % k.shape[2]:
        raise ValueError("flash_attn_varlen_segments expects [batch, tokens, heads, dim] Q and native matching K/V")
    if token_indices.dtype != torch.long or cu_seqlens.dtype != torch.int32:
        raise ValueError("token_indices must be int64 and cu_seqlens int32")
    if max_seqlen < 1 or token_indices.numel() == 0:
        return q.new_zeros(q.shape)
    ids = torch.full((q.shape[0] * q.shape[1],), PAD_SEQUENCE_ID, dtype=torch.long, device=q.device)
    doc = torch.bucketize(torch.arange(token_indices.numel(), device=q.device), cu_seqlens[1:].to(torch.long), right=True)
    ids[token_indices] = doc
    return flash_attn_varlen(q, k, v, ids.view(q.shape[0], q.shape[1]))


# ------------------------------------------------------------------------------------------------ dense blocks with LSE
def flash_attn_dense(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Causal attention of one dense block (differentiable)."""
    return attention(q, k, v, causal=True)


def flash_attn_dense_with_lse(q, k, v, *, q_positions, k_positions, q_sequence_ids=None, k_sequence_ids=None, scale=None) -> FlashAttnBlockOutput:
    """One (query block, key block) step of ring attention: output and log-sum-exp, no autograd."""
    out, lse = attention_block_forward(q, k, v, q_positions=q_positions, k_positions=k_positions, q_sequence_ids=q_sequence_ids,
                                       k_sequence_ids=k_sequence_ids, scale=scale)
    return FlashAttnBlockOutput(out, lse)


def flash_attn_dense_backward(q, k, v, out, lse, dout, *, q_positions, k_positions, q_sequence_ids=None, k_sequence_ids=None, scale=None):
    """Block gradients ``(dq, dk, dv)`` given the GLOBAL output and log-sum-exp of the query rows."""
    return attention_block_backward(q, k, v, out, lse, dout, q_positions=q_positions, k_positions=k_positions,
                                    q_sequence_ids=q_sequence_ids, k_sequence_ids=k_sequence_ids, scale=scale)

"""Attention core of the HDP-balanced schedule: every document of the local packed wave attends over its own ring.

The active wave's :class:`ByteScaleHdpLocalLayout` says where each document's tokens sit in the local ``[rows, width]``
batch and which ranks share it. Documents that live on this rank alone are handled by ONE masked local attention call
(their sequence ids keep them apart); each multi-rank document runs ring attention over its member ranks through
point-to-point exchanges inside the one shared HDP group. All ranks walk the documents in the planner's order, so the
exchanges of different documents never cross (reference ``runtime/layers/hdp_attention.py:29-165``).
"""
from __future__ import annotations

from typing import TYPE_CHECKING

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.ops.attention import attention
from maltos_b200.utils.attention_backend import AttentionBackend, validate_attention_backend
from maltos_b200.utils.constants import PAD_SEQUENCE_ID
from maltos_b200.utils.profiling import span

from .attn_masking_utils import canonical_position_ids, canonical_sequence_ids
from .cp_functional import document_ring_plan, dynamic_flash_ring_attention

if TYPE_CHECKING:
    from maltos_b200.parallel.hdp_helper import ByteScaleHdpLocalLayout


def _validate_hdp_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("HDP attention expects q/k/v shaped [batch, tokens, heads, head_dim]")
    if k.shape != v.shape:
        raise ValueError(f"HDP attention K/V shapes must match, got {tuple(k.shape)} and {tuple(v.shape)}")
    if q.size(0) != k.size(0) or q.size(1) != k.size(1) or q.size(3) != k.size(3):
        raise ValueError("HDP attention Q/K/V batch, token, and head-dim sizes must match")
    if k.size(2) < 1 or q.size(2) % k.size(2):
        raise ValueError("HDP attention Q heads must be a positive multiple of native KV heads")


class HdpBalancedAttentionCore(nn.Module):
    """Drop-in ``attn_core`` (``[B, S, h, D]`` layout, native GQA) installed by ``ByteScaleHdpPlugin``."""

    preserves_native_gqa = True
    layout = "bshd"

    def __init__(self, group: dist.ProcessGroup, attention_backend: str = AttentionBackend.EAGER) -> None:
        super().__init__()
        self.group = group
        self.attention_backend = validate_attention_backend(attention_backend)
        self._active_layout: "ByteScaleHdpLocalLayout | None" = None

    def set_active_schedule(self, layout: "ByteScaleHdpLocalLayout") -> None:
        self._active_layout = layout

    def forward(self, q, k, v, position_offset: int = 0, position_ids=None, sequence_ids=None):
        layout = self._active_layout
        if layout is None:
            raise RuntimeError("HdpBalancedAttentionCore requires an active ByteScaleHdpLocalLayout")
        rank = dist.get_rank(self.group)
        if rank != layout.rank:
            raise RuntimeError(f"HDP attention layout rank={layout.rank} does not match process-group rank={rank}")
        if not layout.documents:   # dummy wave: keep q, k, v in the graph so that every parameter still gets a (zero) gradient
            return q * 0 + (k.sum() + v.sum()) * 0
        _validate_hdp_qkv(q, k, v)
        B, S = q.shape[:2]
        if B != layout.packed_rows:
            raise ValueError("HDP attention batch rows must equal local packed rows")
        pos = canonical_position_ids(position_ids, batch_size=B, seq_len=S, position_offset=position_offset, device=q.device)
        seq = canonical_sequence_ids(sequence_ids, batch_size=B, seq_len=S, device=q.device)
        with span("maltos::hdp_balanced.attention"):
            out = torch.zeros_like(q)
            local_docs = [d for d in layout.documents if len(d.participant_ranks) == 1]
            if local_docs:
                out = out + self._local_documents(q, k, v, pos, seq, layout, local_docs)
            for doc in layout.documents:
                if len(doc.participant_ranks) == 1:
                    continue
                rows, cols = slice(doc.local_row, doc.local_row + 1), slice(doc.local_start, doc.local_end)
                doc_seq = seq[rows, cols] if seq is not None else None
                cache_key = ("ring", str(q.device), doc.document_id)
                plan = layout.attention_metadata_cache.get(cache_key)
                if plan is None:      # host-side knowledge of the document's ring, shared by all layers of the wave
                    plan = document_ring_plan(sequence_length=doc.sequence_length, padded_length=doc.padded_length,
                                              local_length=doc.local_end - doc.local_start, ring_size=len(doc.participant_ranks))
                piece = dynamic_flash_ring_attention(q[rows, cols], k[rows, cols], v[rows, cols], positions=pos[rows, cols],
                                                     sequence_ids=doc_seq, group=self.group, participant_ranks=doc.participant_ranks,
                                                     module_id=id(self), partition_tokens=layout.partition_tokens,
                                                     metadata_cache=layout.attention_metadata_cache, metadata_cache_key=cache_key, plan=plan)
                out = out + _scatter_columns(piece, B, S, doc.local_row, doc.local_start)
            return out

    @staticmethod
    def _local_documents(q, k, v, pos, seq, layout, docs):
        """One masked attention over the whole local batch restricted to the single-rank documents: tokens of other
        documents are marked as padding, so they neither see nor are seen."""
        key = ("local_only_mask", str(q.device))
        keep = layout.attention_metadata_cache.get(key)
        if keep is None:
            keep = torch.zeros(q.shape[:2], dtype=torch.bool, device=q.device)
            for d in docs:
                keep[d.local_row, d.local_start:d.local_end] = True
            layout.attention_metadata_cache[key] = keep
        ids = seq if seq is not None else torch.zeros(q.shape[:2], dtype=torch.long, device=q.device)
        ids = torch.where(keep, ids, torch.full_like(ids, PAD_SEQUENCE_ID))
        # order inside a row decides causality; document ids decide who may look at whom
        order = torch.arange(q.shape[1], device=q.device).unsqueeze(0).expand(q.shape[0], -1)
        res = attention(q, k, v, q_positions=order, k_positions=order, q_sequence_ids=ids, k_sequence_ids=ids)
        return res * keep.unsqueeze(-1).unsqueeze(-1).to(res.dtype)


def _scatter_columns(piece: torch.Tensor, rows: int, width: int, row: int, start: int) -> torch.Tensor:
    """``piece [1, L, h, D]`` placed at ``(row, start)`` of a zero ``[rows, width, h, D]`` tensor (differentiable)."""
    pad_cols = torch.nn.functional.pad(piece, (0, 0, 0, 0, start, width - start - piece.shape[1]))
    return torch.nn.functional.pad(pad_cols, (0, 0, 0, 0, 0, 0, row, rows - row - 1))

"""Attention core in ``[B, S, heads, D]`` layout with native GQA (no ``repeat_interleave`` of K/V, unlike the
reference's ``models/llama.py:145-148``) and one general mask rule that covers dense causal, packed documents and
context-parallel blocks:

    key j is visible to query i  <=>  k_pos[j] <= q_pos[i]  and  k_seq[j] == q_seq[i]  and  k_seq[j] != PAD

Positions / sequence ids default to ``arange`` / one document. On CUDA bf16 the tcgen05 flash kernels in
``csrc/flash_attn.cu`` run (forward returns the log-sum-exp so that ring attention can merge blocks); elsewhere an
fp32 eager restatement is used, which is also the oracle of the kernel tests.
"""
from __future__ import annotations

import math

import torch

from maltos_b200.utils.constants import PAD_SEQUENCE_ID

from . import _lib


def build_visibility_mask(q_positions, k_positions, q_sequence_ids=None, k_sequence_ids=None) -> torch.Tensor:
    """Boolean ``[B, Sq, Sk]`` mask of the rule above."""
    mask = k_positions.unsqueeze(1) <= q_positions.unsqueeze(2)
    if q_sequence_ids is not None and k_sequence_ids is not None:
        same = q_sequence_ids.unsqueeze(2) == k_sequence_ids.unsqueeze(1)
        mask = mask & same & (k_sequence_ids != PAD_SEQUENCE_ID).unsqueeze(1)
    return mask


def attention_reference(q, k, v, *, q_positions=None, k_positions=None, q_sequence_ids=None, k_sequence_ids=None,
                        causal: bool = True, scale: float | None = None, return_lse: bool = False):
    """fp32 eager attention. q ``[B,Sq,hq,D]``, k/v ``[B,Sk,hkv,D]`` -> ``[B,Sq,hq,D]`` (and ``lse [B,hq,Sq]``)."""
    B, Sq, hq, D = q.shape
    Sk, hkv = k.shape[1], k.shape[2]
    g = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3).reshape(B, hkv, g, Sq, D)
    kf = k.float().permute(0, 2, 1, 3).unsqueeze(2)
    vf = v.float().permute(0, 2, 1, 3).unsqueeze(2)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale  # [B,hkv,g,Sq,Sk]
    if q_positions is None and causal:
        q_positions = torch.arange(Sk - Sq, Sk, device=q.device).unsqueeze(0).expand(B, Sq)
        k_positions = torch.arange(Sk, device=q.device).unsqueeze(0).expand(B, Sk)
    if q_positions is not None:
        mask = build_visibility_mask(q_positions, k_positions, q_sequence_ids, k_sequence_ids)
        scores = scores.masked_fill(~mask.view(B, 1, 1, Sq, Sk), float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    probs = torch.exp(scores - lse.unsqueeze(-1))
    probs = torch.nan_to_num(probs, nan=0.0)  # rows with no visible key
    out = torch.matmul(probs, vf).reshape(B, hq, Sq, D).permute(0, 2, 1, 3).to(q.dtype)
    if return_lse:
        return out, lse.reshape(B, hq, Sq)
    return out


def _kernel_eligible(q, k, v) -> bool:
    return (_lib.use_kernels(q) and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
            and q.shape[-1] in (64, 128))


def attention(q, k, v, *, q_positions=None, k_positions=None, q_sequence_ids=None, k_sequence_ids=None,
              causal: bool = True, scale: float | None = None, return_lse: bool = False, packed_causal: bool = False):
    """General masked attention (see module docstring). Differentiable. ``packed_causal``: causality follows the index
    inside the row (positions are ignored) and documents are separated by their sequence ids."""
    if _kernel_eligible(q, k, v):
        from .flash_attn import flash_attention

        return flash_attention(q, k, v, q_positions=q_positions, k_positions=k_positions, q_sequence_ids=q_sequence_ids,
                               k_sequence_ids=k_sequence_ids, causal=causal, scale=scale, return_lse=return_lse,
                               packed_causal=packed_causal)
    if packed_causal or (q_positions is None and q_sequence_ids is not None):
        B, Sq, Sk = q.shape[0], q.shape[1], k.shape[1]
        q_positions = torch.arange(Sk - Sq, Sk, device=q.device).unsqueeze(0).expand(B, Sq)
        k_positions = torch.arange(Sk, device=q.device).unsqueeze(0).expand(B, Sk)
    return attention_reference(q, k, v, q_positions=q_positions, k_positions=k_positions, q_sequence_ids=q_sequence_ids,
                               k_sequence_ids=k_sequence_ids, causal=causal, scale=scale, return_lse=return_lse)


def causal_attention(q, k, v, *, position_ids=None, sequence_ids=None, scale: float | None = None):
    """Self-attention over one local sequence: causal, and document-local when ``sequence_ids`` is given.

    Inside a packed row positions restart per document, so the row index decides causality and the document id the block
    structure; on the GPU that is ONE launch of the flash kernel over the padded rows (no compaction, no host sync)."""
    if sequence_ids is None:
        return attention(q, k, v, causal=True, scale=scale)
    return attention(q, k, v, q_sequence_ids=sequence_ids, k_sequence_ids=sequence_ids, causal=True, scale=scale,
                     packed_causal=True)


# ------------------------------------------------------------------------------------------------ block primitives
def attention_block_forward(q, k, v, *, q_positions, k_positions, q_sequence_ids=None, k_sequence_ids=None, scale=None):
    """One (query block, key block) attention WITHOUT autograd: returns ``(out, lse)`` with ``lse = -inf`` and
    ``out = 0`` for rows that see no key. Building block of ring attention; merged with :func:`merge_attention_blocks`.
    ``q_positions=None`` means every key of the block is visible to every query (no mask is evaluated)."""
    with torch.no_grad():
        if _kernel_eligible(q, k, v):
            from .flash_attn import flash_block_forward

            res = flash_block_forward(q, k, v, q_positions, k_positions, q_sequence_ids, k_sequence_ids, scale)
            if res is not None:
                return res
        out, lse = attention_reference(q, k, v, q_positions=q_positions, k_positions=k_positions, q_sequence_ids=q_sequence_ids,
                                       k_sequence_ids=k_sequence_ids, causal=False, scale=scale, return_lse=True)
        return out, lse


def merge_attention_blocks(out_a, lse_a, out_b, lse_b):
    """Combine two partial softmax results over disjoint key sets. ``out [B,S,h,D]`` fp32, ``lse [B,h,S]`` fp32."""
    lse = torch.logaddexp(lse_a, lse_b)
    wa = torch.exp(lse_a - lse).nan_to_num(0.0).permute(0, 2, 1).unsqueeze(-1)
    wb = torch.exp(lse_b - lse).nan_to_num(0.0).permute(0, 2, 1).unsqueeze(-1)
    return out_a * wa + out_b * wb, lse


def attention_block_backward(q, k, v, out, lse, dout, *, q_positions, k_positions, q_sequence_ids=None, k_sequence_ids=None,
                             scale=None):
    """Gradients of one block given the GLOBAL output and log-sum-exp of the query rows (flash-attention backward
    formulation): ``P = exp(S - lse)``, ``dS = P * (dO V^T - rowsum(dO * O))``. Returns fp32 ``(dq, dk, dv)``.
    ``q_positions=None``: every key is visible to every query."""
    with torch.no_grad():
        if _kernel_eligible(q, k, v):
            from .flash_attn import flash_block_backward

            res = flash_block_backward(q, k, v, out, lse, dout, q_positions, k_positions, q_sequence_ids, k_sequence_ids, scale)
            if res is not None:
                return res
        B, Sq, hq, D = q.shape
        Sk, hkv = k.shape[1], k.shape[2]
        g = hq // hkv
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        qf = q.float().permute(0, 2, 1, 3).reshape(B, hkv, g, Sq, D)
        kf = k.float().permute(0, 2, 1, 3).unsqueeze(2)
        vf = v.float().permute(0, 2, 1, 3).unsqueeze(2)
        of = out.float().permute(0, 2, 1, 3).reshape(B, hkv, g, Sq, D)
        dof = dout.float().permute(0, 2, 1, 3).reshape(B, hkv, g, Sq, D)
        scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
        p = torch.exp(scores - lse.float().reshape(B, hkv, g, Sq, 1))
        if q_positions is not None:
            mask = build_visibility_mask(q_positions, k_positions, q_sequence_ids, k_sequence_ids).view(B, 1, 1, Sq, Sk)
            p = p.masked_fill(~mask, 0.0)
        p = p.nan_to_num(0.0)
        dv = torch.matmul(p.transpose(-1, -2), dof).sum(2)
        dp = torch.matmul(dof, vf.transpose(-1, -2))
        delta = (dof * of).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq = torch.matmul(ds, kf).reshape(B, hq, Sq, D).permute(0, 2, 1, 3)
        dk = torch.matmul(ds.transpose(-1, -2), qf).sum(2).permute(0, 2, 1, 3)
        return dq.contiguous(), dk.contiguous(), dv.permute(0, 2, 1, 3).contiguous()

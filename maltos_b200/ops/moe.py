"""Mixture-of-experts token processing on one device.

``moe_experts_forward`` sends every (token, choice) assignment through its expert and sums the gated results:
assignments are sorted by expert once (stable, so capacity order is token order) and each expert runs on a
contiguous slice. The expert count per slice is read on the host (one sync per call) - the expert-parallel layer
uses capacity-bounded buffers instead when a capacity factor is set.
"""
from __future__ import annotations

import torch


def moe_experts_forward(flat: torch.Tensor, expert_idx: torch.Tensor, gate: torch.Tensor, keep: torch.Tensor | None,
                        experts: list) -> torch.Tensor:
    """``flat [N,H]``, ``expert_idx/gate [N,k]``, ``keep [N,k]`` bool or None, ``experts``: callables ``[n,H]->[n,H]``."""
    N, H = flat.shape
    k = expert_idx.shape[1]
    E = len(experts)
    assign_expert = expert_idx.reshape(-1)
    assign_gate = gate.reshape(-1)
    if keep is not None:
        assign_gate = assign_gate * keep.reshape(-1).to(assign_gate.dtype)
        assign_expert = torch.where(keep.reshape(-1), assign_expert, torch.full_like(assign_expert, E))
    token_of = torch.arange(N, device=flat.device).repeat_interleave(k)
    order = torch.argsort(assign_expert, stable=True)
    sorted_tokens = token_of[order]
    counts = torch.bincount(assign_expert, minlength=E + 1)[:E].tolist()
    gathered = flat.index_select(0, sorted_tokens)
    gates_sorted = assign_gate[order].unsqueeze(1).to(flat.dtype)
    out = torch.zeros_like(flat)
    at = 0
    pieces = []
    for e, n in enumerate(counts):
        if n == 0:
            continue
        pieces.append(experts[e](gathered[at:at + n]) * gates_sorted[at:at + n])
        at += n
    if pieces:
        out = out.index_add(0, sorted_tokens[:at], torch.cat(pieces, dim=0))
    return out

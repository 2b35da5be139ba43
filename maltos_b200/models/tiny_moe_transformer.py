"""Tiny decoder whose FFN is a mixture of experts in every layer (reference ``models/tiny_moe_transformer.py:25-311``).

``TopKMoE`` generalises the reference's ``Top1MoE`` (softmax router, top-1, no capacity limit, Switch-style
load-balance loss ``E * sum_e f_e * mean_prob_e``): ``top_k`` and ``capacity_factor`` are optional; with their
defaults it is the reference block. The expert-parallel plugin replaces it with the dispatching version.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from maltos_b200.parallel.specs import ContextParallelSpec, ExpertParallelSpec, PipelineParallelSpec, TpSpParallelSpec
from maltos_b200.runtime.types import LossOutput, PipelineOutput

from .common import Linear, ParsedBatch, lm_logits, lm_loss
from .tiny_transformer import MLP, CausalSelfAttention, RmsNorm, RoPE, tiny_tp_rules


def load_balance_loss(router_logits: torch.Tensor, expert_idx: torch.Tensor) -> torch.Tensor:
    """``E * sum_e (fraction of assignments to e) * (mean router prob of e)``; ``expert_idx`` is ``[N]`` or ``[N,k]``."""
    n_exp = router_logits.shape[-1]
    probs = router_logits.float().softmax(dim=-1)
    counts = torch.bincount(expert_idx.reshape(-1), minlength=n_exp).float()
    frac = counts / max(expert_idx.numel(), 1)
    return n_exp * (frac * probs.mean(dim=0)).sum()


_top1_load_balance_loss = load_balance_loss


def route_tokens(router_logits: torch.Tensor, top_k: int, renormalize: bool = True):
    """softmax -> top-k. Returns ``(expert_idx [N,k], gate [N,k])``; with k=1 the gate is the raw top probability."""
    probs = router_logits.softmax(dim=-1)
    gate, idx = probs.topk(top_k, dim=-1)
    if top_k > 1 and renormalize:
        gate = gate / gate.sum(dim=-1, keepdim=True)
    return idx, gate


def route_and_balance(router_logits: torch.Tensor, top_k: int, *, need_aux: bool):
    """``(expert_idx [N,k], gate [N,k], load-balance loss or None)``. On CUDA one fused router kernel produces the
    selection, the gates and the statistics of the loss; elsewhere the eager helpers above."""
    from maltos_b200.ops.moe_router import _kernel_ok, load_balance_loss_from_stats, route

    if _kernel_ok(router_logits, top_k):
        idx, gate, mean_prob, counts = route(router_logits, top_k, True)
        return idx, gate, (load_balance_loss_from_stats(mean_prob, counts) if need_aux else None)
    idx, gate = route_tokens(router_logits, top_k)
    aux = load_balance_loss(router_logits, idx if top_k > 1 else idx.squeeze(-1)) if need_aux else None
    return idx, gate, aux


def capacity_keep_mask(expert_idx: torch.Tensor, num_experts: int, capacity: int) -> torch.Tensor:
    """True for assignments that fit: per expert, the first ``capacity`` assignments in token order are kept."""
    flat = expert_idx.reshape(-1)
    onehot = torch.nn.functional.one_hot(flat, num_experts)
    slot = (onehot.cumsum(0) * onehot).sum(-1) - 1
    return (slot < capacity).view_as(expert_idx)


class TopKMoE(nn.Module):
    def __init__(self, dim: int, hidden_size: int, num_experts: int, top_k: int = 1, capacity_factor: float | None = None) -> None:
        super().__init__()
        self._dim, self._hidden_size, self._num_experts = dim, hidden_size, num_experts
        self.top_k = top_k
        self.capacity_factor = capacity_factor
        self.router = Linear(dim, num_experts, bias=False)
        self.experts = nn.ModuleList([MLP(dim, hidden_size) for _ in range(num_experts)])

    @property
    def dim(self) -> int:
        return self._dim

    @property
    def hidden_size(self) -> int:
        return self._hidden_size

    @property
    def num_experts(self) -> int:
        return self._num_experts

    def forward(self, x: torch.Tensor, *, return_aux_loss: bool = False):
        from maltos_b200.ops.moe import moe_experts_forward

        B, S, H = x.shape
        flat = x.reshape(-1, H)
        logits = self.router(flat)
        idx, gate, aux = route_and_balance(logits, self.top_k, need_aux=return_aux_loss)
        keep, cap = None, None
        if self.capacity_factor is not None:
            cap = max(1, int(self.capacity_factor * flat.shape[0] * self.top_k / self._num_experts + 0.999999))
            keep = capacity_keep_mask(idx, self._num_experts, cap)
        out = moe_experts_forward(flat, idx, gate, keep, list(self.experts), capacity=cap).view(B, S, H)
        if not return_aux_loss:
            return out
        return out, aux


Top1MoE = TopKMoE


class MoETransformerBlock(nn.Module):
    def __init__(self, dim, n_heads, n_kv_heads, hidden_size, eps, num_experts, attention_backend: str = "eager",
                 top_k: int = 1, capacity_factor: float | None = None, apply_rope: bool = False):
        super().__init__()
        self.attn = CausalSelfAttention(dim, n_heads, n_kv_heads, attention_backend=attention_backend, apply_rope=apply_rope)
        self.norm1 = RmsNorm(dim, eps)
        self.moe = TopKMoE(dim, hidden_size, num_experts, top_k=top_k, capacity_factor=capacity_factor)
        self.norm2 = RmsNorm(dim, eps)

    def forward(self, x, cos=None, sin=None, position_offset: int = 0, position_ids=None, sequence_ids=None, return_aux_loss: bool = False):
        x = self.attn(self.norm1(x), cos, sin, position_offset=position_offset, position_ids=position_ids, sequence_ids=sequence_ids) + x
        out = self.moe(self.norm2(x), return_aux_loss=return_aux_loss)
        if not return_aux_loss:
            return out + x
        y, aux = out
        return y + x, aux


def _metric(t: torch.Tensor):
    """Metrics stay on the device (no host sync per micro-step); the runtime reads them once per optimizer step."""
    return t.detach().float()


class TinyMoETransformer(nn.Module):
    handles_sequence_parallel_loss = True

    def __init__(self, dim, n_heads, n_kv_heads, hidden_size, eps, n_layers, vocab_size, max_seq_len, num_experts,
                 moe_aux_loss_coef: float = 0.0, attention_backend: str = "eager", top_k: int = 1,
                 capacity_factor: float | None = None, apply_rope: bool = False):
        super().__init__()
        if moe_aux_loss_coef < 0:
            raise ValueError("moe_aux_loss_coef must be >= 0")
        self.embed = nn.Embedding(vocab_size, dim)
        self.rope = RoPE(dim // n_heads, max_seq_len)
        self.layers = nn.ModuleList([
            MoETransformerBlock(dim, n_heads, n_kv_heads, hidden_size, eps, num_experts, attention_backend=attention_backend,
                                top_k=top_k, capacity_factor=capacity_factor, apply_rope=apply_rope)
            for _ in range(n_layers)
        ])
        self.norm = RmsNorm(dim, eps)
        self.lm_head = Linear(dim, vocab_size, bias=False)
        self.moe_aux_loss_coef = float(moe_aux_loss_coef)
        self._total_moe_layers = n_layers

    def forward(self, batch):
        b = ParsedBatch(batch)
        if b.hidden_states is not None:
            x = b.hidden_states
        else:
            if b.input_ids is None:
                raise ValueError("TinyMoETransformer requires input_ids or hidden_states")
            if self.embed is None:
                raise ValueError("TinyMoETransformer PP non-first stage requires hidden_states input")
            x = self.embed(b.input_ids)
        cos, sin = self.rope.cos.float(), self.rope.sin.float()
        want_aux = self.moe_aux_loss_coef > 0
        aux_terms: list[torch.Tensor] = []
        for layer in self.layers:
            out = layer(x, cos, sin, position_offset=b.position_offset, position_ids=b.position_ids,
                        sequence_ids=b.sequence_ids, return_aux_loss=want_aux)
            if want_aux and isinstance(out, tuple):   # identity layers of other PP stages return a bare tensor
                x, aux = out
                aux_terms.append(aux)
            else:
                x = out
        if want_aux:
            balance = torch.stack(aux_terms).sum() / float(self._total_moe_layers) if aux_terms else x.new_zeros((), dtype=torch.float32)
            aux_loss = self.moe_aux_loss_coef * balance
            if b.aux_loss_weight is not None:       # this rank sees 1 / cp of every sequence and the gradients are summed
                aux_loss = aux_loss * float(b.aux_loss_weight)
        if self.norm is None or self.lm_head is None:
            return PipelineOutput(activation=x, auxiliary_loss=aux_loss) if want_aux else x
        h = self.norm(x)
        if b.labels is None:
            return lm_logits(h, self.lm_head)
        if b.input_ids is not None and b.labels.shape != b.input_ids.shape:
            raise ValueError(f"labels shape must match input_ids shape, got {b.labels.shape} vs {b.input_ids.shape}")
        ce = lm_loss(h, self.lm_head, b.labels, b.loss_weight, b.loss_scale)
        if not want_aux:
            return ce
        total = ce + aux_loss
        return LossOutput(loss=total, auxiliary_loss=aux_loss,
                          metrics={"loss/ce": _metric(ce), "moe/load_balance_loss": _metric(balance), "loss/total": _metric(total)})

    def expert_parallel_spec(self) -> ExpertParallelSpec:
        return ExpertParallelSpec(moe_paths=[f"layers.{i}.moe" for i in range(len(self.layers))])

    def pipeline_parallel_spec(self) -> PipelineParallelSpec:
        return PipelineParallelSpec(head_layers=["embed"], pipe_layers=["layers"], tail_layers=["norm", "lm_head"])

    def context_parallel_spec(self) -> ContextParallelSpec:
        return ContextParallelSpec(attention_paths=[f"layers.{i}.attn" for i in range(len(self.layers))])


class TinyMoETransformerTp(TinyMoETransformer):
    """TP shards the attention only; experts stay whole."""

    def tpsp_parallelize_spec(self):
        return TpSpParallelSpec(rules=tiny_tp_rules(len(self.layers), sequence_parallel=False, with_mlp=False), tie_rules=[])


class TinyMoETransformerTpSp(TinyMoETransformer):
    def tpsp_parallelize_spec(self):
        rules = tiny_tp_rules(len(self.layers), sequence_parallel=True, with_mlp=False)
        return TpSpParallelSpec(rules=rules, tie_rules=[])

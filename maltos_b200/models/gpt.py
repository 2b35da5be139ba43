"""GPT-2-style tiny decoder: LayerNorm, GELU FFN, learned positional embedding, tied input/output embeddings.
The plumbing benchmark (DP + ZeRO-1 on CPU/gloo, save -> load -> resume) is specified on this architecture; the
reference has no such model, its runtime simply accepts any loss-returning module."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from maltos_b200.ops.attention import causal_attention
from maltos_b200.utils.losses import causal_cross_entropy

from .common import ParsedBatch


@dataclass(frozen=True)
class GPTConfig:
    vocab_size: int = 512
    d_model: int = 64
    n_heads: int = 4
    d_ff: int = 256
    n_layers: int = 2
    max_seq_len: int = 64
    layer_norm_eps: float = 1e-5
    tie_embeddings: bool = True


class GPTAttention(nn.Module):
    def __init__(self, cfg: GPTConfig) -> None:
        super().__init__()
        self.n_heads = cfg.n_heads
        self.head_dim = cfg.d_model // cfg.n_heads
        self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)

    def forward(self, x, position_ids=None, sequence_ids=None):
        B, S, D = x.shape
        q, k, v = self.qkv(x).view(B, S, 3, self.n_heads, self.head_dim).unbind(dim=2)
        o = causal_attention(q, k, v, position_ids=position_ids, sequence_ids=sequence_ids)
        return self.proj(o.reshape(B, S, D))


class GPTBlock(nn.Module):
    def __init__(self, cfg: GPTConfig) -> None:
        super().__init__()
        self.ln1 = nn.LayerNorm(cfg.d_model, eps=cfg.layer_norm_eps)
        self.attn = GPTAttention(cfg)
        self.ln2 = nn.LayerNorm(cfg.d_model, eps=cfg.layer_norm_eps)
        self.fc1 = nn.Linear(cfg.d_model, cfg.d_ff)
        self.fc2 = nn.Linear(cfg.d_ff, cfg.d_model)

    def forward(self, x, position_ids=None, sequence_ids=None):
        x = x + self.attn(self.ln1(x), position_ids, sequence_ids)
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))


class TinyGPT(nn.Module):
    def __init__(self, cfg: GPTConfig = GPTConfig()) -> None:
        super().__init__()
        self.config = cfg
        self.wte = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.wpe = nn.Embedding(cfg.max_seq_len, cfg.d_model)
        self.layers = nn.ModuleList([GPTBlock(cfg) for _ in range(cfg.n_layers)])
        self.ln_f = nn.LayerNorm(cfg.d_model, eps=cfg.layer_norm_eps)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.wte.weight
        self.apply(self._init)

    @staticmethod
    def _init(m: nn.Module) -> None:
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, batch):
        b = ParsedBatch(batch)
        ids = b.input_ids
        B, S = ids.shape
        pos = b.position_ids if b.position_ids is not None else torch.arange(b.position_offset, b.position_offset + S, device=ids.device)
        x = self.wte(ids) + self.wpe(pos)
        for layer in self.layers:
            x = layer(x, b.position_ids, b.sequence_ids)
        logits = self.lm_head(self.ln_f(x))
        if b.labels is None:
            return logits
        return causal_cross_entropy(logits, b.labels)

    def flops_per_token(self) -> float:
        c = self.config
        return float(3 * (c.n_layers * (8 * c.d_model * c.d_model + 4 * c.d_model * c.d_ff + 4 * c.max_seq_len * c.d_model) + 2 * c.d_model * c.vocab_size))

"""Tiny pre-norm decoder used by the distributed test matrix (RmsNorm, GQA attention, SwiGLU MLP, untied head).

Parameter/buffer names follow the reference's ``models/tiny_transformer.py:27-347``. Like the reference, the RoPE
tables are built (persistent buffers ``rope.cos``/``rope.sin``, part of its checkpoints) but NOT applied unless
``apply_rope=True`` - the reference block never uses them, so parity mode has no positional signal.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from maltos_b200.ops.attention import causal_attention
from maltos_b200.ops.norm import rms_norm
from maltos_b200.ops.rope import rope_qkv_split
from maltos_b200.ops.swiglu import swiglu, swiglu_packed
from maltos_b200.parallel.specs import (ContextParallelSpec, PipelineParallelSpec, TpSpParallelSpec, TpSpShardAxis,
                                        TpSpShardRule)

from .common import Linear, ParsedBatch, lm_logits, lm_loss, project_group, project_out


class _LocalCausalAttentionCore(nn.Module):
    preserves_native_gqa = True
    layout = "bshd"

    def __init__(self, attention_backend: str = "eager") -> None:
        super().__init__()
        self.attention_backend = attention_backend

    def forward(self, q, k, v, position_offset: int = 0, position_ids=None, sequence_ids=None):
        return causal_attention(q, k, v, position_ids=position_ids, sequence_ids=sequence_ids)


class CausalSelfAttention(nn.Module):
    handles_sequence_parallel_input = True

    def __init__(self, dim, n_heads, n_kv_heads, attention_backend: str = "eager", apply_rope: bool = False):
        super().__init__()
        self.head_dim = dim // n_heads
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads or n_heads
        self.apply_rope = apply_rope
        self.q_proj = Linear(dim, dim, bias=False)
        self.k_proj = Linear(dim, self.head_dim * self.n_kv_heads, bias=False)
        self.v_proj = Linear(dim, self.head_dim * self.n_kv_heads, bias=False)
        self.o_proj = Linear(dim, dim, bias=False)
        self.attn_core = _LocalCausalAttentionCore(attention_backend)

    def parameter_fusion_groups(self):
        return [[self.q_proj.weight, self.k_proj.weight, self.v_proj.weight]]

    def forward(self, x, cos=None, sin=None, position_offset: int = 0, position_ids=None, sequence_ids=None):
        qkv, offs = project_group(x, (self.q_proj, self.k_proj, self.v_proj))
        hq = self.q_proj.weight.shape[0] // self.head_dim
        hkv = self.k_proj.weight.shape[0] // self.head_dim
        q, k, v = rope_qkv_split(qkv, cos, sin, num_heads=hq, num_kv_heads=hkv, head_dim=self.head_dim,
                                 position_ids=position_ids, position_offset=position_offset, interleaved=True,
                                 offsets=tuple(offs), rotate=self.apply_rope and cos is not None)
        core = self.attn_core
        if getattr(core, "layout", "bhsd") == "bshd":
            o = core(q, k, v, position_offset, position_ids, sequence_ids)
        else:
            o = core(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), position_offset, position_ids, sequence_ids).transpose(1, 2)
        return project_out(o.reshape(*o.shape[:2], hq * self.head_dim), self.o_proj)


class MLP(nn.Module):
    handles_sequence_parallel_input = True

    def __init__(self, dim, hidden_size):
        super().__init__()
        self.gate = Linear(dim, hidden_size, bias=False)
        self.up = Linear(dim, hidden_size, bias=False)
        self.down = Linear(hidden_size, dim, bias=False)

    def parameter_fusion_groups(self):
        return [[self.gate.weight, self.up.weight]]

    def forward(self, x):
        gu, offs = project_group(x, (self.gate, self.up))
        f = self.gate.weight.shape[0]
        act = swiglu_packed(gu) if (offs[0] == 0 and offs[1] == f) else swiglu(gu[..., offs[0]:offs[0] + f], gu[..., offs[1]:offs[1] + f])
        return project_out(act, self.down)


class RmsNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return rms_norm(x, self.weight, self.eps)


class TransformerBlock(nn.Module):
    def __init__(self, dim, n_heads, n_kv_heads, hidden_size, eps, attention_backend: str = "eager", apply_rope: bool = False):
        super().__init__()
        self.attn = CausalSelfAttention(dim, n_heads, n_kv_heads, attention_backend=attention_backend, apply_rope=apply_rope)
        self.norm1 = RmsNorm(dim, eps)
        self.mlp = MLP(dim, hidden_size)
        self.norm2 = RmsNorm(dim, eps)

    def forward(self, x, cos=None, sin=None, position_offset: int = 0, position_ids=None, sequence_ids=None):
        x = self.attn(self.norm1(x), cos, sin, position_offset=position_offset, position_ids=position_ids, sequence_ids=sequence_ids) + x
        return self.mlp(self.norm2(x)) + x


class RoPE(nn.Module):
    """cos/sin tables ``[max_seq_len, head_dim/2]`` stored as persistent buffers (checkpoint entries)."""

    def __init__(self, head_dim, max_seq_len, base=10000):
        super().__init__()
        inv = 1.0 / (base ** (torch.arange(0, head_dim, 2).float() / head_dim))
        freq = torch.outer(torch.arange(max_seq_len).float(), inv)
        self.register_buffer("cos", torch.cos(freq))
        self.register_buffer("sin", torch.sin(freq))

    def forward(self, start=None, end=None, position_ids=None):
        return self.cos, self.sin


class TinyTransformer(nn.Module):
    handles_sequence_parallel_loss = True

    def __init__(self, dim, n_heads, n_kv_heads, hidden_size, eps, n_layers, vocab_size, max_seq_len,
                 attention_backend: str = "eager", apply_rope: bool = False):
        super().__init__()
        self.embed = nn.Embedding(vocab_size, dim)
        self.rope = RoPE(dim // n_heads, max_seq_len)
        self.layers = nn.ModuleList([
            TransformerBlock(dim, n_heads, n_kv_heads, hidden_size, eps, attention_backend=attention_backend, apply_rope=apply_rope)
            for _ in range(n_layers)
        ])
        self.norm = RmsNorm(dim, eps)
        self.lm_head = Linear(dim, vocab_size, bias=False)

    def _embed(self, b: ParsedBatch) -> torch.Tensor:
        if b.hidden_states is not None:
            return b.hidden_states
        if b.input_ids is None:
            raise ValueError(f"{type(self).__name__} requires input_ids or hidden_states")
        if self.embed is None:
            raise ValueError(f"{type(self).__name__} PP non-first stage requires hidden_states input")
        return self.embed(b.input_ids)

    def forward(self, batch):
        b = ParsedBatch(batch)
        x = self._embed(b)
        cos, sin = self.rope.cos.float(), self.rope.sin.float()
        for layer in self.layers:
            x = layer(x, cos, sin, position_offset=b.position_offset, position_ids=b.position_ids, sequence_ids=b.sequence_ids)
        if self.norm is None or self.lm_head is None:
            return x
        h = self.norm(x)
        if b.labels is None:
            return lm_logits(h, self.lm_head)
        if b.input_ids is not None and b.labels.shape != b.input_ids.shape:
            raise ValueError(f"labels shape must match input_ids shape, got {b.labels.shape} vs {b.input_ids.shape}")
        return lm_loss(h, self.lm_head, b.labels, b.loss_weight, b.loss_scale)

    def pipeline_parallel_spec(self) -> PipelineParallelSpec:
        return PipelineParallelSpec(head_layers=["embed"], pipe_layers=["layers"], tail_layers=["norm", "lm_head"])

    def context_parallel_spec(self) -> ContextParallelSpec:
        return ContextParallelSpec(attention_paths=[f"layers.{i}.attn" for i in range(len(self.layers))])

    def compile_spec(self) -> dict[str, list[str]]:
        return {"mlp": [f"layers.{i}.mlp" for i in range(len(self.layers))]}


def tiny_tp_rules(n_layers: int, *, sequence_parallel: bool, with_mlp: bool = True) -> list[TpSpShardRule]:
    post = "reduce_scatter" if sequence_parallel else "all_reduce"
    dim = 1 if sequence_parallel else -1
    rules: list[TpSpShardRule] = []
    if sequence_parallel:
        rules.append(TpSpShardRule("embed", TpSpShardAxis.SEQUENCE, post_comm="scatter", comm_dim=1))
    for i in range(n_layers):
        a, m = f"layers.{i}.attn", f"layers.{i}.mlp"
        if sequence_parallel:
            rules.append(TpSpShardRule(a, TpSpShardAxis.SEQUENCE, pre_comm="all_gather", comm_dim=1))
        rules += [TpSpShardRule(f"{a}.q_proj", TpSpShardAxis.PARAM_OUT), TpSpShardRule(f"{a}.k_proj", TpSpShardAxis.PARAM_OUT),
                  TpSpShardRule(f"{a}.v_proj", TpSpShardAxis.PARAM_OUT),
                  TpSpShardRule(f"{a}.o_proj", TpSpShardAxis.PARAM_IN, post_comm=post, comm_dim=dim)]
        if with_mlp:
            if sequence_parallel:
                rules.append(TpSpShardRule(m, TpSpShardAxis.SEQUENCE, pre_comm="all_gather", comm_dim=1))
            rules += [TpSpShardRule(f"{m}.gate", TpSpShardAxis.PARAM_OUT), TpSpShardRule(f"{m}.up", TpSpShardAxis.PARAM_OUT),
                      TpSpShardRule(f"{m}.down", TpSpShardAxis.PARAM_IN, post_comm=post, comm_dim=dim)]
    if sequence_parallel:
        rules.append(TpSpShardRule("lm_head", TpSpShardAxis.SEQUENCE, pre_comm="all_gather", comm_dim=1))
    return rules


class TinyTransformerTp(TinyTransformer):
    def tpsp_parallelize_spec(self):
        return TpSpParallelSpec(rules=tiny_tp_rules(len(self.layers), sequence_parallel=False), tie_rules=[])


class TinyTransformerTpSp(TinyTransformer):
    def tpsp_parallelize_spec(self):
        return TpSpParallelSpec(rules=tiny_tp_rules(len(self.layers), sequence_parallel=True), tie_rules=[])

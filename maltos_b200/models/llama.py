"""LLaMA-family decoder (pre-norm, RMSNorm, interleaved-pair RoPE, GQA, SwiGLU), parameter names and config fields
as in the reference's ``models/llama.py:30-369`` so that checkpoints and recipes carry over.

What differs is the execution: q/k/v and gate/up are projection *groups* (one GEMM each), RoPE is fused with the
q/k/v split, K/V keep their native GQA head count inside attention, the second residual add is fused into the
post-attention RMSNorm, SwiGLU is one kernel on the packed gate/up output, and the loss head never materialises the
``[tokens, vocab]`` logits in training.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

from maltos_b200.ops.attention import causal_attention
from maltos_b200.ops.norm import add_rms_norm, rms_norm
from maltos_b200.ops.rope import build_rope_cache, rope_qkv_split
from maltos_b200.ops.swiglu import swiglu_packed, swiglu
from maltos_b200.parallel.specs import (ContextParallelSpec, PipelineParallelSpec, TpSpParallelSpec, TpSpShardAxis,
                                        TpSpShardRule)

from .activation_checkpointing import ActivationCheckpointConfig
from .common import Linear, ParsedBatch, lm_logits, lm_loss, project_group, project_out, run_layer


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int = 512
    intermediate_size: int = 2048
    num_hidden_layers: int = 8
    num_attention_heads: int = 8
    num_key_value_heads: int | None = None
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    attention_backend: str = "sdpa_auto"
    activation_checkpointing: ActivationCheckpointConfig = field(default_factory=ActivationCheckpointConfig)

    def __post_init__(self) -> None:
        from maltos_b200.utils.attention_backend import validate_attention_backend

        validate_attention_backend(self.attention_backend)


class LlamaRMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        """``norm(x)``; with ``residual``: ``(norm(x + residual), x + residual)`` in one pass over the row. Going through
        the module call (rather than reading ``weight`` from outside) keeps parameter-sharding hooks in the loop."""
        if residual is None:
            return rms_norm(x, self.weight, self.eps)
        return add_rms_norm(x, residual, self.weight, self.eps)


class LlamaRotaryEmbedding(nn.Module):
    """fp32 cos/sin tables ``[max_pos, head_dim/2]`` (non-persistent buffers, as in the reference)."""

    def __init__(self, head_dim: int, max_position_embeddings: int, base: float) -> None:
        super().__init__()
        cos, sin = build_rope_cache(max_position_embeddings, head_dim, base)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def _apply(self, fn, recurse=True):
        # the tables stay fp32 when the model is cast to bf16: the kernels read fp32 angles
        cos, sin = self.cos, self.sin
        super()._apply(fn, recurse)
        self.cos = cos.to(self.cos.device)
        self.sin = sin.to(self.sin.device)
        return self


class _LlamaAttentionCore(nn.Module):
    """Local attention core; context-parallel plugins replace this module (``attn_core``)."""

    preserves_native_gqa = True
    layout = "bshd"

    def __init__(self, attention_backend: str = "sdpa_auto") -> None:
        super().__init__()
        self.attention_backend = attention_backend

    def forward(self, q, k, v, position_offset: int = 0, position_ids=None, sequence_ids=None):
        return causal_attention(q, k, v, position_ids=position_ids, sequence_ids=sequence_ids)


class LlamaAttention(nn.Module):
    handles_sequence_parallel_input = True
    rope_interleaved = True

    def __init__(self, config: LlamaConfig) -> None:
        super().__init__()
        if config.hidden_size % config.num_attention_heads:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        self.config = config
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_key_value_heads or config.num_attention_heads
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        self.head_dim = config.hidden_size // config.num_attention_heads
        self.rotary_emb = LlamaRotaryEmbedding(self.head_dim, config.max_position_embeddings, config.rope_theta)
        self.q_proj = Linear(config.hidden_size, self.num_heads * self.head_dim, bias=False)
        self.k_proj = Linear(config.hidden_size, self.num_kv_heads * self.head_dim, bias=False)
        self.v_proj = Linear(config.hidden_size, self.num_kv_heads * self.head_dim, bias=False)
        self.o_proj = Linear(config.hidden_size, config.hidden_size, bias=False)
        self.attn_core = _LlamaAttentionCore(config.attention_backend)

    def parameter_fusion_groups(self):
        return [[self.q_proj.weight, self.k_proj.weight, self.v_proj.weight]]

    def forward(self, x, *, position_offset: int = 0, position_ids=None, sequence_ids=None):
        qkv, offs = project_group(x, (self.q_proj, self.k_proj, self.v_proj))
        hq = self.q_proj.weight.shape[0] // self.head_dim      # local head counts (TP shards the heads)
        hkv = self.k_proj.weight.shape[0] // self.head_dim
        q, k, v = rope_qkv_split(qkv, self.rotary_emb.cos, self.rotary_emb.sin, num_heads=hq, num_kv_heads=hkv,
                                 head_dim=self.head_dim, position_ids=position_ids, position_offset=position_offset,
                                 interleaved=self.rope_interleaved, offsets=tuple(offs))
        core = self.attn_core
        if getattr(core, "layout", "bhsd") == "bshd":
            o = core(q, k, v, position_offset, position_ids, sequence_ids)
        else:  # cores written for the [B, heads, S, D] convention
            o = core(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), position_offset, position_ids, sequence_ids).transpose(1, 2)
        return project_out(o.reshape(*o.shape[:2], hq * self.head_dim), self.o_proj)


class LlamaMLP(nn.Module):
    handles_sequence_parallel_input = True

    def __init__(self, config) -> None:
        super().__init__()
        self.gate_proj = Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = Linear(config.intermediate_size, config.hidden_size, bias=False)

    def parameter_fusion_groups(self):
        return [[self.gate_proj.weight, self.up_proj.weight]]

    def forward(self, x):
        gu, offs = project_group(x, (self.gate_proj, self.up_proj))
        f = self.gate_proj.weight.shape[0]
        if offs[0] == 0 and offs[1] == f:
            act = swiglu_packed(gu)
        else:
            act = swiglu(gu[..., offs[0]:offs[0] + f], gu[..., offs[1]:offs[1] + f])
        return project_out(act, self.down_proj)


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config: LlamaConfig) -> None:
        super().__init__()
        self.self_attn = LlamaAttention(config)
        self.mlp = LlamaMLP(config)
        self.input_layernorm = LlamaRMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_attention_layernorm = LlamaRMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward(self, x, position_offset: int = 0, position_ids=None, sequence_ids=None):
        a = self.self_attn(self.input_layernorm(x), position_offset=position_offset, position_ids=position_ids,
                           sequence_ids=sequence_ids)
        y, x = self.post_attention_layernorm(a, residual=x)   # x <- x + a ; y = norm(x), one pass
        return x + self.mlp(y)


class LlamaForCausalLM(nn.Module):
    handles_sequence_parallel_loss = True

    def __init__(self, config: LlamaConfig) -> None:
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([LlamaDecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.norm = LlamaRMSNorm(config.hidden_size, config.rms_norm_eps)
        self.lm_head = Linear(config.hidden_size, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.embed_tokens.weight

    def forward(self, batch):
        b = ParsedBatch(batch)
        if b.hidden_states is not None:
            x = b.hidden_states
        else:
            if b.input_ids is None:
                raise ValueError("LlamaForCausalLM requires input_ids or hidden_states")
            if self.embed_tokens is None:
                raise ValueError("LlamaForCausalLM PP non-first stage requires hidden_states input")
            x = self.embed_tokens(b.input_ids)
        ckpt = self.config.activation_checkpointing
        for i, layer in enumerate(self.layers):
            x = run_layer(layer, x, use_checkpoint=self.training and ckpt.should_checkpoint_layer(i),
                          position_offset=b.position_offset, position_ids=b.position_ids, sequence_ids=b.sequence_ids)
        if self.norm is None or self.lm_head is None:
            return x
        h = self.norm(x)
        if b.labels is None:
            return lm_logits(h, self.lm_head)
        if b.input_ids is not None and b.labels.shape != b.input_ids.shape:
            raise ValueError(f"labels shape must match input_ids shape, got {b.labels.shape} vs {b.input_ids.shape}")
        return lm_loss(h, self.lm_head, b.labels, b.loss_weight, b.loss_scale)

    # ---- parallel declarations
    def pipeline_parallel_spec(self) -> PipelineParallelSpec:
        return PipelineParallelSpec(head_layers=["embed_tokens"], pipe_layers=["layers"], tail_layers=["norm", "lm_head"])

    def context_parallel_spec(self) -> ContextParallelSpec:
        return ContextParallelSpec(attention_paths=[f"layers.{i}.self_attn" for i in range(len(self.layers))])

    def compile_spec(self) -> dict[str, list[str]]:
        return {"mlp": [f"layers.{i}.mlp" for i in range(len(self.layers))]}

    def flops_per_token(self) -> float:
        c = self.config
        per_layer = 8 * c.hidden_size * c.hidden_size + 6 * c.hidden_size * c.intermediate_size + 4 * c.max_position_embeddings * c.hidden_size
        return float(3 * (c.num_hidden_layers * per_layer + 2 * c.hidden_size * c.vocab_size))


def _tp_rules(n_layers: int, post: str) -> list[TpSpShardRule]:
    rules = []
    for i in range(n_layers):
        a, m = f"layers.{i}.self_attn", f"layers.{i}.mlp"
        rules += [
            TpSpShardRule(f"{a}.q_proj", TpSpShardAxis.PARAM_OUT), TpSpShardRule(f"{a}.k_proj", TpSpShardAxis.PARAM_OUT),
            TpSpShardRule(f"{a}.v_proj", TpSpShardAxis.PARAM_OUT), TpSpShardRule(f"{a}.o_proj", TpSpShardAxis.PARAM_IN, post_comm=post),
            TpSpShardRule(f"{m}.gate_proj", TpSpShardAxis.PARAM_OUT), TpSpShardRule(f"{m}.up_proj", TpSpShardAxis.PARAM_OUT),
            TpSpShardRule(f"{m}.down_proj", TpSpShardAxis.PARAM_IN, post_comm=post),
        ]
    return rules


def _sp_rules(n_layers: int, embed: str, attn: str, mlp: str, head: str, inner) -> list[TpSpShardRule]:
    rules = [TpSpShardRule(embed, TpSpShardAxis.SEQUENCE, post_comm="scatter", comm_dim=1)]
    for i in range(n_layers):
        rules.append(TpSpShardRule(f"layers.{i}.{attn}", TpSpShardAxis.SEQUENCE, pre_comm="all_gather", comm_dim=1))
        rules.append(TpSpShardRule(f"layers.{i}.{mlp}", TpSpShardAxis.SEQUENCE, pre_comm="all_gather", comm_dim=1))
        rules += inner(i)
    rules.append(TpSpShardRule(head, TpSpShardAxis.SEQUENCE, pre_comm="all_gather", comm_dim=1))
    return rules


class LlamaForCausalLMTp(LlamaForCausalLM):
    def tpsp_parallelize_spec(self) -> TpSpParallelSpec:
        return TpSpParallelSpec(rules=_tp_rules(len(self.layers), "all_reduce"), tie_rules=[])


class LlamaForCausalLMTpSp(LlamaForCausalLM):
    def tpsp_parallelize_spec(self) -> TpSpParallelSpec:
        per_layer = _tp_rules(len(self.layers), "reduce_scatter")
        n = len(self.layers)
        inner = lambda i: [r if r.shard_axis is TpSpShardAxis.PARAM_OUT else TpSpShardRule(r.module_path, r.shard_axis, post_comm="reduce_scatter", comm_dim=1)
                           for r in per_layer[7 * i:7 * i + 7]]  # noqa: E731
        return TpSpParallelSpec(rules=_sp_rules(n, "embed_tokens", "self_attn", "mlp", "lm_head", inner), tie_rules=[])

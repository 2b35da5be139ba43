"""OLMo-2 decoder: post-sublayer RMSNorm (``x = residual + norm(sublayer(x))``), QK-norm over the whole
``heads*head_dim`` projection (TP-shardable ``DistributedRMSNorm``), rotate-half RoPE, optional attention bias.
Names and config fields follow the reference's ``models/olmo.py:30-372``."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch.nn as nn

from maltos_b200.ops.rope import apply_rope
from maltos_b200.parallel.specs import (ContextParallelSpec, PipelineParallelSpec, TpSpParallelSpec, TpSpShardAxis,
                                        TpSpShardRule)
from maltos_b200.runtime.layers.distributed_rmsnorm import DistributedRMSNorm

from .activation_checkpointing import ActivationCheckpointConfig
from .common import Linear, ParsedBatch, lm_logits, lm_loss, project_group, project_out, run_layer
from .llama import LlamaMLP, LlamaRMSNorm, LlamaRotaryEmbedding, _LlamaAttentionCore


@dataclass(frozen=True)
class OlmoConfig:
    vocab_size: int = 100352
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int | None = None
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-6
    rope_theta: float = 500000.0
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    attention_backend: str = "sdpa_auto"
    activation_checkpointing: ActivationCheckpointConfig = field(default_factory=ActivationCheckpointConfig)

    def __post_init__(self) -> None:
        from maltos_b200.utils.attention_backend import validate_attention_backend

        validate_attention_backend(self.attention_backend)


class OlmoRMSNorm(LlamaRMSNorm):
    pass


class OlmoRotaryEmbedding(LlamaRotaryEmbedding):
    """Same fp32 half-width angle tables; the rotate-half pairing ``(i, i + D/2)`` is chosen at the call site."""


class OlmoAttention(nn.Module):
    handles_sequence_parallel_input = True

    def __init__(self, config: OlmoConfig) -> None:
        super().__init__()
        if config.hidden_size % config.num_attention_heads:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        self.config = config
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_key_value_heads or config.num_attention_heads
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        self.head_dim = config.hidden_size // config.num_attention_heads
        self.rotary_emb = OlmoRotaryEmbedding(self.head_dim, config.max_position_embeddings, config.rope_theta)
        b = config.attention_bias
        self.q_proj = Linear(config.hidden_size, self.num_heads * self.head_dim, bias=b)
        self.k_proj = Linear(config.hidden_size, self.num_kv_heads * self.head_dim, bias=b)
        self.v_proj = Linear(config.hidden_size, self.num_kv_heads * self.head_dim, bias=b)
        self.o_proj = Linear(config.hidden_size, config.hidden_size, bias=b)
        self.q_norm = DistributedRMSNorm(self.num_heads * self.head_dim, config.rms_norm_eps)
        self.k_norm = DistributedRMSNorm(self.num_kv_heads * self.head_dim, config.rms_norm_eps)
        self.attn_core = _LlamaAttentionCore(config.attention_backend)

    def parameter_fusion_groups(self):
        return [[self.q_proj.weight, self.k_proj.weight, self.v_proj.weight]]

    def forward(self, x, *, position_offset: int = 0, position_ids=None, sequence_ids=None, rotary=None):
        qkv, offs = project_group(x, (self.q_proj, self.k_proj, self.v_proj))
        B, S = qkv.shape[:2]
        nq, nk = self.q_proj.weight.shape[0], self.k_proj.weight.shape[0]
        hq, hkv = nq // self.head_dim, nk // self.head_dim
        q = self.q_norm(qkv[..., offs[0]:offs[0] + nq])
        k = self.k_norm(qkv[..., offs[1]:offs[1] + nk])
        v = qkv[..., offs[2]:offs[2] + nk].reshape(B, S, hkv, self.head_dim)
        cos, sin = rotary if rotary is not None else (self.rotary_emb.cos, self.rotary_emb.sin)
        q = apply_rope(q.reshape(B, S, hq, self.head_dim), cos, sin, position_ids=position_ids, position_offset=position_offset, interleaved=False)
        k = apply_rope(k.reshape(B, S, hkv, self.head_dim), cos, sin, position_ids=position_ids, position_offset=position_offset, interleaved=False)
        core = self.attn_core
        if getattr(core, "layout", "bhsd") == "bshd":
            o = core(q, k, v, position_offset, position_ids, sequence_ids)
        else:
            o = core(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), position_offset, position_ids, sequence_ids).transpose(1, 2)
        return project_out(o.reshape(B, S, hq * self.head_dim), self.o_proj)


class OlmoDecoderLayer(nn.Module):
    def __init__(self, config: OlmoConfig) -> None:
        super().__init__()
        self.self_attn = OlmoAttention(config)
        self.mlp = LlamaMLP(config)
        self.post_attention_layernorm = OlmoRMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_feedforward_layernorm = OlmoRMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward(self, x, position_offset: int = 0, position_ids=None, sequence_ids=None, rotary=None):
        x = x + self.post_attention_layernorm(self.self_attn(x, position_offset=position_offset, position_ids=position_ids,
                                                             sequence_ids=sequence_ids, rotary=rotary))
        return x + self.post_feedforward_layernorm(self.mlp(x))


class OlmoForCausalLM(nn.Module):
    handles_sequence_parallel_loss = True

    def __init__(self, config: OlmoConfig) -> None:
        super().__init__()
        self.config = config
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        head_dim = config.hidden_size // config.num_attention_heads
        # one model-level table shared by all layers
        self.rotary_emb = OlmoRotaryEmbedding(head_dim, config.max_position_embeddings, config.rope_theta)
        self.layers = nn.ModuleList([OlmoDecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.norm = OlmoRMSNorm(config.hidden_size, config.rms_norm_eps)
        self.lm_head = Linear(config.hidden_size, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.embed_tokens.weight

    def forward(self, batch):
        b = ParsedBatch(batch)
        if b.hidden_states is not None:
            x = b.hidden_states
        else:
            if b.input_ids is None:
                raise ValueError("OlmoForCausalLM requires input_ids or hidden_states")
            if self.embed_tokens is None:
                raise ValueError("OlmoForCausalLM PP non-first stage requires hidden_states input")
            x = self.embed_tokens(b.input_ids)
        rotary = (self.rotary_emb.cos, self.rotary_emb.sin)
        ckpt = self.config.activation_checkpointing
        for i, layer in enumerate(self.layers):
            x = run_layer(layer, x, use_checkpoint=self.training and ckpt.should_checkpoint_layer(i),
                          position_offset=b.position_offset, position_ids=b.position_ids, sequence_ids=b.sequence_ids, rotary=rotary)
        if self.norm is None or self.lm_head is None:
            return x
        h = self.norm(x)
        if b.labels is None:
            return lm_logits(h, self.lm_head)
        if b.input_ids is not None and b.labels.shape != b.input_ids.shape:
            raise ValueError(f"labels shape must match input_ids shape, got {b.labels.shape} vs {b.input_ids.shape}")
        return lm_loss(h, self.lm_head, b.labels, b.loss_weight, b.loss_scale)

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


def _olmo_rules(n_layers: int, sequence_parallel: bool) -> list[TpSpShardRule]:
    post = "reduce_scatter" if sequence_parallel else "all_reduce"
    dim = 1 if sequence_parallel else -1
    rules: list[TpSpShardRule] = []
    if sequence_parallel:
        rules.append(TpSpShardRule("embed_tokens", TpSpShardAxis.SEQUENCE, post_comm="scatter", comm_dim=1))
    for i in range(n_layers):
        a, m = f"layers.{i}.self_attn", f"layers.{i}.mlp"
        if sequence_parallel:
            rules.append(TpSpShardRule(a, TpSpShardAxis.SEQUENCE, pre_comm="all_gather", comm_dim=1))
        rules += [TpSpShardRule(f"{a}.{n}", TpSpShardAxis.PARAM_OUT) for n in ("q_proj", "k_proj", "v_proj", "q_norm", "k_norm")]
        rules.append(TpSpShardRule(f"{a}.o_proj", TpSpShardAxis.PARAM_IN, post_comm=post, comm_dim=dim))
        if sequence_parallel:
            rules.append(TpSpShardRule(m, TpSpShardAxis.SEQUENCE, pre_comm="all_gather", comm_dim=1))
        rules += [TpSpShardRule(f"{m}.gate_proj", TpSpShardAxis.PARAM_OUT), TpSpShardRule(f"{m}.up_proj", TpSpShardAxis.PARAM_OUT),
                  TpSpShardRule(f"{m}.down_proj", TpSpShardAxis.PARAM_IN, post_comm=post, comm_dim=dim)]
    if sequence_parallel:
        rules.append(TpSpShardRule("lm_head", TpSpShardAxis.SEQUENCE, pre_comm="all_gather", comm_dim=1))
    return rules


class OlmoForCausalLMTp(OlmoForCausalLM):
    def tpsp_parallelize_spec(self) -> TpSpParallelSpec:
        return TpSpParallelSpec(rules=_olmo_rules(len(self.layers), False), tie_rules=[])


class OlmoForCausalLMTpSp(OlmoForCausalLM):
    def tpsp_parallelize_spec(self) -> TpSpParallelSpec:
        return TpSpParallelSpec(rules=_olmo_rules(len(self.layers), True), tie_rules=[])

"""Building blocks shared by the model files: batch unpacking, projection groups that work on plain ``nn.Linear``
and on the tensor-parallel replacements alike, the loss head, checkpointed layer calls.

Model code stays single-device PyTorch: it calls ``project_group`` / ``project_out`` and declares parallel specs;
whether those calls become one local tcgen05 GEMM, or a fused all-gather->GEMM / GEMM->reduce-scatter kernel over
NVLink, is decided by the modules the TP plugins put in place."""
from __future__ import annotations

from typing import Any, Sequence

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from maltos_b200.ops.cross_entropy import linear_cross_entropy
from maltos_b200.ops.gemm import linear
from maltos_b200.ops.grouped import grouped_linear
from maltos_b200.utils.activation_checkpoint import activation_checkpoint_context_fn
from maltos_b200.utils.constants import (AUX_LOSS_WEIGHT_KEY, HIDDEN_STATES_KEY, IGNORE_INDEX, INPUT_IDS_KEY, LABELS_KEY, LOSS_SCALE_KEY, LOSS_WEIGHT_KEY, POSITION_IDS_KEY,
                                         POSITION_OFFSET_KEY, SEQUENCE_IDS_KEY)
from maltos_b200.utils.losses import causal_cross_entropy


class ParsedBatch:
    __slots__ = ("input_ids", "hidden_states", "labels", "position_offset", "position_ids", "sequence_ids", "loss_weight", "aux_loss_weight", "loss_scale")

    def __init__(self, batch: Any) -> None:
        self.hidden_states = self.labels = self.position_ids = self.sequence_ids = self.loss_weight = None
        self.position_offset = 0
        self.aux_loss_weight = self.loss_scale = None
        if isinstance(batch, dict):
            self.input_ids = batch.get(INPUT_IDS_KEY)
            self.hidden_states = batch.get(HIDDEN_STATES_KEY)
            self.labels = batch.get(LABELS_KEY)
            self.position_offset = int(batch.get(POSITION_OFFSET_KEY, 0) or 0)
            self.position_ids = batch.get(POSITION_IDS_KEY)
            self.sequence_ids = batch.get(SEQUENCE_IDS_KEY)
            self.loss_weight = batch.get(LOSS_WEIGHT_KEY)
            self.aux_loss_weight = batch.get(AUX_LOSS_WEIGHT_KEY)
            self.loss_scale = batch.get(LOSS_SCALE_KEY)
        elif isinstance(batch, (tuple, list)):
            self.input_ids, self.labels = batch
        else:
            self.input_ids = batch


def _is_sequence_parallel(mod: nn.Module) -> bool:
    return bool(getattr(mod, "sequence_parallel", False)) and getattr(mod, "world_size", 1) > 1


def project_group(x: torch.Tensor, modules: Sequence[nn.Module]) -> tuple[torch.Tensor, list[int]]:
    """Apply bias-free linear ``modules`` that share the input ``x``. Returns ``(packed, column offsets)``.

    With sequence-parallel column shards, ``x`` is the local ``[B, S/T, H]`` slice and the result covers the full
    sequence (one all-gather shared by the group, fused into the GEMM on CUDA)."""
    weights = [m.weight for m in modules]
    if any(getattr(m, "bias", None) is not None for m in modules):
        outs = [m(x) for m in modules]
        offs, at = [], 0
        for o in outs:
            offs.append(at)
            at += o.shape[-1]
        return torch.cat(outs, dim=-1), offs
    if _is_sequence_parallel(modules[0]):
        from maltos_b200.runtime.layers.functional import sequence_parallel_grouped_linear

        return sequence_parallel_grouped_linear(x, weights, modules[0].tp_group)
    if getattr(modules[0], "input_is_replicated", False) and getattr(modules[0], "world_size", 1) > 1:
        from maltos_b200.runtime.layers.functional import copy_to_group

        x = copy_to_group(x, modules[0].tp_group)
    return grouped_linear(x, weights)


class Linear(nn.Linear):
    """``nn.Linear`` (same parameters, same checkpoint names) whose forward is the tcgen05 GEMM on CUDA bf16."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, self.bias)


def project_out(x: torch.Tensor, module: nn.Module) -> torch.Tensor:
    """Output projection through the module's own forward (plain, or row-parallel with its communication), so that
    hooks other plugins attach to it (ZeRO-3 gathers, SP gathers) run."""
    return module(x)


def run_layer(layer: nn.Module, x: torch.Tensor, *, use_checkpoint: bool, **kwargs) -> torch.Tensor:
    if use_checkpoint:
        # no layer of these models draws random numbers (no dropout), so the generator state is neither saved nor restored
        return checkpoint(lambda y: layer(y, **kwargs), x, use_reentrant=False, preserve_rng_state=False,
                          context_fn=activation_checkpoint_context_fn)
    return layer(x, **kwargs)


def _local_sequence_slice(t: torch.Tensor, group, local_len: int) -> torch.Tensor:
    import torch.distributed as dist

    rank = dist.get_rank(group)
    return t.narrow(1, rank * local_len, local_len)


def lm_logits(hidden: torch.Tensor, lm_head: nn.Module) -> torch.Tensor:
    """Logits for inference. A sequence-parallel head first all-gathers the hidden states along the sequence."""
    group = getattr(lm_head, "sp_loss_group", None)
    if group is not None:
        from maltos_b200.runtime.layers.functional import all_gather

        hidden = all_gather(hidden, group, 1)
    return lm_head(hidden)


def lm_loss(hidden: torch.Tensor, lm_head: nn.Module, labels: torch.Tensor, loss_weight=None, loss_scale=None) -> torch.Tensor:
    """Mean next-token CE of ``lm_head(hidden)`` vs already-shifted ``labels``.

    Plain bias-free heads use the fused linear+CE op (no ``[tokens, vocab]`` logits kept). When the TP+SP plugin
    marked the head sequence-parallel (``sp_loss_group``), ``hidden`` is this rank's ``[B, S/T, H]`` slice: the
    matching label slice is scored locally and the sum / target count are reduced over the group."""
    group = getattr(lm_head, "sp_loss_group", None)
    if group is not None and labels.shape[1] != hidden.shape[1]:
        labels = _local_sequence_slice(labels, group, hidden.shape[1])
    if isinstance(lm_head, nn.Linear) and lm_head.bias is None and not lm_head._forward_pre_hooks and not lm_head._forward_hooks:
        loss = linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), lm_head.weight, labels.reshape(-1), group=group)
    elif group is None:
        loss = causal_cross_entropy(lm_head(hidden), labels)
    else:
        # The head runs through its own forward (another plugin hooked it, e.g. ZeRO-3 gathers its weight there). Each
        # rank scores its own tokens; the mean must still be taken over the targets of the WHOLE sequence, which the
        # ranks' slices share unevenly in packed rows: local mean x local / global target count, summed over the group.
        from maltos_b200.ops.cross_entropy import _global_count, _GroupSum

        local = causal_cross_entropy(lm_head(hidden), labels)
        flat = labels.reshape(-1)
        local_count = (flat != IGNORE_INDEX).sum()
        global_count = _global_count(flat, IGNORE_INDEX, group).clamp_min(1)
        loss = _GroupSum.apply(local * (local_count.to(local.dtype) / global_count.to(local.dtype)), group)
    if loss_weight is not None:
        loss = loss * float(loss_weight)
    if loss_scale is not None:          # a device scalar: no host read
        loss = loss * loss_scale.to(device=loss.device, dtype=loss.dtype)
    return loss


def init_normal_(module: nn.Module, std: float = 0.02) -> None:
    """normal(0, std) for every matrix / embedding, ones for norm weights, zeros for biases."""
    for m in module.modules():
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=std)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

"""Loss averaged over TARGETS across the data-parallel ranks (opt-in; the reference has no counterpart).

Every rank normalises its cross-entropy by its own number of supervised targets and the data-parallel gradient
reduction averages the ranks: a mean of means. With pre-training batches (every token a target) that is the mean over
tokens; with supervised fine-tuning the ranks hold different numbers of targets and rows with few targets weigh more
than they should. This plugin multiplies each rank's loss by ``local targets x dp / targets of all data-parallel ranks``
(one all-reduce of a device scalar per micro-step, no host read), which turns the average of the ranks' gradients into
the gradient of the token-weighted mean - the loss a single process would compute on the union of the rows. The logged
loss (mean over ranks) becomes that token-weighted mean as well.

Granularity: one micro-step (and, under pipeline parallelism, one pipeline micro-batch: the runner re-derives the scale of
each piece from the per-row counts). Micro-steps of an accumulation window still weigh equally, as in a single process
that accumulates. HDP does this weighting itself and is rejected here.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import RuntimePhase
from maltos_b200.utils.constants import IGNORE_INDEX, LABELS_KEY, LOSS_SCALE_KEY, LOSS_TARGET_COUNTS_KEY

#: per-row targets of the WHOLE rows (over the context-parallel group) behind ``loss_scale``; lets the pipeline runner
#: give each of its micro-batches the exact scale
LOSS_ROW_TARGETS_KEY = "loss_row_targets"


class TokenWeightedLossPlugin(RuntimePlugin):
    def __init__(self) -> None:
        super().__init__(id=PluginId.TOKEN_WEIGHTED_LOSS, name="token_weighted_loss", runs_after={PluginId.CP, PluginId.PP})

    def bind(self, runtime) -> None:
        super().bind(runtime)
        if runtime.has_plugin(PluginId.HDP):
            raise ValueError("TokenWeightedLossPlugin: ByteScale HDP already weights every rank's loss by its targets")
        if runtime.has_plugin(PluginId.CUDA_GRAPH):
            raise ValueError("TokenWeightedLossPlugin issues a collective per micro-step and cannot run inside a recorded graph")

    def on_step_phase(self, phase: RuntimePhase) -> None:
        if phase is not RuntimePhase.PRE_STEP_RUNNER:
            return
        rt = self.runtime
        batch = rt.state.batch
        if not isinstance(batch, dict) or not torch.is_tensor(batch.get(LABELS_KEY)):
            return
        labels = batch[LABELS_KEY]
        counts = batch.get(LOSS_TARGET_COUNTS_KEY)
        if torch.is_tensor(counts):            # rows already cut by context parallelism: column 1 counts the whole row
            rows = counts[:, 1].to(device=labels.device, dtype=torch.float32, non_blocking=True)
        else:
            rows = (labels != IGNORE_INDEX).sum(dim=tuple(range(1, labels.dim()))).to(torch.float32)
        local = rows.sum()
        total = local.clone()
        group = rt.get_group(MeshAxis.DP)
        dp = 1
        if group is not None and dist.get_world_size(group) > 1:
            dp = dist.get_world_size(group)
            dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
        batch[LOSS_SCALE_KEY] = local * float(dp) / total.clamp_min(1.0)
        batch[LOSS_ROW_TARGETS_KEY] = rows


__all__ = ["LOSS_ROW_TARGETS_KEY", "TokenWeightedLossPlugin"]

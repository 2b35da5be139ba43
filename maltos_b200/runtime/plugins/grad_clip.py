"""Global-norm gradient clipping for runtime-owned optimizers (ZeRO plugins clip their own shards through
``RuntimeCore.grad_clip_max_norm``). PRE_STEP: norm^2 = all-reduce over the world of ``sum ||g||^2 / replicas`` in fp64;
gradients are scaled by ``max_norm / (norm + 1e-6)`` when that is < 1 (reference ``runtime/plugins/grad_clip.py:10-85``).
On CUDA the sum of squares is one multi-tensor launch, the coefficient stays on the device and the scaling is a second
launch that is skipped by the kernel itself when the coefficient is 1 - no host synchronisation in the step."""
from __future__ import annotations

import torch
import torch.distributed as dist

from maltos_b200.ops.optim import clip_coefficient, scale_tensors_, sum_of_squares
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import RuntimePhase

_ZERO = (PluginId.ZERO1, PluginId.ZERO2, PluginId.ZERO3)


class GradClipPlugin(RuntimePlugin):
    def __init__(self, max_norm: float) -> None:
        if max_norm <= 0:
            raise ValueError(f"max_norm must be > 0, got {max_norm}")
        super().__init__(id=PluginId.GRAD_CLIP, name="grad_clip",
                         runs_after={PluginId.DP, PluginId.TP, PluginId.TP_SP, PluginId.PP, PluginId.CP, PluginId.EP, PluginId.FP16})
        self.max_norm = float(max_norm)
        self._norm: torch.Tensor | None = None

    def bind(self, runtime) -> None:
        super().bind(runtime)
        if any(runtime.has_plugin(z) for z in _ZERO):
            raise ValueError("GradClipPlugin cannot be combined with a ZeRO plugin; set RuntimeCore.grad_clip_max_norm instead")

    def on_step_phase(self, phase: RuntimePhase) -> None:
        if phase is not RuntimePhase.PRE_STEP:
            return
        rt = self.runtime
        optimizer, _ = rt.get_optimizer_and_scheduler()
        if optimizer is None:
            return
        pairs = None
        lister = getattr(optimizer, "grads_for_clipping", None)
        if callable(lister):
            pairs = lister()
        else:
            pairs = [(p, p.grad) for g in optimizer.param_groups for p in g["params"] if p.grad is not None]
        if not pairs:
            return
        scaler = rt.state.scaler
        if scaler is not None:
            scaler.unscale_(optimizer)
        grads = [g for _, g in pairs]
        weights = [1.0 / rt.grad_norm_replica_factor(p) for p, _ in pairs]
        sq = sum_of_squares(grads, weights)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(sq, op=dist.ReduceOp.SUM)
        coef, norm = clip_coefficient(sq, self.max_norm)
        scale_tensors_(grads, coef)
        self._norm = norm
        rt.state.metadata["grad_norm"] = norm       # a device scalar: read by whoever wants the number (the reference stores a float)

    def collect_metrics(self):
        if self._norm is None:
            return {}
        return {"grad_norm": float(self._norm.item()), "max_norm": self.max_norm}

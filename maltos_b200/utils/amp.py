"""Loss scaling for fp16 when gradients are spread over ranks.

``torch.amp.GradScaler`` decides from the gradients it sees on THIS rank whether a step overflowed. With tensor-parallel
shards or sharded optimizers (ZeRO) an ``inf`` lives on one rank only: that rank would skip the step and halve its scale
while the others step - replicas and loss scales drift apart. :class:`DistributedGradScaler` makes the decision global: the
per-device "found inf" flags are MAX-reduced over the world before anybody looks at them (the reference uses the plain
scaler, ``runtime/plugins/fp16.py:37-46``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class DistributedGradScaler(torch.amp.GradScaler):
    def _unscale_grads_(self, optimizer, inv_scale, found_inf, allow_fp16):
        per_device = super()._unscale_grads_(optimizer, inv_scale, found_inf, allow_fp16)
        if dist.is_initialized() and dist.get_world_size() > 1:
            if not per_device:      # a rank without any gradient in this optimizer still has to join the reduction
                per_device = {found_inf.device: found_inf.clone()}
            for flag in per_device.values():
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        return per_device

    def found_inf(self, optimizer) -> bool:
        """After ``unscale_(optimizer)``: whether any rank saw a non-finite gradient (host read)."""
        state = self._per_optimizer_states.get(id(optimizer))
        if not state:
            return False
        return any(float(v.item()) > 0 for v in state["found_inf_per_device"].values())


__all__ = ["DistributedGradScaler"]

"""ZeRO stage 2: gradients and optimizer state sharded over the data-parallel group (reference
``runtime/plugins/zero2.py:256-290``).

Builds on the stage-1 plugin (same flat buckets, same asynchronous reduce-scatter fired from the gradient hooks, same
peer-memory mode); what changes is where gradients live between micro-steps: each bucket's full-size gradient buffer is a
TEMPORARY pool buffer that exists only during one backward, and what is carried across the accumulation window is the
rank's own shard (``accumulate_on_shard``). A checkpoint taken inside an accumulation window therefore saves the shard
gradients as plugin state.
"""
from __future__ import annotations

from maltos_b200.runtime.buffer_allocator import BufferPolicy, acquire_buffer, release_buffer
from maltos_b200.runtime.plugin import PluginId
from maltos_b200.utils.profiling import span

from .zero1 import Zero1Plugin


class Zero2Plugin(Zero1Plugin):
    accumulate_on_shard = True

    def __init__(self, bucket_mb_size: int = 25, *, peer_memory: bool | None = None) -> None:
        super().__init__(bucket_mb_size, peer_memory=peer_memory, _id=PluginId.ZERO2, _name="zero2")

    def _pre_backward(self, ctx) -> None:
        for b in self.buckets:
            if ctx.accum_start and b.local_param.grad is not None:
                b.local_param.grad.zero_()
            if b.grad is None:
                b.grad_handle = acquire_buffer(shape=(b.data.numel(),), dtype=b.data.dtype, device=b.data.device, policy=BufferPolicy.TEMPORARY)
                b.grad = b.grad_handle.tensor
            b.grad.zero_()
            self._attach_grad_views(b)
            b.pending = len(b.params)
            b.fired = False

    def _post_backward(self, ctx) -> None:
        with span("maltos::zero.grad_sync.wait"):
            self._peer_phase(True)
            for b in self.buckets:
                self._finish(b)
                for p in b.params:
                    p.grad = None
                if b.grad_handle is not None:
                    release_buffer(b.grad_handle)
                if b.peer_grad_ptrs is None:
                    b.grad, b.grad_handle = None, None
            self._peer_phase(False)

    def export_plugin_state(self):
        ctx = self.runtime.state.step_context
        if ctx.microbatch_idx == 0:
            return {}
        return {"bucket_local_grads": [None if b.local_param.grad is None else b.local_param.grad.detach().cpu().clone() for b in self.buckets]}

    def import_plugin_state(self, state) -> None:
        grads = state.get("bucket_local_grads")
        if not isinstance(grads, list):
            return
        for b, g in zip(self.buckets, grads):
            if g is not None:
                b.local_param.grad = g.to(device=b.local_param.device, dtype=b.local_param.dtype)


__all__ = ["Zero2Plugin"]

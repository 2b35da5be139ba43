"""CUDA-graph capture of a launch-bound micro-step.

Small models (and large ones sharded over many GPUs) spend a micro-step in hundreds of short kernels, and the host
needs longer to launch them than the device needs to run them. ``GraphedMicroStep`` records the forward and backward
of one micro-step - this library's kernels are ordinary launches on the current stream, so they are captured like any
other - and replays the whole recording with one driver call. The reference has no counterpart (its answer to launch
overhead is ``torch.compile``, ``runtime/plugins/compile.py:11-144``).

Rules of the recording:

* shapes are static: every call must bring tensors of the shapes of the example batch (they are copied into the
  recording's input buffers);
* gradients ACCUMULATE like in eager execution: the recording owns one gradient tensor per parameter (allocated during
  the capture, overwritten by every replay) and every call adds them to ``param.grad`` with one multi-tensor add;
* the step must not read device values on the host (``.item()``, data-dependent shapes) and must not run collectives
  whose arguments change from call to call (the fused tensor-parallel kernels carry a call sequence number);
* activation checkpointing that saves and restores the random-number state cannot be recorded;
* no autograd graph of an earlier eager step over the same parameters may still be alive (drop the old loss tensors
  first): its gradient-accumulation nodes are bound to the stream they ran on, and the capture stream may not make the
  default stream wait.
"""
from __future__ import annotations

from typing import Callable, Mapping

import torch


class GraphedMicroStep:
    def __init__(self, step_fn: Callable[[Mapping[str, torch.Tensor]], torch.Tensor], parameters, example_batch: Mapping[str, torch.Tensor],
                 *, loss_scale: float = 1.0, warmup: int = 3) -> None:
        """``step_fn(batch) -> scalar loss`` (forward only; the backward of ``loss * loss_scale`` is recorded here)."""
        if not torch.cuda.is_available():
            raise RuntimeError("GraphedMicroStep needs a CUDA device")
        self.step_fn = step_fn
        self.loss_scale = float(loss_scale)
        self.params = [p for p in parameters if p.requires_grad]
        self.static = {k: v.detach().clone() for k, v in example_batch.items() if torch.is_tensor(v)}
        self.extra = {k: v for k, v in example_batch.items() if not torch.is_tensor(v)}
        saved = [p.grad for p in self.params]
        # warm-up on a side stream (lazy initialisations, autotuning and workspace allocations happen here, not in the capture)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                for p in self.params:
                    p.grad = None
                self._run()
        torch.cuda.current_stream().wait_stream(side)
        # gradients are None at capture time: the recorded backward then allocates them from the graph's own memory pool
        # and every replay rewrites them (no in-place accumulation node runs inside the recording)
        for p in self.params:
            p.grad = None
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = self._run()
        self.recorded = [(p, p.grad) for p in self.params if p.grad is not None]
        for p, g in zip(self.params, saved):
            p.grad = g                       # what the caller had before (possibly None)

    def _run(self) -> torch.Tensor:
        loss = self.step_fn({**self.static, **self.extra})
        (loss * self.loss_scale).backward()
        return loss.detach()

    def __call__(self, batch: Mapping[str, torch.Tensor]) -> torch.Tensor:
        """Copies ``batch`` into the recorded inputs, replays forward + backward, returns the (recorded) loss tensor."""
        for k, dst in self.static.items():
            src = batch[k]
            if src.shape != dst.shape or src.dtype != dst.dtype:
                raise ValueError(f"GraphedMicroStep: '{k}' must keep shape {tuple(dst.shape)} and dtype {dst.dtype}, got {tuple(src.shape)} {src.dtype}")
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        have = [(p.grad, g) for p, g in self.recorded if p.grad is not None]
        if have:
            torch._foreach_add_([a for a, _ in have], [g for _, g in have])
        for p, g in self.recorded:
            if p.grad is None:
                p.grad = g.clone()
        return self.loss

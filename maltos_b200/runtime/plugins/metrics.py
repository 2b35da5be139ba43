"""Step-time and memory gauges. ``perf/step_sec`` spans from the first micro-step's PRE_STEP_RUNNER to POST_STEP and is
emitted exactly once per optimizer step (reference ``runtime/plugins/metrics.py:11-59``)."""
from __future__ import annotations

import time

import torch

from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import RuntimePhase


class MetricPlugin(RuntimePlugin):
    def __init__(self, include_cuda_memory: bool = True) -> None:
        super().__init__(id=PluginId.METRICS, name="metrics")
        self.include_cuda_memory = include_cuda_memory
        self._t0: float | None = None
        self._pending: dict = {}

    def on_step_phase(self, phase: RuntimePhase) -> None:
        if phase is RuntimePhase.PRE_STEP_RUNNER:
            if self._t0 is None:
                self._t0 = time.perf_counter()
        elif phase is RuntimePhase.POST_STEP and self._t0 is not None:
            self._pending = {"perf/step_sec": time.perf_counter() - self._t0}
            self._t0 = None
            dev = torch.device(self.runtime.device)
            if self.include_cuda_memory and dev.type == "cuda":
                self._pending["memory/allocated_gb"] = torch.cuda.memory_allocated(dev) / 1e9
                self._pending["memory/reserved_gb"] = torch.cuda.memory_reserved(dev) / 1e9
                self._pending["memory/max_allocated_gb"] = torch.cuda.max_memory_allocated(dev) / 1e9
                self._pending["memory/max_reserved_gb"] = torch.cuda.max_memory_reserved(dev) / 1e9

    def collect_metrics(self):
        out, self._pending = self._pending, {}
        return out

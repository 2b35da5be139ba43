"""``CudaGraphPlugin``: the micro-step (forward + backward) of a single-GPU run recorded into a CUDA graph.

Owns the step runner. The first micro-steps run eagerly (lazy initialisations, workspace allocations), then the step
is recorded once per batch signature (key names, shapes, dtypes) and every later micro-step is one graph replay plus
one multi-tensor add of the recorded gradients into ``param.grad`` (``maltos_b200.utils.cuda_graph``). Batches with a
new signature are recorded again; up to ``max_graphs`` recordings are kept, further signatures run eagerly.

Scope: one process, no communicating plugin (the fused tensor-parallel kernels carry per-call sequence numbers and
NCCL work handles cannot be replayed by this runner), models whose forward reads no device value on the host, and no
activation checkpointing that saves the random-number state. Not part of the reference (its tool against launch
overhead is ``torch.compile``, ``runtime/plugins/compile.py:11-144``).
"""
from __future__ import annotations

from typing import Any

import torch

from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.step_runners.base import DefaultStepRunner
from maltos_b200.runtime.types import LossOutput, RuntimePhase
from maltos_b200.utils.cuda_graph import GraphedMicroStep
from maltos_b200.utils.profiling import span

_COMMUNICATING = {PluginId.TP, PluginId.TP_SP, PluginId.DP, PluginId.PP, PluginId.CP, PluginId.HDP, PluginId.EP, PluginId.ZERO1,
                  PluginId.ZERO2, PluginId.ZERO3, PluginId.FP16}


class GraphedStepRunner(DefaultStepRunner):
    def __init__(self, eager_steps: int = 2, max_graphs: int = 4) -> None:
        self.eager_steps = eager_steps
        self.max_graphs = max_graphs
        self.graphs: dict[tuple, GraphedMicroStep] = {}
        self.seen = 0
        self.replays = 0

    @staticmethod
    def _signature(batch: dict) -> tuple:
        return tuple(sorted((k, tuple(v.shape), str(v.dtype)) for k, v in batch.items() if torch.is_tensor(v)))

    def run(self, runtime, batch: Any) -> torch.Tensor:
        self.seen += 1
        usable = isinstance(batch, dict) and all(torch.is_tensor(v) and v.is_cuda for v in batch.values())
        if not usable or self.seen <= self.eager_steps:
            return super().run(runtime, batch)
        sig = self._signature(batch)
        graph = self.graphs.get(sig)
        if graph is None:
            if len(self.graphs) >= self.max_graphs:
                return super().run(runtime, batch)
            # forget the eager steps' autograd graphs before recording (their accumulation nodes are stream-bound)
            runtime.state.loss = None
            runtime.state.outputs = None
            div = runtime.state.step_context.loss_divisor

            def forward(b):
                out = runtime.model(b)
                return out.loss if isinstance(out, LossOutput) else out

            graph = self.graphs[sig] = GraphedMicroStep(forward, runtime.model.parameters(), batch, loss_scale=1.0 / div)
            graph.loss_divisor = div
        if graph.loss_divisor != runtime.state.step_context.loss_divisor:
            return super().run(runtime, batch)       # the recorded backward is scaled for another accumulation length
        st = runtime.state
        with span("maltos::graph_replay"):
            runtime._run_step_phase(RuntimePhase.PRE_FORWARD)
            runtime._run_step_phase(RuntimePhase.POST_FORWARD)
            runtime._run_step_phase(RuntimePhase.PRE_BACKWARD)
            loss = graph(batch)
            self.replays += 1
            st.outputs = loss
            st.metadata.pop("model_metrics", None)
            st.metadata["raw_loss_for_metrics"] = loss.float().clone()
            st.loss = loss / graph.loss_divisor if graph.loss_divisor != 1 else loss
            runtime._run_step_phase(RuntimePhase.POST_BACKWARD)
        return st.loss


class CudaGraphPlugin(RuntimePlugin):
    def __init__(self, eager_steps: int = 2, max_graphs: int = 4) -> None:
        super().__init__(id=PluginId.CUDA_GRAPH, name="cuda_graph", owns_step_runner=True)
        self.runner = GraphedStepRunner(eager_steps=eager_steps, max_graphs=max_graphs)

    def bind(self, runtime) -> None:
        super().bind(runtime)
        clash = sorted(p.id.value for p in runtime.plugins if p.id in _COMMUNICATING)
        if clash:
            raise ValueError(f"CudaGraphPlugin records single-process steps only; remove it or the plugins {clash}")
        if runtime.mesh.world_size != 1:
            raise ValueError("CudaGraphPlugin needs a mesh of one rank")

    def build_step_runner(self):
        return self.runner

    def collect_metrics(self) -> dict[str, float]:
        return {"cuda_graph/replays": float(self.runner.replays), "cuda_graph/recordings": float(len(self.runner.graphs))}

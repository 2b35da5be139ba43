"""Default step runner: one forward + one backward of the whole model per micro-step, with plugin phases around
each half (semantics of the reference's ``runtime/step_runners/base.py:18-83``)."""
from __future__ import annotations

from typing import TYPE_CHECKING, Any, Protocol

import torch

from maltos_b200.runtime.types import LossOutput, PipelineOutput, RuntimePhase
from maltos_b200.utils.profiling import span

if TYPE_CHECKING:
    from maltos_b200.runtime.core import RuntimeCore


class StepRunner(Protocol):
    def run(self, runtime: "RuntimeCore", batch: Any) -> torch.Tensor: ...


class DefaultStepRunner:
    def run(self, runtime: "RuntimeCore", batch: Any) -> torch.Tensor:
        self.run_forward(runtime, batch)
        if not torch.is_tensor(runtime.state.loss):
            raise TypeError("RuntimeCore expects model(batch) to return a Tensor loss during training.")
        self.run_backward(runtime)
        return runtime.state.loss

    @staticmethod
    def run_forward(runtime: "RuntimeCore", batch: Any) -> None:
        st = runtime.state
        with span("maltos::forward"):
            runtime._run_step_phase(RuntimePhase.PRE_FORWARD)
            try:
                out = runtime.model(batch)
                st.outputs = out
                if isinstance(out, LossOutput):
                    st.loss = out.loss
                    st.metadata["model_metrics"] = dict(out.metrics)
                else:
                    st.metadata.pop("model_metrics", None)
                    st.loss = out if (torch.is_tensor(out) and not isinstance(out, PipelineOutput)) else None
            finally:
                runtime._run_step_phase(RuntimePhase.POST_FORWARD)

    @staticmethod
    def run_backward(runtime: "RuntimeCore", *, grad_output: torch.Tensor | None = None) -> None:
        st = runtime.state
        with span("maltos::backward"):
            runtime._run_step_phase(RuntimePhase.PRE_BACKWARD)
            if grad_output is None:
                if st.loss is None:
                    raise TypeError("RuntimeCore expected runtime.state.loss to be a Tensor before backward()")
                # the metric must show the un-divided loss - and the un-SCALED one: the fp16 plugin has kept it before it
                # multiplied the loss at PRE_BACKWARD (the reference overwrites it here and logs loss x scale under fp16)
                if not st.metadata.pop("loss_scaled_for_backward", False):
                    st.metadata["raw_loss_for_metrics"] = st.loss.detach().float()
                div = st.step_context.loss_divisor
                if div != 1:
                    st.loss = st.loss / div
                st.loss.backward()
            else:
                if not torch.is_tensor(st.outputs):
                    raise TypeError("RuntimeCore expected runtime.state.outputs Tensor for activation backward()")
                st.outputs.backward(grad_output)
            runtime._run_step_phase(RuntimePhase.POST_BACKWARD)

    @staticmethod
    def run_backward_many(runtime: "RuntimeCore", tensors: list[torch.Tensor], grad_tensors: list[torch.Tensor]) -> None:
        """One autograd sweep for several roots (boundary activation + stage-local auxiliary loss)."""
        if len(tensors) != len(grad_tensors):
            raise ValueError("backward tensors and grad_tensors must have the same length")
        with span("maltos::backward"):
            runtime._run_step_phase(RuntimePhase.PRE_BACKWARD)
            torch.autograd.backward(tensors=tensors, grad_tensors=grad_tensors)
            runtime._run_step_phase(RuntimePhase.POST_BACKWARD)

"""fp16 loss scaling: active when the runtime dtype is float16 on CUDA (on CPU only when asked for, which the tests do).
Scales the loss at PRE_BACKWARD through a gradient scaler kept in ``runtime.state.scaler`` (the core steps through it) and
checkpoints the scaler state (reference ``runtime/plugins/fp16.py:10-74``). The scaler is the distributed one: an overflow
on any rank skips the step on every rank (``utils/amp.py``)."""
from __future__ import annotations

import torch

from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import RuntimePhase, SetupPhase


class Fp16Plugin(RuntimePlugin):
    def __init__(self, init_scale: float = 2.0 ** 16, growth_interval: int = 2000, *, allow_cpu: bool = False) -> None:
        super().__init__(id=PluginId.FP16, name="fp16")
        self.init_scale = init_scale
        self.growth_interval = growth_interval
        self.allow_cpu = allow_cpu
        self.scaler = None

    @property
    def active(self) -> bool:
        rt = self.runtime
        return rt is not None and rt.dtype == torch.float16 and (torch.device(rt.device).type == "cuda" or self.allow_cpu)

    def on_setup_phase(self, phase: SetupPhase, model):
        rt = self.runtime
        if phase is SetupPhase.FINALIZE and rt.dtype == torch.float16 and not self.active:
            # fp16 without loss scaling underflows silently: refuse, as the reference does (``fp16.py:28-33``)
            raise ValueError("Fp16Plugin requires CUDA model parameters for float16 training (allow_cpu=True enables the CPU scaler for tests)")
        if phase is SetupPhase.FINALIZE and self.active:
            from maltos_b200.utils.amp import DistributedGradScaler

            self.scaler = DistributedGradScaler(torch.device(self.runtime.device).type, init_scale=self.init_scale,
                                                growth_interval=self.growth_interval)
            self.runtime.state.scaler = self.scaler
        return model

    def on_step_phase(self, phase: RuntimePhase) -> None:
        if phase is RuntimePhase.PRE_BACKWARD and self.scaler is not None:
            st = self.runtime.state
            if st.loss is not None:
                st.metadata["raw_loss_for_metrics"] = st.loss.detach().float()
                st.metadata["loss_scaled_for_backward"] = True
                st.loss = self.scaler.scale(st.loss)

    def export_plugin_state(self):
        return {"scaler": self.scaler.state_dict()} if self.scaler is not None else {}

    def import_plugin_state(self, state) -> None:
        if self.scaler is not None and isinstance(state.get("scaler"), dict):
            self.scaler.load_state_dict(state["scaler"])

    def collect_metrics(self):
        rt = self.runtime
        out = {"dtype": str(rt.dtype).replace("torch.", "") if rt.dtype is not None else "float32"}
        md = rt.state.metadata          # without a scaler (fp32 / bf16): scale None, never an overflow - the reference's keys
        out["loss_scale"] = md.get("loss_scale") if self.scaler is not None else None
        out["overflow"] = bool(md.get("overflow", False)) if self.scaler is not None else False
        return out

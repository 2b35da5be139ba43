"""``CompilePlugin`` keeps the reference's interface (``runtime/plugins/compile.py:11-144``: scope / backend / mode, the
model's ``compile_spec()`` paths, materialization groups for ZeRO-3) but does not invoke a tracing compiler: the scopes it
names (the SwiGLU MLP) already execute as hand-written fused sm_100a kernels (grouped gate/up GEMM -> SwiGLU kernel ->
row GEMM). It validates the scope, records which module paths are covered, and reports them as metrics."""
from __future__ import annotations

import torch.nn as nn

from maltos_b200.parallel.protocols import CompilableModule
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import SetupPhase


class CompilePlugin(RuntimePlugin):
    def __init__(self, scope: str = "mlp", backend: str = "inductor", mode: str = "default") -> None:
        super().__init__(id=PluginId.COMPILE, name="compile", runs_after={PluginId.TP, PluginId.TP_SP, PluginId.PP, PluginId.EP})
        self.scope, self.backend, self.mode = scope, backend, mode
        self.covered_paths: list[str] = []
        self._modules: list[nn.Module] = []

    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        if phase is SetupPhase.TRANSFORM:
            if not isinstance(model, CompilableModule):
                raise ValueError(f"{type(model).__name__} does not declare compile_spec()")
            spec = model.compile_spec()
            if self.scope not in spec:
                raise ValueError(f"compile scope {self.scope!r} not offered by the model (available: {sorted(spec)})")
            self.covered_paths = [p for p in spec[self.scope] if not self.runtime.is_module_path_omitted(p)]
            self._modules = []
            for path in self.covered_paths:
                try:
                    m = model.get_submodule(path)
                except AttributeError:
                    continue
                if m is not None:
                    self._modules.append(m)
        return model

    @property
    def compiled_module_paths(self) -> list[str]:
        """The reference's name for the covered module paths (there: the modules whose ``forward`` was compiled)."""
        return list(self.covered_paths)

    def param_materialization_groups(self):
        """Each covered module's parameters are gathered together by ZeRO-3 (they are used by one fused region)."""
        return tuple((m, tuple(m.parameters())) for m in self._modules if any(True for _ in m.parameters()))

    def collect_metrics(self):
        return {"fused_scopes": len(self._modules), "compile/scope": self.scope, "compile/backend": self.backend, "compile/mode": self.mode,
                "compile/modules": len(self.covered_paths)}

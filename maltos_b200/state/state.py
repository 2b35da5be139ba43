"""Index of everything a checkpoint must capture: trainable parameters and persistent buffers (with the logical
names/shapes needed to re-shard them), optimizer/scheduler state, RNG, step context, dataloader position and
plugin states. Entry field names are the manifest schema (reference ``state/state.py:18-64``)."""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, is_dataclass
from typing import TYPE_CHECKING, Any, Mapping

import torch
import torch.nn as nn

from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.types import StepContext

if TYPE_CHECKING:
    from maltos_b200.runtime.core import RuntimeCore


@dataclass
class RuntimeParamAttrs:
    """Runtime-only: along which mesh axes a parameter is sharded / replicated."""

    sharded_axes: set[MeshAxis] = field(default_factory=set)
    replicated_axes: set[MeshAxis] = field(default_factory=set)


@dataclass
class ModelStateMeta:
    state_key: str
    logical_names: list[str]
    logical_shapes: list[tuple[int, ...]]
    physical_shape: tuple[int, ...]
    dtype: str
    source_rank: int | None = None


@dataclass
class ParamEntry:
    meta: ModelStateMeta
    param: nn.Parameter
    attrs: RuntimeParamAttrs = field(default_factory=RuntimeParamAttrs)


@dataclass
class BufferEntry:
    meta: ModelStateMeta
    tensor: torch.Tensor


@dataclass(frozen=True)
class RngState:
    cpu: torch.Tensor
    cuda: list[torch.Tensor] | None = None


@dataclass(frozen=True)
class TrainerState:
    rng: RngState
    step_context: dict[str, Any] | None = None
    dataloader: dict[str, Any] | None = None
    plugin_states: dict[str, dict[str, Any]] | None = None


@dataclass(frozen=True)
class OptimizerState:
    state: dict[str, Any]


#: key of the runtime's own entry among the plugin states of ``trainer_rank_N.pt`` (plugin ids are the other keys; a loader that
#: does not know a key skips it)
_RUNTIME_STATE_KEY = "runtime"


def _meta_for(name: str, tensor: torch.Tensor) -> ModelStateMeta:
    shape = tuple(tensor.shape)
    return ModelStateMeta(state_key=name, logical_names=[name], logical_shapes=[shape], physical_shape=shape,
                          dtype=str(tensor.dtype))


@dataclass
class StateManager:
    params: dict[str, ParamEntry] = field(default_factory=dict)
    buffers: dict[str, BufferEntry] = field(default_factory=dict)
    _names_by_param: dict[int, str] = field(default_factory=dict, repr=False)
    _runtime: "RuntimeCore | None" = field(default=None, init=False, repr=False)
    _dataloader: Any = field(default=None, init=False, repr=False)

    OPTIMIZER_KEY = "__optimizer_state__."
    SCHEDULER_KEY = "__scheduler_state__."

    # ------------------------------------------------------------------ binding
    def bind(self, runtime: "RuntimeCore") -> None:
        self._runtime = runtime

    def bind_dataloader(self, dataloader) -> None:
        self._dataloader = dataloader

    @property
    def runtime(self) -> "RuntimeCore":
        if self._runtime is None:
            raise RuntimeError("StateManager is not bound to RuntimeCore")
        return self._runtime

    # ------------------------------------------------------------------ registration / lookup
    def register_module(self, model: nn.Module) -> None:
        """(Re)build the index from ``model``: trainable params and buffers that appear in ``state_dict``."""
        self.params.clear()
        self.buffers.clear()
        self._names_by_param.clear()
        for name, p in model.named_parameters():
            if p.requires_grad:
                self.params[name] = ParamEntry(meta=_meta_for(name, p), param=p)
                self._names_by_param[id(p)] = name
        persistent = set(model.state_dict().keys()) - set(self.params)
        for name, buf in model.named_buffers():
            if name in persistent:
                self.buffers[name] = BufferEntry(meta=_meta_for(name, buf), tensor=buf)

    def _resolve_runtime_name(self, name: str) -> str:
        """Accept names with or without a leading ``module.`` (wrapped models)."""
        known = lambda n: n in self.params or n in self.buffers  # noqa: E731
        if known(name):
            return name
        if known("module." + name):
            return "module." + name
        if name.startswith("module.") and known(name[7:]):
            return name[7:]
        return name

    @property
    def param_states(self) -> Mapping[str, ModelStateMeta]:
        return {k: e.meta for k, e in self.params.items()}

    @property
    def buffer_states(self) -> Mapping[str, ModelStateMeta]:
        return {k: e.meta for k, e in self.buffers.items()}

    def update_model_state(self, fq_name: str, *, logical_names=None, logical_shapes=None, physical_shape=None,
                           dtype=None, source_rank=None, sharded_axes=None, replicated_axes=None) -> None:
        name = self._resolve_runtime_name(fq_name)
        entry = self.params.get(name) or self.buffers.get(name)
        if entry is None:
            raise KeyError(f"model state not found: {name}")
        meta = entry.meta
        for attr, value in (("logical_names", logical_names), ("logical_shapes", logical_shapes),
                            ("physical_shape", physical_shape), ("dtype", dtype), ("source_rank", source_rank)):
            if value is not None:
                setattr(meta, attr, value)
        if isinstance(entry, ParamEntry):
            if sharded_axes is not None:
                entry.attrs.sharded_axes = sharded_axes
            if replicated_axes is not None:
                entry.attrs.replicated_axes = replicated_axes

    def get_model_tensor(self, fq_name: str) -> torch.Tensor:
        name = self._resolve_runtime_name(fq_name)
        if name in self.params:
            return self.params[name].param
        if name in self.buffers:
            return self.buffers[name].tensor
        raise KeyError(f"runtime model tensor not found: {name}")

    def get_param_name(self, param: nn.Parameter) -> str:
        try:
            return self._names_by_param[id(param)]
        except KeyError:
            raise KeyError("runtime parameter name not found") from None

    # ------------------------------------------------------------------ optimizer
    def _owner_tag(self) -> str:
        rt = self.runtime
        return "runtime" if rt._optimizer_owner is rt else rt._optimizer_owner.id.value

    def export_optimizer_state(self) -> OptimizerState | None:
        optimizer, scheduler = self.runtime.get_optimizer_and_scheduler()
        if optimizer is None:
            return None
        tag = self._owner_tag()
        payload: dict[str, Any] = {self.OPTIMIZER_KEY + tag: optimizer.state_dict()}
        if scheduler is not None:
            payload[self.SCHEDULER_KEY + tag] = scheduler.state_dict()
        return OptimizerState(state=payload)

    def import_optimizer_state(self, state: OptimizerState) -> None:
        optimizer, scheduler = self.runtime.get_optimizer_and_scheduler()
        if optimizer is None:
            raise ValueError("no optimizer available to load state into")
        tag = self._owner_tag()
        opt_state = state.state.get(self.OPTIMIZER_KEY + tag)
        if opt_state is None:
            raise ValueError(f"no optimizer state found for owner={tag}")
        optimizer.load_state_dict(opt_state)
        sched_state = state.state.get(self.SCHEDULER_KEY + tag)
        if scheduler is not None and sched_state is not None:
            scheduler.load_state_dict(sched_state)

    # ------------------------------------------------------------------ model
    def export_model_state(self):
        return self.runtime._model_state_owner.export_model_state(self)

    def import_model_state(self, model_state: dict[str, torch.Tensor]) -> None:
        self.runtime._model_state_owner.import_model_state(self, model_state)

    # ------------------------------------------------------------------ trainer (rng, step, loader, plugins)
    def export_trainer_state(self) -> TrainerState:
        rt = self.runtime
        rng = RngState(cpu=torch.get_rng_state(),
                       cuda=torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None)
        plugin_states = {}
        for plugin in rt.plugins:
            exported = plugin.export_plugin_state()
            if exported:
                plugin_states[plugin.id.value] = exported
        partial = self._partial_gradients()
        if partial:
            plugin_states[_RUNTIME_STATE_KEY] = {"partial_grads": partial}
        return TrainerState(rng=rng, step_context=asdict(rt.state.step_context),
                            dataloader=self._dataloader_state(), plugin_states=plugin_states or None)

    def import_trainer_state(self, state: TrainerState) -> None:
        rt = self.runtime
        rt.state.step_context = StepContext(**state.step_context) if state.step_context is not None else StepContext()
        torch.set_rng_state(state.rng.cpu)
        if state.rng.cuda is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state_all(state.rng.cuda)
        if self._dataloader is not None and state.dataloader is not None:
            self._dataloader.load_state_dict(state.dataloader)
        if state.plugin_states:
            for plugin in rt.plugins:
                saved = state.plugin_states.get(plugin.id.value)
                if isinstance(saved, dict):
                    plugin.import_plugin_state(saved)
            own = state.plugin_states.get(_RUNTIME_STATE_KEY)
            if isinstance(own, dict) and isinstance(own.get("partial_grads"), dict):
                for name, grad in own["partial_grads"].items():
                    entry = self.params.get(name)
                    if entry is not None and torch.is_tensor(grad):
                        entry.param.grad = grad.to(device=entry.param.device, dtype=entry.param.dtype).reshape(entry.param.shape).clone()

    def _partial_gradients(self) -> dict[str, torch.Tensor]:
        """Gradients accumulated so far when a checkpoint is taken INSIDE an accumulation window and the runtime itself owns
        the optimizer (the sharded-optimizer plugins keep and save their own partial gradients). Without them the resumed
        window would be missing the micro-steps done before the save."""
        rt = self.runtime
        if rt.state.step_context.microbatch_idx == 0 or getattr(rt, "_optimizer_owner", rt) is not rt:
            return {}
        return {name: e.param.grad.detach().to("cpu").clone() for name, e in self.params.items()
                if e.param.requires_grad and e.param.grad is not None}

    def _dataloader_state(self) -> dict[str, Any] | None:
        if self._dataloader is None:
            return None
        st = self._dataloader.state_dict()
        if is_dataclass(st) and not isinstance(st, type):
            return asdict(st)
        if isinstance(st, dict):
            return dict(st)
        raise TypeError(f"dataloader state must be a dataclass or dict, got {type(st)!r}")

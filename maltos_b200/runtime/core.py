"""RuntimeCore: the execution engine.

It owns the process mesh, orders the plugins, drives the three setup phases, runs micro-steps
(``run_step``) and optimizer steps (``step_optimizer``), and collects metrics. Public behaviour follows the
reference's ``runtime/core.py:39-537`` (same constructor fields, methods and phase order), so plugins, trainers
and tools written against it keep working.
"""
from __future__ import annotations

import warnings
from collections.abc import Callable, Iterable
from dataclasses import dataclass, field
from graphlib import TopologicalSorter
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.parallel.plan import ParallelPlan
from maltos_b200.parallel.protocols import FlopsEstimatableModule
from maltos_b200.state.state import ModelStateMeta, StateManager
from maltos_b200.utils.constants import INPUT_IDS_KEY, LOSS_TARGET_COUNTS_KEY
from maltos_b200.utils.profiling import profiled, span

from .mesh import MeshAxis, MeshConfig, ProcessGroupManager
from .optim import MasterWeightsOptimizer
from .plugin import PluginId, RuntimePlugin
from .step_runners.base import DefaultStepRunner
from .types import MetricValue, ParamRole, RuntimePhase, RuntimeState, SetupPhase, StepContext

OptimizerFactory = Callable[[Iterable[nn.Parameter]], torch.optim.Optimizer]
SchedulerFactory = Callable[[torch.optim.Optimizer], Any]

_ZERO_IDS = (PluginId.ZERO1, PluginId.ZERO2, PluginId.ZERO3)


def _rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def order_plugins(plugins: list[RuntimePlugin]) -> list[RuntimePlugin]:
    """Topological order over ``requires`` (hard), ``runs_after`` / ``runs_before`` (only among present plugins)."""
    by_id: dict[PluginId, RuntimePlugin] = {}
    for p in plugins:
        if p.id in by_id:
            raise ValueError(f"duplicate plugin id={p.id.value}")
        by_id[p.id] = p
    graph: dict[PluginId, set[PluginId]] = {pid: set() for pid in by_id}
    for p in plugins:
        absent = set(p.requires) - by_id.keys()
        if absent:
            raise ValueError(f"plugin={p.name} requires missing plugins={sorted(x.value for x in absent)}")
        graph[p.id] |= set(p.requires) | (set(p.runs_after) & by_id.keys())
        for later in p.runs_before:
            if later in by_id:
                graph[later].add(p.id)
    # Deterministic on every rank: among the plugins whose predecessors are all placed, the one declared first goes next.
    # (Feeding sets of ids to a generic sorter breaks ties by the iteration order of those sets, which follows the
    # per-process string hash seed: two ranks could order unconstrained plugins - and their collectives - differently.)
    TopologicalSorter(graph).prepare()          # raises CycleError with the offending cycle
    ordered: list[RuntimePlugin] = []
    placed: set[PluginId] = set()
    remaining = list(plugins)
    while remaining:
        nxt = next(p for p in remaining if graph[p.id] <= placed)
        ordered.append(nxt)
        placed.add(nxt.id)
        remaining.remove(nxt)
    return ordered


def _single_owner(plugins: list[RuntimePlugin], flag: str, what: str):
    owners = [p for p in plugins if getattr(p, flag)]
    if len(owners) > 1:
        raise ValueError(f"RuntimeCore allows only one {what}-owning plugin, got {[p.id.value for p in owners]}")
    return owners[0] if owners else None


@dataclass
class RuntimeCore:
    model: nn.Module
    mesh: MeshConfig = field(default_factory=MeshConfig)
    plan: ParallelPlan = field(default_factory=ParallelPlan)
    device: torch.device | str | None = None
    dtype: torch.dtype | None = None
    grad_accum_steps: int = 1
    grad_clip_max_norm: float | None = None
    optimizer_factory: OptimizerFactory | None = None
    scheduler_factory: SchedulerFactory | None = None
    plugins: list[RuntimePlugin] = field(default_factory=list)
    state_manager: StateManager = field(default_factory=StateManager)
    state: RuntimeState = field(default_factory=RuntimeState)
    _optimizer: Any = field(default=None, init=False, repr=False)
    _scheduler: Any = field(default=None, init=False, repr=False)
    _step_runner: Any = field(default=None, init=False, repr=False)
    _group_manager: ProcessGroupManager | None = field(default=None, init=False, repr=False)
    _closed: bool = field(default=False, init=False, repr=False)
    _omitted_module_paths: set[str] = field(default_factory=set, init=False, repr=False)
    _module_replacements: dict = field(default_factory=dict, init=False, repr=False)
    _param_roles: dict[int, ParamRole] = field(default_factory=dict, init=False, repr=False)
    _optimizer_owner: Any = field(default=None, init=False, repr=False)
    _step_runner_owner: Any = field(default=None, init=False, repr=False)
    _model_state_owner: Any = field(default=None, init=False, repr=False)

    # ------------------------------------------------------------------ construction
    def __post_init__(self) -> None:
        if self.grad_accum_steps < 1:
            raise ValueError(f"grad_accum_steps must be >= 1, got {self.grad_accum_steps}")
        if self.grad_clip_max_norm is not None and self.grad_clip_max_norm <= 0:
            raise ValueError(f"grad_clip_max_norm must be > 0, got {self.grad_clip_max_norm}")
        self.state.step_context = StepContext(grad_accum_steps=self.grad_accum_steps)
        self._group_manager = ProcessGroupManager.from_plan(self.plan, self.mesh)
        self.plugins = order_plugins(list(self.plugins))
        if self.plan.batch_data_cp_aware:
            if self.mesh.cp <= 1:
                raise ValueError("batch_data_cp_aware=True requires mesh.cp > 1")
            if not self.has_plugin(PluginId.CP):
                raise ValueError("batch_data_cp_aware=True requires ContextParallelPlugin")
        self._optimizer_owner = _single_owner(self.plugins, "owns_optimizer", "optimizer") or self
        self._model_state_owner = _single_owner(self.plugins, "owns_model_state", "model-state") or self
        self._step_runner_owner = self._pick_step_runner_owner()

    def _pick_step_runner_owner(self):
        owner = _single_owner(self.plugins, "owns_step_runner", "step-runner")
        strays = [p.id.value for p in self.plugins if not p.owns_step_runner and p.build_step_runner() is not None]
        if strays:
            warnings.warn("plugins returned step runners without declaring owns_step_runner=True; "
                          f"their step runners will be ignored: {strays}", stacklevel=3)
        return owner or self

    def _resolve_plugin_order(self, plugins: list[RuntimePlugin]) -> list[RuntimePlugin]:
        return order_plugins(plugins)

    def has_plugin(self, plugin_id: PluginId) -> bool:
        return any(p.id == plugin_id for p in self.plugins)

    def get_plugin(self, plugin_id: PluginId) -> RuntimePlugin | None:
        return next((p for p in self.plugins if p.id == plugin_id), None)

    # ------------------------------------------------------------------ setup / teardown
    def setup(self, *, checkpoint_path: str | Path | None = None, load_weights_only: bool = False) -> None:
        if load_weights_only and checkpoint_path is None:
            raise ValueError("load_weights_only=True requires checkpoint_path")
        self.device = _device_of(self.model) if self.device is None else torch.device(self.device)
        self.state_manager.bind(self)
        self._param_roles.clear()
        for plugin in self.plugins:
            plugin.bind(self)
        self._refuse_tied_parameters_under_model_splitting()
        self._run_setup_phase(SetupPhase.TRANSFORM)
        self._run_setup_phase(SetupPhase.MATERIALIZE)
        self.state_manager.register_module(self.model)
        self._run_setup_phase(SetupPhase.FINALIZE)
        for plugin in self.plugins:
            plugin.annotate_param_metadata()
        self._resolve_param_checkpoint_metadata()
        self._populate_static_model_metrics()
        self._setup_optimizer_and_scheduler()
        self._step_runner = self._step_runner_owner.build_step_runner()
        if self._step_runner is None:
            if self._step_runner_owner is self:
                raise ValueError("runtime default step runner owner did not provide a step runner")
            raise ValueError(f"plugin={self._step_runner_owner.id.value} declared owns_step_runner=True but did not provide a step runner")
        if checkpoint_path is not None:
            from maltos_b200.state.checkpoint import load_sharded_checkpoint

            load_sharded_checkpoint(self.state_manager, checkpoint_path, weights_only=load_weights_only)

    def _refuse_tied_parameters_under_model_splitting(self) -> None:
        """A parameter that two modules share (tied input / output embeddings) cannot be cut by tensor or pipeline parallelism
        the way the plugins cut modules - one module at a time: the halves would stop being the same tensor, silently (the
        reference accepts it and trains two diverging copies)."""
        splitting = [pid for pid in (PluginId.TP, PluginId.TP_SP, PluginId.PP) if self.has_plugin(pid)]
        if not splitting:
            return
        owners: dict[int, list[str]] = {}
        for name, param in self.model.named_parameters(remove_duplicate=False):
            owners.setdefault(id(param), []).append(name)
        tied = [names for names in owners.values() if len(names) > 1]
        if tied:
            raise ValueError(f"parameters shared between modules {tied[:4]} are not supported with {[p.value for p in splitting]}: "
                             "untie them (tie_word_embeddings=False) or train without tensor / pipeline parallelism")

    def _run_setup_phase(self, phase: SetupPhase) -> None:
        if phase is SetupPhase.MATERIALIZE and self._model_state_owner is self:
            if self.dtype is None:
                self.model.to(self.device)
            else:
                self.model.to(device=self.device, dtype=self.dtype)
        for plugin in self.plugins:
            self.model = plugin.on_setup_phase(phase, self.model)
        if phase is SetupPhase.MATERIALIZE:
            self._fuse_parameter_groups()

    def _fuse_parameter_groups(self) -> None:
        """Lay the weights of every projection group (q/k/v, gate/up) back to back so that the group runs as one
        GEMM. Skipped when a ZeRO plugin owns the parameter storage (it lays parameters out in its own buckets)."""
        if any(self.has_plugin(z) for z in _ZERO_IDS):
            return
        from maltos_b200.ops.grouped import fuse_parameters

        for module in self.model.modules():
            groups = getattr(module, "parameter_fusion_groups", None)
            if not callable(groups):
                continue
            for params in groups():
                params = [p for p in params if isinstance(p, nn.Parameter)]
                if len(params) > 1 and all(p.is_cuda and p.dtype == torch.bfloat16 and p.dim() == 2 for p in params):
                    fuse_parameters(params)

    def _run_step_phase(self, phase: RuntimePhase) -> None:
        for plugin in self.plugins:
            plugin.on_step_phase(phase)

    def _populate_static_model_metrics(self) -> None:
        self.state.static_metrics["perf/world_size"] = self.mesh.world_size
        if isinstance(self.model, FlopsEstimatableModule):
            try:
                self.state.static_metrics["perf/flops_per_token"] = float(self.model.flops_per_token())
            except AttributeError:
                pass

    def close(self) -> None:
        if self._closed:
            return
        failures: list[BaseException] = []
        for plugin in reversed(self.plugins):
            try:
                plugin.close()
            except BaseException as exc:  # noqa: BLE001 - collected and re-raised as a group
                failures.append(exc)
        if self._group_manager is not None:
            try:
                self._group_manager.close()
            except BaseException as exc:  # noqa: BLE001
                failures.append(exc)
        self._closed = True
        if failures:
            raise ExceptionGroup("RuntimeCore.close() failed", failures)

    # ------------------------------------------------------------------ stepping
    def run_step(self, batch: Any) -> tuple[torch.Tensor, bool]:
        """One micro-step (forward + backward). Returns ``(loss, should_step)``."""
        if self._step_runner is None:
            raise AssertionError("RuntimeCore step runner is not initialized; call setup() first")
        with span("maltos::batch_h2d"):
            batch = _to_device(batch, torch.device(self.device))
        st = self.state
        st.batch = batch
        # tokens of the whole accumulation window (the reference reports the last micro-step only, which under-reports the
        # throughput by the accumulation factor); a plugin may correct the micro-step's count in PRE_STEP_RUNNER
        st.metadata["tokens_micro"] = _token_count(batch)
        ctx = st.step_context
        self._run_step_phase(RuntimePhase.PRE_STEP_RUNNER)
        ntok = st.metadata.pop("tokens_micro", None)
        if ntok is not None:
            st.metadata["tokens"] = ntok + (st.metadata.get("tokens") or 0 if ctx.microbatch_idx != 0 else 0)
        with span("maltos::micro_step_runner"):
            loss = self._step_runner.run(self, st.batch)
        self._accumulate_loss_metric()
        return loss, ctx.advance_micro_step()

    def step_optimizer(self) -> None:
        self._run_step_phase(RuntimePhase.PRE_STEP)
        optimizer, scheduler = self.get_optimizer_and_scheduler()
        if optimizer is None:
            raise RuntimeError("step_optimizer() requires a runtime-owned or plugin-owned optimizer")
        prepare = getattr(optimizer, "copy_master_params", None)
        if callable(prepare):
            prepare()
        scaler = self.state.scaler
        if scaler is not None:
            before = scaler.get_scale()
            scaler.step(optimizer)
            scaler.update()
            after = scaler.get_scale()
            self.state.metadata["loss_scale"] = float(after)
            self.state.metadata["overflow"] = bool(after < before)
        else:
            optimizer.step()
            self.state.metadata["loss_scale"] = None
            self.state.metadata["overflow"] = False
        if scheduler is not None:
            scheduler.step()
        optimizer.zero_grad(set_to_none=True)
        self._run_step_phase(RuntimePhase.POST_STEP)
        self.state.step_context.advance_step()

    # ------------------------------------------------------------------ groups & plugin coordination channels
    def get_group(self, axis: MeshAxis):
        return self._group_manager.get_group(axis)

    def get_group_ranks(self, axis: MeshAxis) -> list[int]:
        return self._group_manager.get_group_ranks(axis)

    def mark_module_path_omitted(self, path: str) -> None:
        self._omitted_module_paths.add(path)

    def is_module_path_omitted(self, path: str) -> bool:
        return any(path == o or path.startswith(o + ".") for o in self._omitted_module_paths)

    def add_module_replacement(self, original: type, replacement: type) -> None:
        self._module_replacements.setdefault(original, set()).add(replacement)

    def get_module_replacements(self, original: type) -> set:
        return self._module_replacements.get(original, set())

    def set_param_role(self, param: nn.Parameter, role: ParamRole) -> None:
        self._param_roles[id(param)] = role

    def get_param_role(self, param: nn.Parameter) -> ParamRole:
        return self._param_roles.get(id(param), ParamRole.SHARED)

    def grad_norm_replica_factor(self, param: nn.Parameter, *, sharded_over: frozenset = frozenset()) -> int:
        """How many ranks hold an identical copy of this parameter's gradient (its square is counted once).
        ``sharded_over``: mesh axes over which the CALLER holds different pieces of the gradient (a sharded optimizer's
        shard group); replication along them does not apply to a shard."""
        name = self.state_manager.get_param_name(param)
        sizes = {MeshAxis.DP: self.mesh.dp, MeshAxis.TP: self.mesh.tp, MeshAxis.PP: self.mesh.pp, MeshAxis.CP: self.mesh.cp}
        factor = 1
        for axis in self.state_manager.params[name].attrs.replicated_axes:
            if axis in sharded_over:
                continue
            if axis in sizes:
                factor *= sizes[axis]
            else:
                group = self.get_group(axis)
                if group is not None:
                    factor *= dist.get_world_size(group)
        if factor < 1:
            raise ValueError(f"invalid grad_norm_replica_factor={factor} for param={name}")
        return factor

    # ------------------------------------------------------------------ model state ownership (default owner)
    def export_model_state(self, state_manager: StateManager) -> tuple[dict[str, torch.Tensor], list[ModelStateMeta]]:
        rank = _rank()
        metas = [e.meta for e in state_manager.params.values()] + [e.meta for e in state_manager.buffers.values()]
        tensors: dict[str, torch.Tensor] = {}
        for meta in metas:
            if meta.source_rank is None:
                raise RuntimeError(f"checkpoint source rank not resolved for model state={meta.state_key}")
            if meta.source_rank == rank:
                tensors[meta.state_key] = state_manager.get_model_tensor(meta.state_key).detach().cpu().clone()
        return tensors, metas

    def import_model_state(self, state_manager: StateManager, model_state: dict[str, torch.Tensor]) -> None:
        for key, value in model_state.items():
            name = state_manager._resolve_runtime_name(key)
            if name not in state_manager.params and name not in state_manager.buffers:
                raise KeyError(f"model state not found: {name}")
            dst = state_manager.get_model_tensor(name)
            dst.data.copy_(value.to(device=dst.device, dtype=dst.dtype))

    def model_state_checkpoint_rank(self, fq_name: str, *, rank_id: int) -> int:
        if fq_name in self.state_manager.buffers:
            return rank_id
        attrs = self.state_manager.params[fq_name].attrs
        return self.mesh.infer_checkpoint_rank(rank_id, plan=self.plan, replicated_axes=attrs.replicated_axes)

    def _resolve_param_checkpoint_metadata(self) -> None:
        rank = _rank()
        for name in list(self.state_manager.params) + list(self.state_manager.buffers):
            self.state_manager.update_model_state(name, source_rank=self.model_state_checkpoint_rank(name, rank_id=rank))

    # ------------------------------------------------------------------ optimizer
    def _setup_optimizer_and_scheduler(self) -> None:
        if self._optimizer_owner is not self:
            optimizer, _ = self._optimizer_owner.get_optimizer_and_scheduler()
            if optimizer is None:
                raise ValueError(f"plugin={self._optimizer_owner.id.value} declared owns_optimizer=True but did not provide an optimizer")
            return
        self._optimizer = self.create_optimizer(self.model.parameters())
        self._scheduler = self.create_scheduler(self._optimizer)

    def get_optimizer_and_scheduler(self):
        if self._optimizer_owner is self:
            return self._optimizer, self._scheduler
        return self._optimizer_owner.get_optimizer_and_scheduler()

    def create_optimizer(self, params: Iterable[nn.Parameter]) -> torch.optim.Optimizer:
        if self.optimizer_factory is None:
            raise ValueError("optimizer_factory is required to create an optimizer")
        params = list(params)
        if self.dtype in (None, torch.float32):
            return self.optimizer_factory(params)
        return MasterWeightsOptimizer(params, optimizer_factory=self.optimizer_factory)

    def create_scheduler(self, optimizer):
        return None if self.scheduler_factory is None else self.scheduler_factory(optimizer)

    def should_save_optimizer(self, rank_id: int) -> bool:
        return self.optimizer_checkpoint_rank(rank_id) == rank_id

    def optimizer_checkpoint_rank(self, rank_id: int) -> int:
        owner = self._optimizer_owner
        return self.optimizer_state_source_rank(rank_id) if owner is self else owner.optimizer_state_source_rank(rank_id)

    def optimizer_state_source_rank(self, rank_id: int) -> int:
        if any(self.has_plugin(z) for z in _ZERO_IDS):
            return rank_id
        roles = {self.get_param_role(p) for p in self.model.parameters() if p.requires_grad}
        if len(roles) != 1:
            return rank_id  # nothing trainable, or a mix of shared and expert state: every rank saves
        axis = MeshAxis.EREP if roles == {ParamRole.EXPERT} else MeshAxis.DCP
        return self.mesh.infer_checkpoint_rank(rank_id, plan=self.plan, replicated_axes={axis})

    def build_step_runner(self):
        return DefaultStepRunner()

    # ------------------------------------------------------------------ metrics
    @profiled("maltos::metrics.collect")
    def collect_metrics(self) -> dict[str, MetricValue]:
        md = self.state.metadata
        out: dict[str, MetricValue] = {"step": self.state.step_context.step}
        out.update(self.state.static_metrics)
        total, count = md.get("loss_sum_for_metrics"), md.get("loss_count_for_metrics", 0)
        if torch.is_tensor(total) and isinstance(count, int) and count > 0:
            out["loss"] = float((total / count).item())  # the only host read of the loss per optimizer step
        elif self.state.loss is not None:
            out["loss"] = float(self.state.loss.detach().float().item())
        if "loss" in out and self.mesh.cp > 1 and self.has_plugin(PluginId.CP):
            # every context-parallel rank differentiates its SHARE of the loss (local mean x local / global targets); the
            # logged value is averaged over all ranks, so report cp x share: the average is then the loss of the whole rows
            # (the reference logs the share, i.e. loss / cp)
            out["loss"] *= float(self.mesh.cp)
        model_metrics = md.get("model_metrics")
        if model_metrics is not None:
            if not isinstance(model_metrics, dict):
                raise TypeError("runtime model_metrics metadata must be a dict")
            for k, v in model_metrics.items():
                if k in out:
                    raise ValueError(f"duplicate model metric key={k}")
                out[k] = float(v.item()) if torch.is_tensor(v) else v
        if md.get("tokens") is not None:
            out["train/tokens"] = float(md["tokens"]) / float(self.mesh.tp * self.mesh.pp * self.mesh.cp)
        optimizer, scheduler = self.get_optimizer_and_scheduler()
        if optimizer is not None and optimizer.param_groups:
            out["lr"] = float(optimizer.param_groups[0]["lr"])
        if scheduler is not None:
            out["scheduler_last_epoch"] = int(scheduler.last_epoch)
        for plugin in self.plugins:
            for k, v in plugin.collect_metrics().items():
                full = k if "/" in k else f"{plugin.id.value}/{k}"
                if full in out:
                    raise ValueError(f"duplicate metric key={full}")
                out[full] = v
        return out

    def _accumulate_loss_metric(self) -> None:
        md = self.state.metadata
        raw = md.pop("raw_loss_for_metrics", None)
        if not torch.is_tensor(raw):
            return
        running, n = md.get("loss_sum_for_metrics"), md.get("loss_count_for_metrics")
        fresh = self.state.step_context.microbatch_idx == 0 or not torch.is_tensor(running) or not isinstance(n, int)
        if fresh:  # new window (also after a mid-accumulation resume, where telemetry is not restored)
            md["loss_sum_for_metrics"], md["loss_count_for_metrics"] = raw.clone(), 1
        else:
            running.add_(raw)
            md["loss_count_for_metrics"] = n + 1


# ---------------------------------------------------------------------- helpers
def _token_count(batch: Any) -> int | None:
    first = None
    if isinstance(batch, dict):
        first = batch.get(INPUT_IDS_KEY)
    elif isinstance(batch, (tuple, list)) and batch:
        first = batch[0]
    elif torch.is_tensor(batch):
        first = batch
    return int(first.numel()) if torch.is_tensor(first) else None


_count_batch_tokens = _token_count


def _device_of(module: nn.Module) -> torch.device:
    for t in module.parameters():
        return t.device
    for t in module.buffers():
        return t.device
    return torch.device("cpu")


def _to_device(value: Any, device: torch.device) -> Any:
    if torch.is_tensor(value):
        return value.to(device, non_blocking=True)
    if isinstance(value, dict):     # host-side bookkeeping (per-row target counts) stays on the host
        return {k: (v if k == LOSS_TARGET_COUNTS_KEY else _to_device(v, device)) for k, v in value.items()}
    if isinstance(value, tuple):
        return tuple(_to_device(v, device) for v in value)
    if isinstance(value, list):
        return [_to_device(v, device) for v in value]
    return value


_move_to_device = _to_device


def _global_token_contribution(local_tokens: int, mesh: MeshConfig) -> float:
    return float(local_tokens) / float(mesh.tp * mesh.pp * mesh.cp)

"""Runtime side of ByteScale HDP: installs the dynamic-ring attention cores and runs a batch as ordered waves.

Layout types live in ``parallel/hdp_helper.py``, scheduling and batch building in ``data/bytescale_hdp.py``. The plugin
owns the step runner: one global batch arrives as an envelope of this rank's wave batches; every wave does a forward
and backward inside the same gradient-accumulation window (ranks with nothing to do in a wave run a 1-token dummy batch
so ZeRO / DDP hooks stay aligned). Reference: ``runtime/plugins/hdp.py:30-259``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.parallel.hdp_helper import (BYTESCALE_HDP_SCHEDULE_KEY, BYTESCALE_HDP_WAVES_KEY, ByteScaleHdpBalancedConfig,
                                             ByteScaleHdpLocalLayout)
from maltos_b200.parallel.protocols import ContextParallelizableModule
from maltos_b200.runtime.layers.hdp_attention import HdpBalancedAttentionCore
from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.step_runners import DefaultStepRunner
from maltos_b200.runtime.types import RuntimePhase, SetupPhase
from maltos_b200.utils.attention_backend import AttentionBackend


def _schedule_from_batch(batch) -> ByteScaleHdpLocalLayout:
    if not isinstance(batch, dict):
        raise TypeError("ByteScale HDP requires a dict batch")
    schedule = batch.get(BYTESCALE_HDP_SCHEDULE_KEY)
    if not isinstance(schedule, ByteScaleHdpLocalLayout):
        raise RuntimeError("ByteScaleHdpDataLoader must attach the local schedule")
    return schedule


def _waves_from_batch(batch) -> tuple[dict, ...]:
    if not isinstance(batch, dict):
        raise TypeError("ByteScale HDP requires a dict batch envelope")
    waves = batch.get(BYTESCALE_HDP_WAVES_KEY)
    if not isinstance(waves, tuple) or not waves or not all(isinstance(w, dict) for w in waves):
        raise RuntimeError("ByteScaleHdpDataLoader must attach a non-empty tuple of local waves")
    return waves


def _wave_metrics(layouts: tuple[ByteScaleHdpLocalLayout, ...]) -> dict[str, float | int]:
    docs = [d for lay in layouts for d in lay.documents]
    return {"global_documents": layouts[0].global_document_count, "local_documents": len(docs),
            "local_valid_tokens": sum(lay.valid_tokens for lay in layouts),
            "local_placement_tokens": sum(lay.placement_tokens for lay in layouts),
            "local_padded_slots": sum(lay.padded_slots for lay in layouts),
            "local_attention_work": sum(d.sequence_length * d.local_length for d in docs), "waves": len(layouts)}


@dataclass
class _WaveClock:
    """Time spent in real and in dummy waves of the current optimizer step (CUDA events, resolved at metric time)."""

    count: int = 0
    seconds: float = 0.0
    events: list = field(default_factory=list)

    def add(self, host_seconds: float, cuda_events) -> None:
        self.count += 1
        self.seconds += host_seconds
        if cuda_events is not None:
            self.events.append(cuda_events)

    def drain(self) -> None:
        for start, end in self.events:
            end.synchronize()
            self.seconds += start.elapsed_time(end) / 1e3
        self.events.clear()

    def reset(self) -> None:
        self.count, self.seconds = 0, 0.0
        self.events.clear()


class ByteScaleHdpPlugin(RuntimePlugin):
    def __init__(self, *, config: ByteScaleHdpBalancedConfig) -> None:
        super().__init__(id=PluginId.HDP, name="bytescale_hdp", runs_after={PluginId.TP, PluginId.TP_SP, PluginId.DP},
                         owns_step_runner=True)
        self.config = config
        self._attention_cores: list[HdpBalancedAttentionCore] = []
        self._metrics: dict[str, float | int] = {}
        self._real, self._dummy = _WaveClock(), _WaveClock()

    @property
    def hdp_group(self) -> dist.ProcessGroup:
        group = self.runtime.get_group(MeshAxis.DCP)
        if group is None:
            raise ValueError("ByteScaleHdpPlugin requires a DCP process group")
        return group

    def bind(self, runtime) -> None:
        super().bind(runtime)
        if any(p.id == PluginId.CP for p in runtime.plugins if p is not self):
            raise ValueError("ByteScaleHdpPlugin and ContextParallelPlugin are mutually exclusive")
        if runtime.mesh.dp * runtime.mesh.cp <= 1:
            raise ValueError("ByteScaleHdpPlugin requires DCP world size > 1")
        if runtime.mesh.cp != 1:
            raise ValueError("ByteScale HDP baseline requires cp_size=1; HDP replaces fixed CP")
        if runtime.mesh.pp != 1:
            raise ValueError("ByteScale HDP currently implements FCP's CP-only baseline and requires pp_size=1")

    def on_setup_phase(self, phase: SetupPhase, model: nn.Module) -> nn.Module:
        if phase is not SetupPhase.TRANSFORM or dist.get_world_size(self.hdp_group) <= 1:
            return model
        if not isinstance(model, ContextParallelizableModule):
            raise TypeError("ByteScaleHdpPlugin requires context_parallel_spec()")
        for path in model.context_parallel_spec().attention_paths:
            if self.runtime.is_module_path_omitted(path):
                continue
            block = model.get_submodule(path)
            if not hasattr(block, "attn_core"):
                raise TypeError(f"attention module path={path} has no attn_core")
            core = HdpBalancedAttentionCore(self.hdp_group, attention_backend=getattr(block.attn_core, "attention_backend", AttentionBackend.EAGER))
            block.attn_core = core
            self._attention_cores.append(core)
        if not self._attention_cores:
            raise ValueError("ByteScaleHdpPlugin found no attention cores to transform")
        return model

    def on_step_phase(self, phase: RuntimePhase) -> None:
        state = self.runtime.state
        if phase is RuntimePhase.PRE_STEP_RUNNER:
            if state.step_context.accum_start:
                self._real.reset()
                self._dummy.reset()
            schedules = tuple(_schedule_from_batch(w) for w in _waves_from_batch(state.batch))
            for s in schedules:
                if s.partition_tokens != self.config.partition_tokens:
                    raise ValueError(f"ByteScale dataloader/plugin partition_tokens mismatch: loader={s.partition_tokens} "
                                     f"plugin={self.config.partition_tokens}")
            state.metadata["tokens_micro"] = schedules[0].global_valid_targets
            self._metrics = _wave_metrics(schedules)
        elif phase is RuntimePhase.PRE_FORWARD:
            schedule = _schedule_from_batch(state.batch)
            for core in self._attention_cores:
                core.set_active_schedule(schedule)

    def collect_metrics(self) -> dict[str, float | int]:
        self._real.drain()
        self._dummy.drain()
        out = dict(self._metrics)
        out.update({"dummy_wave_count": self._dummy.count, "real_wave_count": self._real.count,
                    "dummy_wave_sec": self._dummy.seconds, "real_wave_sec": self._real.seconds,
                    "dummy_wave_sec_sum": self._dummy.seconds, "real_wave_sec_sum": self._real.seconds})
        self._metrics = {}
        return out

    def build_step_runner(self):
        return _HdpWaveStepRunner(self)

    def record_wave_overhead(self, *, is_dummy: bool, host_seconds: float, cuda_events) -> None:
        (self._dummy if is_dummy else self._real).add(host_seconds, cuda_events)


class _HdpWaveStepRunner:
    """Forward + backward of every wave of the envelope; the reported loss is the sum of the (pre-weighted) wave losses."""

    def __init__(self, plugin: ByteScaleHdpPlugin) -> None:
        self.plugin = plugin

    def run(self, runtime, batch) -> torch.Tensor:
        waves = _waves_from_batch(batch)
        losses = []
        for i, wave in enumerate(waves):
            runtime.state.step_context.set_hdp_wave(wave_idx=i, wave_count=len(waves))
            runtime.state.batch = wave
            is_dummy = not _schedule_from_batch(wave).documents
            t0 = time.perf_counter()
            events = None
            if torch.cuda.is_available():
                events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                events[0].record()
            DefaultStepRunner.run_forward(runtime, wave)
            if not torch.is_tensor(runtime.state.loss):
                raise TypeError("ByteScale HDP requires each wave to produce a Tensor loss")
            losses.append(runtime.state.loss.detach())
            DefaultStepRunner.run_backward(runtime)
            if events is not None:
                events[1].record()
            self.plugin.record_wave_overhead(is_dummy=is_dummy, host_seconds=0.0 if events else time.perf_counter() - t0, cuda_events=events)
        total = torch.stack(losses).sum()
        runtime.state.loss = total
        runtime.state.metadata["raw_loss_for_metrics"] = total
        return total

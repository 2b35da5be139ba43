"""``torch.profiler`` integration: a wait/warmup/active/repeat schedule stepped at POST_STEP, one Chrome trace per rank
under ``trace_dir/rank_XXXXX/trace.json``; ``rank0_only`` profiles a single rank and barriers around trace boundaries so
the others do not run ahead (reference ``runtime/plugins/torch_profiler.py:12-136``)."""
from __future__ import annotations

from pathlib import Path

import torch
import torch.distributed as dist

from maltos_b200.runtime.plugin import PluginId, RuntimePlugin
from maltos_b200.runtime.types import RuntimePhase, SetupPhase


class TorchProfilerPlugin(RuntimePlugin):
    def __init__(self, trace_dir: str, wait: int = 1, warmup: int = 1, active: int = 2, repeat: int = 1, record_shapes: bool = False,
                 profile_memory: bool = False, with_stack: bool = False, with_flops: bool = False, rank0_only: bool = False) -> None:
        super().__init__(id=PluginId.TORCH_PROFILER, name="torch_profiler")
        self.trace_dir = Path(trace_dir)
        self.wait, self.warmup, self.active, self.repeat = wait, warmup, active, repeat
        self.record_shapes, self.profile_memory, self.with_stack, self.with_flops = record_shapes, profile_memory, with_stack, with_flops
        self.rank0_only = rank0_only
        self._profiler = None
        self._steps = 0
        self.trace_paths: list[Path] = []

    def _rank(self) -> int:
        return dist.get_rank() if dist.is_initialized() else 0

    def _enabled_here(self) -> bool:
        return not self.rank0_only or self._rank() == 0

    def on_setup_phase(self, phase: SetupPhase, model):
        if phase is SetupPhase.FINALIZE and self._enabled_here() and self._profiler is None:
            out_dir = self.trace_dir / f"rank_{self._rank():05d}"
            out_dir.mkdir(parents=True, exist_ok=True)
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)

            def on_trace(prof) -> None:
                idx = len(self.trace_paths)
                path = out_dir / ("trace.json" if idx == 0 else f"trace_{idx}.json")
                prof.export_chrome_trace(str(path))
                self.trace_paths.append(path)

            self._profiler = torch.profiler.profile(
                activities=acts, schedule=torch.profiler.schedule(wait=self.wait, warmup=self.warmup, active=self.active, repeat=self.repeat),
                on_trace_ready=on_trace, record_shapes=self.record_shapes, profile_memory=self.profile_memory,
                with_stack=self.with_stack, with_flops=self.with_flops)
            self._profiler.start()
        return model

    def on_step_phase(self, phase: RuntimePhase) -> None:
        if phase is not RuntimePhase.POST_STEP:
            return
        self._steps += 1
        cycle = self.wait + self.warmup + self.active
        at_boundary = cycle > 0 and self._steps % cycle in (self.wait + self.warmup, 0)
        if self.rank0_only and at_boundary and dist.is_initialized():
            dist.barrier()
        if self._profiler is not None:
            self._profiler.step()
        if self.rank0_only and at_boundary and dist.is_initialized():
            dist.barrier()

    def collect_metrics(self):
        """The reference's keys (``runtime/plugins/torch_profiler.py:88-97``)."""
        enabled = self._profiler is not None
        out_dir = self.trace_dir / f"rank_{self._rank():05d}"
        return {"torch_profiler/enabled": enabled, "torch_profiler/rank0_only": self.rank0_only,
                "torch_profiler/trace_dir": str(out_dir) if enabled else None, "torch_profiler/wait": self.wait,
                "torch_profiler/warmup": self.warmup, "torch_profiler/active": self.active, "torch_profiler/repeat": self.repeat}

    def close(self) -> None:
        if self._profiler is not None:
            self._profiler.stop()
            self._profiler = None

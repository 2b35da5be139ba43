"""Training loop: the Trainer owns cadence (steps, logging, checkpoints, retention), the RuntimeCore owns execution.

``fit`` pulls micro-batches until ``max_steps`` optimizer steps are done; metrics are collected once per optimizer step
and flushed asynchronously (the numbers of interval k are printed at interval k+1), checkpoints are written every
``checkpoint_every`` steps into ``checkpoint_dir/step_XXXXXXXX`` with optional retention (``keep_last`` /
``keep_every_n_steps``) and a free-space guard. Interface of the reference's ``train/trainer.py:25-183``.
"""
from __future__ import annotations

import re
import shutil
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch.distributed as dist

from maltos_b200.data.prefetch import PrefetchDataLoader
from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.state.checkpoint import save_runtime_spec, save_sharded_checkpoint
from maltos_b200.utils.distributed import raise_if_any_rank_failed
from maltos_b200.utils.metrics import MetricAggregator, PendingMetricFlush
from maltos_b200.utils.profiling import span


@dataclass(frozen=True)
class TrainerConfig:
    max_steps: int
    log_every: int = 1
    checkpoint_every: int | None = None
    checkpoint_dir: str | Path | None = None
    resume_from: str | Path | None = None
    load_weights_only: bool = False
    checkpoint_keep_last: int | None = None
    checkpoint_keep_every_n_steps: int | None = None
    checkpoint_min_free_gb: float | None = None
    data_prefetch_batches: int = 0


def _is_log_rank() -> bool:
    return not dist.is_initialized() or dist.get_rank() == 0


def _checkpoint_step_dir(root, step: int) -> Path:
    return Path(root) / f"step_{step:08d}"


def _checkpoint_step_dirs(root: Path) -> list[tuple[int, Path]]:
    if not root.is_dir():
        return []
    out = []
    for p in root.iterdir():
        m = re.fullmatch(r"step_(\d{8})", p.name) if p.is_dir() else None
        if m:
            out.append((int(m.group(1)), p))
    return out


def _apply_checkpoint_retention(root, *, current_step: int, keep_last: int | None, keep_every_n_steps: int | None) -> None:
    if (keep_last is None and keep_every_n_steps is None) or not _is_log_rank():
        return
    found = sorted(_checkpoint_step_dirs(Path(root)))
    keep = {p for s, p in found if s == current_step}
    if keep_last:
        keep |= {p for _, p in found[-keep_last:]}
    if keep_every_n_steps is not None:
        keep |= {p for s, p in found if s % keep_every_n_steps == 0}
    for _, p in found:
        if p not in keep:
            shutil.rmtree(p)


def _validate(config: TrainerConfig, runtime_spec) -> None:
    if config.max_steps < 0:
        raise ValueError(f"max_steps must be >= 0, got {config.max_steps}")
    if config.log_every < 1:
        raise ValueError(f"log_every must be >= 1, got {config.log_every}")
    if config.checkpoint_every is not None:
        if config.checkpoint_every < 1:
            raise ValueError(f"checkpoint_every must be >= 1, got {config.checkpoint_every}")
        if config.checkpoint_dir is None:
            raise ValueError("checkpoint_dir is required when checkpoint_every is set")
        if runtime_spec is None:
            raise ValueError("runtime_spec is required when checkpoint_every is set")
    if config.checkpoint_keep_last is not None and config.checkpoint_keep_last < 0:
        raise ValueError(f"checkpoint_keep_last must be >= 0, got {config.checkpoint_keep_last}")
    if config.checkpoint_keep_every_n_steps is not None and config.checkpoint_keep_every_n_steps < 1:
        raise ValueError(f"checkpoint_keep_every_n_steps must be >= 1, got {config.checkpoint_keep_every_n_steps}")
    if config.checkpoint_min_free_gb is not None and config.checkpoint_min_free_gb < 0:
        raise ValueError(f"checkpoint_min_free_gb must be >= 0, got {config.checkpoint_min_free_gb}")
    if config.data_prefetch_batches not in (0, 1):
        raise ValueError("data_prefetch_batches currently supports only 0 or 1")


class Trainer:
    def __init__(self, *, runtime, dataloader, config: TrainerConfig, logger=None, metric_aggregator: MetricAggregator | None = None,
                 checkpoint_uploader=None, runtime_spec: dict[str, Any] | None = None) -> None:
        _validate(config, runtime_spec)
        self.runtime = runtime
        self.dataloader = PrefetchDataLoader(dataloader) if config.data_prefetch_batches else dataloader
        self.config = config
        self.loggers = [] if logger is None else (logger if isinstance(logger, list) else [logger])
        self.metric_aggregator = metric_aggregator or MetricAggregator()
        self.checkpoint_uploader = checkpoint_uploader
        self.runtime_spec = runtime_spec
        self._last_logged_step = 0
        self._pending_log: PendingMetricFlush | None = None
        self._graceful_stop = False
        self._stop_requested = False
        self._stop_pending = None
        self.stopped_early_at: int | None = None
        self.heartbeat = None

    def setup(self) -> None:
        self.runtime.state_manager.bind_dataloader(self.dataloader)
        self.runtime.setup(checkpoint_path=self.config.resume_from, load_weights_only=self.config.load_weights_only)
        if self.config.checkpoint_every is not None:
            failure = None
            try:
                if _is_log_rank():
                    save_runtime_spec(self.config.checkpoint_dir, self.runtime_spec)
            except Exception as exc:  # noqa: BLE001 - an unwritable checkpoint directory must stop every rank, now
                failure = exc
            raise_if_any_rank_failed(failure, f"writing the runtime spec under {self.config.checkpoint_dir}")
        self._last_logged_step = self.runtime.state.step_context.step

    # ------------------------------------------------------------------ graceful stop (not in the reference)
    def enable_graceful_stop(self, signals=()) -> None:
        """After this call ``request_stop()`` - from any rank, e.g. from the handler installed here for ``signals`` (a
        scheduler's SIGTERM before preemption) - ends ``fit()`` cleanly: all ranks finish the same optimizer step, write a
        checkpoint of it (when a checkpoint directory is configured) and return; ``--resume-from auto`` continues there.
        The ranks agree through one asynchronous one-element all-reduce per optimizer step that is read a step later, when
        it has long finished: no extra synchronisation in the step, and a stop takes effect within two steps."""
        import signal as _signal

        self._graceful_stop = True
        for sig in signals:
            _signal.signal(sig, lambda *_: self.request_stop())

    def enable_heartbeat(self, *, timeout: float, interval: float = 1.0) -> None:
        """Watch the other ranks from a background thread (``utils/heartbeat.py``); ``fit()`` then checks before every
        micro-step and raises ``PeerLostError`` instead of launching into a collective that a dead rank will never join."""
        from maltos_b200.utils.heartbeat import HeartbeatMonitor

        if dist.is_initialized() and dist.get_world_size() > 1:
            self.heartbeat = HeartbeatMonitor.for_default_group(interval=interval, timeout=timeout).start()

    def request_stop(self) -> None:
        self._stop_requested = True

    def _stop_agreed(self) -> bool:
        """Once per optimizer step on every rank: reads the agreement issued a step ago, issues the next one."""
        if not self._graceful_stop:
            return False
        import torch

        from maltos_b200.utils.metrics import _metric_device

        previous, self._stop_pending = self._stop_pending, None
        agreed = False
        if previous is not None:
            work, flag = previous
            if work is not None:
                work.wait()
            agreed = bool(flag.item())
        flag = torch.tensor([1.0 if self._stop_requested else 0.0], device=_metric_device())
        work = None
        if dist.is_initialized() and dist.get_world_size() > 1:
            work = dist.all_reduce(flag, op=dist.ReduceOp.MAX, async_op=True)
        self._stop_pending = (work, flag)
        return agreed

    def _cp_rank(self):
        if not self.runtime.plan.batch_data_cp_aware:
            return None
        return dist.get_rank(self.runtime.get_group(MeshAxis.CP))

    def fit(self) -> None:
        rt = self.runtime
        try:
            while rt.state.step_context.step < self.config.max_steps:
                with span("maltos::data.next_batch"):
                    batch = self.dataloader.next_batch(self._cp_rank())
                if self.heartbeat is not None:
                    self.heartbeat.check()
                _, should_step = rt.run_step(batch)
                if not should_step:
                    continue
                with span("maltos::optimizer_step"):
                    rt.step_optimizer()
                with span("maltos::metrics.aggregate"):
                    self.metric_aggregator.update(rt.collect_metrics())   # one host read of the loss per optimizer step
                self._maybe_log()
                self._maybe_checkpoint()
                if self._stop_agreed():
                    self.stopped_early_at = rt.state.step_context.step
                    self._maybe_checkpoint(force=True)
                    break
            self._flush_pending_log()
        finally:
            if self.heartbeat is not None:
                self.heartbeat.stop()
            rt.close()
            closer = getattr(self.dataloader, "close", None)
            if callable(closer):
                closer()
            if self.checkpoint_uploader is not None:
                self.checkpoint_uploader.close()

    # ------------------------------------------------------------------ logging
    def _emit(self, metrics: dict[str, Any]) -> None:
        if self.loggers and _is_log_rank():
            for lg in self.loggers:
                lg.log(metrics)

    def _maybe_log(self) -> None:
        step = self.runtime.state.step_context.step
        if step == 0 or step % self.config.log_every:
            return
        delta, self._last_logged_step = step - self._last_logged_step, step
        with span("maltos::metrics.flush_async"):
            fresh = self.metric_aggregator.flush_async(step_delta=delta)
        previous, self._pending_log = self._pending_log, fresh
        if previous is not None:
            with span("maltos::metrics.wait_previous"):
                self._emit(previous.wait())

    def _flush_pending_log(self) -> None:
        pending, self._pending_log = self._pending_log, None
        if pending is not None:
            with span("maltos::metrics.wait_final"):
                self._emit(pending.wait())

    # ------------------------------------------------------------------ checkpoints
    def _maybe_checkpoint(self, force: bool = False) -> None:
        every = self.config.checkpoint_every
        step = self.runtime.state.step_context.step
        if every is None or step == 0:
            return
        if force:
            if step % every == 0:
                return                          # the regular save of this step has just been written
        elif step % every:
            return
        target = _checkpoint_step_dir(self.config.checkpoint_dir, step)
        with span("maltos::checkpoint.save"):
            save_sharded_checkpoint(self.runtime.state_manager, target, min_free_gb=self.config.checkpoint_min_free_gb)
        _apply_checkpoint_retention(self.config.checkpoint_dir, current_step=step, keep_last=self.config.checkpoint_keep_last,
                                    keep_every_n_steps=self.config.checkpoint_keep_every_n_steps)
        if self.checkpoint_uploader is not None and _is_log_rank():
            self.checkpoint_uploader.upload_checkpoint(target, step)

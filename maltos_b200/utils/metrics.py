"""Metric aggregation, cross-rank reduction and sinks.

Per optimizer step the trainer feeds ``RuntimeCore.collect_metrics()`` into a :class:`MetricAggregator`. At a logging
boundary every key is reduced locally over the steps of the interval and then across ranks with ONE packed fp64
all-reduce per reduction kind, issued asynchronously and consumed at the next boundary, so logging never stalls the
step that follows. Rules are chosen from the key (reference ``utils/metrics.py:331-354``): ``loss*`` mean/mean;
``*_sec`` sum/max then divided by the number of steps, the interval total kept as ``*_window``; ``*tokens*`` sum/sum;
``*/grad_norm`` and ``memory*`` max/max; ``*/overflow`` any; everything else last value of rank 0. Derived:
``train/tokens_per_sec`` and ``perf/tflops_per_gpu``.
"""
from __future__ import annotations

import concurrent.futures
import json
import re
from dataclasses import dataclass
from enum import Enum
from pathlib import Path
from typing import Any, Protocol

import torch
import torch.distributed as dist

MetricValue = float | int | str | bool | None


class MetricLogger(Protocol):
    def log(self, metrics: dict[str, MetricValue]) -> None: ...


class MetricReduction(str, Enum):
    MEAN = "mean"
    SUM = "sum"
    LAST = "last"
    MAX = "max"
    ANY = "any"
    RANK0 = "rank0"
    NONE = "none"


class MetricStepReduction(str, Enum):
    PER_STEP = "per_step"


@dataclass(frozen=True)
class MetricRule:
    local: MetricReduction = MetricReduction.LAST
    distributed: MetricReduction = MetricReduction.RANK0
    step: MetricStepReduction | None = None


_R = MetricReduction
_LAST0 = MetricRule(_R.LAST, _R.RANK0)
_EXACT_LAST = {"lr", "step", "microbatch_idx", "grad_accum_steps", "scheduler_last_epoch", "should_step_optimizer"}


def _rule_for_key(key: str, rules: dict[str, MetricRule]) -> MetricRule:
    if key in rules:
        return rules[key]
    if key == "loss" or key.startswith("loss/") or key.endswith("/loss") or key.endswith("_loss"):      # moe/load_balance_loss too
        return MetricRule(_R.MEAN, _R.MEAN)
    if key in _EXACT_LAST or key.endswith("/lr"):
        return _LAST0
    if key.endswith("_sec"):
        return MetricRule(_R.SUM, _R.MAX, MetricStepReduction.PER_STEP)
    if key.endswith("_sec_sum") or key.endswith("_wave_count"):
        return MetricRule(_R.SUM, _R.SUM, MetricStepReduction.PER_STEP)
    if key.endswith("/overflow"):
        return MetricRule(_R.ANY, _R.ANY)
    if key.endswith("/grad_norm") or "memory" in key:
        return MetricRule(_R.MAX, _R.MAX)
    if "tokens" in key:
        return MetricRule(_R.SUM, _R.SUM)
    return _LAST0


def _is_number(v) -> bool:
    return isinstance(v, (float, int, bool))


def _reduce_local(values: list[MetricValue], how: MetricReduction) -> MetricValue:
    kept = [v for v in values if v is not None]
    if not kept:
        return None
    if how in (_R.LAST, _R.RANK0, _R.NONE):
        return kept[-1]
    if how is _R.ANY:
        return any(bool(v) for v in kept)
    if not all(_is_number(v) for v in kept):
        return kept[-1]
    nums = [float(v) for v in kept]
    if how is _R.MEAN:
        return sum(nums) / len(nums)
    if how is _R.SUM:
        return sum(nums)
    if how is _R.MAX:
        return max(nums)
    raise ValueError(f"unsupported local metric reduction={how.value}")


def _metric_device() -> torch.device:
    if dist.is_initialized() and dist.get_backend() == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


@dataclass
class PendingMetricSync:
    result: dict[str, MetricValue]
    pending: list                     # (packed tensor, work, [(key, local value)], as_bool)
    reductions: dict[str, MetricReduction]

    def wait(self) -> dict[str, MetricValue]:
        for packed, work, items, as_bool in self.pending:
            work.wait()
            for (key, _), v in zip(items, packed.tolist()):
                if as_bool:
                    self.result[key] = bool(v)
                elif self.reductions[key] is _R.MEAN:
                    self.result[key] = v / dist.get_world_size()
                else:
                    self.result[key] = v
        self.pending.clear()
        return self.result


class DistributedMetricSync:
    def reduce_value(self, value: MetricValue, how: MetricReduction) -> MetricValue:
        return self.reduce_metrics({"_": value}, {"_": how})["_"]

    def reduce_metrics_async(self, metrics: dict[str, MetricValue], reductions: dict[str, MetricReduction]) -> PendingMetricSync:
        if not dist.is_initialized():
            return PendingMetricSync(dict(metrics), [], reductions)
        passthrough: dict[str, MetricValue] = {}
        sums, maxes, anys = [], [], []
        for key, value in metrics.items():
            how = reductions[key]
            if how in (_R.NONE, _R.RANK0, _R.LAST) or value is None or not _is_number(value):
                passthrough[key] = value
            elif how in (_R.MEAN, _R.SUM):
                sums.append((key, float(value)))
            elif how is _R.MAX:
                maxes.append((key, float(value)))
            elif how is _R.ANY:
                anys.append((key, float(bool(value))))
            else:
                raise ValueError(f"unsupported distributed metric reduction={how.value}")
        dev = _metric_device()
        pending = []
        for items, op, as_bool, dtype in ((sums, dist.ReduceOp.SUM, False, torch.float64), (maxes, dist.ReduceOp.MAX, False, torch.float64),
                                          (anys, dist.ReduceOp.MAX, True, torch.int64)):
            if items:
                packed = torch.tensor([v for _, v in items], dtype=dtype, device=dev)
                pending.append((packed, dist.all_reduce(packed, op=op, async_op=True), items, as_bool))
        return PendingMetricSync(passthrough, pending, reductions)

    def reduce_metrics(self, metrics, reductions) -> dict[str, MetricValue]:
        return self.reduce_metrics_async(metrics, reductions).wait()


def _apply_step_reductions(metrics: dict[str, MetricValue], rules: dict[str, MetricRule], *, step_delta: int | None) -> None:
    for key, value in list(metrics.items()):
        if _rule_for_key(key, rules).step is not MetricStepReduction.PER_STEP:
            continue
        if step_delta is None or step_delta < 1:
            raise ValueError(f"step_delta must be >= 1 for per-step metric {key!r}, got {step_delta}")
        if isinstance(value, (float, int)):
            metrics[f"{key}_window"] = float(value)
            metrics[key] = float(value) / float(step_delta)


def _add_derived_metrics(m: dict[str, MetricValue]) -> None:
    tokens = m.get("train/tokens")
    elapsed = m.get("perf/step_sec_window", m.get("perf/step_sec"))
    if isinstance(tokens, (float, int)) and isinstance(elapsed, (float, int)) and elapsed > 0:
        m["train/tokens_per_sec"] = float(tokens) / float(elapsed)
    tps, fpt, world = m.get("train/tokens_per_sec"), m.get("perf/flops_per_token"), m.get("perf/world_size")
    if all(isinstance(x, (float, int)) for x in (tps, fpt, world)) and world > 0:
        m["perf/tflops_per_gpu"] = float(tps) * float(fpt) / float(world) / 1e12


@dataclass
class PendingMetricFlush:
    sync: PendingMetricSync
    rules: dict[str, MetricRule]
    step_delta: int | None

    def wait(self) -> dict[str, MetricValue]:
        out = self.sync.wait()
        _apply_step_reductions(out, self.rules, step_delta=self.step_delta)
        _add_derived_metrics(out)
        return out


class MetricAggregator:
    def __init__(self, rules: dict[str, MetricRule] | None = None, syncer: DistributedMetricSync | None = None) -> None:
        self.rules = rules or {}
        self.syncer = syncer or DistributedMetricSync()
        self._values: dict[str, list[MetricValue]] = {}

    def update(self, metrics: dict[str, MetricValue]) -> None:
        for k, v in metrics.items():
            self._values.setdefault(k, []).append(v)

    def has_values(self) -> bool:
        return bool(self._values)

    def flush_async(self, *, step_delta: int | None = None) -> PendingMetricFlush:
        local = {k: _reduce_local(v, _rule_for_key(k, self.rules).local) for k, v in self._values.items()}
        self._values.clear()
        sync = self.syncer.reduce_metrics_async(local, {k: _rule_for_key(k, self.rules).distributed for k in local})
        return PendingMetricFlush(sync, self.rules, step_delta)

    def flush(self, *, step_delta: int | None = None) -> dict[str, MetricValue]:
        return self.flush_async(step_delta=step_delta).wait()


# ------------------------------------------------------------------------------------------------ sinks
def _format_metric_value(v: MetricValue) -> str:
    return f"{v:.6g}" if isinstance(v, float) else str(v)


_CONSOLE_FIELDS = (
    ("loss", "loss", lambda v: f"{v:.6g}"),
    ("lr", "lr", lambda v: f"{v:.2e}"),
    ("perf/step_sec", "step", lambda v: f"{v:.2f}s"),
    ("train/tokens_per_sec", "throughput", lambda v: f"{v:,.0f} tok/s"),
    ("perf/tflops_per_gpu", "compute", lambda v: f"{v:.1f} TF/GPU"),
    ("zero3/grad_norm", "grad-norm", lambda v: f"{v:.4g}"),
)


def _format_metrics(metrics: dict[str, MetricValue]) -> str:
    """One compact console line with the values worth watching live; everything else only goes to JSONL / W&B."""
    step = metrics.get("step")
    head = f"step {int(step):05d}" if isinstance(step, int) and not isinstance(step, bool) else "step"
    parts = []
    for key, label, fmt in _CONSOLE_FIELDS:
        v = metrics.get(key)
        if isinstance(v, (float, int)) and not isinstance(v, bool):
            parts.append(f"{label} {fmt(float(v))}")
    alloc, peak = metrics.get("memory/allocated_gb"), metrics.get("memory/max_allocated_gb")
    if isinstance(alloc, (float, int)) and isinstance(peak, (float, int)):
        parts.append(f"memory {float(alloc):.1f}/{float(peak):.1f} GiB")
    if parts:
        return f"[{head}] " + " | ".join(parts)
    return " ".join(f"{k}={_format_metric_value(v)}" for k, v in sorted(metrics.items()))


class ConsoleMetricLogger:
    def log(self, metrics: dict[str, MetricValue]) -> None:
        print(_format_metrics(metrics), flush=True)


class JsonlMetricLogger:
    def __init__(self, path) -> None:
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)

    def log(self, metrics: dict[str, MetricValue]) -> None:
        with self.path.open("a", encoding="utf-8") as f:
            f.write(json.dumps(metrics, sort_keys=True) + "\n")


class WandbMetricLogger:
    """Weights & Biases sink; ``wandb`` is imported only when this logger is constructed."""

    def __init__(self, *, project: str, name: str | None = None, entity: str | None = None, run_id: str | None = None,
                 mode: str | None = None, tags: list[str] | None = None, config: dict[str, Any] | None = None) -> None:
        import wandb

        self.wandb = wandb
        self.run = wandb.init(project=project, name=name, entity=entity, id=run_id, resume="allow" if run_id is not None else None,
                              mode=mode, tags=tags, config=config)

    def log(self, metrics: dict[str, MetricValue]) -> None:
        step = metrics.get("step")
        self.wandb.log(metrics, step=int(step) if isinstance(step, int) else None)


def _sanitize_artifact_name(name: str) -> str:
    return re.sub(r"[^A-Za-z0-9_.-]+", "-", name).strip("-._") or "checkpoint"


class WandbCheckpointUploader:
    """Uploads ``step_XXXXXXXX`` directories (plus ``runtime_spec.json``) as artifacts on a background thread; a new
    upload is skipped while the previous one is still running."""

    def __init__(self, logger: WandbMetricLogger, *, every_steps: int, artifact_prefix: str | None = None) -> None:
        if every_steps < 1:
            raise ValueError(f"every_steps must be >= 1, got {every_steps}")
        self.logger = logger
        self.every_steps = every_steps
        self.artifact_prefix = _sanitize_artifact_name(artifact_prefix or logger.run.name or logger.run.id)
        self.executor = concurrent.futures.ThreadPoolExecutor(max_workers=1)
        self._future: concurrent.futures.Future | None = None

    def _reap(self, wait: bool = False) -> None:
        if self._future is None:
            return
        if wait:
            concurrent.futures.wait([self._future])
        if self._future.done() and self._future.exception() is not None:
            print(f"warning: W&B checkpoint upload failed: {self._future.exception()}")

    def upload_checkpoint(self, checkpoint_dir, step: int) -> None:
        if step % self.every_steps:
            return
        self._reap()
        if self._future is not None and not self._future.done():
            print(f"warning: previous W&B checkpoint upload still running; skip step={step}")
            return
        self._future = self.executor.submit(self._upload, Path(checkpoint_dir), step)

    def _upload(self, checkpoint_dir: Path, step: int) -> None:
        art = self.logger.wandb.Artifact(name=f"{self.artifact_prefix}-step-{step:08d}", type="checkpoint",
                                         metadata={"step": step, "path": str(checkpoint_dir)})
        spec = checkpoint_dir.parent / "runtime_spec.json"
        if not spec.is_file():
            raise FileNotFoundError(f"runtime checkpoint spec not found: {spec}")
        art.add_file(str(spec), name="runtime_spec.json")
        art.add_dir(str(checkpoint_dir), name=checkpoint_dir.name)
        self.logger.run.log_artifact(art, aliases=["latest", f"step_{step}"]).wait()

    def close(self) -> None:
        self._reap(wait=True)
        self.executor.shutdown(wait=True)

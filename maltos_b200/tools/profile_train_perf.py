"""Synthetic-data training throughput benchmark for any recipe, runtime spec or named case.

Builds the normal model and ``RuntimeCore`` of a recipe (through the same builders as the training CLI), feeds it
deterministic synthetic causal-LM batches - dense rows, or packed rows of several documents with partial supervision and
tail padding - and times global optimizer steps. The learning rate is 0 by default so the fixed workload cannot
diverge while forward, backward, clipping and the optimizer all run. Step time is the per-step maximum over ranks of a
device-synchronised wall clock. Results go to ``<output-dir>/summary.json`` and ``summary.txt``; ``--profile`` adds a
torch.profiler trace of the timed steps. Command line after the reference's ``tools/profile_train_perf.py:123-203``:

    torchrun --nproc_per_node=8 -m maltos_b200.tools.profile_train_perf --recipe configs/llama3_8b_tp8.yaml --warmup 3 --steps 5
    torchrun --nproc_per_node=8 -m maltos_b200.tools.profile_train_perf --case llama3_8b_tp8 -- --micro-batch-size 2
"""
from __future__ import annotations

import argparse
import json
import math
import platform
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist
import yaml

from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.train import cli as train_cli
from maltos_b200.train.flags import parse_args_from, parse_runtime_spec_args
from maltos_b200.utils.constants import IGNORE_INDEX, INPUT_IDS_KEY, LABELS_KEY, PAD_SEQUENCE_ID, POSITION_IDS_KEY, SEQUENCE_IDS_KEY

DEFAULT_CASE_FILE = Path("configs/profile_train_perf_cases.yaml")
_SYNTHETIC_KEYS = ("packed", "packed_sequences", "segment_count_min", "segment_count_max", "supervised_fraction_min",
                   "supervised_fraction_max", "max_padding_fraction", "delivery", "data_source", "document_length_trace")


@dataclass(frozen=True)
class CaseDefinition:
    name: str
    description: str = ""
    recipe: str | None = None
    runtime_spec: str | None = None
    recipe_overrides: tuple[str, ...] = ()
    synthetic: dict[str, Any] | None = None
    warmup: int | None = None
    steps: int | None = None
    require_calibrated_hdp_cost: bool = False       # refuse the uncalibrated 1 / 0 / 0 cost proxy (measurement cases)


@dataclass(frozen=True)
class SyntheticBatchConfig:
    """Shape of the synthetic input distribution."""

    layout: str = "dense"                   # "dense" rows, or "packed" rows of several documents
    segment_count_min: int = 3
    segment_count_max: int = 7
    supervised_fraction_min: float = 1.0    # share of a document's tokens (its tail) that carry a loss
    supervised_fraction_max: float = 1.0
    max_padding_fraction: float = 0.0       # tail padding of a packed row, uniform in [0, max]
    delivery: str = "host"                  # "host": CPU batches moved by the runtime; "device": created on the device
    document_length_trace: tuple | None = None   # packed rows follow these document lengths (row i uses trace[i % len]) instead of random cuts

    def __post_init__(self) -> None:
        if self.document_length_trace is not None:
            if self.layout != "packed":
                raise ValueError("document_length_trace needs the packed layout")
            if not self.document_length_trace or any(not row or any(int(n) < 2 for n in row) for row in self.document_length_trace):
                raise ValueError("document_length_trace rows must be non-empty lists of document lengths >= 2")
        if self.layout not in ("dense", "packed"):
            raise ValueError(f"synthetic layout must be dense or packed, got {self.layout!r}")
        if not 1 <= self.segment_count_min <= self.segment_count_max:
            raise ValueError("segment counts must satisfy 1 <= min <= max")
        for lo, hi, what in ((self.supervised_fraction_min, self.supervised_fraction_max, "supervised_fraction"),
                             (0.0, self.max_padding_fraction, "max_padding_fraction")):
            if not 0.0 <= lo <= hi <= 1.0:
                raise ValueError(f"{what} must lie in [0, 1] with min <= max")
        if self.delivery not in ("host", "device"):
            raise ValueError(f"delivery must be host or device, got {self.delivery!r}")


# ------------------------------------------------------------------------------------------------ synthetic data
def make_synthetic_batch(*, rows: int, seq_len: int, vocab_size: int, config: SyntheticBatchConfig, generator: torch.Generator,
                         device: torch.device | str = "cpu", row_offset: int = 0) -> dict[str, torch.Tensor]:
    """One ``[rows, seq_len]`` batch with already-shifted labels (and positions / sequence ids when packed)."""
    tokens = torch.randint(0, vocab_size, (rows, seq_len + 1), generator=generator, dtype=torch.long)
    ids, labels = tokens[:, :-1].clone(), tokens[:, 1:].clone()
    if config.layout == "dense":
        return {INPUT_IDS_KEY: ids.to(device), LABELS_KEY: labels.to(device)}
    pos = torch.zeros((rows, seq_len), dtype=torch.long)
    seq = torch.full((rows, seq_len), PAD_SEQUENCE_ID, dtype=torch.long)
    uniform = lambda lo, hi: lo + (hi - lo) * float(torch.rand((), generator=generator))   # noqa: E731
    for r in range(rows):
        if config.document_length_trace is not None:
            lengths = [int(n) for n in config.document_length_trace[(row_offset + r) % len(config.document_length_trace)]]
            if sum(lengths) > seq_len:
                raise ValueError(f"document_length_trace row sums to {sum(lengths)} > seq_len {seq_len}")
            bounds = [0]
            for n in lengths:
                bounds.append(bounds[-1] + n)
            used = bounds[-1]
        else:
            used = seq_len - int(round(uniform(0.0, config.max_padding_fraction) * seq_len))
            n_docs = int(torch.randint(config.segment_count_min, config.segment_count_max + 1, (), generator=generator))
            n_docs = max(1, min(n_docs, used // 2))
            cuts = sorted(set(torch.randperm(max(used - 1, 1), generator=generator)[:n_docs - 1].add(1).tolist())) if n_docs > 1 else []
            bounds = [0, *cuts, used]
        for d, (a, b) in enumerate(zip(bounds, bounds[1:])):
            seq[r, a:b] = d
            pos[r, a:b] = torch.arange(b - a)
            supervised = max(1, int(round(uniform(config.supervised_fraction_min, config.supervised_fraction_max) * (b - a))))
            labels[r, a:b - supervised] = IGNORE_INDEX       # the prompt part carries no loss
            labels[r, b - 1] = IGNORE_INDEX                  # the last token of a document has no target inside it
        labels[r, used:] = IGNORE_INDEX
        ids[r, used:] = 0
    out = {INPUT_IDS_KEY: ids, LABELS_KEY: labels, POSITION_IDS_KEY: pos, SEQUENCE_IDS_KEY: seq}
    return {k: v.to(device) for k, v in out.items()}


class SyntheticBatchStream:
    """Deterministic batch source with the ``next_batch(cp_rank)`` interface of the data loaders. Every DP rank draws from
    its own seeded stream (HDP ranks share one: they need the same global batch)."""

    def __init__(self, *, rows: int, seq_len: int, vocab_size: int, config: SyntheticBatchConfig, seed: int, stream_id: int,
                 device: torch.device, pool: int = 8) -> None:
        gen = torch.Generator().manual_seed(seed * 1000003 + stream_id)
        target = device if config.delivery == "device" else "cpu"
        self.batches = [make_synthetic_batch(rows=rows, seq_len=seq_len, vocab_size=vocab_size, config=config, generator=gen, device=target,
                                             row_offset=i * rows) for i in range(pool)]
        if config.delivery == "host" and device.type == "cuda":
            self.batches = [{k: v.pin_memory() for k, v in b.items()} for b in self.batches]
        self.cursor = 0
        self.consumed_tokens = 0
        self.active_tokens = [int((b[LABELS_KEY] != IGNORE_INDEX).sum()) for b in self.batches]

    def next_batch(self, cp_rank: int | None = None) -> dict[str, torch.Tensor]:
        batch = self.batches[self.cursor % len(self.batches)]
        self.cursor += 1
        self.consumed_tokens += batch[INPUT_IDS_KEY].numel()
        return batch

    def state_dict(self):
        return {"cursor": self.cursor}

    def load_state_dict(self, state) -> None:
        self.cursor = int(state["cursor"])


# ------------------------------------------------------------------------------------------------ cases & arguments
def _load_cases(path: Path) -> dict[str, CaseDefinition]:
    if not path.is_file():
        return {}
    raw = yaml.safe_load(path.read_text(encoding="utf-8")) or {}
    cases = {}
    for name, body in (raw.get("cases") or {}).items():
        body = dict(body or {})
        synthetic = body.get("synthetic")
        if synthetic is not None:
            unknown = set(synthetic) - set(_SYNTHETIC_KEYS)
            if unknown:
                raise ValueError(f"case {name}: unknown synthetic keys {sorted(unknown)}")
        if bool(body.get("recipe")) == bool(body.get("runtime_spec")):
            raise ValueError(f"case {name}: exactly one of recipe / runtime_spec is required")
        cases[name] = CaseDefinition(name=name, description=str(body.get("description", "")), recipe=body.get("recipe"),
                                     runtime_spec=body.get("runtime_spec"),
                                     recipe_overrides=tuple(str(x) for x in (body.get("overrides") or body.get("recipe_overrides") or ())),
                                     synthetic=synthetic, warmup=body.get("warmup"), steps=body.get("steps"),
                                     require_calibrated_hdp_cost=bool(body.get("require_calibrated_hdp_cost", False)))
    return cases


def _parse_tool_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Time synthetic training steps of a recipe, runtime spec or named case.")
    p.add_argument("--recipe", type=str, help="training recipe YAML")
    p.add_argument("--runtime-spec", type=str, help="runtime_spec.json of a checkpoint root")
    p.add_argument("--case-file", type=Path, default=DEFAULT_CASE_FILE)
    p.add_argument("--case", type=str, help="named experiment from --case-file")
    p.add_argument("--list-cases", action="store_true", help="print cases and exit")
    p.add_argument("--warmup", type=int, default=None, help="untimed global optimizer steps")
    p.add_argument("--steps", type=int, default=None, help="timed global optimizer steps")
    p.add_argument("--synthetic-layout", choices=("dense", "packed"), default=None)
    p.add_argument("--packed-input", action=argparse.BooleanOptionalAction, default=None, help="shortcut for --synthetic-layout packed / dense")
    p.add_argument("--packed-sequences", type=int, default=None, help="fixed number of documents per packed row (min = max)")
    p.add_argument("--segment-count-min", type=int, default=None)
    p.add_argument("--segment-count-max", type=int, default=None)
    p.add_argument("--supervised-fraction-min", type=float, default=None)
    p.add_argument("--supervised-fraction-max", type=float, default=None)
    p.add_argument("--max-padding-fraction", type=float, default=None)
    p.add_argument("--delivery", "--synthetic-delivery", dest="delivery", choices=("host", "device", "cuda"), default=None,
                   help="host: pinned CPU batches moved by the runtime (what a data loader delivers); device / cuda: created on the GPU")
    p.add_argument("--data-source", choices=("synthetic", "recipe"), default=None,
                   help="synthetic generator (default) or the recipe's own memory-mapped data loader (needs --data after --)")
    p.add_argument("--seed", type=int, default=1234, help="synthetic data seed")
    p.add_argument("--output-dir", type=Path, default=Path("profiles/train_perf"))
    p.add_argument("--profile", action="store_true", help="export a torch.profiler trace of the timed steps")
    p.add_argument("--profile-all-ranks", action="store_true", help="trace every rank (large); default traces rank 0 only")
    p.add_argument("--profile-record-shapes", action="store_true")
    p.add_argument("--profile-memory", action="store_true")
    p.add_argument("--use-recipe-optimizer", action="store_true", help="keep the recipe's learning rate instead of lr=0")
    p.add_argument("--benchmark-lr", type=float, default=None, help="learning rate of the benchmark (default 0)")
    p.add_argument("recipe_overrides", nargs=argparse.REMAINDER, help="normal training flags after --")
    args = p.parse_args(argv)
    if args.packed_sequences is not None and args.packed_sequences < 2:
        p.error("--packed-sequences must be >= 2")
    if args.delivery == "cuda":
        args.delivery = "device"
    if args.packed_input is not None and args.synthetic_layout is None:
        args.synthetic_layout = "packed" if args.packed_input else "dense"
    return args


def _resolve_case(args: argparse.Namespace, cases: dict[str, CaseDefinition]) -> CaseDefinition:
    chosen = [x for x in (args.recipe, args.runtime_spec, args.case) if x]
    if len(chosen) != 1:
        raise SystemExit("exactly one of --recipe, --runtime-spec, --case is required")
    if args.case:
        if args.case not in cases:
            raise SystemExit(f"unknown case {args.case!r}; available: {sorted(cases)}")
        return cases[args.case]
    return CaseDefinition(name="adhoc", recipe=args.recipe, runtime_spec=args.runtime_spec)


def _training_args(case: CaseDefinition, overrides: list[str]) -> argparse.Namespace:
    extra = [*case.recipe_overrides, *(overrides[1:] if overrides[:1] == ["--"] else overrides)]
    if case.recipe:
        return parse_args_from(["--config", case.recipe, *extra], require_data=False)
    spec = json.loads(Path(case.runtime_spec).read_text(encoding="utf-8"))
    base = parse_runtime_spec_args(spec)
    if not extra:
        return base
    merged = parse_args_from(extra, require_data=False)
    explicit = {a.lstrip("-").replace("-", "_") for a in extra if a.startswith("--")}
    for key in explicit:
        key = key[3:] if key.startswith("no_") else key
        if hasattr(merged, key):
            setattr(base, key, getattr(merged, key))
    return base


def _synthetic_config(args: argparse.Namespace, case: CaseDefinition) -> SyntheticBatchConfig:
    spec = dict(case.synthetic or {})
    layout = args.synthetic_layout or ("packed" if spec.get("packed") else "dense")
    pick = lambda cli, key, default: cli if cli is not None else spec.get(key, default)   # noqa: E731
    packed = layout == "packed"
    fixed = args.packed_sequences if args.packed_sequences is not None else spec.get("packed_sequences")
    if fixed is not None and args.segment_count_min is None and args.segment_count_max is None:
        spec["segment_count_min"] = spec["segment_count_max"] = int(fixed)
    trace = spec.get("document_length_trace")
    delivery = pick(args.delivery, "delivery", "host")
    return SyntheticBatchConfig(
        document_length_trace=None if trace is None or not packed else tuple(tuple(int(n) for n in row) for row in trace),
        layout=layout, segment_count_min=pick(args.segment_count_min, "segment_count_min", 3),
        segment_count_max=pick(args.segment_count_max, "segment_count_max", 7),
        supervised_fraction_min=pick(args.supervised_fraction_min, "supervised_fraction_min", 0.55 if packed else 1.0),
        supervised_fraction_max=pick(args.supervised_fraction_max, "supervised_fraction_max", 0.70 if packed else 1.0),
        max_padding_fraction=pick(args.max_padding_fraction, "max_padding_fraction", 0.02 if packed else 0.0),
        delivery="device" if delivery == "cuda" else delivery)


# ------------------------------------------------------------------------------------------------ run
def _run_global_step(core, batches) -> torch.Tensor:
    loss = None
    cp_rank = None
    if core.plan.batch_data_cp_aware:
        cp_rank = dist.get_rank(core.get_group(MeshAxis.CP))
    for micro in range(core.grad_accum_steps):
        loss, should_step = core.run_step(batches.next_batch(cp_rank))
        if should_step != (micro + 1 == core.grad_accum_steps):
            raise RuntimeError("optimizer-step request does not coincide with the accumulation boundary")
    core.step_optimizer()
    return loss


def _check_finite(loss: torch.Tensor, *, phase: str, step: int) -> float:
    value = float(loss.detach().float().item())
    if not math.isfinite(value):
        raise FloatingPointError(f"non-finite synthetic loss during {phase} step {step}: {value}")
    return value


def _max_over_ranks(local_seconds: list[float], device: torch.device) -> list[float]:
    """A global step is over when the slowest rank is done: the per-step maximum is the distributed latency."""
    t = torch.tensor(local_seconds, dtype=torch.float64, device=device if device.type == "cuda" else "cpu")
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t.cpu().tolist()]


def _flops_per_token(args: argparse.Namespace) -> float | None:
    """Model FLOPs per token of a dense decoder (forward + backward = 6 x matmul parameters + causal attention)."""
    try:
        h, layers, ffn, vocab, seq = args.dim, args.n_layers, args.hidden_size, args.vocab_size, args.seq_len
        kv = (args.n_kv_heads or args.n_heads) * (h // args.n_heads)
        per_layer = 2 * h * h + 2 * h * kv + 3 * h * ffn
        return 6.0 * (layers * per_layer + h * vocab) + 6.0 * layers * seq * h
    except (AttributeError, TypeError):
        return None


def _environment() -> dict[str, Any]:
    """What a number depends on besides the code: interpreter, libraries, devices, launcher and tuning variables, commit."""
    import os
    import subprocess

    env: dict[str, Any] = {"python": platform.python_version(), "torch": torch.__version__, "host": platform.node(),
                           "platform": platform.platform(), "cpu_count": os.cpu_count()}
    if torch.cuda.is_available():
        props = torch.cuda.get_device_properties(torch.cuda.current_device())
        env.update(device=props.name, cuda=torch.version.cuda, devices=torch.cuda.device_count(), sm=f"{props.major}.{props.minor}",
                   sm_count=props.multi_processor_count, device_memory_gib=round(props.total_memory / 2**30, 1))
        try:
            env["nccl"] = ".".join(str(v) for v in torch.cuda.nccl.version())
        except Exception:  # noqa: BLE001 - builds without NCCL
            env["nccl"] = None
    from maltos_b200.ops import _lib

    env["kernel_library"] = str(_lib.library_path()) if _lib.available() else None
    env["variables"] = {k: v for k, v in sorted(os.environ.items())
                        if k.startswith(("MALTOS_B200_", "NCCL_", "TORCH_NCCL_", "CUDA_DEVICE_MAX_CONNECTIONS", "CUDA_VISIBLE_DEVICES", "OMP_NUM_THREADS"))}
    try:
        root = Path(__file__).resolve().parents[2]
        env["commit"] = subprocess.run(["git", "-C", str(root), "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=5).stdout.strip() or None
    except Exception:  # noqa: BLE001 - not a work tree / no git
        env["commit"] = None
    return env


def _trace_summary(config: SyntheticBatchConfig, seq_len: int) -> dict[str, Any] | None:
    """Identity and shape of a fixed document trace (so that two summaries can be checked to describe the same workload)."""
    trace = config.document_length_trace
    if trace is None:
        return None
    import hashlib

    flat = [n for row in trace for n in row]
    return {"sha256": hashlib.sha256(json.dumps([list(r) for r in trace]).encode()).hexdigest()[:16], "rows": len(trace),
            "documents": len(flat), "min_length": min(flat), "max_length": max(flat),
            "active_fraction": sum(flat) / (len(trace) * seq_len)}


class _TimedLoader:
    """Wraps a loader and accumulates the time the training loop waits in ``next_batch`` (data stalls of a step)."""

    def __init__(self, inner) -> None:
        self.inner, self.wait_seconds, self.calls = inner, 0.0, 0

    def next_batch(self, cp_rank=None):
        t0 = time.perf_counter()
        batch = self.inner.next_batch(cp_rank)
        self.wait_seconds += time.perf_counter() - t0
        self.calls += 1
        return batch

    def take(self) -> float:
        w, self.wait_seconds = self.wait_seconds, 0.0
        return w

    def close(self) -> None:
        closer = getattr(self.inner, "close", None)
        if callable(closer):
            closer()


def run(train_args: argparse.Namespace, tool_args: argparse.Namespace, case: CaseDefinition) -> dict[str, Any] | None:
    warmup = tool_args.warmup if tool_args.warmup is not None else (case.warmup if case.warmup is not None else 3)
    steps = tool_args.steps if tool_args.steps is not None else (case.steps if case.steps is not None else 5)
    if warmup < 0 or steps < 1:
        raise SystemExit("--warmup must be >= 0 and --steps >= 1")
    if tool_args.benchmark_lr is not None:
        train_args.lr = tool_args.benchmark_lr
    elif not tool_args.use_recipe_optimizer:
        train_args.lr, train_args.min_lr = 0.0, 0.0        # stable workload: every kernel runs, nothing moves
    synthetic = _synthetic_config(tool_args, case)
    data_source = tool_args.data_source or (case.synthetic or {}).get("data_source") or "synthetic"
    if data_source == "recipe" and not getattr(train_args, "data", None):
        raise SystemExit("--data-source recipe needs the recipe's data: pass --data <shards> after --")
    if case.require_calibrated_hdp_cost and (train_args.hdp_cost_alpha, train_args.hdp_cost_beta, train_args.hdp_cost_gamma) == (1.0, 0.0, 0.0):
        raise SystemExit(f"case {case.name} is a measurement case: pass calibrated --hdp-cost-alpha/-beta/-gamma after -- "
                         "(the 1 / 0 / 0 proxy is refused)")

    train_cli._maybe_init_distributed(train_args)
    device = train_cli._select_device()
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    train_cli.validate_args(train_args, world)
    torch.manual_seed(train_args.seed)
    core = train_cli._build_runtime(train_args, train_cli._build_model(train_args), device)
    core.setup()
    core.model.train()
    try:
        dp_group = core.get_group(MeshAxis.DP)
        dp_rank = dist.get_rank(dp_group) if dp_group is not None else 0
        stream_id = 0 if train_args.hdp_balanced else dp_rank
        stream = None
        if data_source == "recipe":
            _, batches, _ = train_cli._build_dataloader(train_args, dp_rank=dp_rank, cp_token_planner=core.plan.cp_token_planner)
        else:
            batches = stream = SyntheticBatchStream(rows=train_args.micro_batch_size, seq_len=train_args.seq_len, vocab_size=train_args.vocab_size,
                                                    config=synthetic, seed=tool_args.seed, stream_id=stream_id, device=device)
            if train_args.hdp_balanced:
                from maltos_b200.data.bytescale_hdp import ByteScaleHdpDataLoader

                batches = ByteScaleHdpDataLoader(batches, hdp_rank=dp_rank, hdp_world_size=train_args.dp_size,
                                                 config=train_cli._build_hdp_config(train_args))
        if getattr(train_args, "data_prefetch_batches", 0):
            from maltos_b200.data.prefetch import PrefetchDataLoader

            batches = PrefetchDataLoader(batches)          # the next batch (and its HDP schedule) is prepared under the current step
        batches = _TimedLoader(batches)

        def sync() -> None:
            if device.type == "cuda":
                torch.cuda.synchronize(device)

        for i in range(warmup):
            _check_finite(_run_global_step(core, batches), phase="warmup", step=i)
        sync()
        if device.type == "cuda":
            torch.cuda.reset_peak_memory_stats(device)
        profiler = None
        if tool_args.profile and (rank == 0 or tool_args.profile_all_ranks):
            acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if device.type == "cuda" else [])
            profiler = torch.profiler.profile(activities=acts, record_shapes=tool_args.profile_record_shapes,
                                              profile_memory=tool_args.profile_memory)
            profiler.__enter__()
        local, waits, final_loss = [], [], float("nan")
        batches.take()
        for i in range(steps):
            if dist.is_initialized():
                dist.barrier()
            sync()
            t0 = time.perf_counter()
            loss = _run_global_step(core, batches)
            sync()
            local.append(time.perf_counter() - t0)
            waits.append(batches.take())
            final_loss = _check_finite(loss, phase="timed", step=i)
        if profiler is not None:
            profiler.__exit__(None, None, None)
            tool_args.output_dir.mkdir(parents=True, exist_ok=True)
            profiler.export_chrome_trace(str(tool_args.output_dir / f"trace_rank{rank}.json"))
        seconds = _max_over_ranks(local, device)
        data_wait = _max_over_ranks(waits, device)
        peak = torch.tensor([float(torch.cuda.max_memory_allocated(device)) if device.type == "cuda" else 0.0], dtype=torch.float64,
                            device=device if device.type == "cuda" else "cpu")
        if dist.is_initialized() and world > 1:
            dist.all_reduce(peak, op=dist.ReduceOp.MAX)
        if rank != 0:
            return None
        replicas = 1 if train_args.hdp_balanced else train_args.dp_size
        tokens = replicas * train_args.micro_batch_size * train_args.seq_len * train_args.grad_accum_steps
        t = torch.tensor(seconds, dtype=torch.float64)
        mean = float(t.mean())
        fpt = _flops_per_token(train_args)
        summary = {
            "case": case.name, "description": case.description, "recipe": case.recipe, "runtime_spec": case.runtime_spec,
            "world_size": world, "mesh": {k: getattr(train_args, f"{k}_size") for k in ("dp", "tp", "pp", "cp", "ep")},
            "zero_stage": train_args.zero_stage, "use_sp": train_args.use_sp, "precision": train_args.precision,
            "synthetic": asdict(synthetic),
            "synthetic_seed": tool_args.seed, "warmup_steps": warmup, "timed_steps": steps, "step_seconds": seconds,
            "mean_step_seconds": mean, "p50_step_seconds": float(torch.quantile(t, 0.5)), "p90_step_seconds": float(torch.quantile(t, 0.9)),
            "tokens_per_step": tokens, "tokens_per_second": tokens / mean,
            "active_target_fraction": None if stream is None else
            sum(stream.active_tokens) / (len(stream.batches) * train_args.micro_batch_size * train_args.seq_len),
            "data_source": data_source, "data_prefetch_batches": int(getattr(train_args, "data_prefetch_batches", 0) or 0),
            "data_wait_seconds_per_step": sum(data_wait) / len(data_wait), "data_wait_fraction": sum(data_wait) / sum(seconds),
            "document_trace": _trace_summary(synthetic, train_args.seq_len),
            "model_flops_per_token": fpt, "model_tflops_per_gpu": None if fpt is None else tokens / mean * fpt / world / 1e12,
            "peak_memory_gib": float(peak.item()) / 2**30, "final_loss": final_loss, "profiled": bool(tool_args.profile),
            "learning_rate": train_args.lr, "environment": _environment(),
        }
        _write_summary(tool_args.output_dir, summary)
        return summary
    finally:
        core.close()
        closer = getattr(locals().get("batches"), "close", None)
        if callable(closer):
            closer()


def _write_summary(output_dir: Path, summary: dict[str, Any]) -> None:
    output_dir.mkdir(parents=True, exist_ok=True)
    (output_dir / "summary.json").write_text(json.dumps(summary, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    tf = summary["model_tflops_per_gpu"]
    lines = [f"case: {summary['case']}  world={summary['world_size']}  mesh={summary['mesh']}  zero={summary['zero_stage']}  sp={summary['use_sp']}",
             f"steps: warmup={summary['warmup_steps']} timed={summary['timed_steps']}  layout={summary['synthetic']['layout']}",
             f"step time: mean {summary['mean_step_seconds']:.4f}s  p50 {summary['p50_step_seconds']:.4f}s  p90 {summary['p90_step_seconds']:.4f}s",
             f"throughput: {summary['tokens_per_second']:,.0f} tokens/s" + (f"  {tf:.1f} model TFLOP/s/GPU" if tf is not None else ""),
             f"data: {summary['data_source']} prefetch={summary['data_prefetch_batches']} wait {summary['data_wait_seconds_per_step'] * 1e3:.2f} ms/step "
             f"({summary['data_wait_fraction'] * 100:.1f} % of the step)",
             f"peak memory: {summary['peak_memory_gib']:.2f} GiB  final loss: {summary['final_loss']:.4f}"]
    (output_dir / "summary.txt").write_text("\n".join(lines) + "\n", encoding="utf-8")
    print("\n".join(lines))


def main(argv=None) -> None:
    args = _parse_tool_args(argv)
    cases = _load_cases(args.case_file)
    if args.list_cases:
        for name, case in sorted(cases.items()):
            print(f"{name}: {case.description}")
        return
    case = _resolve_case(args, cases)
    train_args = _training_args(case, list(args.recipe_overrides))
    try:
        run(train_args, args, case)
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()

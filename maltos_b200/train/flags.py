"""Command-line flags, YAML recipes and the frozen ``runtime_spec``.

Every flag is one row of ``FLAGS`` (name, type, default, choices, and the ``section.key`` names a YAML recipe may use
for it); the argparse parser, the recipe->flag mapping and the spec field lists are derived from that table. A recipe is
pre-parsed from ``--config`` and becomes parser *defaults*, so explicit flags win. Flag names, defaults, the alias set and
the spec layout (``format = "train_cli_args"``, ``version = 3``, 16 model + 22 runtime fields, strict field check) are
those of the reference (``train/flags.py:12-403``) because recipes and checkpoints carry them. Additional flags of this
framework: ``--pp-schedule``, ``--rope-theta``, ``--moe-top-k``, ``--moe-capacity-factor``, ``--init-std``; they are
deliberately NOT part of the spec so that spec files stay interchangeable.
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass, field
from typing import Any

import yaml

TRAIN_CLI_RUNTIME_SPEC_FORMAT = "train_cli_args"
TRAIN_CLI_RUNTIME_SPEC_VERSION = 3

BOOL = "bool"   # marker type: --x / --no-x


@dataclass(frozen=True)
class Flag:
    name: str                      # destination, e.g. "seq_len" (flag is --seq-len)
    type: Any = str
    default: Any = None
    choices: tuple | None = None
    nargs: str | None = None
    yaml: tuple[str, ...] = field(default_factory=tuple)   # "section.key" aliases in recipes
    help: str | None = None


_ATTN = ("eager", "sdpa_auto", "sdpa_flash", "flash_attn")

FLAGS: tuple[Flag, ...] = (
    # data
    Flag("data", str, None, nargs="+", yaml=("data.paths",), help="token shard .bin files / directories, or a packed SFT dataset directory / meta.json"),
    Flag("data_format", str, "auto", ("auto", "pretrain", "sft"), yaml=("data.format",)),
    Flag("token_dtype", str, "uint32", ("uint16", "uint32", "int64")),
    Flag("seq_len", int, 128, yaml=("data.seq_len",)),
    Flag("micro_batch_size", int, 1, yaml=("data.micro_batch_size",), help="per-DP-rank batch size (global packed batch size with --hdp-balanced)"),
    Flag("data_prefetch_batches", int, 0, (0, 1), yaml=("data.prefetch_batches",)),
    # schedule / optimizer
    Flag("max_steps", int, 10, yaml=("training.max_steps",)),
    Flag("dry_run", BOOL, False, yaml=("training.dry_run",)),
    Flag("grad_accum_steps", int, 1, yaml=("training.grad_accum_steps",)),
    Flag("lr", float, 1e-3, yaml=("training.lr",)),
    Flag("weight_decay", float, 0.0, yaml=("training.weight_decay",)),
    Flag("adam_beta1", float, 0.9, yaml=("training.adam_beta1",)),
    Flag("adam_beta2", float, 0.95, yaml=("training.adam_beta2",)),
    Flag("adam_eps", float, 1e-8, yaml=("training.adam_eps",)),
    Flag("fused_adamw", BOOL, False, yaml=("training.fused_adamw",)),
    Flag("lr_schedule", str, "constant", ("constant", "linear", "cosine"), yaml=("training.lr_schedule",)),
    Flag("warmup_steps", int, 0, yaml=("training.warmup_steps",)),
    Flag("min_lr", float, 0.0, yaml=("training.min_lr",)),
    Flag("seed", int, 42),
    # model
    Flag("model", str, "tiny", ("tiny", "tiny_moe", "llama", "olmo", "olmo2"), yaml=("model.type",)),
    Flag("dim", int, 256, yaml=("model.hidden_size", "model.dim")),
    Flag("n_heads", int, 8, yaml=("model.num_heads", "model.n_heads")),
    Flag("n_kv_heads", int, None, yaml=("model.num_kv_heads", "model.n_kv_heads")),
    Flag("hidden_size", int, 1024, yaml=("model.intermediate_size",)),
    Flag("n_layers", int, 4, yaml=("model.num_layers", "model.n_layers")),
    Flag("num_experts", int, 8, yaml=("model.num_experts",)),
    Flag("moe_aux_loss_coef", float, 0.0, yaml=("model.moe_aux_loss_coef",)),
    Flag("vocab_size", int, 32000, yaml=("model.vocab_size",)),
    Flag("eps", float, 1e-5, yaml=("model.rms_norm_eps", "model.eps")),
    Flag("attention_backend", str, "sdpa_auto", _ATTN, yaml=("model.attention_backend",)),
    Flag("activation_checkpointing", BOOL, False, yaml=("model.activation_checkpointing",)),
    Flag("activation_checkpoint_every_n_layers", int, 1, yaml=("model.activation_checkpoint_every_n_layers",)),
    Flag("rope_theta", float, None, yaml=("model.rope_theta",), help="RoPE base (default: 10000 for llama, 500000 for olmo)"),
    Flag("moe_top_k", int, 1, yaml=("model.moe_top_k",)),
    Flag("moe_capacity_factor", float, None, yaml=("model.moe_capacity_factor",)),
    Flag("init_std", float, None, yaml=("model.init_std",), help="re-initialise matrices with normal(0, std)"),
    # parallelism
    Flag("dp_size", int, 1, yaml=("parallel.dp_size",)),
    Flag("pp_size", int, 1, yaml=("parallel.pp_size",)),
    Flag("pp_microbatches", int, 1, yaml=("parallel.pp_microbatches",)),
    Flag("pp_schedule", str, "afab", ("afab", "1f1b"), yaml=("parallel.pp_schedule",)),
    Flag("cp_size", int, 1, yaml=("parallel.cp_size",)),
    Flag("tp_native_comm_overlap", BOOL, False, yaml=("parallel.tp_native_comm_overlap",),
         help="accepted for compatibility: the fused sm_100a all-gather->GEMM / GEMM->reduce-scatter kernels are the CUDA path"),
    Flag("cp_attn_core", str, "all_gather_kv", ("all_gather_kv", "ring"), yaml=("parallel.cp_attn_core",)),
    Flag("batch_data_cp_aware", BOOL, False, yaml=("parallel.batch_data_cp_aware",)),
    Flag("cp_token_planner", str, None, ("fixed_contiguous", "fixed_zigzag"), yaml=("parallel.cp_token_planner",)),
    Flag("hdp_balanced", BOOL, False, yaml=("parallel.hdp_balanced",)),
    Flag("hdp_partition_tokens", int, None, yaml=("parallel.hdp_partition_tokens",)),
    Flag("hdp_cost_alpha", float, 1.0, yaml=("parallel.hdp_cost_alpha",)),
    Flag("hdp_cost_beta", float, 0.0, yaml=("parallel.hdp_cost_beta",)),
    Flag("hdp_cost_gamma", float, 0.0, yaml=("parallel.hdp_cost_gamma",)),
    Flag("hdp_balance_delta", float, 0.0, yaml=("parallel.hdp_balance_delta",)),
    Flag("tp_size", int, 1, yaml=("parallel.tp_size",)),
    Flag("ep_size", int, 1, yaml=("parallel.ep_size",)),
    Flag("zero_stage", int, 0, (0, 1, 2, 3), yaml=("parallel.zero_stage",)),
    Flag("use_sp", BOOL, False, yaml=("parallel.use_sp",)),
    Flag("ddp_mode", str, None, ("sync", "async", "bucket"), yaml=("parallel.ddp_mode",)),
    # precision / clipping / fused scopes
    Flag("precision", str, "fp32", ("fp32", "bf16", "fp16"), yaml=("training.precision",)),
    Flag("grad_clip", float, None, yaml=("training.grad_clip",)),
    # loss = mean over the targets of ALL data-parallel ranks of a micro-step instead of the mean of the ranks' means
    Flag("token_weighted_loss", BOOL, False, yaml=("training.token_weighted_loss",)),
    Flag("compile", BOOL, False, yaml=("compile.enabled",)),
    Flag("compile_scope", str, "mlp", yaml=("compile.scope",)),
    Flag("compile_mode", str, "default", yaml=("compile.mode",)),
    Flag("cuda_graph", BOOL, False, yaml=("training.cuda_graph",)),   # record the micro-step into a CUDA graph (one process)
    # observability
    Flag("disable_metrics", BOOL, False, yaml=("training.disable_metrics",)),
    Flag("torch_profiler", BOOL, False, yaml=("profiling.torch_profiler",)),
    Flag("torch_profiler_dir", str, "traces/train", yaml=("profiling.torch_profiler_dir",)),
    Flag("torch_profiler_wait", int, 1, yaml=("profiling.torch_profiler_wait",)),
    Flag("torch_profiler_warmup", int, 1, yaml=("profiling.torch_profiler_warmup",)),
    Flag("torch_profiler_active", int, 3, yaml=("profiling.torch_profiler_active",)),
    Flag("torch_profiler_repeat", int, 1, yaml=("profiling.torch_profiler_repeat",)),
    Flag("torch_profiler_record_shapes", BOOL, False, yaml=("profiling.torch_profiler_record_shapes",)),
    Flag("torch_profiler_profile_memory", BOOL, False, yaml=("profiling.torch_profiler_profile_memory",)),
    Flag("torch_profiler_with_stack", BOOL, False, yaml=("profiling.torch_profiler_with_stack",)),
    Flag("torch_profiler_with_flops", BOOL, False, yaml=("profiling.torch_profiler_with_flops",)),
    Flag("torch_profiler_rank0_only", BOOL, False, yaml=("profiling.torch_profiler_rank0_only",)),
    Flag("log_every", int, 1, yaml=("logging.log_every",)),
    Flag("metrics_jsonl", str, None, yaml=("logging.metrics_jsonl",)),
    Flag("run_manifest", str, None, yaml=("logging.run_manifest",)),
    Flag("wandb_project", str, None, yaml=("logging.wandb_project",)),
    Flag("wandb_run_name", str, None, yaml=("logging.wandb_run_name",)),
    Flag("wandb_entity", str, None, yaml=("logging.wandb_entity",)),
    Flag("wandb_run_id", str, None, yaml=("logging.wandb_run_id",)),
    Flag("wandb_mode", str, None, ("online", "offline", "disabled"), yaml=("logging.wandb_mode",)),
    Flag("wandb_tags", str, None, yaml=("logging.wandb_tags",), help="comma-separated W&B tags"),
    Flag("wandb_checkpoint_every", int, None, yaml=("logging.wandb_checkpoint_every",)),
    # checkpoints
    Flag("checkpoint_dir", str, None, yaml=("checkpoint.dir", "checkpoint.checkpoint_dir")),
    Flag("checkpoint_every", int, None, yaml=("checkpoint.every", "checkpoint.checkpoint_every")),
    Flag("checkpoint_keep_last", int, None, yaml=("checkpoint.keep_last", "checkpoint.checkpoint_keep_last")),
    Flag("checkpoint_keep_every_n_steps", int, None, yaml=("checkpoint.keep_every_n_steps", "checkpoint.checkpoint_keep_every_n_steps")),
    Flag("checkpoint_min_free_gb", float, None, yaml=("checkpoint.min_free_gb", "checkpoint.checkpoint_min_free_gb")),
    Flag("resume_from", str, None, yaml=("checkpoint.resume_from",)),
    # SIGTERM / SIGUSR1 end the run cleanly: all ranks finish the same step, save it and exit (resume with --resume-from auto)
    Flag("graceful_stop", BOOL, False, yaml=("checkpoint.graceful_stop",)),
    # seconds without a heartbeat after which a rank is reported lost (host-side check before every micro-step); unset = off
    Flag("heartbeat_timeout", float, None, yaml=("training.heartbeat_timeout",)),
    Flag("load_weights_only", BOOL, False, yaml=("checkpoint.load_weights_only",)),
    # launch
    Flag("backend", str, None),
    Flag("master_addr", str, "127.0.0.1"),
    Flag("master_port", str, "29550"),
)

_RUNTIME_SPEC_MODEL_FIELDS = ("model", "dim", "n_heads", "n_kv_heads", "hidden_size", "n_layers", "num_experts", "moe_aux_loss_coef",
                              "vocab_size", "eps", "seq_len", "attention_backend", "activation_checkpointing",
                              "activation_checkpoint_every_n_layers", "use_sp", "tp_size")
_RUNTIME_SPEC_RUNTIME_FIELDS = ("dp_size", "tp_size", "pp_size", "cp_size", "ep_size", "hdp_balanced", "hdp_partition_tokens",
                                "hdp_cost_alpha", "hdp_cost_beta", "hdp_cost_gamma", "hdp_balance_delta", "pp_microbatches",
                                "cp_attn_core", "batch_data_cp_aware", "cp_token_planner", "zero_stage", "ddp_mode", "precision",
                                "use_sp", "compile", "compile_scope", "compile_mode")

_YAML_TO_DEST = {alias: f.name for f in FLAGS for alias in f.yaml}


def build_arg_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="LLM training recipe.")
    parser.add_argument("--config", type=str, default=None, help="YAML training recipe")
    for f in FLAGS:
        opt = "--" + f.name.replace("_", "-")
        if f.type is BOOL:
            parser.add_argument(opt, action=argparse.BooleanOptionalAction, default=f.default, help=f.help)
            continue
        kw: dict[str, Any] = dict(type=f.type, default=f.default, help=f.help)
        if f.choices is not None:
            kw["choices"] = f.choices
        if f.nargs is not None:
            kw["nargs"] = f.nargs
        parser.add_argument(opt, **kw)
    return parser


def _config_key_to_arg_dest(section: str, key: str) -> str:
    return _YAML_TO_DEST.get(f"{section}.{key}", key)


def _load_config_defaults(path: str) -> dict[str, Any]:
    with open(path, "r", encoding="utf-8") as f:
        raw = yaml.safe_load(f) or {}
    if not isinstance(raw, dict):
        raise ValueError(f"config must be a YAML mapping, got {type(raw)!r}")
    defaults: dict[str, Any] = {"config": path}
    for section, body in raw.items():
        if isinstance(body, dict):
            for key, value in body.items():
                defaults[_config_key_to_arg_dest(section, key)] = value
        else:
            defaults[section] = body
    return defaults


def _preparse_config_path(argv: list[str] | None = None) -> str | None:
    pre = argparse.ArgumentParser(add_help=False)
    pre.add_argument("--config", type=str, default=None)
    return pre.parse_known_args(argv)[0].config


def _validate_data_requirement(args: argparse.Namespace, *, require_data: bool) -> None:
    if require_data and args.data is None:
        raise ValueError("--data is required unless provided by --config")


def parse_args_with_defaults(defaults: dict[str, Any], argv: list[str] | None = None, *, require_data: bool = True) -> argparse.Namespace:
    parser = build_arg_parser()
    parser.set_defaults(**defaults)
    args = parser.parse_args(argv)
    if isinstance(args.data, str):
        args.data = [args.data]
    _validate_data_requirement(args, require_data=require_data)
    return args


def parse_args_from(argv: list[str] | None = None, *, require_data: bool = True) -> argparse.Namespace:
    path = _preparse_config_path(argv)
    return parse_args_with_defaults(_load_config_defaults(path) if path is not None else {}, argv, require_data=require_data)


def parse_args(*, require_data: bool = True) -> argparse.Namespace:
    return parse_args_from(require_data=require_data)


def build_runtime_spec(args: argparse.Namespace) -> dict[str, Any]:
    """The subset of flags that determines the checkpoint layout (model shape + parallel layout)."""
    return {
        "format": TRAIN_CLI_RUNTIME_SPEC_FORMAT,
        "version": TRAIN_CLI_RUNTIME_SPEC_VERSION,
        "model": {k: getattr(args, k) for k in _RUNTIME_SPEC_MODEL_FIELDS},
        "runtime": {k: getattr(args, k) for k in _RUNTIME_SPEC_RUNTIME_FIELDS},
    }


def _validate_runtime_spec_fields(section: str, values: dict[str, Any], expected: tuple[str, ...]) -> None:
    missing, extra = sorted(set(expected) - set(values)), sorted(set(values) - set(expected))
    if missing or extra:
        raise ValueError(f"runtime spec {section} fields mismatch: missing={missing}, extra={extra}")


def parse_runtime_spec_args(spec: dict[str, Any]) -> argparse.Namespace:
    if spec.get("format") != TRAIN_CLI_RUNTIME_SPEC_FORMAT:
        raise ValueError(f"unsupported runtime spec format={spec.get('format')!r}")
    version = int(spec.get("version", 0))
    if version != TRAIN_CLI_RUNTIME_SPEC_VERSION:
        raise ValueError(f"unsupported runtime spec version={version}")
    model, runtime = spec.get("model"), spec.get("runtime")
    if not isinstance(model, dict):
        raise ValueError("runtime spec missing model mapping")
    if not isinstance(runtime, dict):
        raise ValueError("runtime spec missing runtime mapping")
    _validate_runtime_spec_fields("model", model, _RUNTIME_SPEC_MODEL_FIELDS)
    _validate_runtime_spec_fields("runtime", runtime, _RUNTIME_SPEC_RUNTIME_FIELDS)
    for k in set(model) & set(runtime):
        if model[k] != runtime[k]:
            raise ValueError(f"runtime spec field {k!r} disagrees between model and runtime sections")
    ns = {f.name: f.default for f in FLAGS}     # flags outside the spec keep their defaults
    ns.update(model)
    ns.update(runtime)
    return argparse.Namespace(**ns)

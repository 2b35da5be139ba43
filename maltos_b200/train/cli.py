"""Command-line training application (one process per GPU under ``torchrun``).

``main()``: flags/recipe -> process group -> validation -> model -> plugin list + ``RuntimeCore`` -> data loader ->
``Trainer.setup()`` -> run summary / manifest -> ``Trainer.fit()``. The builders are importable on their own
(``_build_model``, ``_build_runtime``, ``_build_dataloader`` ...) because tools and tests assemble runs from them
(reference ``train/cli.py:95-913``).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
from pathlib import Path
from typing import Any

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

from maltos_b200.parallel import (ContextParallelBatchSharder, ParallelPlan, PipelineScheduleConfig,
                                  build_context_token_planner)
from maltos_b200.parallel.context_interfaces import ContextParallelAttentionCoreType
from maltos_b200.parallel.context_token_planner import ContextTokenPlannerType
from maltos_b200.runtime.core import RuntimeCore
from maltos_b200.runtime.mesh import MeshConfig
from maltos_b200.utils.distributed import distributed_barrier, raise_if_any_rank_failed

from .flags import build_runtime_spec, parse_args
from .trainer import Trainer, TrainerConfig


# ------------------------------------------------------------------------------------------------ validation
def validate_args(args: argparse.Namespace, world_size: int) -> None:
    expected = args.dp_size * args.pp_size * args.cp_size * args.tp_size
    if world_size != expected:
        raise ValueError(f"world_size={world_size} must equal dp_size * pp_size * cp_size * tp_size={expected}")
    if args.use_sp and args.tp_size <= 1:
        raise ValueError("--use-sp requires --tp-size > 1")
    if args.use_sp and not args.hdp_balanced and (args.seq_len // max(args.cp_size, 1)) % args.tp_size:
        raise ValueError(f"--use-sp splits the (context-parallel share of the) sequence over the tensor-parallel ranks: "
                         f"--seq-len={args.seq_len} / cp={args.cp_size} must be divisible by --tp-size={args.tp_size}")
    if args.cp_size > 1 and args.seq_len % args.cp_size:
        raise ValueError("--cp-size requires --seq-len divisible by cp_size for CP v0")
    heads, kv_heads = args.n_heads, args.n_kv_heads or args.n_heads
    if heads < 1 or kv_heads < 1 or heads % kv_heads:
        raise ValueError(f"--n-heads={heads} must be a positive multiple of --n-kv-heads={kv_heads}")
    if args.dim % heads:
        raise ValueError(f"--dim={args.dim} must be divisible by --n-heads={heads}")
    if args.tp_size > 1:
        # attention is split by heads (a rank owns whole query heads and the key / value heads they share), the MLP by columns
        for flag, value in (("--n-heads", heads), ("--n-kv-heads", kv_heads), ("--hidden-size", args.hidden_size)):
            if value % args.tp_size:
                raise ValueError(f"{flag}={value} must be divisible by --tp-size={args.tp_size} (key / value heads are not replicated "
                                 "across tensor-parallel ranks)")
    if args.hdp_balanced:
        if args.cp_size != 1:
            raise ValueError("--hdp-balanced requires --cp-size 1; HDP replaces fixed CP")
        if args.pp_size != 1:
            raise ValueError("--hdp-balanced currently implements FCP's CP-only baseline and requires --pp-size 1")
        if args.batch_data_cp_aware:
            raise ValueError("--hdp-balanced is incompatible with --batch-data-cp-aware")
        if args.hdp_partition_tokens is None:
            raise ValueError("--hdp-balanced requires --hdp-partition-tokens")
        if args.hdp_partition_tokens < 1:
            raise ValueError("--hdp-partition-tokens must be positive")
        if args.hdp_partition_tokens % 2:
            raise ValueError("--hdp-partition-tokens must be even for symmetric zigzag partitions")
        _build_hdp_config(args).validate_tp_sp_partition(tp_size=args.tp_size, use_sp=args.use_sp)
    if args.pp_size > 1 and args.pp_microbatches and args.micro_batch_size % args.pp_microbatches:
        raise ValueError(f"--micro-batch-size={args.micro_batch_size} must be divisible by --pp-microbatches={args.pp_microbatches} "
                         "(the pipeline runner cuts every micro-batch into that many pieces)")
    if getattr(args, "token_weighted_loss", False) and args.hdp_balanced:
        raise ValueError("--token-weighted-loss is implied by --hdp-balanced (HDP weights every rank's loss by its targets)")
    if args.ep_size > 1 and args.dp_size % args.ep_size:
        raise ValueError("--ep-size must divide --dp-size")
    if args.ep_size > 1 and args.model != "tiny_moe":
        raise ValueError("--ep-size > 1 requires --model tiny_moe")
    if args.moe_aux_loss_coef < 0:
        raise ValueError("--moe-aux-loss-coef must be >= 0")
    if args.moe_aux_loss_coef > 0 and args.model != "tiny_moe":
        raise ValueError("--moe-aux-loss-coef requires --model tiny_moe")
    if args.zero_stage > 0 and args.dp_size <= 1:
        raise ValueError("--zero-stage > 0 requires --dp-size > 1")
    if args.zero_stage > 0 and args.ddp_mode is not None:
        raise ValueError("--ddp-mode is only valid when --zero-stage is 0")
    if args.wandb_checkpoint_every is not None:
        if args.wandb_checkpoint_every < 1:
            raise ValueError("--wandb-checkpoint-every must be >= 1")
        if args.checkpoint_every is None:
            raise ValueError("--wandb-checkpoint-every requires --checkpoint-every")
        if args.wandb_checkpoint_every % args.checkpoint_every:
            raise ValueError("--wandb-checkpoint-every must be a multiple of --checkpoint-every")
        if args.wandb_project is None or args.wandb_mode == "disabled":
            raise ValueError("--wandb-checkpoint-every requires enabled W&B logging")


def latest_checkpoint(checkpoint_dir) -> Path | None:
    """Newest COMPLETE checkpoint under ``checkpoint_dir``: the highest ``step_XXXXXXXX`` that has a manifest (a directory
    still being written is called ``step_XXXXXXXX.tmp`` and never matches)."""
    if checkpoint_dir is None or not Path(checkpoint_dir).is_dir():
        return None
    steps = sorted(p for p in Path(checkpoint_dir).glob("step_[0-9]*") if p.is_dir() and p.name[5:].isdigit() and (p / "manifest.json").is_file())
    return steps[-1] if steps else None


def resolve_resume_path(resume_from, checkpoint_dir, *, rank: int):
    """``--resume-from latest``: the newest complete checkpoint of ``--checkpoint-dir`` (an error if there is none);
    ``--resume-from auto``: the same, or a fresh start when there is none - the form a restart loop wants (the reference
    takes explicit paths only). Rank 0 looks and tells the others, so that every rank resumes from the same step even
    while a retention policy deletes old checkpoints. Any other value is returned as given."""
    if resume_from not in ("latest", "auto"):
        return resume_from
    found = [None]
    if rank == 0:
        hit = latest_checkpoint(checkpoint_dir)
        found = [None if hit is None else str(hit)]
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.broadcast_object_list(found, src=0)
    if found[0] is None and resume_from == "latest":
        raise ValueError(f"--resume-from latest: no complete checkpoint (step_XXXXXXXX with manifest.json) under --checkpoint-dir={checkpoint_dir}")
    if rank == 0:
        print(f"resume_from={resume_from} -> {found[0] or 'fresh start'}", flush=True)
    return found[0]


# ------------------------------------------------------------------------------------------------ model
def _variant(base, tp, sp, args):
    return sp if args.use_sp else (tp if args.tp_size > 1 else base)


def _build_model(args: argparse.Namespace) -> nn.Module:
    from maltos_b200 import models as M

    ckpt = M.ActivationCheckpointConfig(enabled=bool(args.activation_checkpointing), every_n_layers=args.activation_checkpoint_every_n_layers)
    name = args.model
    if name == "tiny":
        cls = _variant(M.TinyTransformer, M.TinyTransformerTp, M.TinyTransformerTpSp, args)
        model = cls(args.dim, args.n_heads, args.n_kv_heads or args.n_heads, args.hidden_size, args.eps, args.n_layers,
                    args.vocab_size, args.seq_len, attention_backend=args.attention_backend)
    elif name == "tiny_moe":
        cls = _variant(M.TinyMoETransformer, M.TinyMoETransformerTp, M.TinyMoETransformerTpSp, args)
        model = cls(args.dim, args.n_heads, args.n_kv_heads or args.n_heads, args.hidden_size, args.eps, args.n_layers,
                    args.vocab_size, args.seq_len, args.num_experts, moe_aux_loss_coef=args.moe_aux_loss_coef,
                    attention_backend=args.attention_backend, top_k=getattr(args, "moe_top_k", 1) or 1,
                    capacity_factor=getattr(args, "moe_capacity_factor", None),
                    apply_rope=getattr(args, "rope_theta", None) is not None)
    elif name == "llama":
        cls = _variant(M.LlamaForCausalLM, M.LlamaForCausalLMTp, M.LlamaForCausalLMTpSp, args)
        model = cls(M.LlamaConfig(vocab_size=args.vocab_size, hidden_size=args.dim, intermediate_size=args.hidden_size,
                                  num_hidden_layers=args.n_layers, num_attention_heads=args.n_heads, num_key_value_heads=args.n_kv_heads,
                                  max_position_embeddings=args.seq_len, rms_norm_eps=args.eps,
                                  rope_theta=getattr(args, "rope_theta", None) or 10000.0,
                                  attention_backend=args.attention_backend, activation_checkpointing=ckpt))
    elif name in ("olmo", "olmo2"):
        cls = _variant(M.OlmoForCausalLM, M.OlmoForCausalLMTp, M.OlmoForCausalLMTpSp, args)
        model = cls(M.OlmoConfig(vocab_size=args.vocab_size, hidden_size=args.dim, intermediate_size=args.hidden_size,
                                 num_hidden_layers=args.n_layers, num_attention_heads=args.n_heads, num_key_value_heads=args.n_kv_heads,
                                 max_position_embeddings=args.seq_len, rms_norm_eps=args.eps,
                                 rope_theta=getattr(args, "rope_theta", None) or 500000.0,
                                 attention_backend=args.attention_backend, activation_checkpointing=ckpt))
    else:
        raise ValueError(f"unknown model={name}")
    std = getattr(args, "init_std", None)
    if std is not None:
        from maltos_b200.models.common import init_normal_

        init_normal_(model, float(std))
    return model


def _zero3_wrap_classes() -> set[type]:
    from maltos_b200.models.llama import LlamaRMSNorm
    from maltos_b200.models.tiny_transformer import RmsNorm
    from maltos_b200.runtime.layers.distributed_rmsnorm import DistributedRMSNorm

    return {nn.Linear, nn.Embedding, nn.LayerNorm, RmsNorm, LlamaRMSNorm, DistributedRMSNorm}


def _build_hdp_config(args: argparse.Namespace):
    from maltos_b200.parallel.hdp_helper import ByteScaleHdpBalancedConfig, ByteScaleHdpCostModel

    return ByteScaleHdpBalancedConfig(partition_tokens=args.hdp_partition_tokens, balance_delta=args.hdp_balance_delta,
                                      cost_model=ByteScaleHdpCostModel(alpha=args.hdp_cost_alpha, beta=args.hdp_cost_beta, gamma=args.hdp_cost_gamma))


# ------------------------------------------------------------------------------------------------ optimizer / schedule
def _build_optimizer_factory(args: argparse.Namespace):
    if args.lr < 0:
        raise ValueError("--lr must be >= 0")
    if args.weight_decay < 0:
        raise ValueError("--weight-decay must be >= 0")
    if not 0.0 <= args.adam_beta1 < 1.0:
        raise ValueError("--adam-beta1 must be in [0, 1)")
    if not 0.0 <= args.adam_beta2 < 1.0:
        raise ValueError("--adam-beta2 must be in [0, 1)")
    if args.adam_eps <= 0:
        raise ValueError("--adam-eps must be > 0")
    kw = dict(lr=args.lr, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_eps, weight_decay=args.weight_decay)

    def factory(params):
        if args.fused_adamw:
            from maltos_b200.runtime.optim import FusedAdamW   # one multi-tensor sm_100a launch per step on CUDA

            return FusedAdamW(params, **kw)
        return torch.optim.AdamW(params, **kw)

    return factory


def lr_multiplier_fn(args: argparse.Namespace):
    floor = args.min_lr / args.lr if args.lr > 0 else 0.0

    def mult(step: int) -> float:
        if args.warmup_steps > 0 and step < args.warmup_steps:
            return max(0.0, step / args.warmup_steps)
        if args.lr_schedule == "constant":
            return 1.0
        span_steps = max(1, args.max_steps - args.warmup_steps)
        t = min(1.0, max(0.0, (step - args.warmup_steps) / span_steps))
        if args.lr_schedule == "linear":
            return floor + (1.0 - floor) * (1.0 - t)
        if args.lr_schedule == "cosine":
            return floor + (1.0 - floor) * 0.5 * (1.0 + math.cos(math.pi * t))
        raise ValueError(f"unknown lr_schedule={args.lr_schedule}")

    return mult


def _build_scheduler_factory(args: argparse.Namespace):
    if args.warmup_steps < 0:
        raise ValueError("--warmup-steps must be >= 0")
    if args.min_lr < 0:
        raise ValueError("--min-lr must be >= 0")
    if args.min_lr > args.lr:
        raise ValueError("--min-lr must be <= --lr")
    if args.lr_schedule == "constant" and args.warmup_steps == 0:
        return None
    fn = lr_multiplier_fn(args)
    return lambda optimizer: torch.optim.lr_scheduler.LambdaLR(optimizer, fn)


# ------------------------------------------------------------------------------------------------ runtime
def _build_ddp(mode: str):
    from maltos_b200.runtime.plugins.ddp import BucketDataParallelPlugin, DataParallelPlugin

    return BucketDataParallelPlugin() if mode == "bucket" else DataParallelPlugin(async_op=(mode == "async"))


def _build_runtime(args: argparse.Namespace, model: nn.Module, device: torch.device, *, weights_only: bool = False) -> RuntimeCore:
    from maltos_b200.runtime import plugins as _  # noqa: F401
    from maltos_b200.runtime.plugins.compile import CompilePlugin
    from maltos_b200.runtime.plugins.cp import ContextParallelPlugin
    from maltos_b200.runtime.plugins.ep import ExpertParallelPlugin
    from maltos_b200.runtime.plugins.fp16 import Fp16Plugin
    from maltos_b200.runtime.plugins.grad_clip import GradClipPlugin
    from maltos_b200.runtime.plugins.metrics import MetricPlugin
    from maltos_b200.runtime.plugins.pp import PipelineParallelPlugin
    from maltos_b200.runtime.plugins.torch_profiler import TorchProfilerPlugin
    from maltos_b200.runtime.plugins.tp import TensorParallelPlugin
    from maltos_b200.runtime.plugins.tp_sp import TpSpPlugin
    from maltos_b200.runtime.plugins.zero1 import Zero1Plugin
    from maltos_b200.runtime.plugins.zero2 import Zero2Plugin
    from maltos_b200.runtime.plugins.zero3 import Zero3Plugin

    dtype = {"fp32": None, "bf16": torch.bfloat16, "fp16": torch.float16}[args.precision]
    opt_factory = (lambda params: torch.optim.SGD(params, lr=0.0)) if weights_only else _build_optimizer_factory(args)
    sched_factory = None if weights_only else _build_scheduler_factory(args)
    plugins: list = []
    clip_in_core = None
    if args.tp_size > 1 and args.use_sp:
        overlap = bool(getattr(args, "tp_native_comm_overlap", False))
        workspace = None
        if overlap:       # the symmetric transfer buffers are sized and allocated at setup, not inside the first step
            from maltos_b200.runtime.layers.functional import native_comm_overlap_workspace_bytes

            workspace = native_comm_overlap_workspace_bytes(micro_batch_size=args.micro_batch_size, seq_len=args.seq_len // max(args.cp_size, 1),
                                                            hidden_size=args.dim, tp_size=args.tp_size, dtype=dtype or torch.float32)
        plugins.append(TpSpPlugin(native_comm_overlap=overlap, native_comm_overlap_workspace_bytes=workspace))
    elif args.tp_size > 1:
        plugins.append(TensorParallelPlugin())
    if args.hdp_balanced:
        from maltos_b200.runtime.plugins.hdp import ByteScaleHdpPlugin

        plugins.append(ByteScaleHdpPlugin(config=_build_hdp_config(args)))
    elif args.cp_size > 1:
        plugins.append(ContextParallelPlugin())
    if getattr(args, "token_weighted_loss", False):
        from maltos_b200.runtime.plugins.token_weighted_loss import TokenWeightedLossPlugin

        plugins.append(TokenWeightedLossPlugin())
    if args.ep_size > 1:
        plugins.append(ExpertParallelPlugin())
    if args.pp_size > 1:
        plugins.append(PipelineParallelPlugin(schedule=getattr(args, "pp_schedule", "afab") or "afab"))
    if args.zero_stage == 0:
        if args.dp_size > 1:
            plugins.append(_build_ddp(args.ddp_mode or "sync"))
    elif args.zero_stage == 1:
        plugins.append(Zero1Plugin())
    elif args.zero_stage == 2:
        plugins.append(Zero2Plugin())
    else:
        plugins.append(Zero3Plugin(wrap_cls=_zero3_wrap_classes()))
    if args.compile:
        plugins.append(CompilePlugin(scope=args.compile_scope, mode=args.compile_mode))
    if getattr(args, "cuda_graph", False):
        from maltos_b200.runtime.plugins.cuda_graph import CudaGraphPlugin

        plugins.append(CudaGraphPlugin())
    if dtype == torch.float16:
        plugins.append(Fp16Plugin(allow_cpu=torch.device(device).type == "cpu"))     # CPU runs (tests) scale the loss too
    if not weights_only and args.grad_clip is not None:
        if args.zero_stage == 0:
            plugins.append(GradClipPlugin(max_norm=args.grad_clip))
        else:
            clip_in_core = args.grad_clip
    if not weights_only and not args.disable_metrics:
        plugins.append(MetricPlugin())
    if not weights_only and args.torch_profiler:
        plugins.append(TorchProfilerPlugin(trace_dir=args.torch_profiler_dir, wait=args.torch_profiler_wait, warmup=args.torch_profiler_warmup,
                                           active=args.torch_profiler_active, repeat=args.torch_profiler_repeat,
                                           record_shapes=args.torch_profiler_record_shapes, profile_memory=args.torch_profiler_profile_memory,
                                           with_stack=args.torch_profiler_with_stack, with_flops=args.torch_profiler_with_flops,
                                           rank0_only=args.torch_profiler_rank0_only))
    plan = ParallelPlan(
        cp_attn_core=ContextParallelAttentionCoreType(args.cp_attn_core),
        batch_data_cp_aware=args.batch_data_cp_aware,
        cp_token_planner=ContextTokenPlannerType(args.cp_token_planner) if args.cp_token_planner is not None else None,
        pp_schedule=PipelineScheduleConfig(schedule=getattr(args, "pp_schedule", "afab") or "afab", microbatches=args.pp_microbatches),
    )
    mesh = MeshConfig(dp=args.dp_size, tp=args.tp_size, pp=args.pp_size, cp=args.cp_size, ep=args.ep_size)
    return RuntimeCore(model=model, mesh=mesh, plan=plan, device=device, dtype=dtype, grad_accum_steps=args.grad_accum_steps,
                       grad_clip_max_norm=clip_in_core, optimizer_factory=opt_factory, scheduler_factory=sched_factory, plugins=plugins)


# ------------------------------------------------------------------------------------------------ data
def _expand_data_paths(items: list[str]) -> list[Path]:
    out: list[Path] = []
    for item in items:
        p = Path(item)
        if p.is_dir():
            found = sorted(p.glob("*.bin"))
            if not found:
                raise ValueError(f"no .bin token shards under {p}")
            out.extend(found)
        else:
            if not p.is_file():
                raise ValueError(f"token shard not found: {p}")
            out.append(p)
    return out


def _infer_data_format(items: list[str], *, explicit: str) -> str:
    if explicit != "auto":
        return explicit
    if len(items) != 1:
        return "pretrain"
    cand = Path(items[0])
    meta = cand / "meta.json" if cand.is_dir() else cand
    if meta.is_file() and meta.name == "meta.json":
        try:
            if json.loads(meta.read_text(encoding="utf-8")).get("format") == "maltos_sft_packed":
                return "sft"
        except (OSError, json.JSONDecodeError):
            pass
    return "pretrain"


def _resolve_sft_data_source(items: list[str]) -> Path:
    if len(items) != 1:
        raise ValueError("--data-format sft expects a single SFT dataset directory or meta.json path")
    return Path(items[0])


def _build_dataloader(args: argparse.Namespace, *, dp_rank: int, cp_token_planner=None):
    from maltos_b200.data import PackedSFTDataset, PretrainingDataLoader, SFTDataLoader, TokenShardDataset

    hdp_rank = dp_rank
    dp_world = args.dp_size
    if args.hdp_balanced:          # every HDP rank reads the same canonical batch and cuts its own piece
        dp_rank, dp_world = 0, 1
    sharder = None
    if args.batch_data_cp_aware:
        if args.cp_size <= 1:
            raise ValueError("--batch-data-cp-aware requires --cp-size > 1")
        if cp_token_planner is None:
            raise ValueError("--batch-data-cp-aware requires --cp-token-planner")
        sharder = ContextParallelBatchSharder(planner=build_context_token_planner(cp_token_planner), world_size=args.cp_size)
    fmt = _infer_data_format(args.data, explicit=args.data_format)
    if fmt == "pretrain":
        paths = _expand_data_paths(args.data)
        loader = PretrainingDataLoader(TokenShardDataset(paths, dtype=np.dtype(args.token_dtype)), seq_len=args.seq_len,
                                       micro_batch_size=args.micro_batch_size, dp_rank=dp_rank, dp_world_size=dp_world, seed=args.seed,
                                       cp_batch_sharder=sharder)
    else:
        dataset = PackedSFTDataset(_resolve_sft_data_source(args.data))
        if args.seq_len != dataset.seq_len:
            raise ValueError(f"SFT dataset seq_len={dataset.seq_len} must match --seq-len={args.seq_len}")
        paths = list(dataset.shard_paths)
        loader = SFTDataLoader(dataset, micro_batch_size=args.micro_batch_size, dp_rank=dp_rank, dp_world_size=dp_world, seed=args.seed,
                               cp_batch_sharder=sharder)
    if args.hdp_balanced:
        from maltos_b200.data.bytescale_hdp import ByteScaleHdpDataLoader

        loader = ByteScaleHdpDataLoader(loader, hdp_rank=hdp_rank, hdp_world_size=args.dp_size, config=_build_hdp_config(args))
    return paths, loader, fmt


# ------------------------------------------------------------------------------------------------ logging
def _parse_tags(tags) -> list[str] | None:
    if tags is None:
        return None
    if isinstance(tags, list):
        return [str(t) for t in tags]
    out = [t.strip() for t in str(tags).split(",") if t.strip()]
    return out or None


def _build_logging(args: argparse.Namespace, rank: int):
    from maltos_b200.utils.metrics import ConsoleMetricLogger, JsonlMetricLogger, WandbCheckpointUploader, WandbMetricLogger

    if rank != 0:
        return None, None
    loggers: list = [ConsoleMetricLogger()]
    if args.metrics_jsonl:
        loggers.append(JsonlMetricLogger(args.metrics_jsonl))
    uploader = None
    if args.wandb_project and args.wandb_mode != "disabled":
        try:
            wb = WandbMetricLogger(project=args.wandb_project, name=args.wandb_run_name, entity=args.wandb_entity, run_id=args.wandb_run_id,
                                   mode=args.wandb_mode, tags=_parse_tags(args.wandb_tags), config=vars(args))
        except Exception as exc:  # noqa: BLE001 - no key, no network, package missing
            # Only this rank builds loggers: raising here would leave every other rank waiting in the next collective until
            # the process-group timeout. Training goes on with the console / JSONL sinks.
            if os.environ.get("MALTOS_B200_WANDB_REQUIRED", "0") == "1":
                raise
            print(f"WARNING: Weights & Biases logging was requested (project={args.wandb_project!r}, mode={args.wandb_mode!r}) but could not be "
                  f"started: {type(exc).__name__}: {exc}. Continuing without it (--wandb-mode offline|disabled selects that explicitly; "
                  "MALTOS_B200_WANDB_REQUIRED=1 makes this fatal).", file=sys.stderr, flush=True)
            return loggers, None
        loggers.append(wb)
        if args.wandb_checkpoint_every is not None:
            uploader = WandbCheckpointUploader(wb, every_steps=args.wandb_checkpoint_every)
    return loggers, uploader


# ------------------------------------------------------------------------------------------------ run summary / manifest
def _count_trainable_params(model: nn.Module) -> int:
    return sum(p.numel() for p in model.parameters() if p.requires_grad)


def _global_batch_tokens(args: argparse.Namespace) -> int:
    replicas = 1 if args.hdp_balanced else args.dp_size
    return args.micro_batch_size * args.seq_len * args.grad_accum_steps * replicas


def _format_optional_number(value: object) -> str:
    return "n/a" if value is None else (f"{value:,}" if isinstance(value, int) else f"{value:.6g}")


def _git_output(cmd: list[str]) -> str | None:
    try:
        out = subprocess.run(["git", *cmd], cwd=Path(__file__).resolve().parent, capture_output=True, text=True, timeout=10)
    except (OSError, subprocess.SubprocessError):
        return None
    return out.stdout.strip() if out.returncode == 0 else None


def _git_is_dirty() -> bool | None:
    status = _git_output(["status", "--porcelain"])
    return None if status is None else bool(status)


def _build_run_manifest(*, args, runtime: RuntimeCore, initial_trainable_params: int, data_paths, data_format, device, world_size: int) -> dict[str, Any]:
    local_params = sum(p.numel() for p in runtime.model.parameters())
    return {
        "git": {"commit": _git_output(["rev-parse", "HEAD"]), "dirty": _git_is_dirty()},
        "argv": list(sys.argv),
        "args": {k: (v if isinstance(v, (int, float, str, bool, list, type(None))) else str(v)) for k, v in sorted(vars(args).items())},
        "resolved": {
            "world_size": world_size,
            "device": str(device),
            "mesh": {"dp": args.dp_size, "tp": args.tp_size, "pp": args.pp_size, "cp": args.cp_size, "ep": args.ep_size},
            "plugins": [p.id.value for p in runtime.plugins],
            "trainable_params_before_sharding": initial_trainable_params,
            "local_param_elements_rank0": local_params,
            "global_batch_tokens": _global_batch_tokens(args),
            "data_format": data_format,
            "data_paths": [str(p) for p in data_paths],
            "runtime_spec": build_runtime_spec(args),
            "torch": torch.__version__,
        },
    }


def _write_run_manifest(*, rank: int, **kw) -> None:
    if rank != 0:
        return
    path = Path(kw["args"].run_manifest)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(_build_run_manifest(**kw), indent=2, sort_keys=True) + "\n", encoding="utf-8")


def _print_run_summary(*, args, runtime: RuntimeCore, initial_trainable_params: int, data_paths, data_format, device, world_size: int, rank: int) -> None:
    if rank != 0:
        return
    lines = [
        "=== training run ===",
        f"model={args.model} params={initial_trainable_params:,} dim={args.dim} layers={args.n_layers} heads={args.n_heads}/{args.n_kv_heads or args.n_heads} ffn={args.hidden_size} vocab={args.vocab_size}",
        f"mesh dp={args.dp_size} tp={args.tp_size}{'+sp' if args.use_sp else ''} pp={args.pp_size} cp={args.cp_size} ep={args.ep_size} world={world_size} device={device}",
        f"plugins={[p.id.value for p in runtime.plugins]}",
        f"precision={args.precision} zero={args.zero_stage} grad_accum={args.grad_accum_steps} grad_clip={_format_optional_number(args.grad_clip)}",
        f"data format={data_format} shards={len(data_paths)} seq_len={args.seq_len} micro_batch={args.micro_batch_size} global_batch_tokens={_global_batch_tokens(args):,}",
        f"optimizer adamw{'(fused sm_100a)' if args.fused_adamw else ''} lr={args.lr:g} schedule={args.lr_schedule} warmup={args.warmup_steps} max_steps={args.max_steps}",
    ]
    print("\n".join(lines), flush=True)


# ------------------------------------------------------------------------------------------------ process setup
def _maybe_init_distributed(args: argparse.Namespace) -> None:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1 or dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", args.master_addr)
    os.environ.setdefault("MASTER_PORT", str(args.master_port))
    backend = args.backend or ("nccl" if torch.cuda.is_available() else "gloo")
    dist.init_process_group(backend=backend)


def _select_device() -> torch.device:
    if torch.cuda.is_available():
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        return torch.device("cuda", local)
    return torch.device("cpu")


def main(argv: list[str] | None = None) -> None:
    from .flags import parse_args_from

    args = parse_args_from(argv) if argv is not None else parse_args()
    _maybe_init_distributed(args)
    device = _select_device()
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    validate_args(args, world)
    torch.manual_seed(args.seed)           # same seed on every rank: identical initial weights everywhere
    if device.type == "cuda":
        torch.cuda.manual_seed_all(args.seed)
    mesh = MeshConfig(dp=args.dp_size, pp=args.pp_size, cp=args.cp_size, tp=args.tp_size, ep=args.ep_size)
    dp_rank = mesh.rank_coordinates(rank)[0]
    model = _build_model(args)
    n_params = _count_trainable_params(model)
    args.resume_from = resolve_resume_path(args.resume_from, args.checkpoint_dir, rank=rank)
    runtime = _build_runtime(args, model, device)
    # data paths are per host: a mount missing on one node must stop every rank here, not leave the others in the first barrier
    failure, built = None, (None, None, None)
    try:
        built = _build_dataloader(args, dp_rank=dp_rank, cp_token_planner=runtime.plan.cp_token_planner)
    except Exception as exc:  # noqa: BLE001 - re-raised on every rank
        failure = exc
    raise_if_any_rank_failed(failure, "opening the training data")
    data_paths, loader, data_format = built
    loggers, uploader = (None, None) if args.dry_run else _build_logging(args, rank)
    trainer = Trainer(
        runtime=runtime, dataloader=loader, logger=loggers, checkpoint_uploader=uploader, runtime_spec=build_runtime_spec(args),
        config=TrainerConfig(max_steps=args.max_steps, log_every=args.log_every, checkpoint_every=args.checkpoint_every,
                             checkpoint_dir=args.checkpoint_dir, resume_from=args.resume_from, load_weights_only=args.load_weights_only,
                             checkpoint_keep_last=args.checkpoint_keep_last, checkpoint_keep_every_n_steps=args.checkpoint_keep_every_n_steps,
                             checkpoint_min_free_gb=args.checkpoint_min_free_gb, data_prefetch_batches=args.data_prefetch_batches))
    trainer.setup()
    if getattr(args, "graceful_stop", False):
        import signal

        trainer.enable_graceful_stop(signals=(signal.SIGTERM, signal.SIGUSR1))
    if getattr(args, "heartbeat_timeout", None):
        trainer.enable_heartbeat(timeout=float(args.heartbeat_timeout), interval=min(1.0, float(args.heartbeat_timeout) / 4))
    common = dict(args=args, runtime=runtime, initial_trainable_params=n_params, data_paths=data_paths, data_format=data_format,
                  device=device, world_size=world)
    _print_run_summary(rank=rank, **common)
    if args.run_manifest is not None:
        _write_run_manifest(rank=rank, **common)
    if args.dry_run:
        if rank == 0:
            print("dry_run=true")
        runtime.close()
    else:
        trainer.fit()
        if trainer.stopped_early_at is not None and rank == 0:
            print(f"stopped on request after step {trainer.stopped_early_at}", flush=True)
    if dist.is_initialized():
        distributed_barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

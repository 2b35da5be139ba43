"""Convert between runtime checkpoints (per-rank, layout-specific) and logical checkpoints (whole tensors, safetensors).

``runtime-to-logical --checkpoint <step dir> --output <dir>``: single process; the recipe is read from the runtime spec
stored next to the checkpoint.

``logical-to-runtime --config recipe.yaml --checkpoint <logical dir> --output <root> [-- overrides]``: run with the
target layout's world size (``torchrun``); every rank writes its own model artifact of a weights-only checkpoint
``<root>/step_00000000`` plus the runtime spec. Same command line as the reference's ``tools/convert_checkpoint.py:48-66``.
"""
from __future__ import annotations

import argparse
from pathlib import Path

import torch
import torch.distributed as dist

from maltos_b200.state.checkpoint import load_runtime_spec, save_runtime_spec, save_sharded_checkpoint_from_model_state
from maltos_b200.state.logical_checkpoint import (LogicalCheckpointTensorReader, _build_runtime_model_state_from_logical_tensors,
                                                  iter_logical_tensors_from_runtime_checkpoint, save_logical_checkpoint)
from maltos_b200.train import cli as train_cli
from maltos_b200.train.flags import build_runtime_spec, parse_args_from, parse_runtime_spec_args
from maltos_b200.utils.distributed import distributed_barrier


def build_arg_parser_for_convert() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="Convert between runtime and logical checkpoints.")
    sub = parser.add_subparsers(dest="command", required=True)
    r2l = sub.add_parser("runtime-to-logical")
    r2l.add_argument("--checkpoint", type=str, required=True, help="Source runtime checkpoint dir.")
    r2l.add_argument("--output", type=str, required=True, help="Output logical checkpoint dir.")
    l2r = sub.add_parser("logical-to-runtime")
    l2r.add_argument("--config", type=str, required=True, help="Recipe YAML for the target runtime.")
    l2r.add_argument("--checkpoint", type=str, required=True, help="Source logical checkpoint dir.")
    l2r.add_argument("--output", type=str, required=True, help="Output runtime checkpoint dir.")
    l2r.add_argument("recipe_overrides", nargs=argparse.REMAINDER, help="Optional recipe overrides after '--', reusing the training flags.")
    return parser


def _recipe_args(args: argparse.Namespace) -> argparse.Namespace:
    if args.command == "runtime-to-logical":
        return parse_runtime_spec_args(load_runtime_spec(args.checkpoint))
    overrides = list(args.recipe_overrides)
    if overrides[:1] == ["--"]:
        overrides = overrides[1:]
    return parse_args_from(["--config", args.config, *overrides], require_data=False)


def runtime_to_logical(recipe: argparse.Namespace, checkpoint_dir: Path, output_dir: Path) -> None:
    model = train_cli._build_model(recipe)
    sizes = {k: int(getattr(recipe, k, 1)) for k in ("ep_size", "dp_size", "tp_size", "pp_size", "cp_size")}
    tensors = dict(iter_logical_tensors_from_runtime_checkpoint(checkpoint_dir, model=model, **sizes))
    save_logical_checkpoint(output_dir, tensors)
    print(f"saved logical checkpoint to {output_dir}")


def logical_to_runtime(runtime, checkpoint_dir: Path, output_dir: Path, *, recipe: argparse.Namespace, rank: int) -> None:
    """Weights only: optimizer, scheduler, RNG and data-loader state are not part of a logical checkpoint."""
    reader = LogicalCheckpointTensorReader(checkpoint_dir)
    model_state, entries = _build_runtime_model_state_from_logical_tensors(runtime, reader)
    if rank == 0:
        save_runtime_spec(output_dir, build_runtime_spec(recipe))
    if dist.is_initialized():
        distributed_barrier()
    save_sharded_checkpoint_from_model_state(runtime.state_manager, output_dir / "step_00000000", model_state=model_state,
                                             rank_entries=entries, include_training_state=False)
    if rank == 0:
        print(f"saved runtime checkpoint to {output_dir}")
    if dist.is_initialized():
        distributed_barrier()


def main(argv=None) -> None:
    torch.set_grad_enabled(False)
    args = build_arg_parser_for_convert().parse_args(argv)
    recipe = _recipe_args(args)
    if args.command == "runtime-to-logical":
        runtime_to_logical(recipe, Path(args.checkpoint), Path(args.output))
        return
    train_cli._maybe_init_distributed(recipe)
    device = train_cli._select_device()
    rank = dist.get_rank() if dist.is_initialized() else 0
    runtime = train_cli._build_runtime(recipe, train_cli._build_model(recipe), device, weights_only=True)
    runtime.setup()
    try:
        logical_to_runtime(runtime, Path(args.checkpoint), Path(args.output), recipe=recipe, rank=rank)
    finally:
        runtime.close()
        if dist.is_initialized():
            distributed_barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()

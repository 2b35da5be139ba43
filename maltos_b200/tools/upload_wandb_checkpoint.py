"""Upload runtime checkpoints (``<root>/step_XXXXXXXX`` plus ``runtime_spec.json``) to Weights & Biases as artifacts.

    python -m maltos_b200.tools.upload_wandb_checkpoint --checkpoint-dir workspace/llama_50m/checkpoints/runtime \\
        --steps 1000 2000 --project maltos --artifact-prefix llama-50m-dp2-tp2-sp-zero3

One artifact per step, named ``<prefix>-step-XXXXXXXX``, aliased ``step_<n>`` (and ``latest`` for the highest step).
Same flags as the reference's ``tools/upload_wandb_checkpoint.py:18-37``. Needs the ``wandb`` package and network access.
"""
from __future__ import annotations

import argparse
import re
from pathlib import Path


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Upload a local checkpoint directory to W&B as an artifact.")
    p.add_argument("--checkpoint-dir", required=True, type=str, help="Checkpoint root directory")
    p.add_argument("--steps", required=True, type=int, nargs="+", help="Checkpoint steps to upload")
    p.add_argument("--project", required=True, type=str, help="W&B project")
    p.add_argument("--entity", type=str, default=None, help="W&B entity/team")
    p.add_argument("--run-id", type=str, default=None, help="Existing W&B run id to attach artifacts to")
    p.add_argument("--resume", type=str, default="allow", choices=("allow", "must", "never", "auto"))
    p.add_argument("--run-name", type=str, default=None, help="Temporary W&B run name for the upload")
    p.add_argument("--artifact-prefix", type=str, default=None, help="Artifact name prefix. Defaults to checkpoint root name")
    p.add_argument("--artifact-type", type=str, default="checkpoint")
    p.add_argument("--alias", action="append", default=[], help="Extra artifact alias. Can be passed multiple times")
    p.add_argument("--wait", action=argparse.BooleanOptionalAction, default=True)
    return p.parse_args(argv)


def sanitize_artifact_name(name: str) -> str:
    clean = re.sub(r"[^A-Za-z0-9_.-]+", "-", name).strip("-._")
    if not clean:
        raise ValueError(f"invalid artifact name: {name!r}")
    return clean


def plan_uploads(root: Path, steps: list[int], prefix: str, extra_aliases: list[str]) -> list[dict]:
    """What will be uploaded, validated up front: one entry per step with directory, artifact name, aliases, file count."""
    if not root.is_dir():
        raise ValueError(f"checkpoint root directory does not exist: {root}")
    if not (root / "runtime_spec.json").is_file():
        raise ValueError(f"runtime checkpoint spec not found: {root / 'runtime_spec.json'}")
    plan = []
    for step in steps:
        step_dir = root / f"step_{step:08d}"
        if not step_dir.is_dir():
            raise ValueError(f"checkpoint step directory does not exist: {step_dir}")
        if not (step_dir / "manifest.json").is_file():
            raise ValueError(f"checkpoint manifest not found: {step_dir / 'manifest.json'}")
        aliases = [*extra_aliases, f"step_{step}"] + (["latest"] if step == max(steps) else [])
        plan.append({"step": step, "dir": step_dir, "name": f"{prefix}-step-{step:08d}", "aliases": aliases,
                     "files": sum(1 for f in step_dir.rglob("*") if f.is_file())})
    return plan


def main(argv=None) -> None:
    args = parse_args(argv)
    root = Path(args.checkpoint_dir)
    prefix = sanitize_artifact_name(args.artifact_prefix or root.name)
    plan = plan_uploads(root, list(args.steps), prefix, list(args.alias))
    import wandb

    init = {"project": args.project, "entity": args.entity, "job_type": "checkpoint-upload"}
    if args.run_id is not None:
        init.update(id=args.run_id, resume=args.resume)
    if args.run_name is not None or args.run_id is None:
        init["name"] = args.run_name or f"upload-{prefix}"
    run = wandb.init(**init)
    try:
        for item in plan:
            artifact = wandb.Artifact(name=item["name"], type=args.artifact_type,
                                      metadata={"step": item["step"], "path": str(item["dir"]), "files": item["files"]})
            artifact.add_file(str(root / "runtime_spec.json"), name="runtime_spec.json")
            artifact.add_dir(str(item["dir"]), name=item["dir"].name)
            logged = run.log_artifact(artifact, aliases=item["aliases"])
            if args.wait:
                logged.wait()
            print(f"uploaded {item['dir']} to {args.project}/{item['name']} aliases={item['aliases']}")
    finally:
        run.finish()


if __name__ == "__main__":
    main()

"""Sharded runtime checkpoints.

Layout (identical to the reference, ``state/checkpoint.py:86-250``, so either implementation loads the other's):

    <root>/runtime_spec.json
    <root>/step_XXXXXXXX/manifest.json          rank 0; json.dump(indent=2)
    <root>/step_XXXXXXXX/model_rank_R.pt        dict[state_key -> CPU tensor]
    <root>/step_XXXXXXXX/optim_rank_R.pt        only ranks that are their own optimizer source
    <root>/step_XXXXXXXX/trainer_rank_R.pt      asdict(TrainerState)

Writes go to ``step_XXXXXXXX.tmp`` and rank 0 renames after a barrier, so a crash never leaves a half-written
checkpoint under the final name.
"""
from __future__ import annotations

import json
import shutil
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Literal

import torch
import torch.distributed as dist

from maltos_b200.runtime.types import PpStatus, RuntimePhase
from maltos_b200.utils.distributed import distributed_barrier, raise_if_any_rank_failed

from .state import ModelStateMeta, OptimizerState, RngState, StateManager, TrainerState

MANIFEST_VERSION = 1
ArtifactKind = Literal["model", "optimizer", "trainer"]


@dataclass(frozen=True)
class CheckpointArtifact:
    kind: ArtifactKind
    rank: int
    path: str
    source_rank: int | None = None


@dataclass(frozen=True)
class RankCheckpointMetadata:
    rank: int
    entries: list[ModelStateMeta]


@dataclass(frozen=True)
class CheckpointManifest:
    version: int
    world_size: int
    ranks: list[RankCheckpointMetadata]
    optimizer_source_ranks: list[int]
    artifacts: list[CheckpointArtifact]


def _rank_world() -> tuple[int, int]:
    if dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _meta_from_json(d: dict[str, Any]) -> ModelStateMeta:
    src = d.get("source_rank")
    return ModelStateMeta(
        state_key=d["state_key"],
        logical_names=[str(n) for n in d["logical_names"]],
        logical_shapes=[tuple(s) for s in d["logical_shapes"]],
        physical_shape=tuple(d["physical_shape"]),
        dtype=d["dtype"],
        source_rank=None if src is None else int(src),
    )


# ------------------------------------------------------------------------------------------------ save
def save_sharded_checkpoint(state_manager: StateManager, path, *, min_free_gb: float | None = None) -> None:
    _save(state_manager, Path(path), min_free_gb, None, None, True)


def save_sharded_checkpoint_from_model_state(state_manager: StateManager, path, *, model_state: dict[str, torch.Tensor],
                                             rank_entries: list[ModelStateMeta], include_training_state: bool = True,
                                             min_free_gb: float | None = None) -> None:
    """Write a checkpoint whose model part is given explicitly (used by the logical -> runtime converter)."""
    _save(state_manager, Path(path), min_free_gb, model_state, rank_entries, include_training_state)


def _save(sm: StateManager, final_dir: Path, min_free_gb, model_override, entries_override, with_training: bool) -> None:
    # A refusal or an I/O error on one rank (the directory exists, the disk is full) stops ALL ranks at the next agreement
    # point: a rank that raised alone would leave the others waiting in the barrier behind it.
    rank, _ = _rank_world()
    tmp_dir = final_dir.with_name(final_dir.name + ".tmp")
    failure = None
    try:
        if min_free_gb is not None:
            _check_min_free_space(final_dir.parent, min_free_gb)
        if rank == 0:
            if final_dir.exists():
                if any(final_dir.iterdir()):
                    raise FileExistsError(f"checkpoint already exists: {final_dir}")
                final_dir.rmdir()
            if tmp_dir.exists():
                shutil.rmtree(tmp_dir)
            tmp_dir.parent.mkdir(parents=True, exist_ok=True)
    except Exception as exc:  # noqa: BLE001 - re-raised on every rank
        failure = exc
    raise_if_any_rank_failed(failure, f"preparing checkpoint directory {final_dir}")
    written = None
    try:
        written = _write_local_files(sm, tmp_dir, model_override, entries_override, with_training)
    except Exception as exc:  # noqa: BLE001
        failure = exc
    raise_if_any_rank_failed(failure, f"writing checkpoint files under {tmp_dir}")
    _write_manifest(sm, tmp_dir, *written)
    if rank == 0:
        tmp_dir.rename(final_dir)
    distributed_barrier()


def _write_local_files(sm: StateManager, out_dir: Path, model_override, entries_override, with_training: bool):
    """This rank's ``.pt`` files; returns ``(entries, artifacts)`` as JSON-ready lists for the manifest."""
    runtime = sm.runtime
    rank, _ = _rank_world()
    out_dir.mkdir(parents=True, exist_ok=True)

    if model_override is not None and entries_override is not None:
        tensors = {k: v.detach().cpu().contiguous() for k, v in model_override.items()}
        entries = [ModelStateMeta(e.state_key, list(e.logical_names), list(e.logical_shapes), tuple(e.physical_shape),
                                  e.dtype, e.source_rank) for e in entries_override]
    else:
        tensors, entries = sm.export_model_state()

    artifacts: list[dict[str, Any]] = []
    model_file = f"model_rank_{rank}.pt"
    torch.save(tensors, out_dir / model_file)
    artifacts.append(asdict(CheckpointArtifact("model", rank, model_file)))

    if with_training:
        opt = sm.export_optimizer_state()
        if opt is not None and runtime.should_save_optimizer(rank):
            optim_file = f"optim_rank_{rank}.pt"
            torch.save(opt.state, out_dir / optim_file)
            artifacts.append(asdict(CheckpointArtifact("optimizer", rank, optim_file, source_rank=rank)))
        trainer_file = f"trainer_rank_{rank}.pt"
        torch.save(asdict(sm.export_trainer_state()), out_dir / trainer_file)
        artifacts.append(asdict(CheckpointArtifact("trainer", rank, trainer_file)))

    return [asdict(e) for e in entries], artifacts


def _write_manifest(sm: StateManager, out_dir: Path, entry_dicts, artifacts) -> None:
    """Collective: rank 0 gathers every rank's entries and artifacts and writes ``manifest.json``."""
    runtime = sm.runtime
    rank, world = _rank_world()
    if dist.is_initialized():
        all_entries = [None] * world if rank == 0 else None
        all_artifacts = [None] * world if rank == 0 else None
        dist.gather_object(entry_dicts, all_entries, dst=0)
        dist.gather_object(artifacts, all_artifacts, dst=0)
    else:
        all_entries, all_artifacts = [entry_dicts], [artifacts]

    if rank == 0:
        manifest = CheckpointManifest(
            version=MANIFEST_VERSION,
            world_size=world,
            ranks=[RankCheckpointMetadata(r, [_meta_from_json(e) for e in (ents or [])]) for r, ents in enumerate(all_entries)],
            optimizer_source_ranks=[runtime.optimizer_checkpoint_rank(r) for r in range(world)],
            artifacts=[CheckpointArtifact(**a) for per_rank in all_artifacts for a in (per_rank or [])],
        )
        with open(out_dir / "manifest.json", "w", encoding="utf-8") as f:
            json.dump(asdict(manifest), f, indent=2)
    distributed_barrier()


# ------------------------------------------------------------------------------------------------ load
def load_checkpoint_manifest(checkpoint_dir) -> CheckpointManifest:
    with open(Path(checkpoint_dir) / "manifest.json", "r", encoding="utf-8") as f:
        raw = json.load(f)
    version = int(raw.get("version", 0))
    if version != MANIFEST_VERSION:
        raise ValueError(f"unsupported checkpoint manifest version={version}")
    if "artifacts" not in raw:
        raise ValueError("manifest missing artifacts field")
    return CheckpointManifest(
        version=version,
        world_size=int(raw["world_size"]),
        ranks=[RankCheckpointMetadata(int(r["rank"]), [_meta_from_json(e) for e in r["entries"]]) for r in raw["ranks"]],
        optimizer_source_ranks=[int(x) for x in raw["optimizer_source_ranks"]],
        artifacts=[CheckpointArtifact(a["kind"], int(a["rank"]), a["path"],
                                      None if a.get("source_rank") is None else int(a["source_rank"]))
                   for a in raw["artifacts"]],
    )


def _artifact(manifest: CheckpointManifest, kind: str, rank: int) -> CheckpointArtifact | None:
    return next((a for a in manifest.artifacts if a.kind == kind and a.rank == rank), None)


def _read_artifact(path):
    """One ``.pt`` file of a checkpoint; an unreadable file (truncated by a crash or a full disk, damaged in transit) is
    reported with its path instead of the archive reader's message."""
    try:
        return torch.load(path, map_location="cpu", weights_only=True)
    except FileNotFoundError:
        raise
    except Exception as exc:  # noqa: BLE001 - zip / pickle errors of any kind
        raise ValueError(f"checkpoint file {path} cannot be read (truncated or corrupt?): {type(exc).__name__}: {exc}") from exc


def load_sharded_checkpoint(state_manager: StateManager, path, *, weights_only: bool = False) -> None:
    runtime = state_manager.runtime
    ckpt = Path(path)
    rank, _ = _rank_world()
    # Reading is file work without collectives, and every rank reads different files: one of them may fail alone (a file
    # cut short, a missing mount). All ranks learn of it here, before the first collective of the import.
    model_state = trainer_blob = optim_blob = None
    failure = None
    try:
        manifest = load_checkpoint_manifest(ckpt)
        _validate_manifest_for_runtime(manifest, runtime, weights_only=weights_only)
        model_state = _gather_model_entries(ckpt, manifest, manifest.ranks[rank], rank)
        if not weights_only:
            t_art = _artifact(manifest, "trainer", rank)
            if t_art is None:
                raise ValueError(f"manifest missing trainer artifact for rank={rank}")
            with torch.serialization.safe_globals([PpStatus]):
                trainer_blob = _read_artifact(ckpt / t_art.path)
            o_art = _artifact(manifest, "optimizer", manifest.optimizer_source_ranks[rank])
            if o_art is not None:
                optim_blob = _read_artifact(ckpt / o_art.path)
    except Exception as exc:  # noqa: BLE001 - re-raised below, on every rank
        failure = exc
    raise_if_any_rank_failed(failure, f"reading checkpoint {ckpt}")

    state_manager.import_model_state(model_state)
    optimizer, _ = runtime.get_optimizer_and_scheduler()
    resync = getattr(optimizer, "sync_master_params_from_model", None)
    if callable(resync):
        resync()
    if optim_blob is not None:
        state_manager.import_optimizer_state(OptimizerState(state=optim_blob))
    if trainer_blob is not None:
        rng = trainer_blob["rng"]
        state_manager.import_trainer_state(TrainerState(
            rng=RngState(cpu=rng["cpu"], cuda=rng.get("cuda")),
            step_context=trainer_blob.get("step_context"),
            dataloader=trainer_blob.get("dataloader"),
            plugin_states=trainer_blob.get("plugin_states"),
        ))
    # plugins that re-derive their shards after a load must not round restored fp32 master weights through the model dtype
    runtime.state.metadata["optimizer_state_restored"] = optim_blob is not None
    runtime._run_step_phase(RuntimePhase.POST_LOAD)
    distributed_barrier()


def _gather_model_entries(ckpt: Path, manifest: CheckpointManifest, rank_meta: RankCheckpointMetadata, rank: int) -> dict[str, torch.Tensor]:
    opened: dict[int, dict[str, torch.Tensor]] = {}
    out: dict[str, torch.Tensor] = {}
    for entry in rank_meta.entries:
        src = entry.source_rank
        if src is None:
            raise ValueError(f"manifest missing model source rank for entry={entry.state_key}, rank={rank}")
        art = _artifact(manifest, "model", src)
        if art is None:
            raise ValueError(f"manifest missing model artifact for source rank={src} (used by rank={rank}, entry={entry.state_key})")
        if src not in opened:
            opened[src] = _read_artifact(ckpt / art.path)
        if entry.state_key not in opened[src]:
            raise ValueError(f"model state missing entry={entry.state_key} in source rank={src} artifact")
        out[entry.state_key] = opened[src][entry.state_key]
    return out


def _validate_manifest_for_runtime(manifest: CheckpointManifest, runtime, *, weights_only: bool = False) -> None:
    rank, world = _rank_world()
    n = manifest.world_size
    if n != world:
        raise ValueError(f"checkpoint world_size mismatch: checkpoint={n}, runtime={world}")
    if len(manifest.ranks) != n:
        raise ValueError(f"manifest ranks length mismatch: expected={n}, got={len(manifest.ranks)}")
    if len(manifest.optimizer_source_ranks) != n:
        raise ValueError(f"manifest optimizer_source_ranks length mismatch: expected={n}, got={len(manifest.optimizer_source_ranks)}")
    if rank >= n:
        raise ValueError(f"runtime rank out of range: rank={rank}, world_size={n}")
    seen: set[tuple[str, int]] = set()
    for a in manifest.artifacts:
        if (a.kind, a.rank) in seen:
            raise ValueError(f"duplicate artifact in manifest: kind={a.kind}, rank={a.rank}")
        seen.add((a.kind, a.rank))
    for r in range(n):
        if ("model", r) not in seen:
            raise ValueError(f"manifest missing model artifact for rank={r}")
        if not weights_only and ("trainer", r) not in seen:
            raise ValueError(f"manifest missing trainer artifact for rank={r}")
    for rm in manifest.ranks:
        for e in rm.entries:
            if e.source_rank is None:
                raise ValueError(f"manifest missing model source rank for entry={e.state_key}, rank={rm.rank}")
            if not 0 <= e.source_rank < n:
                raise ValueError(f"manifest model source rank out of range: rank={rm.rank}, entry={e.state_key}, source_rank={e.source_rank}")
            if ("model", e.source_rank) not in seen:
                raise ValueError(f"manifest missing model artifact for source rank={e.source_rank} (used by rank={rm.rank}, entry={e.state_key})")
    if weights_only:
        return
    optim_ranks = {a.rank for a in manifest.artifacts if a.kind == "optimizer"}
    if not optim_ranks:
        return
    for r, src in enumerate(manifest.optimizer_source_ranks):
        if not 0 <= src < n:
            raise ValueError(f"manifest optimizer source rank out of range: rank={r}, source_rank={src}")
        if src not in optim_ranks:
            raise ValueError(f"manifest missing optimizer artifact for source rank={src} (used by rank={r})")
    for r in range(n):
        expected = runtime.optimizer_checkpoint_rank(r)
        if expected != manifest.optimizer_source_ranks[r]:
            raise ValueError("optimizer source mapping mismatch between runtime and checkpoint manifest: "
                             f"rank={r}, runtime={expected}, checkpoint={manifest.optimizer_source_ranks[r]}")


# ------------------------------------------------------------------------------------------------ runtime spec
def save_runtime_spec(checkpoint_root, runtime_spec: dict[str, Any]) -> None:
    if not isinstance(runtime_spec, dict) or not runtime_spec:
        raise ValueError("runtime_spec must be a non-empty mapping")
    root = Path(checkpoint_root)
    root.mkdir(parents=True, exist_ok=True)
    target = root / "runtime_spec.json"
    if target.exists():
        if load_runtime_spec(root) != runtime_spec:
            raise ValueError(f"runtime spec already exists with different contents: {target}")
        return
    tmp = root / "runtime_spec.json.tmp"
    with tmp.open("w", encoding="utf-8") as f:
        json.dump(runtime_spec, f, indent=2)
        f.write("\n")
    tmp.replace(target)


def load_runtime_spec(checkpoint) -> dict[str, Any]:
    p = Path(checkpoint)
    for cand in (p / "runtime_spec.json", p.parent / "runtime_spec.json"):
        if cand.is_file():
            with cand.open("r", encoding="utf-8") as f:
                spec = json.load(f)
            if not isinstance(spec, dict) or not spec:
                raise ValueError("runtime_spec.json must contain a non-empty mapping")
            return spec
    raise ValueError(f"runtime spec not found for {p}; expected runtime_spec.json in the checkpoint root")


def _check_min_free_space(path: Path, min_free_gb: float) -> None:
    if min_free_gb < 0:
        raise ValueError(f"min_free_gb must be >= 0, got {min_free_gb}")
    path.mkdir(parents=True, exist_ok=True)
    free_gb = shutil.disk_usage(path).free / 1e9
    if free_gb < min_free_gb:
        raise RuntimeError(f"insufficient free space for checkpoint: path={path} free_gb={free_gb:.2f} required_gb={min_free_gb:.2f}")

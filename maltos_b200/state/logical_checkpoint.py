"""Logical (layout-free) model checkpoints in safetensors form, and conversion from / to runtime checkpoints.

A *logical* checkpoint stores every parameter and buffer once, whole, under its model name: either one
``model.safetensors`` or HF-style shards ``model-0000i-of-0000n.safetensors`` with ``model.safetensors.index.json``
(``{"metadata": {"format": "logical_model", "version": 1, "total_size": ...}, "weight_map": {name: shard}}``). HF
checkpoints that prefix names with ``model.`` (all but ``lm_head.weight``) are read transparently.

A *runtime* checkpoint stores what each rank holds: TP-sharded slices, several parameters packed into one entry, or
``1/N`` slices of flat ZeRO-3 buckets. The two directions here:

* :func:`iter_logical_tensors_from_runtime_checkpoint` reads a runtime checkpoint's manifest, un-packs entries,
  concatenates ZeRO-3 bucket slices over their owner ranks and TP slices along the axis the model's TP/SP spec names;
* :func:`_build_runtime_model_state_from_logical_tensors` cuts the logical tensors into exactly the entries the running
  ``RuntimeCore`` of THIS rank would save, so a weights-only runtime checkpoint can be written for any layout.

Same file format and public functions as the reference's ``state/logical_checkpoint.py:1-704``.
"""
from __future__ import annotations

import json
import math
from collections.abc import Mapping
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import TYPE_CHECKING, Iterable, Iterator

import torch
import torch.distributed as dist

from maltos_b200.parallel.specs import TpSpShardAxis
from maltos_b200.runtime.mesh import MeshAxis
from maltos_b200.state.checkpoint import CheckpointManifest, _read_artifact, load_checkpoint_manifest
from maltos_b200.state.state import ModelStateMeta

if TYPE_CHECKING:
    from maltos_b200.runtime.core import RuntimeCore

_LOGICAL_SINGLE_NAME = "model.safetensors"
_LOGICAL_INDEX_NAME = "model.safetensors.index.json"
_DEFAULT_LOGICAL_SHARD_SIZE_BYTES = 5 * 1024 * 1024 * 1024
_ZERO3_PREFIX = "zero3_bucket_"


@dataclass(frozen=True)
class LogicalCheckpointManifest:
    metadata: dict[str, str | int]
    weight_map: dict[str, str]


# ------------------------------------------------------------------------------------------------ names
def _logical_tensor_name(checkpoint_name: str) -> str:
    return checkpoint_name[len("model."):] if checkpoint_name.startswith("model.") else checkpoint_name


def _checkpoint_tensor_name(logical_name: str) -> str:
    return logical_name if logical_name == "lm_head.weight" else f"model.{logical_name}"


def _resolve_checkpoint_tensor_name(keys, logical_name: str) -> str:
    """The name under which ``logical_name`` is stored among ``keys`` (plain, or with the HF ``model.`` prefix)."""
    if logical_name in keys:
        return logical_name
    prefixed = _checkpoint_tensor_name(logical_name)
    return prefixed if prefixed in keys else logical_name


def _load_logical_index(index_path: Path) -> LogicalCheckpointManifest:
    raw = json.loads(index_path.read_text(encoding="utf-8"))
    metadata, weight_map = raw.get("metadata"), raw.get("weight_map")
    if not isinstance(metadata, dict):
        raise ValueError(f"logical checkpoint index missing metadata: {index_path}")
    if not isinstance(weight_map, dict) or not weight_map:
        raise ValueError(f"logical checkpoint index missing weight_map: {index_path}")
    fmt = metadata.get("format")
    if fmt is not None:     # HF indexes carry no format tag and are accepted as they are
        if fmt != "logical_model":
            raise ValueError(f"unsupported logical checkpoint format={fmt!r}")
        if int(metadata.get("version", 0)) != 1:
            raise ValueError(f"unsupported logical checkpoint version={int(metadata.get('version', 0))}")
    normalized: dict[str, str] = {}
    stored_as: dict[str, str] = {}
    for stored, shard in weight_map.items():
        name = _logical_tensor_name(str(stored))
        if stored_as.setdefault(name, str(stored)) != str(stored):
            raise ValueError(f"logical checkpoint index maps multiple tensors to logical name={name}: {stored_as[name]}, {stored}")
        normalized[name] = str(shard)
    return LogicalCheckpointManifest({str(k): v for k, v in metadata.items()}, normalized)


class _LogicalStore:
    """Read access to a logical checkpoint directory in either of its two forms."""

    def __init__(self, path: str | Path) -> None:
        self.dir = Path(path)
        index, single = self.dir / _LOGICAL_INDEX_NAME, self.dir / _LOGICAL_SINGLE_NAME
        if index.is_file():
            self.weight_map: dict[str, str] | None = _load_logical_index(index).weight_map
        elif single.is_file():
            self.weight_map = None
        else:
            raise ValueError(f"logical checkpoint not found in {self.dir}; expected {_LOGICAL_INDEX_NAME} or {_LOGICAL_SINGLE_NAME}")

    def _open(self, file_name: str):
        from safetensors import safe_open

        return safe_open(str(self.dir / file_name), framework="pt", device="cpu")

    def names(self) -> frozenset[str]:
        if self.weight_map is not None:
            return frozenset(self.weight_map)
        with self._open(_LOGICAL_SINGLE_NAME) as f:
            return frozenset(_logical_tensor_name(k) for k in f.keys())

    def get(self, name: str) -> torch.Tensor:
        if self.weight_map is None:
            with self._open(_LOGICAL_SINGLE_NAME) as f:
                if name not in f.keys():
                    raise KeyError(f"logical checkpoint missing tensor={name}")
                return f.get_tensor(name)
        shard = self.weight_map.get(name)
        if shard is None:
            raise KeyError(f"logical checkpoint missing tensor={name}")
        with self._open(shard) as f:
            return f.get_tensor(_resolve_checkpoint_tensor_name(f.keys(), name))

    def items(self) -> Iterator[tuple[str, torch.Tensor]]:
        """All tensors, one shard file open at a time, names sorted inside each shard."""
        if self.weight_map is None:
            with self._open(_LOGICAL_SINGLE_NAME) as f:
                for k in sorted(f.keys()):
                    yield k, f.get_tensor(k)
            return
        per_shard: dict[str, list[str]] = {}
        for name, shard in self.weight_map.items():
            per_shard.setdefault(shard, []).append(name)
        for shard in sorted(per_shard):
            with self._open(shard) as f:
                keys = set(f.keys())
                for name in sorted(per_shard[shard]):
                    stored = _resolve_checkpoint_tensor_name(keys, name)
                    if stored not in keys:
                        raise ValueError(f"logical checkpoint shard={shard} missing tensor={stored}")
                    yield name, f.get_tensor(stored)


class LogicalCheckpointTensorReader(Mapping[str, torch.Tensor]):
    """Mapping view that opens each requested tensor on demand. Logical-to-runtime conversion runs once per target rank;
    holding the whole model in every process would multiply host memory by the world size although a rank needs only
    its own slices."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        self._store = _LogicalStore(path)
        self._names = self._store.names()

    def __getitem__(self, name: str) -> torch.Tensor:
        if name not in self._names:
            raise KeyError(f"logical checkpoint missing tensor={name}")
        return self._store.get(name)

    def __iter__(self):
        return iter(self._names)

    def __len__(self) -> int:
        return len(self._names)


# ------------------------------------------------------------------------------------------------ logical I/O
def _plan_logical_shards(tensors: dict[str, torch.Tensor], *, max_shard_size_bytes: int) -> list[dict[str, torch.Tensor]]:
    """Greedy split in name order; a tensor larger than the limit gets a shard of its own."""
    shards: list[dict[str, torch.Tensor]] = [{}]
    used = 0
    for name, t in tensors.items():
        size = t.numel() * t.element_size()
        if shards[-1] and used + size > max_shard_size_bytes:
            shards.append({})
            used = 0
        shards[-1][name] = t
        used += size
    return shards


def save_logical_checkpoint(path: str | Path, tensors: dict[str, torch.Tensor], *,
                            max_shard_size_bytes: int = _DEFAULT_LOGICAL_SHARD_SIZE_BYTES) -> None:
    from safetensors.torch import save_file

    if max_shard_size_bytes < 1:
        raise ValueError(f"max_shard_size_bytes must be >= 1, got {max_shard_size_bytes}")
    out = Path(path)
    out.mkdir(parents=True, exist_ok=True)
    host = {name: t.detach().cpu().contiguous() for name, t in sorted(tensors.items())}
    shards = _plan_logical_shards(host, max_shard_size_bytes=max_shard_size_bytes)
    weight_map: dict[str, str] = {}
    for i, shard in enumerate(shards, start=1):
        file_name = f"model-{i:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, str(out / file_name))
        weight_map.update({name: file_name for name in shard})
    index = LogicalCheckpointManifest(
        metadata={"format": "logical_model", "version": 1, "total_size": sum(t.numel() * t.element_size() for t in host.values())},
        weight_map=weight_map)
    (out / _LOGICAL_INDEX_NAME).write_text(json.dumps(asdict(index), indent=2, sort_keys=True) + "\n", encoding="utf-8")


def load_logical_checkpoint(path: str | Path) -> dict[str, torch.Tensor]:
    store = _LogicalStore(path)
    if store.weight_map is None:
        from safetensors.torch import load_file

        return load_file(str(store.dir / _LOGICAL_SINGLE_NAME), device="cpu")
    return dict(store.items())


def load_logical_tensor(path: str | Path, name: str) -> torch.Tensor:
    return _LogicalStore(path).get(name)


def iter_logical_checkpoint_tensors(path: str | Path) -> Iterable[tuple[str, torch.Tensor]]:
    return _LogicalStore(path).items()


# ------------------------------------------------------------------------------------------------ tensor-parallel layout
def _tp_shard_rules(model) -> dict[str, str]:
    """``{"<module path>.weight" / ".bias": PARAM_OUT | PARAM_IN}`` from the model's TP/SP spec (empty without one)."""
    if not hasattr(model, "tpsp_parallelize_spec"):
        return {}
    rules: dict[str, str] = {}
    for rule in model.tpsp_parallelize_spec().rules:
        if rule.shard_axis in (TpSpShardAxis.PARAM_OUT, TpSpShardAxis.PARAM_IN):
            rules[f"{rule.module_path}.weight"] = rule.shard_axis
            rules[f"{rule.module_path}.bias"] = rule.shard_axis
    return rules


def _local_tensor_for_runtime_tensor(*, name: str, logical: torch.Tensor, shard_rules: dict[str, str], tp_rank: int,
                                     tp_world_size: int) -> torch.Tensor:
    axis = shard_rules.get(name)
    if axis == TpSpShardAxis.PARAM_OUT:
        n = logical.size(0) // tp_world_size
        return logical[tp_rank * n:(tp_rank + 1) * n]
    if axis == TpSpShardAxis.PARAM_IN:
        n = logical.size(1) // tp_world_size
        return logical[:, tp_rank * n:(tp_rank + 1) * n]
    return logical


def _assemble_logical_tensor(*, name: str, pieces: list[tuple[int, torch.Tensor]], shard_rules: dict[str, str],
                             target_shape: tuple[int, ...]) -> torch.Tensor:
    """Join the per-rank pieces of one tensor (ordered by owner rank) along its TP axis; replicas must agree."""
    axis = shard_rules.get(name)
    if len(pieces) == 1:
        only = pieces[0][1]
        if tuple(only.shape) == tuple(target_shape):
            return only
        if axis is None:
            raise ValueError(f"logical tensor={name} has local shape={tuple(only.shape)} but expected full shape={target_shape}")
    ordered = [t for _, t in sorted(pieces, key=lambda item: item[0])]
    if axis == TpSpShardAxis.PARAM_OUT:
        full = torch.cat(ordered, dim=0)
    elif axis == TpSpShardAxis.PARAM_IN:
        full = torch.cat(ordered, dim=1)
    elif len(ordered) == 1:
        full = ordered[0]
    else:
        if all(tuple(t.shape) == tuple(target_shape) for t in ordered) and all(torch.equal(ordered[0], t) for t in ordered[1:]):
            return ordered[0]
        raise ValueError(f"logical tensor={name} has {len(ordered)} runtime pieces but no shard metadata to combine them")
    if tuple(full.shape) != tuple(target_shape):
        raise ValueError(f"logical tensor={name} shape mismatch after reconstruction: expected={target_shape}, got={tuple(full.shape)}")
    return full


# ------------------------------------------------------------------------------------------------ runtime -> logical
def _is_zero3_entry(entry: ModelStateMeta) -> bool:
    return entry.state_key.startswith(_ZERO3_PREFIX)


def _rank_coordinates(*, rank: int, dp_size: int, pp_size: int, cp_size: int, tp_size: int) -> tuple[int, int, int, int]:
    """(dp, pp, cp, tp) indices of a global rank in the ``[dp][pp][cp][tp]`` rank order (TP innermost)."""
    rest, tp_idx = divmod(rank, tp_size)
    rest, cp_idx = divmod(rest, cp_size)
    dp_idx, pp_idx = divmod(rest, pp_size)
    if not 0 <= dp_idx < dp_size:
        raise ValueError(f"rank={rank} out of range for mesh dp={dp_size}, pp={pp_size}, cp={cp_size}, tp={tp_size}")
    return dp_idx, pp_idx, cp_idx, tp_idx


def _owned_model_entries(manifest: CheckpointManifest) -> list[tuple[int, ModelStateMeta]]:
    owned = []
    for rank_meta in manifest.ranks:
        for entry in rank_meta.entries:
            if entry.source_rank is None:
                raise ValueError(f"manifest missing model source rank for entry={entry.state_key}, rank={rank_meta.rank}")
            if entry.source_rank == rank_meta.rank:
                owned.append((rank_meta.rank, entry))
    return owned


def _find_model_artifact(manifest: CheckpointManifest, rank: int):
    return next((a for a in manifest.artifacts if a.kind == "model" and a.rank == rank), None)


def _split_entry_tensor(entry: ModelStateMeta, tensor: torch.Tensor) -> Iterable[tuple[str, torch.Tensor]]:
    """Un-pack an entry that stores several logical tensors back to back."""
    if len(entry.logical_names) == 1:
        yield entry.logical_names[0], tensor
        return
    flat = tensor.contiguous().view(-1)
    at = 0
    for name, shape in zip(entry.logical_names, entry.logical_shapes, strict=True):
        n = int(math.prod(shape))
        if at + n > flat.numel():
            raise ValueError(f"checkpoint entry={entry.state_key} too small to unpack logical tensor={name} with shape={shape}")
        yield name, flat[at:at + n].view(shape)
        at += n
    if at != flat.numel():
        raise ValueError(f"checkpoint entry={entry.state_key} packed tensor size mismatch: consumed={at}, total={flat.numel()}")


class _RankFiles:
    """Lazily loaded model artifacts of a runtime checkpoint, one per owner rank."""

    def __init__(self, checkpoint_dir: Path, manifest: CheckpointManifest) -> None:
        self.dir, self.manifest = checkpoint_dir, manifest
        self._cache: dict[int, dict[str, torch.Tensor]] = {}

    def entry(self, rank: int, state_key: str) -> torch.Tensor:
        if rank not in self._cache:
            artifact = _find_model_artifact(self.manifest, rank)
            if artifact is None:
                raise ValueError(f"manifest missing model artifact for rank={rank}")
            self._cache[rank] = _read_artifact(self.dir / artifact.path)
        state = self._cache[rank]
        if state_key not in state:
            raise ValueError(f"model state missing entry={state_key} in source rank={rank} artifact")
        return state[state_key]


def iter_logical_tensors_from_runtime_checkpoint(checkpoint_dir: str | Path, *, model, ep_size: int = 1, dp_size: int = 1,
                                                 tp_size: int = 1, pp_size: int = 1, cp_size: int = 1) -> Iterable[tuple[str, torch.Tensor]]:
    """Yield ``(name, full tensor)`` for every entry of ``model.state_dict()`` rebuilt from a runtime checkpoint.

    ``model`` is the untransformed model of the checkpoint's recipe (it supplies names, shapes, dtypes and TP rules).
    """
    from maltos_b200.runtime.layers.moe import ExpertParallelMoE

    checkpoint_dir = Path(checkpoint_dir)
    if any(isinstance(m, ExpertParallelMoE) for m in model.modules()):
        raise NotImplementedError("offline logical checkpoint conversion does not yet support ExpertParallelMoE models")
    manifest = load_checkpoint_manifest(checkpoint_dir)
    rules = _tp_shard_rules(model)
    reference_state = model.state_dict()
    files = _RankFiles(checkpoint_dir, manifest)

    pieces: dict[str, list[tuple[int, torch.Tensor]]] = {}
    first_writer: dict[tuple[str, int, int], int] = {}
    zero3_groups: dict[tuple, list[tuple[int, ModelStateMeta]]] = {}
    for owner, entry in sorted(_owned_model_entries(manifest), key=lambda item: item[0]):
        if _is_zero3_entry(entry):
            # The slices of one bucket live on the ranks that differ only in the sharding (dp / cp) coordinates. Every
            # tensor-parallel coordinate has a bucket of its own, also for tensors that are replicated over that axis (their
            # copies are compared when the tensor is assembled); expert buckets of different expert-parallel ranks differ in
            # their (global) names.
            _, pp_idx, _, tp_idx = _rank_coordinates(rank=owner, dp_size=dp_size, pp_size=pp_size, cp_size=cp_size, tp_size=tp_size)
            key = ("zero3", pp_idx, tp_idx, tuple(entry.logical_names), tuple(entry.logical_shapes))
            zero3_groups.setdefault(key, []).append((owner, entry))
            continue
        _, pp_idx, _, tp_idx = _rank_coordinates(rank=owner, dp_size=dp_size, pp_size=pp_size, cp_size=cp_size, tp_size=tp_size)
        for name in entry.logical_names:
            # a tensor that several data / context-parallel replicas wrote (a checkpoint whose writer left those axes
            # unmarked) is taken once per pipeline and tensor-parallel coordinate: from its lowest writer
            first = first_writer.setdefault((name, pp_idx, tp_idx), owner)
            if first != owner:
                break
        else:
            for name, local in _split_entry_tensor(entry, files.entry(owner, entry.state_key)):
                pieces.setdefault(name, []).append((owner, local.detach().cpu().contiguous()))

    for members in zero3_groups.values():
        exemplar = members[0][1]
        owners = sorted(r for r, _ in members)
        flat = torch.cat([files.entry(r, exemplar.state_key).detach().cpu().contiguous().view(-1) for r in owners])
        at = 0
        for name, shape in zip(exemplar.logical_names, exemplar.logical_shapes, strict=True):
            n = int(math.prod(shape))
            if at + n > flat.numel():
                raise ValueError(f"zero3 bucket={exemplar.state_key} too small to unpack logical tensor={name} with shape={shape}")
            pieces.setdefault(name, []).append((owners[0], flat[at:at + n].view(shape)))
            at += n

    missing = sorted(set(reference_state) - set(pieces))
    if missing:
        raise ValueError(f"runtime checkpoint missing logical tensors: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
    for name in sorted(reference_state):
        full = _assemble_logical_tensor(name=name, pieces=pieces[name], shard_rules=rules, target_shape=tuple(reference_state[name].shape))
        yield name, full.to(dtype=reference_state[name].dtype).cpu().contiguous()


# ------------------------------------------------------------------------------------------------ logical -> runtime
def _find_zero3_like_plugin(runtime: "RuntimeCore"):
    """The plugin that owns the model state as flat sharded buckets, if the runtime has one."""
    for plugin in runtime.plugins:
        if all(hasattr(plugin, attr) for attr in ("materialize_model", "reshard_model", "buckets")):
            return plugin
    return None


def _validate_supported_runtime_for_import(runtime: "RuntimeCore") -> None:
    # Runtimes already transformed for PP / EP are fine: the entries' metadata carries the runtime -> logical names.
    return


def _runtime_model_state_entries(runtime: "RuntimeCore") -> list[ModelStateMeta]:
    """Metadata of every model-state entry this rank would write into a runtime checkpoint."""
    sm = runtime.state_manager
    buffer_entries = [e.meta for e in sm.buffers.values()]
    zero3 = _find_zero3_like_plugin(runtime)
    if zero3 is None:
        return [e.meta for e in sm.params.values()] + buffer_entries
    rank = dist.get_rank() if dist.is_initialized() else 0
    buckets = [ModelStateMeta(state_key=f"{_ZERO3_PREFIX}{b.index}", logical_names=_bucket_names(zero3, b),
                              logical_shapes=[tuple(s) for s in b.param_shapes], physical_shape=tuple(b.local_param.shape),
                              dtype=str(b.local_param.dtype), source_rank=rank) for b in zero3.buckets]
    return buckets + buffer_entries


def _build_runtime_entry_tensor(*, runtime: "RuntimeCore", entry: ModelStateMeta, tensors: Mapping[str, torch.Tensor],
                                shard_rules: dict[str, str], tp_rank: int, tp_world_size: int) -> torch.Tensor:
    target = runtime.state_manager.get_model_tensor(entry.state_key)
    packed = len(entry.logical_names) > 1
    parts = []
    for name, shape in zip(entry.logical_names, entry.logical_shapes, strict=True):
        if name not in tensors:
            raise KeyError(f"logical checkpoint missing tensor={name}")
        local = _local_tensor_for_runtime_tensor(name=name, logical=tensors[name], shard_rules=shard_rules, tp_rank=tp_rank,
                                                 tp_world_size=tp_world_size)
        if not packed and tuple(local.shape) != tuple(target.shape):
            raise ValueError(f"logical tensor shape mismatch for {name}: expected local shape={tuple(target.shape)}, got={tuple(local.shape)}")
        if packed and local.numel() != int(math.prod(shape)):
            raise ValueError(f"logical tensor size mismatch for {name}: expected local numel={int(math.prod(shape))}, got={local.numel()}")
        parts.append(local.detach().cpu().contiguous())
    out = parts[0] if not packed else torch.cat([t.reshape(-1) for t in parts]).view(entry.physical_shape)
    if tuple(out.shape) != tuple(entry.physical_shape):
        raise ValueError(f"runtime checkpoint tensor shape mismatch for {entry.state_key}: expected={entry.physical_shape}, got={tuple(out.shape)}")
    return out.to(dtype=target.dtype).cpu().contiguous()


def _bucket_names(plugin, bucket) -> list[str]:
    """Checkpoint names of a flat bucket's tensors (logical names where a plugin renamed parameters, e.g. experts)."""
    mapper = getattr(plugin, "bucket_checkpoint_names", None)
    return list(mapper(bucket)) if mapper is not None else list(bucket.logical_names)


def _build_zero3_bucket_tensor(*, bucket, names: list[str], tensors: Mapping[str, torch.Tensor], shard_rules: dict[str, str], tp_rank: int,
                               tp_world_size: int, expected_shape: tuple[int, ...]) -> torch.Tensor:
    """This rank's slice of a flat ZeRO-3 bucket filled from logical tensors (padding stays zero)."""
    total = getattr(bucket, "buffer_size", None) or bucket.padded
    flat = torch.zeros(total, dtype=bucket.local_param.dtype, device="cpu")
    at = 0
    for name, n, shape in zip(names, bucket.param_numels, bucket.param_shapes, strict=True):
        if name not in tensors:
            raise KeyError(f"logical checkpoint missing tensor={name}")
        local = _local_tensor_for_runtime_tensor(name=name, logical=tensors[name], shard_rules=shard_rules, tp_rank=tp_rank,
                                                 tp_world_size=tp_world_size)
        if tuple(local.shape) != tuple(shape):
            raise ValueError(f"logical tensor shape mismatch for {name}: expected local shape={tuple(shape)}, got={tuple(local.shape)}")
        flat[at:at + n].copy_(local.to(dtype=flat.dtype).reshape(-1))
        at += n
    per_rank = int(math.prod(expected_shape))
    lo = bucket.group_context.rank * per_rank
    return flat[lo:lo + per_rank].view(expected_shape).contiguous()


def _build_runtime_model_state_from_logical_tensors(runtime: "RuntimeCore", tensors: Mapping[str, torch.Tensor]):
    """``(model_state, entries)`` of this rank for ``save_sharded_checkpoint_from_model_state``."""
    _validate_supported_runtime_for_import(runtime)
    rank = dist.get_rank() if dist.is_initialized() else 0
    entries = _runtime_model_state_entries(runtime)
    rules = _tp_shard_rules(runtime.model)
    tp_group = runtime.get_group(MeshAxis.TP)
    tp_rank = dist.get_rank(tp_group) if tp_group is not None else 0
    tp_world = dist.get_world_size(tp_group) if tp_group is not None else 1
    zero3 = _find_zero3_like_plugin(runtime)
    buckets = {f"{_ZERO3_PREFIX}{b.index}": b for b in getattr(zero3, "buckets", [])}
    state: dict[str, torch.Tensor] = {}
    for entry in entries:
        if entry.source_rank != rank:
            continue
        if _is_zero3_entry(entry):
            bucket = buckets.get(entry.state_key)
            if bucket is None:
                raise ValueError(f"zero3 runtime bucket metadata missing for state_key={entry.state_key}")
            state[entry.state_key] = _build_zero3_bucket_tensor(bucket=bucket, names=list(entry.logical_names), tensors=tensors, shard_rules=rules, tp_rank=tp_rank,
                                                                tp_world_size=tp_world, expected_shape=entry.physical_shape)
        else:
            state[entry.state_key] = _build_runtime_entry_tensor(runtime=runtime, entry=entry, tensors=tensors, shard_rules=rules,
                                                                 tp_rank=tp_rank, tp_world_size=tp_world)
    return state, entries

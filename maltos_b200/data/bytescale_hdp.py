"""ByteScale HDP: scheduling documents onto ranks in balanced waves, and building each rank's packed wave batches.

Planning is a pure function of the canonical global batch, so every rank computes the same global placement and keeps
only its own part (:class:`ByteScaleHdpLocalLayout`). Steps (reference ``data/bytescale_hdp.py:42-330``):

1. documents sorted by length (descending) are cut into consecutive buckets of about one rank-share of predicted cost;
2. per bucket, waves are filled greedily: among all unplaced documents that still fit, take the one that leaves the
   least free capacity on its chosen ranks (ties: larger local chunk, then bucket order);
3. a document of length L uses ``d = ceil(L / partition_tokens)`` ranks, chosen among the ranks with enough room as the
   ones whose predicted time lags the maximum by more than ``balance_delta`` (fastest first), topped up by the fastest
   others; it is padded to a multiple of ``2 d`` and split zigzag (rank ``i`` gets chunks ``i`` and ``2d-1-i``);
4. every chosen rank is charged ``(alpha L^2 + beta L) / d + gamma``.

A rank without documents in a wave still gets a 1-token dummy batch so that collective-bearing module hooks (ZeRO, DDP)
fire the same number of times everywhere.
"""
from __future__ import annotations

from dataclasses import dataclass
from fractions import Fraction
from typing import Any, Sequence

import torch

from maltos_b200.parallel.hdp_helper import (BYTESCALE_HDP_SCHEDULE_KEY, BYTESCALE_HDP_WAVES_KEY, ByteScaleHdpBalancedConfig,
                                             ByteScaleHdpLocalDocument, ByteScaleHdpLocalLayout, DocumentIndices)
from maltos_b200.utils.constants import (IGNORE_INDEX, INPUT_IDS_KEY, LABELS_KEY, LOSS_WEIGHT_KEY, PAD_SEQUENCE_ID, POSITION_IDS_KEY,
                                         SEQUENCE_IDS_KEY)

SCHEDULER_NAME = "bytescale_dp_balance_reproduction"


@dataclass(frozen=True)
class _Placement:
    document_id: int
    source: DocumentIndices
    sequence_length: int
    padded_length: int
    participant_ranks: tuple[int, ...]

    @property
    def local_length(self) -> int:
        return self.padded_length // len(self.participant_ranks)


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


def _zigzag_positions(padded_length: int, degree: int, local_rank: int) -> tuple[int, ...]:
    chunk = padded_length // (2 * degree)
    mirror = 2 * degree - 1 - local_rank
    return tuple(range(local_rank * chunk, (local_rank + 1) * chunk)) + tuple(range(mirror * chunk, (mirror + 1) * chunk))


def _best_fit_row(remaining: Sequence[int], length: int, capacity: int) -> tuple[int, int]:
    """(row, start column) of the fullest row that still takes ``length`` tokens; a new row when none does."""
    fits = [(space, row) for row, space in enumerate(remaining) if space >= length]
    if not fits:
        return len(remaining), 0
    space, row = min(fits)
    return row, capacity - space


def _bucket_by_profiled_cost(ordered: Sequence[tuple[int, DocumentIndices]], world_size: int, *,
                             config: ByteScaleHdpBalancedConfig) -> tuple[tuple[tuple[int, DocumentIndices], ...], ...]:
    """Consecutive buckets of at most one rank-share of the total predicted cost (a document is never split; one that
    exceeds the share is a bucket of its own)."""
    costs = [config.cost_model.sequence_cost(len(src.source_indices)) for _, src in ordered]
    target = max(Fraction(1), sum(costs, start=Fraction(0)) / world_size)
    buckets: list[list[tuple[int, DocumentIndices]]] = []
    filled = Fraction(0)
    for item, cost in zip(ordered, costs):
        if not buckets or (buckets[-1] and filled + cost > target):
            buckets.append([])
            filled = Fraction(0)
        buckets[-1].append(item)
        filled += cost
    return tuple(tuple(b) for b in buckets)


def _select_algorithm_2_workers(predicted_times: Sequence[Fraction], *, worker_count: int, balance_delta: float,
                                eligible_ranks: Sequence[int]) -> tuple[int, ...] | None:
    """``worker_count`` ranks for one document, or None when fewer ranks have room."""
    eligible = set(eligible_ranks)
    if len(eligible) < worker_count:
        return None
    by_time = lambda r: (predicted_times[r], r)   # noqa: E731
    slowest = max(predicted_times, default=Fraction(0))
    delta = Fraction(str(balance_delta))
    targets = sorted((r for r in eligible if slowest - predicted_times[r] > delta), key=by_time)
    chosen = targets if targets else sorted(eligible, key=by_time)
    if len(chosen) < worker_count:
        chosen = chosen + sorted((r for r in eligible if r not in set(targets)), key=by_time)
    return tuple(sorted(chosen[:worker_count]))


def _select_best_fit_document(remaining: Sequence[tuple[int, DocumentIndices]], *, remaining_capacity: Sequence[int],
                              predicted_times: Sequence[Fraction], world_size: int,
                              config: ByteScaleHdpBalancedConfig) -> tuple[int, _Placement] | None:
    """Scan every unplaced document of the bucket; the tightest fit wins."""
    best_key, best = None, None
    for idx, (doc_id, src) in enumerate(remaining):
        length = len(src.source_indices)
        degree = config.participant_count(length, world_size=world_size)
        padded = _round_up(length, 2 * degree)
        local = padded // degree
        ranks = _select_algorithm_2_workers(predicted_times, worker_count=degree, balance_delta=config.balance_delta,
                                            eligible_ranks=[r for r, cap in enumerate(remaining_capacity) if cap >= local])
        if ranks is None:
            continue
        key = (sum(remaining_capacity[r] - local for r in ranks), -local, idx)
        if best_key is None or key < best_key:
            best_key, best = key, (idx, _Placement(doc_id, src, length, padded, ranks))
    return best


def _plan_waves(indices: Sequence[DocumentIndices], world_size: int, config: ByteScaleHdpBalancedConfig) -> list[tuple[_Placement, ...]]:
    """The global plan: one tuple of placements per wave, identical on every rank."""
    times = [Fraction(0)] * world_size
    ordered = sorted(enumerate(indices), key=lambda item: (-len(item[1].source_indices), item[0]))
    waves: list[tuple[_Placement, ...]] = []
    for bucket in _bucket_by_profiled_cost(ordered, world_size, config=config):
        todo = list(bucket)
        while todo:
            room = [config.partition_tokens] * world_size
            wave: list[_Placement] = []
            while todo:
                pick = _select_best_fit_document(todo, remaining_capacity=room, predicted_times=times, world_size=world_size,
                                                 config=config)
                if pick is None:
                    break
                idx, placement = pick
                todo.pop(idx)
                wave.append(placement)
                share = config.cost_model.participant_cost(placement.sequence_length, len(placement.participant_ranks))
                for r in placement.participant_ranks:
                    room[r] -= placement.local_length
                    times[r] = times[r] + share
            if not wave:
                raise AssertionError("validated document could not fit an empty HDP wave")
            waves.append(tuple(wave))
    return waves


def _local_layout_for_wave(placements: Sequence[_Placement], *, rank: int, world_size: int, config: ByteScaleHdpBalancedConfig,
                           global_valid_targets: int, global_document_count: int, wave_index: int,
                           wave_count: int) -> ByteScaleHdpLocalLayout:
    rows_free: list[int] = []
    mine: list[ByteScaleHdpLocalDocument] = []
    for pl in placements:
        if rank not in pl.participant_ranks:
            continue
        ring = pl.participant_ranks
        me = ring.index(rank)
        row, start = _best_fit_row(rows_free, pl.local_length, config.partition_tokens)
        if row == len(rows_free):
            rows_free.append(config.partition_tokens)
        rows_free[row] -= pl.local_length
        positions = _zigzag_positions(pl.padded_length, len(ring), me)
        real = [p < pl.sequence_length for p in positions]
        mine.append(ByteScaleHdpLocalDocument(
            document_id=pl.document_id, source_row=pl.source.source_row, sequence_length=pl.sequence_length,
            padded_length=pl.padded_length, participant_ranks=ring,
            prev_rank=ring[(me - 1) % len(ring)] if len(ring) > 1 else None,
            next_rank=ring[(me + 1) % len(ring)] if len(ring) > 1 else None,
            local_row=row, local_start=start, local_end=start + pl.local_length,
            source_indices=tuple(pl.source.source_indices[p] if ok else None for p, ok in zip(positions, real)),
            document_positions=tuple(p if ok else None for p, ok in zip(positions, real))))
    if mine and len(rows_free) != 1:
        raise AssertionError("HDP wave packing exceeded its resident-token capacity")
    return ByteScaleHdpLocalLayout(rank=rank, hdp_world_size=world_size, partition_tokens=config.partition_tokens,
                                   scheduler_name=SCHEDULER_NAME, documents=tuple(mine), packed_rows=len(rows_free),
                                   packed_width=config.partition_tokens, global_valid_targets=global_valid_targets,
                                   global_document_count=global_document_count, wave_index=wave_index, wave_count=wave_count)


def schedule_document_waves(indices: Sequence[DocumentIndices], *, rank: int, world_size: int, config: ByteScaleHdpBalancedConfig,
                            global_valid_targets: int) -> tuple[ByteScaleHdpLocalLayout, ...]:
    """This rank's layouts of all waves of one global batch, in execution order."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank={rank} outside world_size={world_size}")
    waves = _plan_waves(indices, world_size, config)
    return tuple(_local_layout_for_wave(w, rank=rank, world_size=world_size, config=config, global_valid_targets=global_valid_targets,
                                        global_document_count=len(indices), wave_index=i, wave_count=len(waves))
                 for i, w in enumerate(waves))


def schedule_documents(indices: Sequence[DocumentIndices], *, rank: int, world_size: int, config: ByteScaleHdpBalancedConfig,
                       global_valid_targets: int) -> ByteScaleHdpLocalLayout:
    """The single wave of a batch that needs only one; multi-wave schedules must go through the loader envelope."""
    layouts = schedule_document_waves(indices, rank=rank, world_size=world_size, config=config, global_valid_targets=global_valid_targets)
    if len(layouts) != 1:
        raise ValueError("ByteScale schedule contains multiple waves; use the HDP dataloader envelope instead of schedule_documents()")
    return layouts[0]


# ------------------------------------------------------------------------------------------------ materialisation
def _dummy_batch(source_batch: dict[str, torch.Tensor], layout: ByteScaleHdpLocalLayout) -> dict[str, Any]:
    ids = source_batch[INPUT_IDS_KEY]
    one = lambda fill, dtype: torch.full((1, 1), fill, dtype=dtype, device=ids.device)   # noqa: E731
    return {INPUT_IDS_KEY: one(0, ids.dtype), LABELS_KEY: one(IGNORE_INDEX, torch.long), POSITION_IDS_KEY: one(0, torch.long),
            SEQUENCE_IDS_KEY: one(PAD_SEQUENCE_ID, torch.long), LOSS_WEIGHT_KEY: 0.0, BYTESCALE_HDP_SCHEDULE_KEY: layout}


def _materialize_bytescale_local_wave(batch: dict[str, torch.Tensor], layout: ByteScaleHdpLocalLayout, *, world_size: int) -> dict[str, Any]:
    if not layout.documents:
        return _dummy_batch(batch, layout)
    ids, labels, positions = batch[INPUT_IDS_KEY], batch.get(LABELS_KEY), batch.get(POSITION_IDS_KEY)
    shape, dev = (layout.packed_rows, layout.packed_width), ids.device
    out: dict[str, Any] = {INPUT_IDS_KEY: torch.zeros(shape, dtype=ids.dtype, device=dev),
                           LABELS_KEY: torch.full(shape, IGNORE_INDEX, dtype=torch.long, device=dev),
                           POSITION_IDS_KEY: torch.zeros(shape, dtype=torch.long, device=dev),
                           SEQUENCE_IDS_KEY: torch.full(shape, PAD_SEQUENCE_ID, dtype=torch.long, device=dev)}
    for doc in layout.documents:
        keep = [i for i, s in enumerate(doc.source_indices) if s is not None]
        if not keep:
            continue
        cols = torch.tensor([doc.local_start + i for i in keep], dtype=torch.long, device=dev)
        src = torch.tensor([doc.source_indices[i] for i in keep], dtype=torch.long, device=dev)
        out[INPUT_IDS_KEY][doc.local_row, cols] = ids[doc.source_row, src]
        if torch.is_tensor(labels):
            out[LABELS_KEY][doc.local_row, cols] = labels[doc.source_row, src].to(torch.long)
        if torch.is_tensor(positions):
            out[POSITION_IDS_KEY][doc.local_row, cols] = positions[doc.source_row, src].to(torch.long)
        else:
            out[POSITION_IDS_KEY][doc.local_row, cols] = torch.tensor([doc.document_positions[i] for i in keep], dtype=torch.long, device=dev)
        out[SEQUENCE_IDS_KEY][doc.local_row, cols] = doc.document_id
    local_targets = int((out[LABELS_KEY] != IGNORE_INDEX).sum().item())
    # the model averages over LOCAL targets; this weight turns the sum over ranks and waves into the global mean
    out[LOSS_WEIGHT_KEY] = world_size * local_targets / layout.global_valid_targets if layout.global_valid_targets else 0.0
    out[BYTESCALE_HDP_SCHEDULE_KEY] = layout
    return out


def build_bytescale_local_batches(batch: dict[str, torch.Tensor], *, rank: int, world_size: int,
                                  config: ByteScaleHdpBalancedConfig):
    """``(wave batches, wave layouts)`` of rank ``rank`` for one canonical global batch."""
    indices = DocumentIndices.from_batch(batch)
    labels = batch.get(LABELS_KEY)
    targets = int((labels != IGNORE_INDEX).sum().item()) if torch.is_tensor(labels) else 0
    layouts = schedule_document_waves(indices, rank=rank, world_size=world_size, config=config, global_valid_targets=targets)
    return tuple(_materialize_bytescale_local_wave(batch, lay, world_size=world_size) for lay in layouts), layouts


def build_bytescale_local_batch(batch: dict[str, torch.Tensor], *, rank: int, world_size: int, config: ByteScaleHdpBalancedConfig):
    waves, layouts = build_bytescale_local_batches(batch, rank=rank, world_size=world_size, config=config)
    if len(waves) != 1:
        raise ValueError("ByteScale schedule contains multiple waves; use build_bytescale_local_batches() or ByteScaleHdpDataLoader")
    return waves[0], layouts[0]


class ByteScaleHdpDataLoader:
    """Wraps a loader of canonical GLOBAL batches (same batch on every HDP rank) and yields this rank's wave envelope
    ``{BYTESCALE_HDP_WAVES_KEY: (wave batch, ...)}``. Checkpoint state is the wrapped loader's."""

    def __init__(self, loader: Any, *, hdp_rank: int, hdp_world_size: int, config: ByteScaleHdpBalancedConfig) -> None:
        self.loader, self.hdp_rank, self.hdp_world_size, self.config = loader, hdp_rank, hdp_world_size, config

    @property
    def consumed_tokens(self):
        return self.loader.consumed_tokens

    def next_batch(self, cp_rank: int | None = None):
        if cp_rank is not None:
            raise ValueError("ByteScale HDP is on DP; cp_rank must be None")
        waves, _ = build_bytescale_local_batches(self.loader.next_batch(None), rank=self.hdp_rank, world_size=self.hdp_world_size,
                                                 config=self.config)
        return {BYTESCALE_HDP_WAVES_KEY: waves}

    def state_dict(self):
        return self.loader.state_dict()

    def load_state_dict(self, state):
        return self.loader.load_state_dict(state)

    def close(self) -> None:
        close = getattr(self.loader, "close", None)
        if close is not None:
            close()

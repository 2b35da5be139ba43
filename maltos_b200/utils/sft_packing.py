"""Packing tokenised SFT examples into fixed-length rows and writing them as binary shards.

Every output row has ``seq_len`` tokens and four aligned fields: ``input_ids`` (uint32), ``labels`` (int32, next-token
targets, ``IGNORE_INDEX`` where the next token is not supervised, at an example's last token and on padding),
``position_ids`` (int32, restarting at 0 for each example) and ``sequence_ids`` (int32, index of the example inside its
row, ``PAD_SEQUENCE_ID`` on padding). Examples never straddle rows: longer ones are cut into ``seq_len`` pieces first.
Two placement strategies: ``next_fit`` (streaming, one open row) and ``best_fit_decreasing`` over a bounded window of
pending pieces. A shard file stores the four ``[rows, seq_len]`` arrays back to back; the metadata written by
:func:`export_packing_metadata` records dtype, byte offset and shape of each so the loader can memory-map them.
File format and statistics follow the reference's ``utils/sft_packing.py:1-433``.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import numpy as np

from maltos_b200.utils.constants import IGNORE_INDEX, INPUT_IDS_KEY, LABELS_KEY, PAD_SEQUENCE_ID, POSITION_IDS_KEY, SEQUENCE_IDS_KEY
from maltos_b200.utils.sft_messages import EncodedSFTExample

INPUT_DTYPE = np.uint32
LABEL_DTYPE = np.int32
POSITION_DTYPE = np.int32
SEQUENCE_DTYPE = np.int32

PACKING_ALGORITHMS = {"next_fit", "best_fit_decreasing"}
_FIELD_ORDER = ((INPUT_IDS_KEY, INPUT_DTYPE), (LABELS_KEY, LABEL_DTYPE), (POSITION_IDS_KEY, POSITION_DTYPE), (SEQUENCE_IDS_KEY, SEQUENCE_DTYPE))


@dataclass(frozen=True)
class PackedSFTField:
    dtype: str
    offset: int
    shape: tuple[int, int]

    def to_metadata(self) -> dict[str, object]:
        return {"dtype": self.dtype, "offset": self.offset, "shape": list(self.shape)}


@dataclass(frozen=True)
class PackedSFTShard:
    shard_idx: int
    path: str
    sequences: int
    input_field: PackedSFTField
    label_field: PackedSFTField
    position_field: PackedSFTField
    sequence_field: PackedSFTField

    def to_metadata(self) -> dict[str, object]:
        fields = {INPUT_IDS_KEY: self.input_field, LABELS_KEY: self.label_field, POSITION_IDS_KEY: self.position_field,
                  SEQUENCE_IDS_KEY: self.sequence_field}
        return {"shard_idx": self.shard_idx, "path": self.path, "sequences": self.sequences,
                "fields": {k: f.to_metadata() for k, f in fields.items()}}


@dataclass(frozen=True)
class PackedSFTSummary:
    raw_tokens: int
    raw_supervised_tokens: int
    packed_sequences: int
    packed_input_tokens: int
    packed_supervised_tokens: int
    padded_tokens: int
    dropped_tail_tokens: int
    shards: list[PackedSFTShard]

    def stats_metadata(self) -> dict[str, object]:
        return {"raw_tokens": self.raw_tokens, "raw_supervised_tokens": self.raw_supervised_tokens,
                "packed_sequences": self.packed_sequences, "packed_input_tokens": self.packed_input_tokens,
                "packed_supervised_tokens": self.packed_supervised_tokens, "padded_tokens": self.padded_tokens,
                "dropped_tail_tokens": self.dropped_tail_tokens, "num_shards": len(self.shards)}


# ------------------------------------------------------------------------------------------------ pure helpers
def resolve_pad_token_id(tokenizer) -> int:
    for candidate in (tokenizer.pad_token_id, tokenizer.eos_token_id):
        if candidate is not None:
            return int(candidate)
    raise ValueError("tokenizer must define pad_token_id or eos_token_id for packed SFT output")


def split_example_to_seq_len(example: EncodedSFTExample, *, seq_len: int) -> list[EncodedSFTExample]:
    n = len(example.token_ids)
    if n <= seq_len:
        return [example]
    return [EncodedSFTExample(list(example.token_ids[a:a + seq_len]), list(example.supervised_mask[a:a + seq_len]))
            for a in range(0, n, seq_len)]


def pack_segments_best_fit_decreasing(segments: list[EncodedSFTExample], *, seq_len: int) -> list[list[EncodedSFTExample]]:
    """Longest piece first (ties in arrival order); each goes to the open bin it fills most tightly, else a new bin."""
    order = sorted(range(len(segments)), key=lambda i: (-len(segments[i].token_ids), i))
    bins: list[list[EncodedSFTExample]] = []
    free: list[int] = []
    for i in order:
        need = len(segments[i].token_ids)
        fits = [(room - need, b) for b, room in enumerate(free) if room >= need]
        if fits:
            _, b = min(fits)
            bins[b].append(segments[i])
            free[b] -= need
        else:
            bins.append([segments[i]])
            free.append(seq_len - need)
    return bins


def _segment_columns(segment: EncodedSFTExample, sequence_id: int):
    """(input_ids, labels, position_ids, sequence_ids) of one piece as numpy vectors, and its supervised-label count."""
    ids = np.asarray(segment.token_ids, dtype=np.int64)
    sup = np.asarray(segment.supervised_mask, dtype=bool)
    labels = np.full(ids.shape, IGNORE_INDEX, dtype=np.int64)
    if ids.size > 1:
        nxt = sup[1:]
        labels[:-1][nxt] = ids[1:][nxt]
    return ids, labels, np.arange(ids.size, dtype=np.int64), np.full(ids.shape, sequence_id, dtype=np.int64), int(sup[1:].sum())


def _tokens_in(segments) -> int:
    return sum(len(s.token_ids) for s in segments)


class PackedSFTWriter:
    """Collects examples with :meth:`add_example`, writes shards as rows fill up, :meth:`finish` returns the summary."""

    def __init__(self, *, output_dir: Path, seq_len: int, sequences_per_shard: int, max_sequences: int | None, pad_token_id: int,
                 packing_algorithm: str = "best_fit_decreasing", packing_buffer_size: int = 4096) -> None:
        if packing_algorithm not in PACKING_ALGORITHMS:
            raise ValueError(f"unsupported packing_algorithm={packing_algorithm!r}; expected one of {sorted(PACKING_ALGORITHMS)}")
        if packing_buffer_size < 1:
            raise ValueError(f"packing_buffer_size must be >= 1, got {packing_buffer_size}")
        self.output_dir = Path(output_dir)
        self.seq_len = seq_len
        self.sequences_per_shard = sequences_per_shard
        self.max_sequences = max_sequences
        self.pad_token_id = pad_token_id
        self.packing_algorithm = packing_algorithm
        self.packing_buffer_size = packing_buffer_size

        self._open_row: list[EncodedSFTExample] = []      # next_fit: pieces of the row being filled
        self._window: list[EncodedSFTExample] = []        # best_fit_decreasing: pieces waiting for the next bin packing
        self._rows: list[np.ndarray] = []                 # finished rows of the current shard, each [4, seq_len] int64
        self.shards: list[PackedSFTShard] = []
        self.raw_tokens = self.raw_supervised_tokens = 0
        self.packed_sequences = self.packed_supervised_tokens = 0
        self.padded_tokens = self.dropped_tail_tokens = 0
        self.reached_sequence_limit = False

    # ------------------------------------------------------------------ public
    def add_example(self, example: EncodedSFTExample) -> None:
        if self.reached_sequence_limit:
            return
        if len(example.token_ids) != len(example.supervised_mask):
            raise ValueError("token_ids and supervised_mask must have the same length")
        if len(example.token_ids) < 2:
            return
        self.raw_tokens += len(example.token_ids)
        self.raw_supervised_tokens += sum(int(f) for f in example.supervised_mask)
        for piece in split_example_to_seq_len(example, seq_len=self.seq_len):
            if self.reached_sequence_limit:
                return
            if self.packing_algorithm == "next_fit":
                self._place_next_fit(piece)
            else:
                self._window.append(piece)
                if len(self._window) >= self.packing_buffer_size:
                    self._pack_window()

    def finish(self) -> PackedSFTSummary:
        if self.packing_algorithm == "next_fit":
            if self._open_row:
                if self._has_budget():
                    self._emit_row(self._open_row)
                else:
                    self.dropped_tail_tokens += _tokens_in(self._open_row)
                self._open_row = []
        else:
            self._pack_window()
        self._write_shard()
        return PackedSFTSummary(raw_tokens=self.raw_tokens, raw_supervised_tokens=self.raw_supervised_tokens,
                                packed_sequences=self.packed_sequences, packed_input_tokens=self.packed_sequences * self.seq_len,
                                packed_supervised_tokens=self.packed_supervised_tokens, padded_tokens=self.padded_tokens,
                                dropped_tail_tokens=self.dropped_tail_tokens, shards=list(self.shards))

    # ------------------------------------------------------------------ placement
    def _has_budget(self) -> bool:
        return self.max_sequences is None or self.packed_sequences < self.max_sequences

    def _place_next_fit(self, piece: EncodedSFTExample) -> None:
        if len(piece.token_ids) > self.seq_len:
            raise ValueError(f"segment length exceeds seq_len: {len(piece.token_ids)} > {self.seq_len}")
        if self._open_row and _tokens_in(self._open_row) + len(piece.token_ids) > self.seq_len:
            self._close_open_row()
        if not self._has_budget():
            self.reached_sequence_limit = True
            self.dropped_tail_tokens += len(piece.token_ids)
            return
        self._open_row.append(piece)
        if _tokens_in(self._open_row) == self.seq_len:
            self._close_open_row()

    def _close_open_row(self) -> None:
        if not self._open_row:
            return
        if not self._has_budget():
            # the row stays open (and is counted as dropped by finish) once the sequence budget is used up
            self.reached_sequence_limit = True
            self.dropped_tail_tokens += _tokens_in(self._open_row)
            return
        self._emit_row(self._open_row)
        self._open_row = []

    def _pack_window(self) -> None:
        if not self._window:
            return
        bins = pack_segments_best_fit_decreasing(self._window, seq_len=self.seq_len)
        self._window = []
        for b, pieces in enumerate(bins):
            if not self._has_budget():
                self.reached_sequence_limit = True
                self.dropped_tail_tokens += sum(_tokens_in(rest) for rest in bins[b:])
                return
            self._emit_row(pieces)

    # ------------------------------------------------------------------ output
    def _emit_row(self, pieces: list[EncodedSFTExample]) -> None:
        row = np.empty((4, self.seq_len), dtype=np.int64)
        row[0], row[1], row[2], row[3] = self.pad_token_id, IGNORE_INDEX, 0, PAD_SEQUENCE_ID
        at = 0
        for sid, piece in enumerate(pieces):
            ids, labels, pos, seq, n_sup = _segment_columns(piece, sid)
            if at + ids.size > self.seq_len:
                raise ValueError(f"packed sequence length exceeds seq_len: {at + ids.size} > {self.seq_len}")
            row[0, at:at + ids.size], row[1, at:at + ids.size] = ids, labels
            row[2, at:at + ids.size], row[3, at:at + ids.size] = pos, seq
            self.packed_supervised_tokens += n_sup
            at += ids.size
        self.padded_tokens += self.seq_len - at
        self._rows.append(row)
        self.packed_sequences += 1
        if len(self._rows) >= self.sequences_per_shard:
            self._write_shard()

    def _write_shard(self) -> None:
        if not self._rows:
            return
        stack = np.stack(self._rows)   # [rows, 4, seq_len]
        idx = len(self.shards)
        path = self.output_dir / f"shard_{idx:05d}.bin"
        fields, offset = [], 0
        with path.open("wb") as f:
            for col, (_, dtype) in enumerate(_FIELD_ORDER):
                arr = np.ascontiguousarray(stack[:, col, :]).astype(dtype)
                arr.tofile(f)
                fields.append(PackedSFTField(np.dtype(dtype).name, offset, (int(arr.shape[0]), int(arr.shape[1]))))
                offset += int(arr.nbytes)
        self.shards.append(PackedSFTShard(idx, path.name, int(stack.shape[0]), *fields))
        print(f"wrote shard={idx:05d} sequences={stack.shape[0]:,} path={path.name}")
        self._rows = []


def export_packing_metadata(*, summary: PackedSFTSummary, seq_len: int, sequences_per_shard: int, packing_algorithm: str,
                            packing_buffer_size: int) -> dict[str, object]:
    field_layout = {key: {"dtype": np.dtype(dtype).name} for key, dtype in _FIELD_ORDER}
    field_layout[LABELS_KEY]["ignore_index"] = IGNORE_INDEX
    field_layout[SEQUENCE_IDS_KEY]["pad_sequence_id"] = PAD_SEQUENCE_ID
    name = "example_aware_windowed_best_fit_decreasing" if packing_algorithm == "best_fit_decreasing" else "example_aware_next_fit"
    return {
        "layout": {"seq_len": seq_len, "row_length": seq_len, "record_stride": seq_len, "fields": field_layout},
        "strategy": {"algorithm": packing_algorithm, "buffer_size": packing_buffer_size, "name": name,
                     "sequences_per_shard": sequences_per_shard},
        "stats": summary.stats_metadata(),
        "shards": [s.to_metadata() for s in summary.shards],
    }

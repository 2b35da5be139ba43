"""SFT message encoding, packing and the shard-preparation tool, read back through the SFT dataset reader."""
import json
from types import SimpleNamespace

import numpy as np
import pytest

from maltos_b200.data.sft import PackedSFTDataset
from maltos_b200.tools import prepare_sft_shards
from maltos_b200.utils.constants import IGNORE_INDEX, PAD_SEQUENCE_ID
from maltos_b200.utils.sft_messages import EncodedSFTExample, encode_sft_example, extract_messages, normalize_message_content
from maltos_b200.utils.sft_packing import PackedSFTWriter, pack_segments_best_fit_decreasing, split_example_to_seq_len


class CharTokenizer:
    """One token per character (code point + 3); ids 0/1/2 are pad/eos/unused."""

    pad_token_id = 0
    eos_token_id = 1
    chat_template = None

    def encode(self, text, add_special_tokens=False):
        return [ord(c) + 3 for c in text]

    def __len__(self):
        return 260


def _ex(n, sup_from=0, base=10):
    return EncodedSFTExample(list(range(base, base + n)), [0] * sup_from + [1] * (n - sup_from))


def test_message_extraction_and_plain_encoding():
    row = {"messages": json.dumps([{"role": "user", "content": [{"type": "text", "text": "hi"}, "!"]},
                                   {"role": "assistant", "content": {"text": "yo"}}, {"role": "user", "content": ""}])}
    msgs = extract_messages(row, "messages")
    assert msgs == [{"role": "user", "content": "hi!"}, {"role": "assistant", "content": "yo"}]
    with pytest.raises(ValueError):
        normalize_message_content([{"type": "image", "url": "x"}])
    enc = encode_sft_example(row, tokenizer=CharTokenizer(), messages_column="messages", prompt_column="prompt",
                             completion_column="completion", apply_chat_template=False, assistant_only_loss=True, append_eos=True)
    text_len = len("user: hi!") + 1 + len("assistant: yo") + 1
    assert len(enc.token_ids) == text_len == len(enc.supervised_mask)
    assert sum(enc.supervised_mask) == len("yo") + 1          # assistant content + its eos
    assert enc.supervised_mask[-3:] == [1, 1, 1] and enc.supervised_mask[-4] == 0
    none = encode_sft_example({"prompt": "q", "completion": ""}, tokenizer=CharTokenizer(), messages_column="messages",
                              prompt_column="prompt", completion_column="completion", apply_chat_template=False,
                              assistant_only_loss=True, append_eos=True)
    assert none is None
    with pytest.raises(ValueError):
        encode_sft_example({"prompt": "q", "completion": "a"}, tokenizer=CharTokenizer(), messages_column="messages",
                           prompt_column="prompt", completion_column="completion", apply_chat_template=True,
                           assistant_only_loss=True, append_eos=True)


def test_split_and_best_fit_decreasing():
    parts = split_example_to_seq_len(_ex(10), seq_len=4)
    assert [len(p.token_ids) for p in parts] == [4, 4, 2]
    bins = pack_segments_best_fit_decreasing([_ex(5), _ex(3), _ex(7), _ex(2), _ex(1)], seq_len=8)
    assert sorted(sorted(len(s.token_ids) for s in b) for b in bins) == [[1, 7], [2], [3, 5]]
    assert all(sum(len(s.token_ids) for s in b) <= 8 for b in bins)


@pytest.mark.parametrize("algorithm", ["next_fit", "best_fit_decreasing"])
def test_writer_rows_and_reader_roundtrip(tmp_path, algorithm):
    w = PackedSFTWriter(output_dir=tmp_path, seq_len=8, sequences_per_shard=2, max_sequences=None, pad_token_id=0,
                        packing_algorithm=algorithm, packing_buffer_size=3)
    examples = [_ex(5, 2, 100), _ex(3, 1, 200), _ex(1), _ex(11, 0, 300), _ex(4, 4, 400)]
    for e in examples:
        w.add_example(e)
    summary = w.finish()
    assert summary.raw_tokens == 5 + 3 + 11 + 4                      # the 1-token example is ignored
    assert summary.packed_input_tokens == summary.packed_sequences * 8
    assert summary.packed_input_tokens - summary.padded_tokens == summary.raw_tokens
    assert sum(s.sequences for s in summary.shards) == summary.packed_sequences
    from maltos_b200.utils.sft_packing import export_packing_metadata

    meta = {"format": "maltos_sft_packed", "format_version": 2,
            "packing": export_packing_metadata(summary=summary, seq_len=8, sequences_per_shard=2, packing_algorithm=algorithm,
                                               packing_buffer_size=3)}
    (tmp_path / "meta.json").write_text(json.dumps(meta))
    ds = PackedSFTDataset(tmp_path)
    rows, _, _ = ds.read_rows(0, 0, len(ds))
    ids, labels, pos, seq = (rows[k] for k in ("input_ids", "labels", "position_ids", "sequence_ids"))
    n_sup = 0
    for r in range(len(ds)):
        for c in range(8):
            if seq[r, c] == PAD_SEQUENCE_ID:
                assert labels[r, c] == IGNORE_INDEX and ids[r, c] == 0 and pos[r, c] == 0
                continue
            same_next = c + 1 < 8 and seq[r, c + 1] == seq[r, c]
            assert pos[r, c] == (pos[r, c - 1] + 1 if c and seq[r, c - 1] == seq[r, c] else 0)
            if labels[r, c] != IGNORE_INDEX:
                assert same_next and labels[r, c] == ids[r, c + 1]
                n_sup += 1
    assert n_sup == summary.packed_supervised_tokens
    # supervised targets: every supervised token that is not the first of its piece
    assert 0 < n_sup <= summary.raw_supervised_tokens


def test_sequence_budget_is_respected(tmp_path):
    w = PackedSFTWriter(output_dir=tmp_path, seq_len=4, sequences_per_shard=8, max_sequences=2, pad_token_id=0,
                        packing_algorithm="next_fit")
    for _ in range(5):
        w.add_example(_ex(4))
    s = w.finish()
    assert s.packed_sequences == 2 and w.reached_sequence_limit and s.dropped_tail_tokens >= 4


def test_prepare_tool_end_to_end(tmp_path):
    src = tmp_path / "rows.jsonl"
    with src.open("w") as f:
        for i in range(20):
            f.write(json.dumps({"prompt": f"question {i}", "completion": "answer " * (1 + i % 3)}) + "\n")
    out = tmp_path / "packed"
    args = prepare_sft_shards.parse_args(["--dataset", str(src), "--tokenizer-name-or-path", "char", "--output-dir", str(out),
                                          "--seq-len", "64", "--sequences-per-shard", "4", "--no-apply-chat-template"])
    from maltos_b200.tools._prep_common import _read_local_file

    summary = prepare_sft_shards.run(args, CharTokenizer(), _read_local_file(src))
    meta = json.loads((out / "meta.json").read_text())
    assert meta["format"] == "maltos_sft_packed" and meta["format_version"] == 2
    assert meta["source"]["stats"] == {"examples_seen": 20, "examples_encoded": 20, "examples_skipped": 0}
    assert meta["packing"]["stats"]["packed_sequences"] == summary.packed_sequences == len(PackedSFTDataset(out))
    assert meta["packing"]["strategy"]["name"] == "example_aware_windowed_best_fit_decreasing"

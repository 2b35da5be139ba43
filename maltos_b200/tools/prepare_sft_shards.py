"""Prepare packed fixed-length SFT shards (``shard_00000.bin`` ... plus ``meta.json``) for ``SFTDataLoader``.

Rows (chat transcripts or prompt/completion pairs) are tokenised with :mod:`maltos_b200.utils.sft_messages`, packed with
:mod:`maltos_b200.utils.sft_packing` and described by a ``maltos_sft_packed`` version-2 metadata file. Command line and
metadata schema follow the reference's ``tools/prepare_sft_shards.py:18-71,220-268``.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

from maltos_b200.tools._prep_common import Progress, format_duration, load_tokenizer, open_rows
from maltos_b200.utils.sft_messages import encode_sft_example
from maltos_b200.utils.sft_packing import PACKING_ALGORITHMS, PackedSFTSummary, PackedSFTWriter, export_packing_metadata, resolve_pad_token_id


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Prepare fixed-length SFT input/label shards for the SFT dataloader.")
    p.add_argument("--dataset", type=str, required=True, help="HF dataset id, local dataset path, or json/jsonl/parquet/csv file")
    p.add_argument("--config", type=str, default=None, help="Optional HF dataset config")
    p.add_argument("--split", type=str, default="train")
    p.add_argument("--messages-column", type=str, default="messages")
    p.add_argument("--prompt-column", type=str, default="prompt")
    p.add_argument("--completion-column", type=str, default="completion")
    p.add_argument("--tokenizer-name-or-path", type=str, required=True)
    p.add_argument("--chat-template-file", type=str, default=None,
                   help="Optional local Jinja chat template file to override tokenizer.chat_template")
    p.add_argument("--output-dir", type=str, required=True)
    p.add_argument("--seq-len", type=int, required=True, help="Packed training sequence length")
    p.add_argument("--sequences-per-shard", type=int, default=8192)
    p.add_argument("--max-examples", type=int, default=None)
    p.add_argument("--max-sequences", type=int, default=None)
    p.add_argument("--expected-vocab-size", type=int, default=None)
    p.add_argument("--packing-algorithm", type=str, default="best_fit_decreasing", choices=sorted(PACKING_ALGORITHMS),
                   help="Sequence packing algorithm. best_fit_decreasing is a bounded-window offline bin packer.")
    p.add_argument("--packing-buffer-size", type=int, default=4096,
                   help="Number of segmented examples to buffer before running best_fit_decreasing.")
    p.add_argument("--assistant-only-loss", action=argparse.BooleanOptionalAction, default=True)
    p.add_argument("--apply-chat-template", action=argparse.BooleanOptionalAction, default=True,
                   help="Render message/prompt-completion rows through tokenizer chat template when available")
    p.add_argument("--append-eos", action=argparse.BooleanOptionalAction, default=True,
                   help="Append eos when using plain prompt/completion fallback")
    p.add_argument("--streaming", action="store_true")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--shuffle-buffer-size", type=int, default=10_000)
    p.add_argument("--log-every-examples", type=int, default=1_000)
    return p.parse_args(argv)


def _validate(args: argparse.Namespace) -> None:
    for name in ("seq_len", "sequences_per_shard", "packing_buffer_size", "log_every_examples"):
        if getattr(args, name) < 1:
            raise ValueError(f"{name} must be >= 1, got {getattr(args, name)}")
    for name in ("max_examples", "max_sequences"):
        value = getattr(args, name)
        if value is not None and value < 1:
            raise ValueError(f"{name} must be >= 1, got {value}")


def build_meta(args: argparse.Namespace, *, vocab_size: int, eos_token_id, counts: dict[str, int], summary: PackedSFTSummary) -> dict:
    return {
        "format": "maltos_sft_packed",
        "format_version": 2,
        "source": {
            "dataset": {"path": args.dataset, "config": args.config, "split": args.split},
            "tokenizer": {"name_or_path": args.tokenizer_name_or_path, "vocab_size": vocab_size, "eos_token_id": eos_token_id},
            "columns": {"messages": args.messages_column, "prompt": args.prompt_column, "completion": args.completion_column},
            "processing": {"assistant_only_loss": bool(args.assistant_only_loss), "apply_chat_template": bool(args.apply_chat_template),
                           "append_eos": bool(args.append_eos), "chat_template_file": args.chat_template_file},
            "stats": dict(counts),
        },
        "packing": export_packing_metadata(summary=summary, seq_len=args.seq_len, sequences_per_shard=args.sequences_per_shard,
                                           packing_algorithm=args.packing_algorithm, packing_buffer_size=args.packing_buffer_size),
    }


def _report(progress: Progress, counts: dict[str, int], packer: PackedSFTWriter, final: bool = False) -> None:
    elapsed = progress.elapsed()
    print(f"[{'done' if final else 'progress'}] examples={counts['examples_seen']:,} encoded={counts['examples_encoded']:,} "
          f"skipped={counts['examples_skipped']:,} raw_tokens={packer.raw_tokens:,} "
          f"raw_supervised_tokens={packer.raw_supervised_tokens:,} packed_sequences={packer.packed_sequences:,} "
          f"packed_tokens={packer.packed_sequences * packer.seq_len:,} packed_supervised_tokens={packer.packed_supervised_tokens:,} "
          f"padded_tokens={packer.padded_tokens:,} elapsed={format_duration(elapsed)} "
          f"examples/sec={counts['examples_seen'] / elapsed:,.1f} tokens/sec={packer.raw_tokens / elapsed:,.0f}")


def run(args: argparse.Namespace, tokenizer, rows) -> PackedSFTSummary:
    """Pack ``rows`` with ``tokenizer`` into ``args.output_dir`` and write ``meta.json``; returns the packing summary."""
    out = Path(args.output_dir)
    out.mkdir(parents=True, exist_ok=True)
    packer = PackedSFTWriter(output_dir=out, seq_len=args.seq_len, sequences_per_shard=args.sequences_per_shard,
                             max_sequences=args.max_sequences, pad_token_id=resolve_pad_token_id(tokenizer),
                             packing_algorithm=args.packing_algorithm, packing_buffer_size=args.packing_buffer_size)
    counts = {"examples_seen": 0, "examples_encoded": 0, "examples_skipped": 0}
    progress = Progress(args.log_every_examples)
    for row in rows:
        if args.max_examples is not None and counts["examples_seen"] >= args.max_examples:
            break
        counts["examples_seen"] += 1
        enc = encode_sft_example(row, tokenizer=tokenizer, messages_column=args.messages_column, prompt_column=args.prompt_column,
                                 completion_column=args.completion_column, apply_chat_template=args.apply_chat_template,
                                 assistant_only_loss=args.assistant_only_loss, append_eos=args.append_eos)
        if enc is None:
            counts["examples_skipped"] += 1
        else:
            counts["examples_encoded"] += 1
            packer.add_example(enc)
        if progress.due(counts["examples_seen"]):
            _report(progress, counts, packer)
        if packer.reached_sequence_limit:
            break
    summary = packer.finish()
    meta = build_meta(args, vocab_size=len(tokenizer), eos_token_id=tokenizer.eos_token_id, counts=counts, summary=summary)
    (out / "meta.json").write_text(json.dumps(meta, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    _report(progress, counts, packer, final=True)
    print(f"wrote {summary.packed_sequences:,} sequences ({summary.packed_input_tokens:,} input tokens, "
          f"{summary.packed_supervised_tokens:,} supervised targets) to {out}")
    return summary


def main(argv=None) -> None:
    args = parse_args(argv)
    _validate(args)
    tok = load_tokenizer(args.tokenizer_name_or_path, args.expected_vocab_size)
    if args.chat_template_file is not None:
        tok.chat_template = Path(args.chat_template_file).read_text(encoding="utf-8")
    print(f"tokenizer={args.tokenizer_name_or_path} vocab_size={len(tok)} eos_id={tok.eos_token_id} pad_id={resolve_pad_token_id(tok)} "
          f"chat_template={'yes' if getattr(tok, 'chat_template', None) else 'no'} packing={args.packing_algorithm} "
          f"buffer={args.packing_buffer_size}")
    rows = open_rows(args.dataset, config=args.config, split=args.split, streaming=args.streaming, seed=args.seed,
                     shuffle_buffer_size=args.shuffle_buffer_size)
    run(args, tok, rows)


if __name__ == "__main__":
    main()

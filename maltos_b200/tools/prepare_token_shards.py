"""Tokenise a text dataset into flat ``uint32`` shards (``tokens_00000.bin`` ...) for ``PretrainingDataLoader``.

Documents are concatenated with an end-of-text token between them; a shard holds exactly ``--tokens-per-shard`` tokens
except the last. Same command line as the reference's ``tools/prepare_token_shards.py:11-28``.
"""
from __future__ import annotations

import argparse
from pathlib import Path

import numpy as np

from maltos_b200.tools._prep_common import Progress, format_duration, load_tokenizer, open_rows


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Tokenize text into uint32 .bin shards for PretrainingDataLoader.")
    p.add_argument("--dataset", type=str, required=True, help="HF dataset id or local dataset path")
    p.add_argument("--config", type=str, default=None, help="Optional HF dataset config")
    p.add_argument("--split", type=str, default="train")
    p.add_argument("--column", type=str, default="text")
    p.add_argument("--tokenizer-name-or-path", type=str, required=True)
    p.add_argument("--output-dir", type=str, required=True)
    p.add_argument("--tokens-per-shard", type=int, default=100_000_000)
    p.add_argument("--max-tokens", type=int, default=None)
    p.add_argument("--expected-vocab-size", type=int, default=None)
    p.add_argument("--eos-token", type=str, default=None)
    p.add_argument("--streaming", action="store_true")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--shuffle-buffer-size", type=int, default=10_000)
    p.add_argument("--log-every-tokens", type=int, default=1_000_000)
    return p.parse_args(argv)


class TokenShardWriter:
    """Accumulates token ids in a preallocated ``uint32`` buffer and writes a file each time it is full."""

    def __init__(self, output_dir: Path, tokens_per_shard: int) -> None:
        self.output_dir = output_dir
        self.buf = np.empty(tokens_per_shard, dtype=np.uint32)
        self.fill = 0
        self.index = 0

    def extend(self, ids) -> None:
        arr = np.asarray(ids, dtype=np.uint32)
        at = 0
        while at < arr.size:
            take = min(arr.size - at, self.buf.size - self.fill)
            self.buf[self.fill:self.fill + take] = arr[at:at + take]
            self.fill += take
            at += take
            if self.fill == self.buf.size:
                self.flush()

    def flush(self) -> None:
        if self.fill == 0:
            return
        path = self.output_dir / f"tokens_{self.index:05d}.bin"
        self.buf[:self.fill].tofile(path)
        print(f"wrote {path} tokens={self.fill}")
        self.index += 1
        self.fill = 0


def _report(progress: Progress, tokens: int, docs: int, target: int | None, final: bool = False) -> None:
    elapsed = progress.elapsed()
    rate = tokens / elapsed
    line = (f"[{'done' if final else 'progress'}] tokens={tokens:,} docs={docs:,} elapsed={format_duration(elapsed)} "
            f"tokens/sec={rate:,.0f}")
    if target is not None and tokens > 0:
        line += f" target={target:,} eta={format_duration(max(target - tokens, 0) / max(rate, 1e-9))}"
    print(line)


def main(argv=None) -> None:
    args = parse_args(argv)
    for name in ("tokens_per_shard", "log_every_tokens"):
        if getattr(args, name) < 1:
            raise ValueError(f"{name} must be >= 1, got {getattr(args, name)}")
    if args.max_tokens is not None and args.max_tokens < 1:
        raise ValueError(f"max_tokens must be >= 1, got {args.max_tokens}")
    out = Path(args.output_dir)
    out.mkdir(parents=True, exist_ok=True)
    tok = load_tokenizer(args.tokenizer_name_or_path, args.expected_vocab_size)
    eos = tok.convert_tokens_to_ids(args.eos_token) if args.eos_token is not None else tok.eos_token_id
    print(f"tokenizer={args.tokenizer_name_or_path} vocab_size={len(tok)} eos_id={eos}")
    rows = open_rows(args.dataset, config=args.config, split=args.split, streaming=args.streaming, seed=args.seed,
                     shuffle_buffer_size=args.shuffle_buffer_size)
    writer = TokenShardWriter(out, args.tokens_per_shard)
    progress = Progress(args.log_every_tokens)
    tokens = docs = 0
    for row in rows:
        text = row.get(args.column)
        if not isinstance(text, str) or not text:
            continue
        ids = tok.encode(text, add_special_tokens=False)
        if eos is not None:
            ids.append(int(eos))
        docs += 1
        if args.max_tokens is not None:
            ids = ids[:args.max_tokens - tokens]
        writer.extend(ids)
        tokens += len(ids)
        if progress.due(tokens):
            _report(progress, tokens, docs, args.max_tokens)
        if args.max_tokens is not None and tokens >= args.max_tokens:
            break
    writer.flush()
    _report(progress, tokens, docs, args.max_tokens, final=True)
    print(f"wrote {tokens:,} tokens to {out}")


if __name__ == "__main__":
    main()

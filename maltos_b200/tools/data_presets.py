"""Environment-driven presets for the two data-preparation tools.

``python -m maltos_b200.tools.data_presets pretrain`` and ``... sft [olmo|custom]`` build the argument list of
``prepare_token_shards`` / ``prepare_sft_shards`` from a preset table; every value can be overridden by an environment
variable of the same name (``TOKENIZER``, ``DATASET``, ``OUTPUT_DIR``, ``SEQ_LEN`` ...), the interface of the reference's
shell drivers ``tools/pretrain_data.sh:9-36`` and ``tools/sft_data.sh:9-161``. ``--print`` shows the command instead of
running it. ``pretrain_data.sh`` / ``sft_data.sh`` beside this file are two-line wrappers for users of those names.
"""
from __future__ import annotations

import os
import sys

PRETRAIN = {
    "TOKENIZER": "NousResearch/Llama-2-7b-hf", "DATASET": "HuggingFaceFW/fineweb-edu", "DATASET_CONFIG": "sample-10BT", "SPLIT": "train",
    "TEXT_COLUMN": "text", "OUTPUT_DIR": "workspace/pretrain/data/fineweb_500m", "MAX_TOKENS": "500000000",
    "TOKENS_PER_SHARD": "100000000", "EXPECTED_VOCAB_SIZE": "32000",
}

_SFT_COMMON = {
    "DATASET_CONFIG": "", "SPLIT": "train", "MESSAGES_COLUMN": "messages", "PROMPT_COLUMN": "prompt", "COMPLETION_COLUMN": "completion",
    "SEQ_LEN": "4096", "SEQUENCES_PER_SHARD": "8192", "MAX_EXAMPLES": "", "MAX_SEQUENCES": "", "EXPECTED_VOCAB_SIZE": "",
    "PACKING_ALGORITHM": "best_fit_decreasing", "PACKING_BUFFER_SIZE": "4096", "ASSISTANT_ONLY_LOSS": "true", "APPLY_CHAT_TEMPLATE": "true",
    "APPEND_EOS": "true", "STREAMING": "false", "SHUFFLE_BUFFER_SIZE": "10000", "LOG_EVERY_EXAMPLES": "1000",
}
SFT = {
    # the public Open Instruct 13B recipe: tokenizer of the base model, the -0225 mixture, masked chat template
    "olmo": dict(_SFT_COMMON, TOKENIZER="allenai/OLMo-2-1124-13B", DATASET="allenai/tulu-3-sft-olmo-2-mixture-0225",
                 CHAT_TEMPLATE_FILE="configs/chat_templates/olmo2_sft_masked.jinja", OUTPUT_DIR="workspace/olmo2_13b_sft/data/olmo2_13b_sft", SEED="8"),
    "custom": dict(_SFT_COMMON, TOKENIZER="", DATASET="", CHAT_TEMPLATE_FILE="", OUTPUT_DIR="workspace/sft/data/sft", SEED="42"),
}
_ALIASES = {"olmo2": "olmo", "olmo2_13b_sft": "olmo", "none": "custom"}


def _resolved(defaults: dict, env) -> dict:
    return {k: (env.get(k) if env.get(k) not in (None, "") else v) for k, v in defaults.items()}


def _flag(argv: list, name: str, value: str) -> None:
    if value != "":
        argv += [name, value]


def pretrain_argv(env=os.environ) -> list:
    v = _resolved(PRETRAIN, env)
    argv = ["--dataset", v["DATASET"], "--split", v["SPLIT"], "--column", v["TEXT_COLUMN"], "--tokenizer-name-or-path", v["TOKENIZER"],
            "--expected-vocab-size", v["EXPECTED_VOCAB_SIZE"], "--output-dir", v["OUTPUT_DIR"], "--max-tokens", v["MAX_TOKENS"],
            "--tokens-per-shard", v["TOKENS_PER_SHARD"], "--streaming"]
    if "DATASET_CONFIG" in env and env["DATASET_CONFIG"] == "":
        return argv                                   # explicitly emptied: no dataset configuration
    _flag(argv, "--config", v["DATASET_CONFIG"])
    return argv


def sft_argv(preset: str = "olmo", env=os.environ) -> list:
    preset = _ALIASES.get(preset, preset)
    if preset not in SFT:
        raise SystemExit(f"unknown PRESET={preset}; expected one of: olmo, olmo2, olmo2_13b_sft, custom, none")
    v = _resolved(SFT[preset], env)
    for need in ("TOKENIZER", "DATASET"):
        if not v[need]:
            raise SystemExit(f"{need} must be set when PRESET={preset}")
    argv = ["--dataset", v["DATASET"], "--split", v["SPLIT"], "--messages-column", v["MESSAGES_COLUMN"], "--prompt-column", v["PROMPT_COLUMN"],
            "--completion-column", v["COMPLETION_COLUMN"], "--tokenizer-name-or-path", v["TOKENIZER"], "--output-dir", v["OUTPUT_DIR"],
            "--seq-len", v["SEQ_LEN"], "--sequences-per-shard", v["SEQUENCES_PER_SHARD"], "--packing-algorithm", v["PACKING_ALGORITHM"],
            "--packing-buffer-size", v["PACKING_BUFFER_SIZE"], "--seed", v["SEED"], "--shuffle-buffer-size", v["SHUFFLE_BUFFER_SIZE"],
            "--log-every-examples", v["LOG_EVERY_EXAMPLES"]]
    for name, key in (("--config", "DATASET_CONFIG"), ("--chat-template-file", "CHAT_TEMPLATE_FILE"), ("--max-examples", "MAX_EXAMPLES"),
                      ("--max-sequences", "MAX_SEQUENCES"), ("--expected-vocab-size", "EXPECTED_VOCAB_SIZE")):
        _flag(argv, name, v[key])
    for name, key in (("assistant-only-loss", "ASSISTANT_ONLY_LOSS"), ("apply-chat-template", "APPLY_CHAT_TEMPLATE"), ("append-eos", "APPEND_EOS")):
        argv.append(f"--{name}" if v[key] == "true" else f"--no-{name}")
    if v["STREAMING"] == "true":
        argv.append("--streaming")
    return argv


def main(argv=None) -> None:
    args = list(sys.argv[1:] if argv is None else argv)
    show = "--print" in args
    args = [a for a in args if a != "--print"]
    if not args or args[0] not in ("pretrain", "sft"):
        raise SystemExit("usage: data_presets.py {pretrain | sft [olmo|custom]} [--print] [extra tool flags]")
    kind, rest = args[0], args[1:]
    if kind == "pretrain":
        from maltos_b200.tools import prepare_token_shards as tool

        tool_argv = pretrain_argv() + rest
    else:
        from maltos_b200.tools import prepare_sft_shards as tool

        preset = os.environ.get("PRESET", "olmo")
        if rest and not rest[0].startswith("-"):
            preset, rest = rest[0], rest[1:]
        tool_argv = sft_argv(preset) + rest
        print(f"preset={_ALIASES.get(preset, preset)} output_dir={tool_argv[tool_argv.index('--output-dir') + 1]}")
    if show:
        print(" ".join([tool.__name__.rsplit(".", 1)[-1], *tool_argv]))
        return
    tool.main(tool_argv)


if __name__ == "__main__":
    main()

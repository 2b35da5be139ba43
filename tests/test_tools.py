"""Command-line tools that run without a GPU: synthetic throughput profiler and the upload planner."""
import json

import pytest
import torch

from maltos_b200.tools import profile_train_perf as ptp
from maltos_b200.tools.upload_wandb_checkpoint import plan_uploads, sanitize_artifact_name
from maltos_b200.utils.constants import IGNORE_INDEX, PAD_SEQUENCE_ID


def test_packed_synthetic_batch_is_well_formed():
    cfg = ptp.SyntheticBatchConfig(layout="packed", segment_count_min=2, segment_count_max=5, supervised_fraction_min=0.4,
                                   supervised_fraction_max=0.6, max_padding_fraction=0.1)
    b = ptp.make_synthetic_batch(rows=4, seq_len=128, vocab_size=50, config=cfg, generator=torch.Generator().manual_seed(0))
    ids, labels, pos, seq = b["input_ids"], b["labels"], b["position_ids"], b["sequence_ids"]
    for r in range(4):
        pad = seq[r] == PAD_SEQUENCE_ID
        assert (labels[r][pad] == IGNORE_INDEX).all() and (ids[r][pad] == 0).all()
        docs = seq[r][~pad]
        assert (docs[1:] >= docs[:-1]).all() and 2 <= int(docs.max()) + 1 <= 5
        starts = torch.nonzero(torch.cat([torch.tensor([True]), docs[1:] != docs[:-1]])).flatten()
        assert (pos[r][starts] == 0).all()
        # a supervised target is the next token of the same document
        sup = torch.nonzero(labels[r] != IGNORE_INDEX).flatten()
        assert len(sup) > 0 and all(seq[r, i] == seq[r, i + 1] and labels[r, i] == ids[r, i + 1] for i in sup.tolist() if i + 1 < 128 and not pad[i + 1])
    with pytest.raises(ValueError):
        ptp.SyntheticBatchConfig(layout="ragged")


def test_case_file_and_profiler_run(tmp_path):
    recipe = tmp_path / "r.yaml"
    recipe.write_text("seed: 1\ndata: {seq_len: 32, micro_batch_size: 2}\nmodel: {type: llama, hidden_size: 64, num_heads: 4, num_kv_heads: 2, "
                      "intermediate_size: 128, num_layers: 2, vocab_size: 128}\ntraining: {grad_accum_steps: 2, lr: 0.001}\n")
    cases = tmp_path / "cases.yaml"
    cases.write_text(f"cases:\n  tiny:\n    description: tiny\n    recipe: {recipe}\n    synthetic: {{packed: true}}\n    warmup: 1\n    steps: 2\n")
    assert set(ptp._load_cases(cases)) == {"tiny"}
    ptp.main(["--case-file", str(cases), "--case", "tiny", "--output-dir", str(tmp_path / "out")])
    summary = json.loads((tmp_path / "out" / "summary.json").read_text())
    assert summary["timed_steps"] == 2 and summary["tokens_per_step"] == 2 * 32 * 2 and summary["learning_rate"] == 0.0
    assert summary["synthetic"]["layout"] == "packed" and summary["tokens_per_second"] > 0
    assert (tmp_path / "out" / "summary.txt").read_text().startswith("case: tiny")


def test_upload_plan_validation(tmp_path):
    assert sanitize_artifact_name("my run/1") == "my-run-1"
    with pytest.raises(ValueError):
        sanitize_artifact_name("///")
    root = tmp_path / "ckpt"
    (root / "step_00000002").mkdir(parents=True)
    with pytest.raises(ValueError):
        plan_uploads(root, [2], "p", [])
    (root / "runtime_spec.json").write_text("{}")
    with pytest.raises(ValueError):
        plan_uploads(root, [2], "p", [])
    (root / "step_00000002" / "manifest.json").write_text("{}")
    (root / "step_00000004").mkdir()
    (root / "step_00000004" / "manifest.json").write_text("{}")
    plan = plan_uploads(root, [2, 4], "p", ["best"])
    assert [i["name"] for i in plan] == ["p-step-00000002", "p-step-00000004"]
    assert plan[0]["aliases"] == ["best", "step_2"] and plan[1]["aliases"] == ["best", "step_4", "latest"]


def test_bench_micro_batch_defaults():
    """The benchmark's micro-batch default is the same for both arms: 2 on one GPU (with a fallback to 1 when it does not
    fit), 1 on several GPUs; explicit values win and switch the fallback off."""
    import importlib.util
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("bench_module", Path(__file__).resolve().parents[1] / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.parse_args([]).micro_batch == 2
    assert bench.parse_args(["--gpus", "4"]).micro_batch == 1
    ref = bench.parse_args(["--impl", "reference"])
    assert ref.micro_batch == 2 and ref.micro_batch_auto
    assert bench.parse_args(["--impl", "reference", "--gpus", "8"]).micro_batch == 1
    assert not bench.parse_args(["--micro-batch", "2"]).micro_batch_auto
    assert bench.parse_args(["--small"]).micro_batch == 1
    assert bench.parse_args(["--micro-batch", "4"]).micro_batch == 4


def test_data_presets_build_the_tool_arguments_from_the_environment(capsys):
    from maltos_b200.tools import data_presets as dp

    argv = dp.pretrain_argv({})
    assert argv[argv.index("--config") + 1] == "sample-10BT" and "--streaming" in argv
    argv = dp.pretrain_argv({"DATASET": "my/data", "DATASET_CONFIG": "", "MAX_TOKENS": "1000"})
    assert "--config" not in argv and argv[argv.index("--dataset") + 1] == "my/data" and argv[argv.index("--max-tokens") + 1] == "1000"
    olmo = dp.sft_argv("olmo2_13b_sft", {})
    assert olmo[olmo.index("--seed") + 1] == "8" and "--assistant-only-loss" in olmo and "--chat-template-file" in olmo
    custom = dp.sft_argv("custom", {"TOKENIZER": "tok", "DATASET": "ds", "APPEND_EOS": "false", "STREAMING": "true", "MAX_EXAMPLES": "5"})
    assert "--no-append-eos" in custom and "--streaming" in custom and custom[custom.index("--max-examples") + 1] == "5"
    assert "--chat-template-file" not in custom
    import pytest

    with pytest.raises(SystemExit, match="TOKENIZER must be set"):
        dp.sft_argv("custom", {})
    with pytest.raises(SystemExit, match="unknown PRESET"):
        dp.sft_argv("nope", {})
    dp.main(["pretrain", "--print"])
    assert capsys.readouterr().out.startswith("prepare_token_shards --dataset")
    # the tools accept what the presets produce
    from maltos_b200.tools import prepare_sft_shards, prepare_token_shards

    ns = prepare_token_shards.parse_args(dp.pretrain_argv({}))
    assert ns.max_tokens == 500000000 and ns.streaming
    ns = prepare_sft_shards.parse_args(olmo)
    assert ns.seq_len == 4096 and ns.assistant_only_loss


def _tiny_recipe(tmp_path):
    recipe = tmp_path / "r.yaml"
    recipe.write_text("seed: 1\ndata: {seq_len: 32, micro_batch_size: 2}\nmodel: {type: llama, hidden_size: 64, num_heads: 4, num_kv_heads: 2, "
                      "intermediate_size: 128, num_layers: 2, vocab_size: 128}\ntraining: {grad_accum_steps: 2, lr: 0.001}\n")
    return recipe


def test_profiler_document_trace_fixed_segments_and_metadata(tmp_path):
    recipe = _tiny_recipe(tmp_path)
    cases = tmp_path / "cases.yaml"
    cases.write_text(f"cases:\n  traced:\n    recipe: {recipe}\n    synthetic:\n      packed: true\n      document_length_trace:\n        - [16, 8, 4]\n"
                     f"        - [30]\n    warmup: 0\n    steps: 1\n  measured:\n    recipe: {recipe}\n    require_calibrated_hdp_cost: true\n")
    ptp.main(["--case-file", str(cases), "--case", "traced", "--output-dir", str(tmp_path / "out")])
    summary = json.loads((tmp_path / "out" / "summary.json").read_text())
    trace = summary["document_trace"]
    assert trace["rows"] == 2 and trace["documents"] == 4 and trace["max_length"] == 30 and abs(trace["active_fraction"] - 58 / 64) < 1e-9
    assert summary["data_source"] == "synthetic" and 0.0 <= summary["data_wait_fraction"] < 1.0
    env = summary["environment"]
    assert {"python", "torch", "host", "platform", "variables", "commit", "kernel_library"} <= set(env)
    # rows follow the trace in order, across batches
    cfg = ptp.SyntheticBatchConfig(layout="packed", document_length_trace=((16, 8, 4), (30,)))
    b = ptp.make_synthetic_batch(rows=2, seq_len=32, vocab_size=50, config=cfg, generator=torch.Generator().manual_seed(0), row_offset=1)
    assert int((b["sequence_ids"][0] != PAD_SEQUENCE_ID).sum()) == 30 and int(b["sequence_ids"][1].max()) == 2
    assert (b["sequence_ids"][1][28:] == PAD_SEQUENCE_ID).all()
    with pytest.raises(ValueError, match="sums to"):
        ptp.make_synthetic_batch(rows=1, seq_len=16, vocab_size=50, config=cfg, generator=torch.Generator().manual_seed(0))
    with pytest.raises(ValueError, match="packed layout"):
        ptp.SyntheticBatchConfig(layout="dense", document_length_trace=((4,),))
    # a measurement case refuses the uncalibrated cost proxy
    with pytest.raises(SystemExit, match="calibrated"):
        ptp.main(["--case-file", str(cases), "--case", "measured", "--output-dir", str(tmp_path / "out2")])
    # compatibility spellings of the flags
    args = ptp._parse_tool_args(["--recipe", str(recipe), "--packed-input", "--packed-sequences", "4", "--synthetic-delivery", "cuda"])
    cfg = ptp._synthetic_config(args, ptp.CaseDefinition(name="x", recipe=str(recipe)))
    assert cfg.layout == "packed" and cfg.segment_count_min == cfg.segment_count_max == 4 and cfg.delivery == "device"


def test_profiler_can_time_the_recipes_own_loader(tmp_path):
    import numpy as np

    recipe = _tiny_recipe(tmp_path)
    np.random.default_rng(0).integers(0, 128, size=4000, dtype=np.uint32).tofile(tmp_path / "tokens_00000.bin")
    ptp.main(["--recipe", str(recipe), "--data-source", "recipe", "--warmup", "0", "--steps", "2", "--output-dir", str(tmp_path / "out"), "--",
              "--data", str(tmp_path / "tokens_00000.bin"), "--data-prefetch-batches", "1"])
    summary = json.loads((tmp_path / "out" / "summary.json").read_text())
    assert summary["data_source"] == "recipe" and summary["data_prefetch_batches"] == 1 and summary["active_target_fraction"] is None
    assert summary["timed_steps"] == 2 and summary["tokens_per_second"] > 0
    with pytest.raises(SystemExit, match="--data"):
        ptp.main(["--recipe", str(recipe), "--data-source", "recipe", "--output-dir", str(tmp_path / "o2")])


def test_bench_line_carries_every_key_of_the_contract():
    """`python bench.py` prints ONE JSON line with the agreed keys (checked on the tiny CPU plumbing configuration, for both
    arms when the reference is installed)."""
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    arms = [[]] + ([["--impl", "reference"]] if (root / "baseline" / "_ref" / "runtime" / "core.py").exists() else [])
    for arm in arms:
        out = subprocess.run([sys.executable, "bench.py", "--small", "--device", "cpu", "--steps", "2", "--warmup", "1", *arm], cwd=root,
                             capture_output=True, text=True, timeout=900)
        assert out.returncode == 0, out.stderr[-2000:]
        lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
        assert len(lines) == 1, out.stdout[-2000:]
        row = json.loads(lines[0])
        for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype",
                    "data", "config", "clocks", "e2e", "gpu_launches", "impl"):
            assert key in row, (arm, key)
        assert row["steps"] == 2 and row["warmup"] == 1 and row["n_gpus"] == 1 and row["higher_is_better"] is True
        assert row["impl"] == ("reference" if arm else "ours")
        assert {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} <= set(row["e2e"]) and row["e2e"]["h2d_bytes_per_step"] > 0
        assert {"micro_batch", "grad_accum", "global_batch", "seq_len"} <= set(row["config"])
        assert row["config"]["micro_batch"] * row["config"]["grad_accum"] == row["config"]["global_batch"]


def test_every_recipe_and_every_profiler_case_validates():
    """All YAML recipes in ``configs/`` and all named profiler cases parse, and their parallel layout passes the CLI's
    validation for the world size they ask for."""
    from pathlib import Path

    from maltos_b200.train import cli, flags

    root = Path(__file__).resolve().parents[1]
    recipes = sorted(p for p in (root / "configs").glob("*.yaml") if p.name != "profile_train_perf_cases.yaml")
    assert len(recipes) >= 8
    for recipe in recipes:
        a = flags.parse_args_from(["--config", str(recipe)], require_data=False)
        cli.validate_args(a, a.dp_size * a.tp_size * a.pp_size * a.cp_size)
    import os

    here = os.getcwd()
    os.chdir(root)      # cases name their recipes relative to the repository root
    try:
        cases = ptp._load_cases(root / "configs" / "profile_train_perf_cases.yaml")
        assert len(cases) >= 12
        for case in cases.values():
            a = ptp._training_args(case, [])
            cli.validate_args(a, a.dp_size * a.tp_size * a.pp_size * a.cp_size)
            ptp._synthetic_config(ptp._parse_tool_args(["--case", case.name]), case)
    finally:
        os.chdir(here)


def test_doctor_reports_the_installation_and_finds_every_entry_point(capsys):
    """Without a CUDA device the tool still loads the kernel library (it has no link-time dependency on the driver) and
    checks that every ``mb_*`` entry point the package calls is exported; exit code 0 = nothing a CUDA run needs is missing."""
    from maltos_b200.tools import doctor

    report = doctor.collect()
    lib = report["library"]
    if lib["present"]:
        assert lib["loads"] and lib["entry_points_called"] >= 30 and lib["entry_points_missing"] == [], lib
    assert report["mode"].startswith("cpu") == (not report["devices"])
    assert doctor.main(["--json"]) == (1 if [p for p in report["problems"] if not p.startswith("no peer access")] else 0)
    assert '"library"' in capsys.readouterr().out

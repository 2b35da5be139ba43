"""Logical (safetensors) checkpoints: file-format round trips and runtime <-> logical conversion across layouts."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import yaml

from tests.dist_utils import free_port
from maltos_b200.state.logical_checkpoint import (LogicalCheckpointTensorReader, iter_logical_checkpoint_tensors, load_logical_checkpoint,
                                                  load_logical_tensor, save_logical_checkpoint)

ROOT = Path(__file__).resolve().parents[1]
MODEL = {"type": "llama", "hidden_size": 64, "num_heads": 4, "num_kv_heads": 2, "intermediate_size": 128, "num_layers": 2,
         "vocab_size": 256}


def test_logical_file_roundtrip_sharded_and_hf_prefix(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {f"layers.{i}.w": torch.randn(16, 8, generator=g) for i in range(5)}
    tensors["lm_head.weight"] = torch.randn(4, 8, generator=g).bfloat16()
    save_logical_checkpoint(tmp_path / "a", tensors, max_shard_size_bytes=16 * 8 * 4 * 2)
    index = json.loads((tmp_path / "a" / "model.safetensors.index.json").read_text())
    assert index["metadata"]["format"] == "logical_model" and index["metadata"]["version"] == 1
    assert len(set(index["weight_map"].values())) == 3 and all("-of-00003" in f for f in index["weight_map"].values())
    back = load_logical_checkpoint(tmp_path / "a")
    assert set(back) == set(tensors) and all(torch.equal(back[k], tensors[k]) for k in tensors)
    assert torch.equal(load_logical_tensor(tmp_path / "a", "layers.3.w"), tensors["layers.3.w"])
    assert dict(iter_logical_checkpoint_tensors(tmp_path / "a")).keys() == tensors.keys()
    reader = LogicalCheckpointTensorReader(tmp_path / "a")
    assert len(reader) == 6 and torch.equal(reader["lm_head.weight"], tensors["lm_head.weight"])
    with pytest.raises(KeyError):
        reader["nope"]
    # an HF-style index: no format tag, names prefixed with "model." except lm_head.weight
    from safetensors.torch import save_file

    hf = tmp_path / "hf"
    hf.mkdir()
    save_file({"model.embed.weight": tensors["layers.0.w"], "lm_head.weight": tensors["lm_head.weight"]}, str(hf / "x.safetensors"))
    (hf / "model.safetensors.index.json").write_text(json.dumps(
        {"metadata": {"total_size": 1}, "weight_map": {"model.embed.weight": "x.safetensors", "lm_head.weight": "x.safetensors"}}))
    hf_back = load_logical_checkpoint(hf)
    assert set(hf_back) == {"embed.weight", "lm_head.weight"} and torch.equal(hf_back["embed.weight"], tensors["layers.0.w"])
    with pytest.raises(ValueError):
        load_logical_checkpoint(tmp_path / "missing")


def _run(cmd, nproc=1):
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=str(ROOT))
    if nproc > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(free_port())] + cmd
    else:
        cmd = [sys.executable] + cmd
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=420)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    return out.stdout


def _recipe(path, parallel):
    cfg = {"seed": 1, "data": {"seq_len": 32, "micro_batch_size": 2}, "model": MODEL, "parallel": parallel,
           "training": {"max_steps": 2, "grad_accum_steps": 1, "lr": 1e-3}}
    path.write_text(yaml.safe_dump(cfg))
    return path


def test_runtime_logical_runtime_across_layouts(tmp_path):
    data = tmp_path / "tokens"
    data.mkdir()
    np.random.default_rng(0).integers(0, 256, size=6000, dtype=np.uint32).tofile(data / "tokens_00000.bin")
    # 1. train two steps as DP2 + ZeRO-3 and keep the runtime checkpoint
    src = _recipe(tmp_path / "src.yaml", {"dp_size": 2, "zero_stage": 3})
    _run(["-m", "maltos_b200.tools.train", "--config", str(src), "--data", str(data), "--checkpoint-dir", str(tmp_path / "rt_a"),
          "--checkpoint-every", "2", "--log-every", "1"], nproc=2)
    step_a = tmp_path / "rt_a" / "step_00000002"
    assert (step_a / "manifest.json").is_file()
    # 2. runtime -> logical (single process, recipe read from the runtime spec)
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "runtime-to-logical", "--checkpoint", str(step_a), "--output", str(tmp_path / "logical_a")])
    logical_a = load_logical_checkpoint(tmp_path / "logical_a")
    assert len(logical_a) > 10 and all(t.dtype == torch.float32 for t in logical_a.values())
    # 3. logical -> runtime for a TP2 + SP layout, then back to logical: every tensor must survive bit for bit
    dst = _recipe(tmp_path / "dst.yaml", {"tp_size": 2, "use_sp": True})
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "logical-to-runtime", "--config", str(dst), "--checkpoint", str(tmp_path / "logical_a"),
          "--output", str(tmp_path / "rt_b")], nproc=2)
    step_b = tmp_path / "rt_b" / "step_00000000"
    manifest = json.loads((step_b / "manifest.json").read_text())
    assert manifest["world_size"] == 2 and not [a for a in manifest["artifacts"] if a["kind"] == "optimizer"]
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "runtime-to-logical", "--checkpoint", str(step_b), "--output", str(tmp_path / "logical_b")])
    logical_b = load_logical_checkpoint(tmp_path / "logical_b")
    assert set(logical_a) == set(logical_b)
    for name in logical_a:
        assert torch.equal(logical_a[name], logical_b[name]), name


def test_expert_parallel_checkpoint_to_pipeline_layout_and_resume(tmp_path):
    """MoE trained with experts spread over two ranks -> logical (experts under their GLOBAL names) -> a two-stage pipeline
    layout -> logical again, bit for bit; and training continues from the converted checkpoint with the loss it would have
    had in the original layout."""
    moe = {"type": "tiny_moe", "hidden_size": 64, "num_heads": 4, "num_kv_heads": 2, "intermediate_size": 96, "num_layers": 2, "vocab_size": 256,
           "num_experts": 4, "moe_aux_loss_coef": 0.0}

    def recipe(path, parallel, steps):
        cfg = {"seed": 1, "data": {"seq_len": 32, "micro_batch_size": 2}, "model": moe, "parallel": parallel,
               "training": {"max_steps": steps, "grad_accum_steps": 1, "lr": 1e-3}}
        path.write_text(yaml.safe_dump(cfg))
        return path

    data = tmp_path / "tokens"
    data.mkdir()
    np.random.default_rng(0).integers(0, 256, size=6000, dtype=np.uint32).tofile(data / "tokens_00000.bin")
    src = recipe(tmp_path / "src.yaml", {"dp_size": 2, "ep_size": 2, "zero_stage": 1}, 2)
    _run(["-m", "maltos_b200.tools.train", "--config", str(src), "--data", str(data), "--checkpoint-dir", str(tmp_path / "rt_a"),
          "--checkpoint-every", "2", "--log-every", "1"], nproc=2)
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "runtime-to-logical", "--checkpoint", str(tmp_path / "rt_a" / "step_00000002"),
          "--output", str(tmp_path / "logical_a")])
    logical_a = load_logical_checkpoint(tmp_path / "logical_a")
    experts = sorted({n.split("experts.")[1].split(".")[0] for n in logical_a if ".experts." in n})
    assert experts == ["0", "1", "2", "3"], experts                          # global expert ids, none missing, none local
    dst = recipe(tmp_path / "dst.yaml", {"pp_size": 2, "pp_microbatches": 2}, 3)
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "logical-to-runtime", "--config", str(dst), "--checkpoint", str(tmp_path / "logical_a"),
          "--output", str(tmp_path / "rt_b")], nproc=2)
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "runtime-to-logical", "--checkpoint", str(tmp_path / "rt_b" / "step_00000000"),
          "--output", str(tmp_path / "logical_b")])
    logical_b = load_logical_checkpoint(tmp_path / "logical_b")
    assert set(logical_a) == set(logical_b)
    for name in logical_a:
        assert torch.equal(logical_a[name], logical_b[name]), name
    # weights-only continuation in the pipeline layout runs and produces finite losses from the converted weights
    out = _run(["-m", "maltos_b200.tools.train", "--config", str(dst), "--data", str(data), "--resume-from", str(tmp_path / "rt_b" / "step_00000000"),
                "--load-weights-only", "--log-every", "1"], nproc=2)
    losses = [float(l.split("loss ")[1].split(" ")[0]) for l in out.splitlines() if l.startswith("[step")]
    assert len(losses) == 3 and all(l == l and l < 6.0 for l in losses), out[-1500:]


def test_zero3_buckets_under_tensor_and_expert_parallelism_convert_to_logical(tmp_path):
    """ZeRO-3 shards over the data-parallel ranks of ONE tensor-parallel coordinate, and expert buckets of different
    expert-parallel ranks hold different experts: the converter must take the slices of a bucket from the ranks of one
    coordinate (not interleave the copies) and find the experts under their global names. Checked by the loss the converted
    weights give in a single process against the loss the original layout gives with the same weights and data."""
    moe = {"type": "tiny_moe", "hidden_size": 64, "num_heads": 4, "num_kv_heads": 2, "intermediate_size": 96, "num_layers": 2, "vocab_size": 256,
           "num_experts": 4, "moe_aux_loss_coef": 0.0}

    def recipe(path, parallel, steps, micro_batch):
        cfg = {"seed": 1, "data": {"seq_len": 32, "micro_batch_size": micro_batch}, "model": moe, "parallel": parallel,
               "training": {"max_steps": steps, "grad_accum_steps": 1, "lr": 1e-3}}
        path.write_text(yaml.safe_dump(cfg))
        return path

    def losses_of(out):
        return [float(l.split("loss ")[1].split(" ")[0]) for l in out.splitlines() if l.startswith("[step")]

    data = tmp_path / "tokens"
    data.mkdir()
    np.random.default_rng(0).integers(0, 256, size=20000, dtype=np.uint32).tofile(data / "tokens_00000.bin")
    src = recipe(tmp_path / "src.yaml", {"dp_size": 2, "tp_size": 2, "use_sp": True, "ep_size": 2, "zero_stage": 3}, 2, 2)
    _run(["-m", "maltos_b200.tools.train", "--config", str(src), "--data", str(data), "--checkpoint-dir", str(tmp_path / "rt_a"),
          "--checkpoint-every", "2", "--log-every", "1"], nproc=4)
    step_a = tmp_path / "rt_a" / "step_00000002"
    manifest = json.loads((step_a / "manifest.json").read_text())
    names = {n for r in manifest["ranks"] for e in r["entries"] for n in e["logical_names"]}
    assert not [n for n in names if "local_experts" in n] and any(".experts.3." in n for n in names)
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "runtime-to-logical", "--checkpoint", str(step_a), "--output", str(tmp_path / "logical")])
    single = recipe(tmp_path / "single.yaml", {}, 1, 4)
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "logical-to-runtime", "--config", str(single), "--checkpoint", str(tmp_path / "logical"),
          "--output", str(tmp_path / "rt_b")])
    one_step = recipe(tmp_path / "src1.yaml", {"dp_size": 2, "tp_size": 2, "use_sp": True, "ep_size": 2, "zero_stage": 3}, 1, 2)
    want = losses_of(_run(["-m", "maltos_b200.tools.train", "--config", str(one_step), "--data", str(data), "--resume-from", str(step_a),
                           "--load-weights-only", "--log-every", "1"], nproc=4))
    got = losses_of(_run(["-m", "maltos_b200.tools.train", "--config", str(single), "--data", str(data), "--resume-from",
                          str(tmp_path / "rt_b" / "step_00000000"), "--load-weights-only", "--log-every", "1"]))
    assert len(want) == len(got) == 1 and abs(want[0] - got[0]) < 2e-4, (want, got)
    # and back into the sharded layout: logical -> ZeRO-3 + TP + EP runtime -> logical is the identity
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "logical-to-runtime", "--config", str(src), "--checkpoint", str(tmp_path / "logical"),
          "--output", str(tmp_path / "rt_c")], nproc=4)
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "runtime-to-logical", "--checkpoint", str(tmp_path / "rt_c" / "step_00000000"),
          "--output", str(tmp_path / "logical_c")])
    a, c = load_logical_checkpoint(tmp_path / "logical"), load_logical_checkpoint(tmp_path / "logical_c")
    assert set(a) == set(c) and all(torch.equal(a[n], c[n]) for n in a)


def test_zero1_checkpoint_is_written_once_per_tensor_parallel_rank_and_converts(tmp_path):
    """ZeRO-1/2 keep full weights on every data-parallel rank: one replica writes them (tensor-parallel shards: one writer
    per TP rank), and the offline converter joins exactly one piece per TP rank (buffers, which every rank writes, are
    taken from the lowest writer of each TP rank)."""
    def recipe(path, parallel, steps, micro_batch):
        cfg = {"seed": 1, "data": {"seq_len": 32, "micro_batch_size": micro_batch}, "model": MODEL, "parallel": parallel,
               "training": {"max_steps": steps, "grad_accum_steps": 1, "lr": 1e-3}}
        path.write_text(yaml.safe_dump(cfg))
        return path

    data = tmp_path / "tokens"
    data.mkdir()
    np.random.default_rng(0).integers(0, 256, size=20000, dtype=np.uint32).tofile(data / "tokens_00000.bin")
    src = recipe(tmp_path / "src.yaml", {"dp_size": 2, "tp_size": 2, "use_sp": True, "zero_stage": 1}, 2, 2)
    _run(["-m", "maltos_b200.tools.train", "--config", str(src), "--data", str(data), "--checkpoint-dir", str(tmp_path / "rt_a"),
          "--checkpoint-every", "2", "--log-every", "1"], nproc=4)
    step_a = tmp_path / "rt_a" / "step_00000002"
    manifest = json.loads((step_a / "manifest.json").read_text())
    writers = {e["source_rank"] for r in manifest["ranks"] for e in r["entries"] if e["state_key"].endswith("proj.weight")}
    assert writers == {0, 1}, writers                       # the two TP ranks of data-parallel replica 0
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "runtime-to-logical", "--checkpoint", str(step_a), "--output", str(tmp_path / "logical")])
    logical = load_logical_checkpoint(tmp_path / "logical")
    # the same training as ZeRO-0 in one process gives the same weights (fp32, summation order aside)
    single = recipe(tmp_path / "single.yaml", {}, 2, 4)
    _run(["-m", "maltos_b200.tools.train", "--config", str(single), "--data", str(data), "--checkpoint-dir", str(tmp_path / "rt_s"),
          "--checkpoint-every", "2", "--log-every", "1"])
    _run(["-m", "maltos_b200.tools.convert_checkpoint", "runtime-to-logical", "--checkpoint", str(tmp_path / "rt_s" / "step_00000002"),
          "--output", str(tmp_path / "logical_s")])
    want = load_logical_checkpoint(tmp_path / "logical_s")
    assert set(want) == set(logical)
    for name in want:
        assert torch.allclose(want[name], logical[name], atol=2e-5), (name, (want[name] - logical[name]).abs().max())

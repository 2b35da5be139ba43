"""Combinations of parallel axes through the training CLI on 4 gloo ranks must reproduce the single-process losses
(same global batch, fp32): DP x TP+SP with ZeRO-3, PP x TP (1F1B), CP(ring) x TP+SP, DP x PP with ZeRO-1."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from tests.dist_utils import free_port

ROOT = Path(__file__).resolve().parents[1]
MODEL = ["--model", "llama", "--dim", "64", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "128", "--n-layers", "4", "--vocab-size", "256",
         "--seq-len", "32", "--lr", "1e-3", "--grad-clip", "1.0", "--log-every", "1", "--max-steps", "3", "--seed", "3"]


@pytest.fixture(scope="module")
def data(tmp_path_factory):
    d = tmp_path_factory.mktemp("tokens")
    np.random.default_rng(1).integers(0, 256, size=30000, dtype=np.uint32).tofile(d / "tokens_00000.bin")
    return d


def _losses(data, extra, nproc):
    env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONPATH=str(ROOT))
    base = ["-m", "maltos_b200.tools.train", "--data", str(data), *MODEL, *extra]
    if nproc > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(free_port()), *base]
    else:
        cmd = [sys.executable, *base]
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    vals = [float(l.split("loss ")[1].split(" ")[0]) for l in out.stdout.splitlines() if l.startswith("[step")]
    assert len(vals) == 3, out.stdout[-2000:]
    return vals


@pytest.fixture(scope="module")
def reference(data):
    # global batch of 4 sequences per optimizer step, as one micro-batch on one process
    return _losses(data, ["--micro-batch-size", "4", "--grad-accum-steps", "1"], 1)


CASES = {
    "dp2_tp2_sp_zero3": ["--dp-size", "2", "--tp-size", "2", "--use-sp", "--zero-stage", "3", "--micro-batch-size", "2", "--grad-accum-steps", "1"],
    "pp2_tp2_1f1b": ["--pp-size", "2", "--tp-size", "2", "--pp-schedule", "1f1b", "--pp-microbatches", "2", "--micro-batch-size", "4",
                     "--grad-accum-steps", "1"],
    "cp2_ring_tp2_sp": ["--cp-size", "2", "--cp-attn-core", "ring", "--tp-size", "2", "--use-sp", "--micro-batch-size", "4", "--grad-accum-steps", "1"],
    # the loader itself hands every context-parallel rank its zigzag share (no sharding inside the runtime)
    "cp2_ring_loader_sharded_tp2_sp": ["--cp-size", "2", "--cp-attn-core", "ring", "--cp-token-planner", "fixed_zigzag", "--batch-data-cp-aware",
                                       "--tp-size", "2", "--use-sp", "--micro-batch-size", "4", "--grad-accum-steps", "1"],
    "dp2_cp2_allgather_loader_sharded_prefetch": ["--dp-size", "2", "--cp-size", "2", "--cp-attn-core", "all_gather_kv", "--cp-token-planner",
                                                  "fixed_contiguous", "--batch-data-cp-aware", "--data-prefetch-batches", "1", "--micro-batch-size", "2",
                                                  "--grad-accum-steps", "1"],
    # balanced hybrid data parallelism: all four ranks cut their waves from the same canonical batch of 4 rows
    "dp4_hdp_balanced_zero1": ["--dp-size", "4", "--hdp-balanced", "--hdp-partition-tokens", "16", "--zero-stage", "1", "--micro-batch-size", "4",
                               "--grad-accum-steps", "1"],
    "dp2_pp2_zero1_accum": ["--dp-size", "2", "--pp-size", "2", "--zero-stage", "1", "--pp-microbatches", "1", "--micro-batch-size", "1",
                            "--grad-accum-steps", "2"],
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_axis_combination_matches_single_process(name, data, reference):
    got = _losses(data, CASES[name], 4)
    # first step: same parameters, only the summation order differs from the single process; later steps also see the
    # order of the gradient reductions, amplified by Adam's normalisation (runs are bit-reproducible from run to run)
    assert abs(got[0] - reference[0]) < 1e-4, (name, got, reference)
    assert max(abs(a - b) for a, b in zip(got, reference)) < 1e-3, (name, got, reference)


@pytest.mark.parametrize("loader_sharded", [False, True])
def test_logged_tokens_cover_the_accumulation_window_once(loader_sharded, data, tmp_path):
    """dp2 x cp2, two micro-batches of 2 rows x 32 tokens per optimizer step: 2 (dp) x 2 (accum) x 2 x 32 = 256 tokens, however
    the rows reach the context-parallel ranks; and the logged loss is the loss of the whole rows, not a rank's share."""
    import json

    out = tmp_path / "metrics.jsonl"
    flags = ["--dp-size", "2", "--cp-size", "2", "--cp-attn-core", "ring", "--cp-token-planner", "fixed_zigzag", "--micro-batch-size", "2",
             "--grad-accum-steps", "2", "--metrics-jsonl", str(out)] + (["--batch-data-cp-aware"] if loader_sharded else [])
    losses = _losses(data, flags, 4)
    rows = [json.loads(l) for l in out.read_text().splitlines()]
    assert [r["train/tokens"] for r in rows] == [256.0, 256.0, 256.0]
    single = _losses(data, ["--micro-batch-size", "8", "--grad-accum-steps", "1"], 1)
    assert abs(losses[0] - single[0]) < 1e-4, (losses, single)

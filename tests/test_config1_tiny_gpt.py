"""The plumbing benchmark as specified (GPT-style tiny decoder, 2 gloo ranks, DP + ZeRO-1, fp32, 10 steps with gradient
accumulation 2 and clipping 1.0, save -> load -> resume) under this runtime and, with the same model file, under the
reference's runtime as the oracle."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from tests.dist_utils import free_port

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"


def _run(extra):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port",
           str(free_port()), str(ROOT / "tests" / "config1_tiny_gpt.py"), *extra]
    env = dict(os.environ, OMP_NUM_THREADS="1", GLOO_SOCKET_IFNAME="lo", PYTHONPATH=str(ROOT))
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=420)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("LOSSES ")][-1]
    return json.loads(line[len("LOSSES "):])


def test_ten_steps_and_resume_equivalence(tmp_path):
    full = _run(["--steps", "10"])
    assert len(full) == 10 and all(3.0 < v < 8.0 for v in full) and full[-1] < full[0]      # ln(512) = 6.24 at the start
    head = _run(["--steps", "6", "--save-at", "6", "--ckpt", str(tmp_path)])
    assert head == full[:6]
    tail = _run(["--steps", "10", "--resume", str(tmp_path / "step_00000006")])
    assert tail == full[6:]


@pytest.mark.skipif(not (REF / "runtime" / "core.py").exists(), reason="reference not installed under baseline/_ref")
def test_same_model_under_the_reference_runtime(tmp_path):
    ours = _run(["--steps", "10"])
    ref = _run(["--steps", "10", "--impl", "reference"])
    assert len(ref) == 10
    assert max(abs(a - b) for a, b in zip(ours, ref)) < 1e-5, (ours, ref)

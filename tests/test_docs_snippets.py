"""The two scripts of ``docs/USER_GUIDE.md`` run as written: the single-process one in-process, the multi-process one on
two gloo ranks under ``torch.distributed.run``."""
import re
import subprocess
import sys
from pathlib import Path

from tests.dist_utils import free_port

ROOT = Path(__file__).resolve().parents[1]


def _python_blocks():
    text = (ROOT / "docs" / "USER_GUIDE.md").read_text(encoding="utf-8")
    return re.findall(r"```python\n(.*?)```", text, flags=re.S)


def test_single_process_script_of_the_guide_runs(tmp_path):
    blocks = _python_blocks()
    assert len(blocks) == 2
    script = tmp_path / "guide_single.py"
    script.write_text(blocks[0])
    out = subprocess.run([sys.executable, str(script)], cwd=ROOT, capture_output=True, text=True, timeout=300,
                         env={"PYTHONPATH": str(ROOT), "PATH": "/usr/bin:/bin", "OMP_NUM_THREADS": "1"})
    assert out.returncode == 0, out.stderr[-2000:]
    steps = [l for l in out.stdout.splitlines() if l.startswith("[step")]
    assert [l.split("]")[0] for l in steps] == ["[step 00002", "[step 00004", "[step 00006"]


def test_multi_process_script_of_the_guide_runs(tmp_path):
    script = tmp_path / "guide_multi.py"
    script.write_text(_python_blocks()[1].replace("CHECKPOINT_DIR", repr(str(tmp_path / "ckpt"))))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), str(script)]
    import os

    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", GLOO_SOCKET_IFNAME="lo"))
    assert out.returncode == 0, (out.stdout + out.stderr)[-3000:]
    assert "[step 00004]" in out.stdout
    written = sorted(p.name for p in (tmp_path / "ckpt" / "step_00000004").iterdir())
    assert written == ["manifest.json", "model_rank_0.pt", "model_rank_1.pt", "optim_rank_0.pt", "optim_rank_1.pt",
                       "trainer_rank_0.pt", "trainer_rank_1.pt"]

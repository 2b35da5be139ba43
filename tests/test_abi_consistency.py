"""Static check of the Python <-> C boundary: every ``mb_*`` entry point that Python calls is exported by a ``csrc/*.cu``
file, and every call passes exactly as many arguments as the C prototype declares (ctypes would not notice a mismatch:
a missing trailing argument becomes whatever is in the register)."""
import ast
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "maltos_b200"


def _c_prototypes() -> dict[str, int]:
    protos = {}
    for src in sorted((PKG / "csrc").glob("*.cu")):
        text = re.sub(r"//[^\n]*", "", src.read_text(encoding="utf-8"))
        for m in re.finditer(r"MB_API\s+[\w\s\*]+?\b(mb_\w+)\s*\(([^)]*)\)\s*\{", text, flags=re.S):
            params = m.group(2).strip()
            protos[m.group(1)] = 0 if params in ("", "void") else len([p for p in params.split(",") if p.strip()])
    return protos


def _python_calls():
    calls = []
    for py in sorted(PKG.rglob("*.py")) + [ROOT / "bench.py", ROOT / "__graft_entry__.py"]:
        tree = ast.parse(py.read_text(encoding="utf-8"))
        for node in ast.walk(tree):
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr.startswith("mb_"):
                if any(isinstance(a, ast.Starred) for a in node.args):
                    continue
                calls.append((py.relative_to(ROOT), node.lineno, node.func.attr, len(node.args)))
    return calls


def test_every_called_entry_point_exists_with_the_same_number_of_arguments():
    protos = _c_prototypes()
    assert len(protos) >= 40, sorted(protos)
    calls = _python_calls()
    assert len(calls) >= 40
    problems = []
    for path, line, name, nargs in calls:
        if name not in protos:
            problems.append(f"{path}:{line}: {name} is not exported by any csrc/*.cu")
        elif protos[name] != nargs:
            problems.append(f"{path}:{line}: {name} called with {nargs} arguments, the C prototype has {protos[name]}")
    assert not problems, "\n".join(problems)


def test_probe_only_entry_points_are_not_called_from_the_package():
    called = {name for _, _, name, _ in _python_calls()}
    assert not called & {"mb_gemm_set_trace", "mb_gemm_set_debug_mode", "mb_gemm_set_debug_stages", "mb_gemm_set_debug_max_pairs",
                         "mb_gemm_debug_descriptor", "mb_flash_probe_read", "mb_pull_probe_read"}


def test_every_polling_loop_in_the_kernels_has_a_deadline_and_nothing_traps():
    """A wait on an mbarrier, a flag or a peer must give up after a time limit and report through the status words (a
    hung kernel takes the GPU with it): every open-ended loop that polls has a ``globaltimer`` deadline within its body,
    and no kernel source uses ``__trap()`` or a device ``assert``."""
    import re

    polls = re.compile(r"try_wait|ld_acquire|acquire_sys|x_tag\[|volatile")
    opened = re.compile(r"\bwhile\s*\((?!0\))")
    checked = 0
    csrc = ROOT / "maltos_b200" / "csrc"
    for path in sorted(csrc.glob("*.cu")) + sorted(csrc.glob("*.cuh")) + sorted(csrc.glob("*.h")):
        lines = path.read_text().splitlines()
        for i, line in enumerate(lines):
            code = line.split("//")[0]
            assert "__trap" not in code, (path.name, i + 1)
            assert not re.search(r"(?<!static_)\bassert\s*\(", code), (path.name, i + 1)
            if not opened.search(code):
                continue
            body = "\n".join(l.split("//")[0] for l in lines[i:i + 14])
            if not polls.search(body):
                continue                 # a host loop or a search over indices
            checked += 1
            assert re.search(r"globaltimer_ns\(\)\s*-\s*t0\s*>\s*limit", body), f"{path.name}:{i + 1}: polling loop without a deadline"
    assert checked >= 4


def test_no_source_names_a_multicast_bulk_load_or_a_batched_memcpy_call():
    """Two things this code base must never contain: a TMA / bulk LOAD with the cluster-multicast qualifier (``tcgen05.commit`` with
    that qualifier is a barrier arrive, not a load, and is used by the CTA-pair GEMM), and the batched memcpy entry points of
    the CUDA runtime / driver (built from pieces here so that this file does not name them either)."""
    batched = [a + "Memcpy" + b + "Batch" + "Async" for a in ("cuda", "cu") for b in ("", "3D")]
    for path in sorted(ROOT.rglob("*")):
        if path.suffix not in (".py", ".cu", ".cuh", ".h", ".cpp", ".sh", ".yaml") or any(part in ("_work", "baseline", "gpurun_out", ".git") for part in path.parts):
            continue
        text = path.read_text(errors="ignore")
        for name in batched:
            assert name not in text, (path, name)
        needle = "multicast" + "::cluster"
        for i, line in enumerate(text.splitlines()):
            if needle in line:
                assert "cp.async" + ".bulk" not in line and "tcgen05.commit" in line, (path, i + 1)

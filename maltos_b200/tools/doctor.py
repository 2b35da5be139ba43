"""``python -m maltos_b200.tools.doctor``: what this installation can do, in one screen.

Checks, in order: the Python side (torch, its CUDA and NCCL versions), the kernel library (present? newer than every
source it was built from? does it load and export the entry points the package calls?), the devices (sm_100 parts, memory,
peer access between every pair - the one-sided kernels need it inside a tensor / expert / context-parallel group), and the
switches set in the environment. Exit code 0 when everything a CUDA run needs is in place, or when there is no CUDA device
and the CPU paths are all there is; 1 when a CUDA device is present but the library is missing, stale or incomplete.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import re
import sys
from pathlib import Path


def _called_entry_points(package_root: Path) -> set[str]:
    names: set[str] = set()
    for path in package_root.rglob("*.py"):
        names |= set(re.findall(r"\.\s*(mb_[a-z0-9_]+)\s*\(", path.read_text(encoding="utf-8")))
    return names


def collect() -> dict:
    import torch

    from maltos_b200 import build as build_mod

    report: dict = {"python": sys.version.split()[0], "torch": torch.__version__, "torch_cuda": torch.version.cuda}
    try:
        report["nccl"] = ".".join(str(v) for v in torch.cuda.nccl.version())
    except Exception as exc:  # noqa: BLE001 - a build without NCCL
        report["nccl"] = f"unavailable ({type(exc).__name__})"
    lib = build_mod.LIB_PATH
    sources = sorted(build_mod.CSRC.glob("*.cu")) + sorted(build_mod.CSRC.glob("*.cuh")) + sorted(build_mod.CSRC.glob("*.h"))
    library = {"path": str(lib), "present": lib.exists(), "sources": len(sources)}
    if lib.exists():
        newer = [s.name for s in sources if s.stat().st_mtime > lib.stat().st_mtime]
        library["stale_against"] = newer
        try:
            handle = ctypes.CDLL(str(lib))
            wanted = sorted(_called_entry_points(build_mod.PKG_DIR))
            library["entry_points_called"] = len(wanted)
            library["entry_points_missing"] = [n for n in wanted if not hasattr(handle, n)]
            library["loads"] = True
        except OSError as exc:
            library["loads"] = False
            library["load_error"] = str(exc)
    report["library"] = library
    devices = []
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            devices.append({"index": i, "name": p.name, "capability": f"{p.major}.{p.minor}", "memory_gib": round(p.total_memory / 2**30, 1),
                            "sms": p.multi_processor_count})
        report["peer_access"] = [[bool(i == j or torch.cuda.can_device_access_peer(i, j)) for j in range(n)] for i in range(n)]
    report["devices"] = devices
    report["switches"] = {k: v for k, v in sorted(os.environ.items()) if k.startswith("MALTOS_B200_")}
    problems = []
    if devices:
        if any(d["capability"] != "10.0" for d in devices):
            problems.append("a visible device is not sm_100: the kernels are built for sm_100a only")
        if not library["present"]:
            problems.append("kernel library missing: run `python -m maltos_b200.build`")
        elif not library.get("loads"):
            problems.append(f"kernel library does not load: {library.get('load_error')}")
        else:
            if library["stale_against"]:
                problems.append(f"kernel library is older than {library['stale_against']}: run `python -m maltos_b200.build`")
            if library["entry_points_missing"]:
                problems.append(f"kernel library lacks {library['entry_points_missing']}: rebuild it")
        if "peer_access" in report and not all(all(row) for row in report["peer_access"]):
            problems.append("no peer access between some devices: groups that span them use NCCL instead of the one-sided kernels")
    report["problems"] = problems
    report["mode"] = "cuda" if devices else "cpu only (fp32 restatements, gloo)"
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--json", action="store_true", help="print the report as one JSON object")
    args = ap.parse_args(argv)
    report = collect()
    if args.json:
        print(json.dumps(report))
    else:
        lib = report["library"]
        print(f"python {report['python']}  torch {report['torch']}  cuda {report['torch_cuda']}  nccl {report['nccl']}")
        print(f"library {lib['path']}: " + ("missing" if not lib["present"] else
              f"present, loads={lib.get('loads')}, stale against {lib.get('stale_against') or 'nothing'}, "
              f"{lib.get('entry_points_called', 0) - len(lib.get('entry_points_missing', []))}/{lib.get('entry_points_called', 0)} entry points"))
        for d in report["devices"]:
            print(f"  cuda:{d['index']} {d['name']} sm_{d['capability'].replace('.', '')} {d['memory_gib']} GiB {d['sms']} SMs")
        if "peer_access" in report:
            print("  peer access: " + ("all pairs" if all(all(r) for r in report["peer_access"]) else json.dumps(report["peer_access"])))
        print(f"mode: {report['mode']}")
        for k, v in report["switches"].items():
            print(f"  {k}={v}")
        for p in report["problems"]:
            print(f"PROBLEM: {p}")
    fatal = [p for p in report["problems"] if not p.startswith("no peer access")]
    return 1 if fatal else 0


if __name__ == "__main__":
    sys.exit(main())

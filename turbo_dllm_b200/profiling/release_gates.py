"""Release gates: source-policy checks that must hold before a build is published.

* single_trainer        – exactly one module defines the training step loop
* no_config_aliases     – only `config.run_spec` parses train.yaml
* no_sys_path_mutation  – package code never edits sys.path
* sm100_only_flags      – every nvcc invocation targets compute_100a/sm_100a
* no_compat_layers      – no Triton / tilelang / torch.compile on package code paths
* bounded_device_waits  – no `__trap`, device `assert(` or unbounded `while (true)` without the
                          library's bounded-wait helpers in CUDA sources
* native_manifest       – the in-tree kernel binary matches its manifest (when built)
* no_cluster_broadcast_loads – no cluster-broadcast qualifier on any bulk/tensor load in CUDA sources

`dllm-release-gate` prints one JSON report and exits 1 when a gate fails.
Counterpart of dllm_parallel/core/profiling/release_gates.py:26-635.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from dataclasses import dataclass
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent


@dataclass
class GateResult:
    name: str
    ok: bool
    detail: str = ""


def _py_files():
    return [p for p in PKG.rglob("*.py") if "__pycache__" not in p.parts]


def _cu_files():
    return list((PKG / "csrc").glob("*.cu")) + list((PKG / "csrc").glob("*.cuh")) + list((PKG / "csrc").glob("*.h"))


def gate_single_trainer() -> GateResult:
    hits = [str(p.relative_to(PKG)) for p in _py_files() if re.search(r"^def run_training\(", p.read_text(), re.M)]
    return GateResult("single_trainer", hits == ["training/trainer.py"], f"step loop defined in {hits}")


def gate_no_config_aliases() -> GateResult:
    hits = [str(p.relative_to(PKG)) for p in _py_files()
            if re.search(r"^def load_run_spec\(", p.read_text(), re.M)]
    return GateResult("no_config_aliases", hits == ["config/run_spec.py"], f"loaders: {hits}")


def gate_no_sys_path_mutation() -> GateResult:
    hits = [str(p.relative_to(PKG)) for p in _py_files() if re.search(r"sys\.path\.(insert|append)", p.read_text())
            and p.name != "release_gates.py"]
    return GateResult("no_sys_path_mutation", not hits, f"offenders: {hits}")


def gate_sm100_only_flags() -> GateResult:
    text = (PKG / "kernels" / "build.py").read_text()
    archs = set(re.findall(r"arch=compute_(\w+),code=sm_(\w+)", text))
    return GateResult("sm100_only_flags", archs == {("100a", "100a")}, f"arch flags: {sorted(archs)}")


# the one place a tracing compiler may appear: the stock-PyTorch baseline column of the attention benchmark,
# which times FlexAttention next to this library's kernels and is called by nothing in the package
BASELINE_ONLY = {"benchmarks/attention_bench.py"}


def gate_no_compat_layers() -> GateResult:
    pat = re.compile(r"^\s*(import triton|from triton|import tilelang|from tilelang)|torch\.compile\(", re.M)
    hits = [str(p.relative_to(PKG)) for p in _py_files() if pat.search(p.read_text()) and p.name != "release_gates.py"
            and str(p.relative_to(PKG)) not in BASELINE_ONLY]
    return GateResult("no_compat_layers", not hits, f"offenders: {hits}")


def gate_bounded_device_waits() -> GateResult:
    bad = []
    for p in _cu_files():
        t = p.read_text()
        if re.search(r"__trap\s*\(|\bassert\s*\(", t):
            bad.append(f"{p.name}: trap/assert")
        for m in re.finditer(r"while\s*\(\s*(true|1)\s*\)", t):
            window = t[m.start(): m.start() + 600]
            if "budget" not in window and "globaltimer" not in window:
                bad.append(f"{p.name}: unbounded loop at offset {m.start()}")
    return GateResult("bounded_device_waits", not bad, "; ".join(bad))


def gate_no_cluster_broadcast_loads() -> GateResult:
    """No bulk / tensor LOAD (`cp.async.bulk…`) may carry the cluster-broadcast qualifier. The qualifier on
    `tcgen05.commit` (an mbarrier arrival in both CTAs of a pair, no memory is loaded) is allowed."""
    needle = "multi" + "cast"
    bad = []
    for p in _cu_files():
        for n, line in enumerate(p.read_text().splitlines(), 1):
            if needle in line and "cp.async.bulk" in line:
                bad.append(f"{p.name}:{n}")
            elif needle in line and "tcgen05.commit" not in line:
                bad.append(f"{p.name}:{n} (outside a tcgen05.commit)")
    return GateResult("no_cluster_broadcast_loads", not bad, f"offenders: {bad}")


def gate_native_manifest() -> GateResult:
    from ..kernels import native

    if not native.library_path().exists():
        return GateResult("native_manifest", True, "library not built (source tree)")
    problems = native.verify_packaged_kernels()
    return GateResult("native_manifest", not problems, "; ".join(problems))


GATES = [gate_single_trainer, gate_no_config_aliases, gate_no_sys_path_mutation, gate_sm100_only_flags,
         gate_no_compat_layers, gate_bounded_device_waits, gate_no_cluster_broadcast_loads, gate_native_manifest]


def run_gates() -> list[GateResult]:
    return [g() for g in GATES]


def main(argv=None) -> int:
    argparse.ArgumentParser(prog="dllm-release-gate").parse_args(argv)
    res = run_gates()
    print(json.dumps({"ok": all(r.ok for r in res), "gates": [r.__dict__ for r in res]}, indent=1))
    return 0 if all(r.ok for r in res) else 1


if __name__ == "__main__":
    raise SystemExit(main())

"""Checks of built distributions (wheel / sdist) before they are published.

A *portable* artifact (what goes to a package index) must contain the package's sources, recipes and kernel
sources and must NOT contain native binaries or machine-specific paths; a *gpu* artifact (the sm_100a wheel
attached to a release) must additionally carry the kernel library and the manifest that pins it.

    python -m turbo_dllm_b200.profiling.portable_artifacts --kind portable dist/*.whl dist/*.tar.gz

Counterpart of dllm_parallel/core/profiling/portable_artifacts.py:14-117.
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import tarfile
import zipfile
from dataclasses import dataclass, field

REQUIRED_SUFFIXES = (
    "turbo_dllm_b200/__init__.py", "turbo_dllm_b200/config/schema.py", "turbo_dllm_b200/training/trainer.py",
    "turbo_dllm_b200/cli/main.py", "turbo_dllm_b200/recipes/manifest.yaml", "turbo_dllm_b200/csrc/api.h",
    "turbo_dllm_b200/csrc/gemm_sm100.cu", "turbo_dllm_b200/kernels/build.py",
)
GPU_REQUIRED_SUFFIXES = ("turbo_dllm_b200/_C/libtdllm_kernels.so", "turbo_dllm_b200/_C/native_kernels.json")
BINARY_SUFFIXES = (".so", ".o", ".a", ".cubin", ".fatbin", ".pyd", ".dll", ".dylib")
# text that must not travel: build-machine paths and work-in-progress markers
FORBIDDEN_TOKENS = (re.compile(rb"/home/[a-z0-9_]+/"), re.compile(rb"/root/[a-zA-Z0-9_]+"), re.compile(rb"_work/"))
TEXT_SUFFIXES = (".py", ".yaml", ".yml", ".toml", ".md", ".cu", ".cuh", ".h", ".sh", ".json", ".txt")


@dataclass
class ArtifactReport:
    path: str
    kind: str
    files: int = 0
    problems: list[str] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return not self.problems


def _members(path: str):
    """(name, reader) pairs of a wheel (zip) or an sdist (tar.gz)."""
    if path.endswith(".whl") or path.endswith(".zip"):
        with zipfile.ZipFile(path) as z:
            for n in z.namelist():
                if not n.endswith("/"):
                    yield n, z.read(n)
    elif path.endswith(".tar.gz") or path.endswith(".tgz"):
        with tarfile.open(path, "r:gz") as t:
            for m in t.getmembers():
                if m.isfile():
                    yield m.name, t.extractfile(m).read()
    else:
        raise ValueError(f"{path}: not a wheel or an sdist")


def check_artifact(path: str, kind: str = "portable") -> ArtifactReport:
    if kind not in ("portable", "gpu"):
        raise ValueError("kind must be 'portable' or 'gpu'")
    rep = ArtifactReport(path, kind)
    names = []
    for name, data in _members(path):
        names.append(name)
        rep.files += 1
        if name.endswith(BINARY_SUFFIXES) and not (kind == "gpu" and name.endswith(GPU_REQUIRED_SUFFIXES[0])):
            rep.problems.append(f"native binary in a {kind} artifact: {name}")
        if name.endswith(TEXT_SUFFIXES):
            for pat in FORBIDDEN_TOKENS:
                m = pat.search(data)
                if m:
                    rep.problems.append(f"{name}: forbidden token {m.group(0)[:40]!r}")
                    break
    for suffix in REQUIRED_SUFFIXES + (GPU_REQUIRED_SUFFIXES if kind == "gpu" else ()):
        if not any(n.endswith(suffix) for n in names):
            rep.problems.append(f"required file missing: {suffix}")
    return rep


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m turbo_dllm_b200.profiling.portable_artifacts")
    ap.add_argument("--kind", choices=("portable", "gpu"), default="portable")
    ap.add_argument("artifacts", nargs="+")
    a = ap.parse_args(argv)
    reports = [check_artifact(p, a.kind) for p in a.artifacts]
    print(json.dumps([{"path": r.path, "kind": r.kind, "files": r.files, "ok": r.ok, "problems": r.problems}
                      for r in reports], indent=1))
    return 0 if all(r.ok for r in reports) else 1


if __name__ == "__main__":
    sys.exit(main())

"""Ahead-of-time build of the sm_100a kernel library (`dllm-build-kernels`).

Compiles every `csrc/*.cu` with nvcc for `compute_100a/sm_100a` (relocatable device code, one
object per source, in parallel), links `_C/libtdllm_kernels.so` in-tree and writes
`_C/native_kernels.json` with source/binary hashes, flags and toolchain versions, so that the
runtime can refuse a stale or foreign binary.

Reference counterpart: dllm_parallel/core/kernels/build.py:38-108 (AOT build + manifest) and
dllm_parallel/core/kernels/_native_specs.py:46-143 (sources, flags); the reference goes through
torch cpp_extension and TORCH_CUDA_ARCH_LIST, this build calls nvcc directly because the
library has a plain C ABI and no torch dependency.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import json
import os
import shutil
import subprocess
import sys
import time
from pathlib import Path

PKG_ROOT = Path(__file__).resolve().parent.parent
CSRC = PKG_ROOT / "csrc"
OUT_DIR = PKG_ROOT / "_C"
LIB_NAME = "libtdllm_kernels.so"
MANIFEST_NAME = "native_kernels.json"
# the checked variant (-DTDLLM_KERNEL_CHECKS: index checks that record instead of accessing) lives beside the
# regular library and is loaded when DLLM_KERNEL_CHECKS=1
CHECKED_LIB_NAME = "libtdllm_kernels_checked.so"
CHECKED_MANIFEST_NAME = "native_kernels_checked.json"
CHECK_FLAGS = ["-DTDLLM_KERNEL_CHECKS=1"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-rdc=true",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


def find_nvcc() -> str:
    cand = os.environ.get("TDLLM_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: set TDLLM_NVCC or put nvcc on PATH")
    return cand


INCLUDED_ONLY = {"attention_bwd_dq_sm100.cu", "attention_bwd_dkv_sm100.cu", "attention_bwd_fused_sm100.cu"}  # pulled in by attention_bwd_host.cu


def sources() -> list[Path]:
    return [p for p in sorted(CSRC.glob("*.cu")) if p.name not in INCLUDED_ONLY]


def all_source_files() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _sha256(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def source_hashes() -> dict[str, str]:
    return {f.name: _sha256(f) for f in all_source_files()}


def checks_requested() -> bool:
    return os.environ.get("DLLM_KERNEL_CHECKS", os.environ.get("TDLLM_KERNEL_CHECKS", "0")) == "1"


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool, extra: tuple = ()) -> tuple[str, str]:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-Xptxas", "-v", "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return src.name, proc.stderr


def is_current(checks: bool = False) -> bool:
    man = OUT_DIR / (CHECKED_MANIFEST_NAME if checks else MANIFEST_NAME)
    lib = OUT_DIR / (CHECKED_LIB_NAME if checks else LIB_NAME)
    if not man.exists() or not lib.exists():
        return False
    try:
        data = json.loads(man.read_text())
    except Exception:
        return False
    return data.get("sources") == source_hashes() and data.get("binary_sha256") == _sha256(lib)


def build(force: bool = False, verbose: bool = False, checks: bool = False) -> Path:
    """Builds the library if sources changed (or `force`). Returns the path of the .so. `checks` builds the
    checked variant (its own objects, library and manifest; the regular build is untouched)."""
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    lib = OUT_DIR / (CHECKED_LIB_NAME if checks else LIB_NAME)
    if not force and is_current(checks):
        return lib
    nvcc = find_nvcc()
    obj_dir = OUT_DIR / ("obj_checked" if checks else "obj")
    extra = tuple(CHECK_FLAGS) if checks else ()
    obj_dir.mkdir(exist_ok=True)
    t0 = time.time()
    srcs = sources()
    ptxas: dict[str, str] = {}
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        futs = [ex.submit(_compile_one, nvcc, s, obj_dir / (s.stem + ".o"), verbose, extra) for s in srcs]
        for f in futs:
            name, log = f.result()
            ptxas[name] = log
    objs = [str(obj_dir / (s.stem + ".o")) for s in srcs]
    link = [nvcc, *ARCH_FLAGS, "-shared", "-Xcompiler", "-fPIC", "-o", str(lib), *objs]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    ver = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout.strip().splitlines()[-1]
    manifest = {
        "format": "turbo_dllm_b200.native_kernels.v1",
        "library": lib.name,
        "arch": "sm_100a",
        "flags": ARCH_FLAGS + NVCC_FLAGS + list(extra),
        "kernel_checks": bool(checks),
        "nvcc": ver,
        "sources": source_hashes(),
        "binary_sha256": _sha256(lib),
        "built_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
        "build_seconds": round(time.time() - t0, 2),
    }
    (OUT_DIR / (CHECKED_MANIFEST_NAME if checks else MANIFEST_NAME)).write_text(json.dumps(manifest, indent=1, sort_keys=True))
    (OUT_DIR / ("ptxas_checked.log" if checks else "ptxas.log")).write_text("\n".join(f"== {k}\n{v}" for k, v in ptxas.items()))
    if verbose:
        print((OUT_DIR / ("ptxas_checked.log" if checks else "ptxas.log")).read_text())
    return lib


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="dllm-build-kernels", description=__doc__.splitlines()[0])
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/spill report")
    ap.add_argument("--checks", action="store_true",
                    help="build the checked variant (-DTDLLM_KERNEL_CHECKS), loaded when DLLM_KERNEL_CHECKS=1")
    args = ap.parse_args(argv)
    try:
        lib = build(force=args.force, verbose=args.verbose, checks=args.checks)
    except RuntimeError as e:
        print(str(e), file=sys.stderr)
        return 2
    print(json.dumps({"library": str(lib), "current": is_current(args.checks), "kernel_checks": args.checks}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

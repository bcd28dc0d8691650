"""Release automation for the sm_100a wheel: manifest with hashes, artifact checks, software bill of materials.

    python packaging/release.py manifest --dist dist --out dist/release_manifest.json
    python packaging/release.py verify   --manifest dist/release_manifest.json
    python packaging/release.py sbom     --out dist/sbom.json

`manifest` records every file of `dist/` (name, bytes, SHA-256), the bundle key (`gpu-sm100a-cu129-cp312`), the
toolchain and the kernel library's own manifest; `verify` re-hashes the files and runs the artifact checks;
`sbom` lists the Python distributions the package imports with their installed versions. Publication order for
a release is: wheels first, the bundle catalog entry last (an installer that reads the catalog never sees a
half-uploaded bundle). Counterpart of the reference's release scripts (.github/scripts/gpu_release.py:19-460,
publish_gpu_assets.py:21-75, scripts/verify/gpu_release_assets.py:28-90).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
BUNDLE_KEY = "gpu-sm100a-cu129-cp312"


def sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for c in iter(lambda: f.read(1 << 20), b""):
            h.update(c)
    return h.hexdigest()


def build_manifest(dist: str) -> dict:
    from turbo_dllm_b200 import __version__

    files = []
    for name in sorted(os.listdir(dist)):
        p = os.path.join(dist, name)
        if os.path.isfile(p) and name != "release_manifest.json":
            files.append({"name": name, "bytes": os.path.getsize(p), "sha256": sha256(p)})
    kernels = None
    man = os.path.join(ROOT, "turbo_dllm_b200", "_C", "native_kernels.json")
    if os.path.exists(man):
        kernels = json.load(open(man))
    return {"format": "turbo_dllm_b200.release_manifest.v1", "bundle": BUNDLE_KEY, "version": __version__,
            "created_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "files": files,
            "native_kernels": kernels, "publication_order": ["wheels", "release_manifest.json", "bundle catalog"]}


def verify(manifest_path: str) -> list[str]:
    from turbo_dllm_b200.profiling.portable_artifacts import check_artifact

    man = json.load(open(manifest_path))
    base = os.path.dirname(os.path.abspath(manifest_path))
    problems = []
    if man.get("format") != "turbo_dllm_b200.release_manifest.v1":
        problems.append(f"unexpected manifest format {man.get('format')!r}")
    for f in man.get("files", []):
        p = os.path.join(base, f["name"])
        if not os.path.exists(p):
            problems.append(f"missing {f['name']}")
        elif sha256(p) != f["sha256"]:
            problems.append(f"{f['name']}: SHA-256 differs from the manifest")
        elif f["name"].endswith(".whl"):
            problems += [f"{f['name']}: {x}" for x in check_artifact(p, "gpu" if "sm100" in man["bundle"] else "portable").problems]
    return problems


def sbom() -> dict:
    from importlib import metadata

    wanted = ("torch", "numpy", "pyyaml", "einops", "safetensors", "transformers", "wandb")
    comps = []
    for name in wanted:
        try:
            comps.append({"name": name, "version": metadata.version(name)})
        except metadata.PackageNotFoundError:
            comps.append({"name": name, "version": None})
    return {"format": "turbo_dllm_b200.sbom.v1", "components": comps, "python": sys.version.split()[0]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="packaging/release.py")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("manifest")
    p.add_argument("--dist", default="dist")
    p.add_argument("--out")
    p = sub.add_parser("verify")
    p.add_argument("--manifest", required=True)
    p = sub.add_parser("sbom")
    p.add_argument("--out")
    a = ap.parse_args(argv)
    if a.cmd == "manifest":
        m = build_manifest(a.dist)
        text = json.dumps(m, indent=1, sort_keys=True)
        open(a.out, "w").write(text) if a.out else print(text)
        return 0
    if a.cmd == "verify":
        problems = verify(a.manifest)
        print(json.dumps({"ok": not problems, "problems": problems}, indent=1))
        return 0 if not problems else 1
    s = sbom()
    text = json.dumps(s, indent=1)
    open(a.out, "w").write(text) if a.out else print(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

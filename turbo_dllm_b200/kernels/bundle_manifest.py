"""GPU bundle catalog: coordinated binary wheels per (python, cuda, torch, arch).

A catalog (JSON, `format: dllm.gpu_bundle_catalog.v1`) lists bundles; each bundle names its
environment key and a list of wheel assets with URL and SHA-256. `detect_environment()` reads the
running interpreter / torch / CUDA / device capability, `select_bundle` picks the matching entry,
`install_bundle` downloads (or copies from a local path), verifies the hashes and calls pip.
This framework ships one wheel family (`turbo-dllm-b200`, sm_100a); the machinery still takes an
arbitrary catalog so mirrors and future architectures work.

Counterpart of dllm_parallel/core/kernels/bundle_manifest.py:42-620.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import urllib.request

CATALOG_FORMAT = "dllm.gpu_bundle_catalog.v1"


class BundleError(RuntimeError):
    pass


def detect_environment() -> dict:
    env = {"python": f"cp{sys.version_info.major}{sys.version_info.minor}", "platform": sys.platform}
    try:
        import torch

        env["torch"] = torch.__version__.split("+")[0]
        env["cuda"] = (torch.version.cuda or "").replace(".", "")
        if torch.cuda.is_available():
            major, minor = torch.cuda.get_device_capability()
            env["arch"] = f"sm{major}{minor}"
    except ImportError:
        env["torch"] = None
    return env


def bundle_key(env: dict) -> str:
    return f"gpu-{env.get('arch', 'sm100')}-cu{env.get('cuda', '')}-{env.get('python', '')}"


def load_catalog(path_or_url: str | None) -> dict:
    if not path_or_url:
        raise BundleError("no bundle catalog given (--catalog PATH_OR_URL)")
    if os.path.exists(path_or_url):
        data = json.load(open(path_or_url))
    else:
        with urllib.request.urlopen(path_or_url, timeout=30) as r:   # noqa: S310 (user-supplied catalog URL)
            data = json.load(r)
    if data.get("format") != CATALOG_FORMAT:
        raise BundleError(f"unexpected catalog format {data.get('format')!r}")
    return data


def select_bundle(catalog: dict, env: dict | None = None) -> dict:
    env = env or detect_environment()
    key = bundle_key(env)
    for b in catalog.get("bundles", []):
        if b.get("key") == key:
            return b
    raise BundleError(f"catalog has no bundle for {key}; available: {[b.get('key') for b in catalog.get('bundles', [])]}")


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def fetch_asset(asset: dict, dest_dir: str) -> str:
    name = asset["name"]
    out = os.path.join(dest_dir, name)
    src = asset["url"]
    if os.path.exists(src):
        shutil.copyfile(src, out)
    else:
        with urllib.request.urlopen(src, timeout=120) as r, open(out, "wb") as f:   # noqa: S310
            shutil.copyfileobj(r, f)
    got = _sha256(out)
    if got != asset["sha256"]:
        os.unlink(out)
        raise BundleError(f"{name}: sha256 {got} differs from catalog {asset['sha256']}")
    return out


def install_bundle(catalog_path: str | None, dry_run: bool = False, pip_runner=None) -> int:
    catalog = load_catalog(catalog_path)
    bundle = select_bundle(catalog)
    print(json.dumps({"bundle": bundle["key"], "assets": [a["name"] for a in bundle["assets"]], "dry_run": dry_run}))
    if dry_run:
        return 0
    with tempfile.TemporaryDirectory() as td:
        wheels = [fetch_asset(a, td) for a in bundle["assets"]]
        run = pip_runner or (lambda cmd: subprocess.run(cmd).returncode)
        return run([sys.executable, "-m", "pip", "install", "--no-deps", *wheels])

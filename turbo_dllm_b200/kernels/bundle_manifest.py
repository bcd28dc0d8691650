"""GPU bundle catalog: coordinated binary wheels per (python, cuda, torch, arch).

A catalog (JSON, `format: dllm.gpu_bundle_catalog.v1`) lists bundles; each bundle names its
environment key and a list of wheel assets with URL and SHA-256. `detect_environment()` reads the
running interpreter / torch / CUDA / device capability, `select_bundle` picks the matching entry,
`install_bundle` downloads (or copies from a local path), verifies the hashes and calls pip.
This framework ships one wheel family (`turbo-dllm-b200`, sm_100a); the machinery still takes an
arbitrary catalog so mirrors and future architectures work.

A bundle also has a manifest of its own (`format: dllm.gpu_bundle.v1`): package version, source revision, Python
ABI, platform, CUDA version, the compute capabilities its kernels were built for, and per wheel name / URL / size /
SHA-256. `create_bundle_manifest` writes one from built wheels, `validate_bundle_manifest` checks the schema (wheel
file names, HTTPS URLs whose last component is the wheel name, hash and size formats, no duplicates) and the host
(`BundleEnvironment`), `create_bundle_catalog` collects the manifests of a release, `resolve_bundle` picks the
manifest for a host from a catalog, and the module's CLI drives all of it.

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
BUNDLE_FORMAT = "dllm.gpu_bundle.v1"
DISTRIBUTION = "turbo_dllm_b200"
MAX_JSON_BYTES = 4 << 20


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


# ------------------------------------------------------------------ per-bundle manifests
import re
from dataclasses import asdict, dataclass
from pathlib import PurePosixPath
from urllib.parse import urlparse

_SHA = re.compile(r"^[0-9a-f]{64}$")
_REV = re.compile(r"^[0-9a-f]{7,40}$")


@dataclass(frozen=True)
class BundleEnvironment:
    package_version: str
    python_abi: str
    platform: str
    cuda: str
    compute_capability: str


def detect_bundle_environment() -> BundleEnvironment:
    """Python ABI, platform, CUDA runtime and the first visible GPU of this host."""
    import platform as _platform

    if sys.platform != "linux":
        raise BundleError("GPU bundles are built for Linux")
    try:
        import torch
    except ImportError as e:
        raise BundleError("PyTorch must be installed before a GPU bundle") from e
    if not torch.cuda.is_available() or torch.version.cuda is None:
        raise BundleError("a visible CUDA GPU and a CUDA build of PyTorch are required")
    from .. import __version__

    major, minor = torch.cuda.get_device_capability()
    return BundleEnvironment(__version__, f"cp{sys.version_info.major}{sys.version_info.minor}",
                             f"linux_{_platform.machine().lower()}", ".".join(torch.version.cuda.split(".")[:2]),
                             f"{major}.{minor}")


def _wheel_distribution(name: str) -> str:
    if PurePosixPath(name).name != name or not name.endswith(".whl") or name.count("-") < 4:
        raise BundleError(f"invalid wheel name: {name!r}")
    return name.split("-")[0].lower().replace(".", "_")


def create_bundle_manifest(wheels: list[str], *, package_version: str, source_revision: str, python_abi: str,
                           platform: str, cuda: str, architectures: list[str], base_url: str,
                           allow_local: bool = False) -> dict:
    """Manifest of one bundle from wheel files on disk; URLs are `base_url/<wheel name>` (HTTPS, or a file:// mirror
    with `allow_local`)."""
    artifacts = []
    for w in wheels:
        name = os.path.basename(w)
        _wheel_distribution(name)
        artifacts.append({"name": name, "url": f"{base_url.rstrip('/')}/{name}", "sha256": _sha256(w),
                          "size": os.path.getsize(w)})
    man = {"format": BUNDLE_FORMAT, "package_version": package_version, "source_revision": source_revision,
           "python_abi": python_abi, "platform": platform, "cuda": cuda, "architectures": sorted(architectures),
           "artifacts": artifacts}
    validate_bundle_schema(man, allow_local)
    return man


def validate_bundle_schema(man: dict, allow_local: bool = False) -> list[dict]:
    """Identity and artifact rules that need no GPU. Returns the artifacts."""
    if man.get("format") != BUNDLE_FORMAT:
        raise BundleError(f"unsupported bundle manifest format {man.get('format')!r}")
    if not _REV.match(str(man.get("source_revision", ""))):
        raise BundleError("bundle source_revision must be a git revision")
    archs = man.get("architectures")
    if not isinstance(archs, list) or not archs or not all(re.match(r"^\d+\.\d+a?$", str(a)) for a in archs):
        raise BundleError("bundle architectures must list compute capabilities such as '10.0'")
    arts = man.get("artifacts")
    if not isinstance(arts, list) or not arts:
        raise BundleError("bundle has no artifacts")
    names = set()
    for a in arts:
        if not isinstance(a, dict):
            raise BundleError("bundle artifact entries must be objects")
        name = str(a.get("name", ""))
        _wheel_distribution(name)
        if name in names:
            raise BundleError(f"duplicate wheel name: {name}")
        names.add(name)
        url = urlparse(str(a.get("url", "")))
        local = allow_local and url.scheme in ("", "file")
        if not local and (url.scheme != "https" or not url.netloc):
            raise BundleError(f"artifact URL must use HTTPS: {name}")
        if PurePosixPath(url.path).name != name:
            raise BundleError(f"artifact URL file name does not match {name}")
        if not _SHA.match(str(a.get("sha256", ""))):
            raise BundleError(f"invalid SHA-256 for {name}")
        if not isinstance(a.get("size"), int) or isinstance(a.get("size"), bool) or a["size"] <= 0:
            raise BundleError(f"invalid artifact size for {name}")
    if not any(_wheel_distribution(n) == DISTRIBUTION for n in names):
        raise BundleError(f"bundle does not carry the {DISTRIBUTION} wheel")
    return arts


def validate_bundle_manifest(man: dict, environment: BundleEnvironment | None = None, allow_local: bool = False) -> list[dict]:
    """Schema plus host compatibility: package version, Python ABI, platform, CUDA and compute capability."""
    arts = validate_bundle_schema(man, allow_local)
    host = environment or detect_bundle_environment()
    for label, have, want in (("package version", host.package_version, man.get("package_version")),
                              ("Python ABI", host.python_abi, man.get("python_abi")),
                              ("platform", host.platform, man.get("platform")), ("CUDA", host.cuda, man.get("cuda"))):
        if have != str(want):
            raise BundleError(f"GPU bundle {label} mismatch: host {have!r}, bundle {want!r}")
    caps = {str(a).rstrip("a") for a in man["architectures"]}
    if host.compute_capability not in caps:
        raise BundleError(f"GPU bundle compute capability mismatch: host {host.compute_capability!r}, bundle {sorted(caps)}")
    return arts


def create_bundle_catalog(release: str, manifests: list[dict], manifest_urls: list[str]) -> dict:
    """Catalog of a release: one entry per bundle manifest with the fields a host is matched on."""
    if len(manifests) != len(manifest_urls) or not manifests:
        raise BundleError("a catalog needs one URL per bundle manifest")
    entries, seen = [], set()
    for man, url in zip(manifests, manifest_urls):
        validate_bundle_schema(man, allow_local=True)
        ident = (man["python_abi"], man["platform"], man["cuda"], tuple(man["architectures"]))
        if ident in seen:
            raise BundleError(f"two bundles for {ident}")
        seen.add(ident)
        entries.append({"manifest_url": url, "package_version": man["package_version"], "python_abi": man["python_abi"],
                        "platform": man["platform"], "cuda": man["cuda"], "architectures": man["architectures"]})
    return {"format": CATALOG_FORMAT, "release": release, "bundle_manifests": entries, "bundles": []}


def read_json(source: str) -> dict:
    """A manifest or catalog from a path or URL, size-limited."""
    if os.path.exists(source):
        data = open(source, "rb").read(MAX_JSON_BYTES + 1)
    else:
        with urllib.request.urlopen(source, timeout=30) as r:   # noqa: S310 (user-supplied catalog URL)
            data = r.read(MAX_JSON_BYTES + 1)
    if len(data) > MAX_JSON_BYTES:
        raise BundleError(f"{source} is larger than {MAX_JSON_BYTES} bytes")
    return json.loads(data)


def resolve_bundle(catalog: dict, environment: BundleEnvironment | None = None, reader=read_json) -> dict:
    """The bundle manifest of `catalog` that fits this host (validated against it)."""
    host = environment or detect_bundle_environment()
    fits = [e for e in catalog.get("bundle_manifests", [])
            if e.get("python_abi") == host.python_abi and e.get("platform") == host.platform and e.get("cuda") == host.cuda
            and host.compute_capability in {str(a).rstrip("a") for a in e.get("architectures", [])}
            and e.get("package_version") == host.package_version]
    if not fits:
        have = [(e.get("python_abi"), e.get("cuda"), e.get("architectures")) for e in catalog.get("bundle_manifests", [])]
        raise BundleError(f"release {catalog.get('release')!r} has no bundle for {asdict(host)}; available: {have}")
    man = reader(fits[0]["manifest_url"])
    validate_bundle_manifest(man, host, allow_local=True)
    return man


def install_bundle_manifest(man: dict, environment: BundleEnvironment | None = None, dry_run: bool = False,
                            pip_runner=None, allow_local: bool = False) -> int:
    arts = validate_bundle_manifest(man, environment, allow_local)
    if dry_run:
        print(json.dumps({"artifacts": [a["name"] for a in arts], "dry_run": True}))
        return 0
    with tempfile.TemporaryDirectory() as td:
        wheels = []
        for a in arts:
            path = fetch_asset({"name": a["name"], "url": a["url"].removeprefix("file://"), "sha256": a["sha256"]}, td)
            if os.path.getsize(path) != a["size"]:
                raise BundleError(f"{a['name']}: size differs from the manifest")
            wheels.append(path)
        run = pip_runner or (lambda cmd: subprocess.run(cmd).returncode)
        return run([sys.executable, "-m", "pip", "install", "--no-deps", *wheels])


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="python -m turbo_dllm_b200.kernels.bundle_manifest")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("create", help="write the manifest of one bundle from built wheels")
    p.add_argument("wheels", nargs="+")
    for f in ("--package-version", "--source-revision", "--python-abi", "--platform", "--cuda", "--base-url", "--output"):
        p.add_argument(f, required=True)
    p.add_argument("--architectures", nargs="+", default=["10.0a"])
    p = sub.add_parser("catalog", help="collect bundle manifests into a release catalog")
    p.add_argument("--release", required=True)
    p.add_argument("--manifest", nargs=2, action="append", metavar=("PATH", "URL"), required=True)
    p.add_argument("--output", required=True)
    p = sub.add_parser("validate")
    p.add_argument("manifest")
    p.add_argument("--schema-only", action="store_true")
    p = sub.add_parser("install")
    p.add_argument("source", help="bundle manifest or release catalog (path or URL)")
    p.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    try:
        if a.cmd == "create":
            man = create_bundle_manifest(a.wheels, package_version=a.package_version, source_revision=a.source_revision,
                                         python_abi=a.python_abi, platform=a.platform, cuda=a.cuda,
                                         architectures=a.architectures, base_url=a.base_url)
            json.dump(man, open(a.output, "w"), indent=1)
        elif a.cmd == "catalog":
            cat = create_bundle_catalog(a.release, [read_json(p) for p, _ in a.manifest], [u for _, u in a.manifest])
            json.dump(cat, open(a.output, "w"), indent=1)
        elif a.cmd == "validate":
            man = read_json(a.manifest)
            (validate_bundle_schema if a.schema_only else validate_bundle_manifest)(man)
            print(json.dumps({"ok": True, "artifacts": len(man["artifacts"])}))
        else:
            doc = read_json(a.source)
            man = resolve_bundle(doc) if doc.get("format") == CATALOG_FORMAT else doc
            return install_bundle_manifest(man, dry_run=a.dry_run)
        return 0
    except (BundleError, OSError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    raise SystemExit(main())

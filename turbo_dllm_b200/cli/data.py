"""`dllm data prepare | inspect | validate | stats` (cf. dllm_parallel/cli/data.py:25-110)."""
from __future__ import annotations

import argparse
import json
import sys


def run_data(argv) -> int:
    from ..data.artifacts import ArtifactError, artifact_stats, load_manifest, validate_artifact
    from ..data.prepare import PreparationError, load_preparation_spec, prepare_dataset

    ap = argparse.ArgumentParser(prog="dllm data")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("prepare")
    p.add_argument("--config", required=True, help="prepare.yaml (format dllm.data.prepare.v1)")
    for name in ("inspect", "validate", "stats"):
        q = sub.add_parser(name)
        q.add_argument("path")
        if name == "validate":
            q.add_argument("--no-hashes", action="store_true")
    a = ap.parse_args(argv)
    try:
        if a.cmd == "prepare":
            m = prepare_dataset(load_preparation_spec(a.config))
            print(json.dumps({"format": m["format"], "samples": m["sample_count"], "tokens": m["token_count"],
                              "dataset_fingerprint": m["metadata"]["dataset_fingerprint"]}))
        elif a.cmd == "inspect":
            m = load_manifest(a.path)
            print(json.dumps({k: m[k] for k in ("format", "version", "created_at", "sample_count", "token_count",
                                                "files", "stats")}, indent=1))
            print(json.dumps({"metadata": m["metadata"]}, indent=1))
        elif a.cmd == "validate":
            m = validate_artifact(a.path, check_hashes=not a.no_hashes)
            print(json.dumps({"valid": True, "format": m["format"],
                              "dataset_fingerprint": m["metadata"]["dataset_fingerprint"]}))
        else:
            print(json.dumps(artifact_stats(a.path), indent=1))
        return 0
    except (ArtifactError, PreparationError, FileNotFoundError, FileExistsError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2

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
    p.add_argument("--output", default=None, help="overrides output.path")
    p.add_argument("--overwrite", action="store_true", help="overrides output.overwrite")
    p.add_argument("--json", action="store_true", help="machine-readable output (the default output already is JSON)")
    for name in ("inspect", "validate", "stats"):
        q = sub.add_parser(name)
        q.add_argument("path")
        q.add_argument("--json", action="store_true")
        if name == "validate":
            q.add_argument("--no-hashes", action="store_true")
            q.add_argument("--config", default=None, help="train.yaml: also check that this run can read the artifact")
    a = ap.parse_args(argv)
    try:
        if a.cmd == "prepare":
            spec = load_preparation_spec(a.config)
            if a.output is not None or a.overwrite:
                spec = spec.with_output(a.output, True if a.overwrite else None)
            m = prepare_dataset(spec)
            print(json.dumps({"format": m["format"], "samples": m["sample_count"], "tokens": m["token_count"],
                              "dataset_fingerprint": m["metadata"]["dataset_fingerprint"], "stats": m["stats"]}))
        elif a.cmd == "inspect":
            m = load_manifest(a.path)
            print(json.dumps({k: m[k] for k in ("format", "version", "created_at", "sample_count", "token_count",
                                                "files", "stats")}, indent=1))
            print(json.dumps({"metadata": m["metadata"]}, indent=1))
        elif a.cmd == "validate":
            m = validate_artifact(a.path, check_hashes=not a.no_hashes)
            res = {"valid": True, "format": m["format"], "dataset_fingerprint": m["metadata"]["dataset_fingerprint"]}
            if a.config:
                from ..config.run_spec import load_run_spec
                from ..data.artifacts import validate_artifact_for_run
                from ..models.config import model_config_from_run_spec

                spec = load_run_spec(a.config).validate()
                cfg = model_config_from_run_spec(spec)
                res["run"] = validate_artifact_for_run(a.path, vocab_size=cfg.vocab_size, mask_token_id=cfg.mask_token_id,
                                                       block_size=spec.objective.block_size, seq_len=spec.model.seq_len)
            print(json.dumps(res))
        else:
            print(json.dumps(artifact_stats(a.path), indent=1))
        return 0
    except (ArtifactError, PreparationError, FileNotFoundError, FileExistsError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2

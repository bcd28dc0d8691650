"""`dllm dflash …`: prepare-features, export, validate-export, serve-sglang, serve-vllm,
verify-sglang, verify-vllm (cf. dllm_parallel/cli/dflash.py:13-110)."""
from __future__ import annotations

import argparse
import json
import shlex
import sys


def run_dflash(argv) -> int:
    from ..config.run_spec import RunSpecError, load_run_spec
    from ..models import export as ex
    from ..serving import dflash_servers as srv

    ap = argparse.ArgumentParser(prog="dllm dflash")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("prepare-features", help="run the frozen target over a dataset and store hidden states")
    p.add_argument("--config", required=True)
    p.add_argument("--output", required=True)
    p.add_argument("--batches", type=int, default=8)
    p = sub.add_parser("export")
    p.add_argument("--config", required=True)
    p.add_argument("--checkpoint", required=True)
    p.add_argument("--output", required=True)
    p = sub.add_parser("validate-export")
    p.add_argument("path")
    for name in ("serve-sglang", "serve-vllm"):
        p = sub.add_parser(name)
        p.add_argument("--target-model", required=True)
        p.add_argument("--draft", required=True)
        p.add_argument("--port", type=int, default=30000 if name == "serve-sglang" else 8000)
        p.add_argument("--tp", type=int, default=1)
        p.add_argument("--num-speculative-tokens", type=int, default=15)
    for name in ("verify-sglang", "verify-vllm"):
        p = sub.add_parser(name)
        p.add_argument("--base-url", required=True)
        p.add_argument("--model", required=True)
        p.add_argument("--min-acceptance-length", type=float, default=1.5)
    a = ap.parse_args(argv)
    try:
        if a.cmd == "prepare-features":
            from ..data.dflash_features import capture_features

            man = capture_features(load_run_spec(a.config).validate(), a.output, a.batches)
            print(json.dumps(man))
            return 0
        if a.cmd == "export":
            from ..checkpoint import load_training_checkpoint
            from ..training.session import TrainingSession

            spec = load_run_spec(a.config).validate()
            s = TrainingSession(spec)
            load_training_checkpoint(a.checkpoint, "latest", s, rank=0, world_size=1, restore_rng=False)
            print(json.dumps({"files": sorted(ex.export_dflash_drafter(s.model, spec, a.output)["files"])}))
            return 0
        if a.cmd == "validate-export":
            import os

            # a DFlash2 export carries config.json with its architecture; check its tensor inventory too
            is_v2 = os.path.exists(os.path.join(a.path, "config.json"))
            problems = ex.validate_dflash2_export(a.path) if is_v2 else ex.validate_dflash_export(a.path)
            print(json.dumps({"ok": not problems, "problems": problems}))
            return 0 if not problems else 1
        if a.cmd in ("serve-sglang", "serve-vllm"):
            build = srv.build_sglang_command if a.cmd == "serve-sglang" else srv.build_vllm_command
            cmd = build(target_model=a.target_model, draft_export=a.draft, port=a.port, tp=a.tp,
                        num_speculative_tokens=a.num_speculative_tokens)
            print(" ".join(shlex.quote(c) for c in cmd))
            return 0
        res = srv.verify_acceptance(a.base_url, a.model, ["The capital of France is", "def fib(n):"],
                                    a.min_acceptance_length)
        print(json.dumps(res))
        return 0 if res["ok"] else 1
    except (RunSpecError, FileNotFoundError, ValueError, OSError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2

"""`dllm` command dispatcher: bundle, checkpoint, config, data, dflash, doctor, init, launch, recipe, train.

User errors (bad config, unknown recipe, missing path) exit with code 2; the launch command
propagates the trainer's exit code. Counterpart of dllm_parallel/cli/main.py:17-304.
"""
from __future__ import annotations

import argparse
import json
import sys

from ..config.run_spec import RunSpecError, load_run_spec


def _doctor(args) -> int:
    from ..diagnostics import inspect_training_runtime

    spec = load_run_spec(args.config) if args.config else None
    rep = inspect_training_runtime(spec, portable_only=args.portable)
    if args.json:
        print(json.dumps(rep.to_dict(), indent=1))
    else:
        for c in rep.checks:
            mark = "ok " if c.ok else ("FAIL" if c.required else "warn")
            print(f"[{mark}] {c.name}: {c.detail}" + (f"  -> {c.remediation}" if not c.ok and c.remediation else ""))
        print("ready" if rep.ready else "not ready")
    return 0 if rep.ready else 1


def _recipe(args) -> int:
    from .. import recipes

    if args.action == "list":
        for r in recipes.list_recipes(args.kind):
            print(f"{r['name']:32s} {r['kind']:8s} {r['description']}")
        return 0
    if args.action == "show":
        print(recipes.recipe_text(args.name), end="")
        return 0
    dest = recipes.copy_recipe(args.name, args.destination or f"{args.name}.yaml")
    print(dest)
    return 0


def _config(args) -> int:
    spec = load_run_spec(args.config)
    spec.validate(world_size=args.world_size)
    if args.print:
        print(spec.to_yaml(), end="")
    else:
        print(json.dumps({"valid": True, "model_id": spec.model.id, "objective": spec.objective.name,
                          "model_parallel_size": spec.model_parallel_size()}))
    return 0


def _bundle(args) -> int:
    from ..kernels import bundle_manifest as bm

    if args.action == "detect":
        print(json.dumps(bm.detect_environment(), indent=1))
        return 0
    if args.action == "list":
        print(json.dumps(bm.load_catalog(args.catalog), indent=1))
        return 0
    return bm.install_bundle(args.catalog, dry_run=args.dry_run)


def _train(args, rest) -> int:
    from ..training.trainer import main as train_main

    train_main(rest)
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="dllm", description="B200-native block-diffusion LM training")
    sub = ap.add_subparsers(dest="command", required=True)
    p = sub.add_parser("doctor", help="check that this machine can train")
    p.add_argument("--config")
    p.add_argument("--portable", action="store_true")
    p.add_argument("--json", action="store_true")
    p = sub.add_parser("recipe", help="packaged recipes")
    p.add_argument("action", choices=("list", "show", "copy"))
    p.add_argument("name", nargs="?")
    p.add_argument("destination", nargs="?")
    p.add_argument("--kind", choices=("smoke", "example", "prod"))
    p = sub.add_parser("config", help="validate / print a run spec")
    p.add_argument("action", choices=("validate",))
    p.add_argument("config")
    p.add_argument("--world-size", type=int)
    p.add_argument("--print", action="store_true")
    p = sub.add_parser("bundle", help="GPU wheel bundles")
    p.add_argument("action", choices=("detect", "list", "install"))
    p.add_argument("--catalog")
    p.add_argument("--dry-run", action="store_true")
    from .launch import add_launch_arguments

    add_launch_arguments(sub.add_parser("launch", help="start training workers"))
    sub.add_parser("train", help="run the trainer in this process (dllm-train flags follow)", add_help=False)
    sub.add_parser("data", help="prepare / inspect / validate / stats", add_help=False)
    sub.add_parser("dflash", help="DFlash feature capture, export and serving helpers", add_help=False)
    sub.add_parser("init", help="write a starter project", add_help=False)
    sub.add_parser("checkpoint", help="inspect / validate checkpoints", add_help=False)
    return ap


PASSTHROUGH = {"train", "data", "dflash", "init", "checkpoint"}


def run(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        if argv and argv[0] in PASSTHROUGH:
            cmd, rest = argv[0], argv[1:]
            if cmd == "train":
                return _train(None, rest)
            if cmd == "data":
                from .data import run_data

                return run_data(rest)
            if cmd == "dflash":
                from .dflash import run_dflash

                return run_dflash(rest)
            if cmd == "init":
                from .init import run_init

                return run_init(rest)
            from ..checkpoint import main as ckpt_main

            return ckpt_main(rest)
        args = build_parser().parse_args(argv)
        if args.command == "doctor":
            return _doctor(args)
        if args.command == "recipe":
            if args.action != "list" and not args.name:
                raise RunSpecError("recipe show/copy needs a recipe name")
            return _recipe(args)
        if args.command == "config":
            return _config(args)
        if args.command == "bundle":
            return _bundle(args)
        if args.command == "launch":
            from .launch import run_launch

            return run_launch(args)
        return 2
    except (RunSpecError, KeyError, FileExistsError, FileNotFoundError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2


def main() -> None:
    raise SystemExit(run())


if __name__ == "__main__":
    main()

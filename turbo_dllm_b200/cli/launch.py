"""`dllm launch`: validate a run spec against the requested world and start the workers.

Builds either `python -m turbo_dllm_b200.training` (one process) or a
`python -m torch.distributed.run` command (nnodes / nproc-per-node / node-rank / master address /
rendezvous / max-restarts / monitor-interval; elastic `min:max` node counts need a rendezvous
endpoint), builds the child environment (`DLLM_RUN_DIR`, `DLLM_CACHE_DIR`,
`PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True`), checks world size against the topology,
optionally checks that the assigned GPUs are idle, prints `DLLM_RUN_DIR / DLLM_CACHE_DIR /
DLLM_COMMAND`, and propagates the child's exit code. `--dry-run` stops after printing.

Counterpart of dllm_parallel/cli/launch.py:41-121 (command), :124-163 (environment), :182-209
(world-size validation), :251-343 (execution).
"""
from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys
import tempfile
import time

from ..config.run_spec import RunSpecError, load_run_spec

TRAIN_MODULE = "turbo_dllm_b200.training"


def add_launch_arguments(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--config", help="train.yaml run spec")
    ap.add_argument("--recipe", help="name of a packaged recipe (see `dllm recipe list`)")
    ap.add_argument("--nnodes", default="1", help="node count, or MIN:MAX for elastic jobs")
    ap.add_argument("--nproc-per-node", type=int, default=1)
    ap.add_argument("--node-rank", type=int, default=0)
    ap.add_argument("--master-addr", default="127.0.0.1")
    ap.add_argument("--master-port", type=int, default=29500)
    ap.add_argument("--rdzv-endpoint")
    ap.add_argument("--rdzv-id", default="dllm")
    ap.add_argument("--rdzv-backend", default="c10d")
    ap.add_argument("--max-restarts", type=int, default=0)
    ap.add_argument("--monitor-interval", type=float, default=5.0)
    ap.add_argument("--run-dir")
    ap.add_argument("--cache-dir")
    ap.add_argument("--gpu-preflight", choices=("auto", "idle", "off"), default="auto")
    ap.add_argument("--runtime-preflight", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("overrides", nargs=argparse.REMAINDER, help="-- followed by dllm-train flags")


def parse_nnodes(value: str) -> tuple[int, int]:
    lo, sep, hi = str(value).partition(":")
    try:
        a = int(lo)
        b = int(hi) if sep else a
    except ValueError:
        raise RunSpecError(f"--nnodes {value!r} is not N or MIN:MAX") from None
    if a < 1 or b < a:
        raise RunSpecError(f"--nnodes {value!r} is not a valid node range")
    return a, b


def build_launch_command(args, config_path: str, extra: list[str]) -> list[str]:
    lo, hi = parse_nnodes(args.nnodes)
    elastic = lo != hi
    if elastic and not args.rdzv_endpoint:
        raise RunSpecError("elastic --nnodes MIN:MAX needs --rdzv-endpoint")
    train = ["-m", TRAIN_MODULE, "--config", config_path, *extra]
    if hi == 1 and args.nproc_per_node == 1 and not args.max_restarts:
        return [sys.executable, *train]
    cmd = [sys.executable, "-m", "torch.distributed.run", f"--nnodes={args.nnodes}",
           f"--nproc-per-node={args.nproc_per_node}", f"--max-restarts={args.max_restarts}",
           f"--monitor-interval={args.monitor_interval}"]
    if args.rdzv_endpoint:
        cmd += [f"--rdzv-endpoint={args.rdzv_endpoint}", f"--rdzv-id={args.rdzv_id}",
                f"--rdzv-backend={args.rdzv_backend}"]
    else:
        cmd += [f"--node-rank={args.node_rank}", f"--master-addr={args.master_addr}",
                f"--master-port={args.master_port}"]
    return cmd + train


def build_launch_environment(args, base_env=None) -> dict:
    env = dict(os.environ if base_env is None else base_env)
    run_dir = args.run_dir or env.get("DLLM_RUN_DIR") or os.path.join(
        os.getcwd(), "runs", time.strftime("%Y%m%d-%H%M%S"))
    cache_dir = args.cache_dir or env.get("DLLM_CACHE_DIR") or os.path.join(
        os.path.expanduser("~"), ".cache", "turbo_dllm_b200")
    env["DLLM_RUN_DIR"] = run_dir
    env["DLLM_CACHE_DIR"] = cache_dir
    env.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    env.setdefault("HF_HOME", os.path.join(cache_dir, "huggingface"))
    env.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
    return env


def apply_parallel_environment(spec, env: dict, world_size: int | None = None) -> dict:
    """Adds what the run spec's parallel features need (parallel/preflight.py) to the launch environment."""
    from ..parallel.preflight import prepare_parallel_environment, validate_supported_training_axes

    validate_supported_training_axes(spec)
    env.update(prepare_parallel_environment(spec, env, world_size))
    return env


def validate_launch_world_size(spec, args) -> int:
    lo, hi = parse_nnodes(args.nnodes)
    for nodes in sorted({lo, hi}):
        world = nodes * args.nproc_per_node
        spec.validate(world_size=world)
    return hi * args.nproc_per_node


def require_idle_assigned_gpus(nproc: int, command_runner=None) -> None:
    """Refuses to start when an assigned GPU already runs compute processes (injectable runner)."""
    run = command_runner or (lambda cmd: subprocess.run(cmd, capture_output=True, text=True, timeout=30))
    try:
        res = run(["nvidia-smi", "--query-compute-apps=gpu_uuid,pid,used_memory", "--format=csv,noheader"])
    except (OSError, subprocess.SubprocessError) as e:
        raise RunSpecError(f"GPU preflight could not run nvidia-smi: {e}") from None
    if getattr(res, "returncode", 1) != 0:
        raise RunSpecError("GPU preflight: nvidia-smi failed: " + str(getattr(res, "stderr", "")).strip())
    busy = [l for l in str(res.stdout).splitlines() if l.strip()]
    if busy:
        raise RunSpecError("GPU preflight: assigned GPUs are not idle:\n  " + "\n  ".join(busy))


def run_launch(args) -> int:
    from ..recipes import recipe_text

    extra = [a for a in (args.overrides or []) if a != "--"]
    tmp = None
    try:
        if args.recipe:
            tmp = tempfile.NamedTemporaryFile("w", suffix=".yaml", prefix=f"recipe_{args.recipe}_", delete=False)
            tmp.write(recipe_text(args.recipe))
            tmp.close()
            config_path = tmp.name
        elif args.config:
            config_path = args.config
        else:
            raise RunSpecError("dllm launch needs --config or --recipe")
        spec = load_run_spec(config_path)
        world = validate_launch_world_size(spec, args)
        cmd = build_launch_command(args, config_path, extra)
        env = apply_parallel_environment(spec, build_launch_environment(args), world)
        print(f"DLLM_RUN_DIR={env['DLLM_RUN_DIR']}")
        print(f"DLLM_CACHE_DIR={env['DLLM_CACHE_DIR']}")
        print("DLLM_COMMAND=" + " ".join(shlex.quote(c) for c in cmd), flush=True)
        if args.dry_run:
            return 0
        if args.runtime_preflight:
            from ..diagnostics import inspect_training_runtime

            inspect_training_runtime(spec).require_ready()
        if args.gpu_preflight == "idle" or (args.gpu_preflight == "auto" and os.environ.get("SLURM_JOB_ID")):
            require_idle_assigned_gpus(args.nproc_per_node)
        os.makedirs(env["DLLM_RUN_DIR"], exist_ok=True)
        return subprocess.run(cmd, env=env).returncode
    except RunSpecError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    finally:
        if tmp is not None and (args.dry_run or True):
            try:
                os.unlink(tmp.name)
            except OSError:
                pass

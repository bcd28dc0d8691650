"""Rank-aware checkpoint save / load.

Layout (kept from the reference so tooling and users can move over):
    <dir>/metadata.json                         written by rank 0 LAST, atomically (tmp + rename)
    <dir>/<tag>/rank_{r:05d}_of_{w:05d}.pt      one shard per rank: model, optimizer, client_state
Tags are `step_{:08d}` (or `duration_{pct:03d}pct_step_{:08d}`); `latest` resolves through
metadata.json. A checkpoint is complete only once metadata.json names it, which happens after
every rank's shard exists; a rank that fails writes `rank_*.error` and publication is refused.
`keep_last_n` prunes older tags. Loading requires the same world size and topology (no
resharding). `async_save` snapshots tensors to host memory and writes from a thread.

Counterparts: dllm_parallel/core/checkpoint/__init__.py:86-239 (save), :318-400 (load), :403-445
(tags / pruning), format.py:63-115 (client_state keys, topology), :171-211 (metadata), :258-296
(topology validation), io.py:20-67 (shard names, atomic writes).
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import random
import shutil
import sys
import tempfile
import threading
import time
from typing import Any

import torch
import torch.distributed as dist

FORMAT = "dllm_parallel.distributed_checkpoint.v1"
BACKEND = "rank_local"


def shard_name(rank: int, world: int) -> str:
    return f"rank_{rank:05d}_of_{world:05d}.pt"


def step_tag(step: int) -> str:
    return f"step_{step:08d}"


def _atomic_write_json(path: str, payload: dict) -> None:
    d = os.path.dirname(path)
    fd, tmp = tempfile.mkstemp(prefix=".tmp_", dir=d)
    with os.fdopen(fd, "w") as f:
        json.dump(payload, f, indent=1, sort_keys=True, default=str)
    os.replace(tmp, path)


def _atomic_torch_save(obj: Any, path: str) -> None:
    d = os.path.dirname(path)
    fd, tmp = tempfile.mkstemp(prefix="tmp_", suffix=".partial", dir=d)
    with os.fdopen(fd, "wb") as f:
        torch.save(obj, f)
    os.replace(tmp, path)


def capture_rng_state() -> dict:
    st = {"python": random.getstate(), "torch_cpu": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["torch_cuda"] = torch.cuda.get_rng_state_all()
    return st


def restore_rng_state(st: dict) -> None:
    random.setstate(st["python"])
    torch.set_rng_state(st["torch_cpu"])
    if torch.cuda.is_available() and "torch_cuda" in st and len(st["torch_cuda"]) == torch.cuda.device_count():
        torch.cuda.set_rng_state_all(st["torch_cuda"])


def topology_record(spec, world: int, runtime) -> dict:
    t = spec.topology
    rec = {"layout": runtime.plan.layout if runtime is not None else "dp",
           "placement": runtime.plan.placement if runtime is not None else "single_node",
           "data_parallel_size": runtime.data_parallel_size if runtime is not None else world,
           "context_parallel_size": t.context_parallel_size if runtime is not None else 1,
           "block_parallel_size": t.block_parallel_size if runtime is not None else 1,
           "tensor_parallel_size": t.tensor_parallel_size, "expert_parallel_size": t.expert_parallel_size,
           "pipeline_parallel_size": t.pipeline_parallel_size, "sequence_parallel": t.sequence_parallel,
           "cp_bp_policy": {"clean_kv_layout": spec.kernel.cp_bp_clean_kv_layout,
                            "clean_kv_transport": spec.kernel.cp_bp_clean_kv_transport}}
    if runtime is not None:
        rec["process_groups"] = {k: v for k, v in runtime.groups.ranks.items()}
    return rec


def _to_cpu(obj):
    if torch.is_tensor(obj):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


_pending: list[threading.Thread] = []
_pending_errors: list[str] = []


def wait_for_async_saves() -> None:
    while _pending:
        _pending.pop().join()
    if _pending_errors:
        msg = "; ".join(_pending_errors)
        _pending_errors.clear()
        raise RuntimeError(f"asynchronous checkpoint save failed: {msg}")


def _barrier(group) -> None:
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier(group=group) if group is not None else dist.barrier()


def save_training_checkpoint(directory: str, session, *, step: int, rank: int, world_size: int, runtime=None,
                             spec=None, tag: str | None = None, control_group=None,
                             async_save: bool | None = None) -> str:
    spec = spec or session.spec
    tag = tag or step_tag(step)
    tag_dir = os.path.join(directory, tag)
    os.makedirs(tag_dir, exist_ok=True)
    client_state = {
        "step": step, "rank": rank, "world_size": world_size,
        "topology": topology_record(spec, world_size, runtime),
        "objective_state": session.objective.state_dict(), "dataloader_state": session.data.state_dict(),
        "scheduler_state": session.scheduler.state_dict(), "config": spec.to_dict(),
        "kernel_metadata": _kernel_metadata(), "run_metadata": _run_metadata(),
        "profiler_metadata": {}, "backbone_state": {"family": session.cfg.family},
        "rng_state": capture_rng_state(),
    }
    st = session.state_dict()
    payload = {"model": st["model"], "optimizer": st["optimizer"], "client_state": client_state}
    for key in ("expert_model", "expert_optimizer"):
        if key in st:
            payload[key] = st[key]
    path = os.path.join(tag_dir, shard_name(rank, world_size))
    err_path = os.path.join(tag_dir, f"rank_{rank:05d}.error")
    use_async = spec.checkpointing.async_checkpoint_save if async_save is None else async_save

    def write(obj):
        try:
            _atomic_torch_save(obj, path)
        except Exception as e:  # surfaced by publication and by wait_for_async_saves()
            open(err_path, "w").write(f"{type(e).__name__}: {e}")
            _pending_errors.append(f"rank {rank}: {e}")

    if use_async:
        snap = _to_cpu(payload)
        th = threading.Thread(target=write, args=(snap,), daemon=True)
        th.start()
        _pending.append(th)
        th.join()  # publication below needs the shard; the device was released after the snapshot
    else:
        write(payload)
    _barrier(control_group)
    if rank == 0:
        publish_metadata(directory, tag, step, world_size, client_state, spec)
    _barrier(control_group)
    return tag


def publish_metadata(directory: str, tag: str, step: int, world_size: int, client_state: dict, spec) -> None:
    tag_dir = os.path.join(directory, tag)
    errors = glob.glob(os.path.join(tag_dir, "rank_*.error"))
    missing = [r for r in range(world_size) if not os.path.exists(os.path.join(tag_dir, shard_name(r, world_size)))]
    if errors or missing:
        open(os.path.join(tag_dir, "checkpoint.error"), "w").write(
            json.dumps({"errors": [os.path.basename(e) for e in errors], "missing_ranks": missing}))
        raise RuntimeError(f"checkpoint {tag} is incomplete: missing ranks {missing}, errors {errors}")
    meta = {"format": FORMAT, "latest_tag": tag, "step": step, "world_size": world_size,
            "topology": client_state["topology"], "config": client_state["config"],
            "objective_state": _jsonable(client_state["objective_state"]),
            "dataloader_state": _jsonable(client_state["dataloader_state"]),
            "scheduler_state": client_state["scheduler_state"], "kernel_metadata": client_state["kernel_metadata"],
            "run_metadata": client_state["run_metadata"], "profiler_metadata": {},
            "backbone_state": client_state["backbone_state"], "checkpoint_backend": BACKEND,
            "model_state_scope": "replicated_flat_parameters",
            "rank_state_pattern": "rank_{rank:05d}_of_{world_size:05d}.pt",
            "created_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
    _atomic_write_json(os.path.join(directory, "metadata.json"), meta)
    keep = spec.checkpointing.keep_last_n
    if keep and keep > 0:
        prune_checkpoints(directory, keep, protect=tag)


def _jsonable(state: dict) -> dict:
    return {k: (v if isinstance(v, (int, float, str, bool, type(None))) else f"<{type(v).__name__}>")
            for k, v in state.items()}


def list_tags(directory: str) -> list[str]:
    tags = [d for d in os.listdir(directory) if os.path.isdir(os.path.join(directory, d))
            and (d.startswith("step_") or d.startswith("duration_"))]
    return sorted(tags, key=lambda t: int(t.rsplit("_", 1)[-1]))


def prune_checkpoints(directory: str, keep_last_n: int, protect: str | None = None) -> list[str]:
    tags = list_tags(directory)
    victims = [t for t in tags[:-keep_last_n] if t != protect] if keep_last_n < len(tags) else []
    for t in victims:
        shutil.rmtree(os.path.join(directory, t), ignore_errors=True)
    return victims


def read_metadata(directory: str) -> dict:
    path = os.path.join(directory, "metadata.json")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{directory} has no metadata.json: not a complete checkpoint directory")
    meta = json.load(open(path))
    if meta.get("format") != FORMAT:
        raise ValueError(f"unsupported checkpoint format {meta.get('format')!r}")
    return meta


def resolve_tag(directory: str, tag: str) -> str:
    return read_metadata(directory)["latest_tag"] if tag == "latest" else tag


def validate_topology(meta: dict, spec, world_size: int, runtime) -> None:
    if int(meta["world_size"]) != world_size:
        raise ValueError(f"checkpoint was written by {meta['world_size']} ranks, this job has {world_size}: "
                         "resharding checkpoints is not implemented")
    have = topology_record(spec, world_size, runtime)
    want = meta["topology"]
    for key in ("data_parallel_size", "context_parallel_size", "block_parallel_size", "tensor_parallel_size",
                "expert_parallel_size", "pipeline_parallel_size", "sequence_parallel", "layout"):
        if want.get(key) != have.get(key):
            raise ValueError(f"checkpoint topology mismatch on {key}: checkpoint {want.get(key)!r}, "
                             f"job {have.get(key)!r} (resharding checkpoints is not implemented)")


def load_training_checkpoint(directory: str, tag: str, session, *, rank: int, world_size: int, runtime=None,
                             restore_rng: bool = True) -> dict:
    meta = read_metadata(directory)
    validate_topology(meta, session.spec, world_size, runtime)
    tag = resolve_tag(directory, tag)
    path = os.path.join(directory, tag, shard_name(rank, world_size))
    if not os.path.exists(path):
        raise FileNotFoundError(f"missing checkpoint shard {path}")
    payload = torch.load(path, map_location=session.device, weights_only=False)
    cs = payload["client_state"]
    session.load_state_dict({**{k: payload[k] for k in ("expert_model", "expert_optimizer") if k in payload},
                             "model": payload["model"], "optimizer": payload["optimizer"],
                             "scheduler": cs["scheduler_state"], "objective": cs["objective_state"],
                             "data": cs["dataloader_state"], "steps_done": cs["step"]})
    if restore_rng:
        restore_rng_state(cs["rng_state"])
    return {"step": cs["step"], "tag": tag, "metadata": meta}


def _kernel_metadata() -> dict:
    try:
        from ..kernels import native

        man = native.manifest() or {}
        return {"library": man.get("library"), "arch": man.get("arch"), "binary_sha256": man.get("binary_sha256")}
    except Exception:
        return {}


def _run_metadata() -> dict:
    from .. import __version__

    return {"package_version": __version__, "torch": torch.__version__, "python": sys.version.split()[0]}


def validate_checkpoint(directory: str, tag: str = "latest") -> dict:
    """Structural check: metadata present, every rank shard exists and loads its client_state."""
    meta = read_metadata(directory)
    tag = resolve_tag(directory, tag)
    world = int(meta["world_size"])
    problems = []
    for r in range(world):
        p = os.path.join(directory, tag, shard_name(r, world))
        if not os.path.exists(p):
            problems.append(f"missing {os.path.basename(p)}")
    if glob.glob(os.path.join(directory, tag, "*.error")):
        problems.append("error markers present")
    return {"directory": directory, "tag": tag, "world_size": world, "step": meta["step"], "ok": not problems,
            "problems": problems}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="dllm-checkpoint")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("inspect", "validate"):
        sp = sub.add_parser(name)
        sp.add_argument("directory")
        sp.add_argument("--tag", default="latest")
    a = ap.parse_args(argv)
    try:
        if a.cmd == "inspect":
            meta = read_metadata(a.directory)
            print(json.dumps({k: meta[k] for k in ("format", "latest_tag", "step", "world_size", "topology",
                                                   "checkpoint_backend")}, indent=1))
            print(json.dumps({"tags": list_tags(a.directory)}))
            return 0
        res = validate_checkpoint(a.directory, a.tag)
        print(json.dumps(res, indent=1))
        return 0 if res["ok"] else 1
    except (FileNotFoundError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    raise SystemExit(main())

"""Rank-aware checkpoint save / load.

Layout (kept from the reference so tooling and users can move over):
    <dir>/metadata.json                         written by rank 0 LAST, atomically (tmp + rename)
    <dir>/<tag>/rank_{r:05d}_of_{w:05d}.pt      one shard per rank: model, optimizer, client_state
Tags are `step_{:08d}` (or `duration_{pct:03d}pct_step_{:08d}`); `latest` resolves through
metadata.json. A checkpoint is complete only once metadata.json names it, which happens after
every rank's shard exists; a rank that fails writes `rank_*.error` and publication is refused.
`keep_last_n` prunes older tags. Loading requires the same world size and topology (no
resharding). Asynchronous saves snapshot tensors to host memory and write from a thread that also publishes
(rank 0) once every shard has appeared; adapter (LoRA) runs can store a model-only checkpoint of the trainable
tensors alone.

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
MODEL_ONLY_FILENAME = "mp_rank_00_model_states.pt"
MODEL_ONLY_MANIFEST = "model_only_manifest.json"
MODEL_ONLY_FORMAT = "dllm_parallel.model_only_checkpoint.v1"


def wait_for_async_saves() -> None:
    """Joins every writer thread started by an asynchronous save and raises if one of them failed."""
    while _pending:
        _pending.pop().join()
    if _pending_errors:
        msg = "; ".join(_pending_errors)
        _pending_errors.clear()
        raise RuntimeError(f"asynchronous checkpoint save failed: {msg}")


def _barrier(group) -> None:
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier(group=group) if group is not None else dist.barrier()


def _remove(path: str) -> None:
    try:
        os.unlink(path)
    except FileNotFoundError:
        pass


def _incomplete(tag_dir: str, world_size: int) -> tuple[list[str], list[int]]:
    errors = sorted(glob.glob(os.path.join(tag_dir, "rank_*.error")))
    missing = [r for r in range(world_size) if not os.path.exists(os.path.join(tag_dir, shard_name(r, world_size)))]
    return errors, missing


def _publish_or_mark(directory: str, tag: str, step: int, world_size: int, client_state: dict, spec) -> str | None:
    """Rank 0: publishes metadata.json when every shard is there, otherwise writes `checkpoint.error` and
    returns its text. Never raises for an incomplete checkpoint: the caller lets every rank see the marker."""
    tag_dir = os.path.join(directory, tag)
    errors, missing = _incomplete(tag_dir, world_size)
    if errors or missing:
        msg = json.dumps({"errors": [os.path.basename(e) for e in errors], "missing_ranks": missing})
        open(os.path.join(tag_dir, "checkpoint.error"), "w").write(msg)
        return msg
    publish_metadata(directory, tag, step, world_size, client_state, spec)
    return None


def save_training_checkpoint(directory: str, session, *, step: int, rank: int, world_size: int, runtime=None,
                             spec=None, tag: str | None = None, control_group=None,
                             async_save: bool | None = None, shard_timeout_s: float = 600.0) -> str:
    """Every rank writes its shard; rank 0 publishes `metadata.json` once all shards exist.

    Failure protocol: a rank whose write fails leaves `rank_{r}.error`; rank 0 then writes `checkpoint.error`
    instead of publishing, all ranks pass the closing barrier, and EVERY rank raises. Markers of an earlier
    attempt at the same tag are cleared first. Synchronous saves use two barriers of `control_group`.
    Asynchronous saves (`checkpointing.async_checkpoint_save`) snapshot the state to host memory, return at
    once, and write from a thread; rank 0's thread publishes when the other ranks' shards have appeared on the
    shared file system (no collective runs off the main thread). `wait_for_async_saves()` joins and reports;
    the next save and the end of training call it. LoRA runs with `checkpointing.model_only` write the
    adapter-only layout instead (`save_model_only_checkpoint`)."""
    spec = spec or session.spec
    if getattr(session, "lora", None) is not None and spec.checkpointing.model_only:
        return save_model_only_checkpoint(directory, session, step=step, rank=rank, world_size=world_size,
                                          runtime=runtime, spec=spec, tag=tag, control_group=control_group)
    wait_for_async_saves()
    tag = tag or step_tag(step)
    tag_dir = os.path.join(directory, tag)
    os.makedirs(tag_dir, exist_ok=True)
    err_path = os.path.join(tag_dir, f"rank_{rank:05d}.error")
    _remove(err_path)
    if rank == 0:
        _remove(os.path.join(tag_dir, "checkpoint.error"))
    client_state = {
        "step": step, "rank": rank, "world_size": world_size,
        "topology": topology_record(spec, world_size, runtime),
        "objective_state": session.objective.state_dict(), "dataloader_state": session.data.state_dict(),
        "scheduler_state": session.scheduler.state_dict(), "config": spec.to_dict(),
        "kernel_metadata": _kernel_metadata(), "run_metadata": _run_metadata(),
        "profiler_metadata": {}, "backbone_state": {"family": session.cfg.family},
        "rng_state": capture_rng_state(),
    }
    if getattr(session, "sharded", None) is not None:
        client_state["checkpoint_backend"] = "fsdp_sharded_rank_local"
        client_state["model_state_scope"] = "sharded_flat_parameters"
    st = session.state_dict()
    payload = {"model": st["model"], "optimizer": st["optimizer"], "client_state": client_state}
    for key in ("expert_model", "expert_optimizer", "adapter"):
        if key in st:
            payload[key] = st[key]
    path = os.path.join(tag_dir, shard_name(rank, world_size))
    use_async = spec.checkpointing.async_checkpoint_save if async_save is None else async_save

    def write(obj) -> bool:
        try:
            _atomic_torch_save(obj, path)
            return True
        except Exception as e:
            open(err_path, "w").write(f"{type(e).__name__}: {e}")
            return False

    if use_async:
        snap = _to_cpu(payload)
        _barrier(control_group)      # stale markers are gone everywhere before any writer can leave a new one

        def work():
            ok = write(snap)
            if not ok:
                _pending_errors.append(f"rank {rank}: shard write failed ({open(err_path).read()})")
            if rank != 0:
                return
            deadline = time.time() + shard_timeout_s
            while time.time() < deadline:
                errors, missing = _incomplete(tag_dir, world_size)
                if errors or not missing:
                    break
                time.sleep(0.05)
            msg = _publish_or_mark(directory, tag, step, world_size, client_state, spec)
            if msg is not None:
                _pending_errors.append(f"checkpoint {tag} is incomplete: {msg}")

        th = threading.Thread(target=work, daemon=True)
        th.start()
        _pending.append(th)
        return tag
    _barrier(control_group)          # stale markers cleared on every rank
    write(payload)
    _barrier(control_group)
    if rank == 0:
        _publish_or_mark(directory, tag, step, world_size, client_state, spec)
    _barrier(control_group)
    marker = os.path.join(tag_dir, "checkpoint.error")
    if os.path.exists(marker):
        raise RuntimeError(f"checkpoint {tag} is incomplete: {open(marker).read()}")
    return tag


def _file_sha256(path: str) -> str:
    import hashlib

    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def save_model_only_checkpoint(directory: str, session, *, step: int, rank: int, world_size: int, runtime=None,
                               spec=None, tag: str | None = None, control_group=None) -> str:
    """Adapter-only checkpoint: rank 0 stores ONE copy of every trainable tensor (the LoRA pairs; they are
    replicated over data-, context- and block-parallel ranks) as `<tag>/mp_rank_00_model_states.pt` plus
    `<tag>/model_only_manifest.json` (format, size, SHA-256, tensor inventory, tied-alias map). Frozen base
    weights, optimizer, scheduler, RNG and data-loader state are left out on purpose, and the published
    metadata says so (`checkpoint_backend: adapter_model_only`), so such a checkpoint seeds fine-tuning or
    export but is not a restart point. Layout of dllm_parallel/core/checkpoint/__init__.py:473-741."""
    spec = spec or session.spec
    lora = getattr(session, "lora", None)
    if lora is None:
        raise ValueError("model-only checkpoints store adapters: the session has none")
    tag = tag or step_tag(step)
    final_dir = os.path.join(directory, tag)
    os.makedirs(directory, exist_ok=True)
    _barrier(control_group)
    problem = None
    if rank == 0:
        tmp_dir = os.path.join(directory, f".{tag}.model-only.tmp")
        try:
            if os.path.exists(final_dir) or os.path.exists(tmp_dir):
                raise FileExistsError(f"checkpoint tag already exists: {final_dir}")
            os.makedirs(tmp_dir)
            module = {n: p.detach().to("cpu", copy=True) for n, p in lora.flat.params.items()}
            # tensors that share storage are stored once under their first name
            seen, shared = {}, {}
            for n, p in lora.flat.params.items():
                key = (p.data_ptr(), tuple(p.shape))
                if key in seen:
                    shared[n] = seen[key]
                    module.pop(n)
                else:
                    seen[key] = n
            state = {"step": int(step), "module": module, "shared_params": shared,
                     "model_state_scope": "trainable_parameters",
                     "client_state": {"step": int(step), "backbone_state": {"family": session.cfg.family},
                                      "config": spec.to_dict(), "checkpoint_backend": "adapter_model_only",
                                      "model_state_scope": "trainable_parameters",
                                      "adapter": {"rank": spec.adapter.rank, "alpha": spec.adapter.alpha,
                                                  "targets": list(spec.adapter.targets or ("attention", "mlp")),
                                                  "scale": lora.scale}}}
            spath = os.path.join(tmp_dir, MODEL_ONLY_FILENAME)
            _atomic_torch_save(state, spath)
            manifest = {"format": MODEL_ONLY_FORMAT, "step": int(step), "filename": MODEL_ONLY_FILENAME,
                        "bytes": os.path.getsize(spath), "sha256": _file_sha256(spath),
                        "tensor_count": len(module), "parameter_count": int(sum(t.numel() for t in module.values())),
                        "tensors": {n: {"shape": list(t.shape), "dtype": str(t.dtype).replace("torch.", "")}
                                    for n, t in module.items()},
                        "shared_params": shared}
            with open(os.path.join(tmp_dir, MODEL_ONLY_MANIFEST), "w") as f:
                f.write(json.dumps(manifest, indent=2, sort_keys=True) + "\n")
            os.replace(tmp_dir, final_dir)
            meta = {"format": FORMAT, "latest_tag": tag, "step": int(step), "world_size": world_size,
                    "topology": topology_record(spec, world_size, runtime), "config": spec.to_dict(),
                    "objective_state": {}, "dataloader_state": {}, "scheduler_state": {}, "rng_state": {},
                    "kernel_metadata": _kernel_metadata(), "run_metadata": _run_metadata(), "profiler_metadata": {},
                    "backbone_state": {"family": session.cfg.family}, "checkpoint_backend": "adapter_model_only",
                    "model_state_scope": "trainable_parameters", "model_only_manifest": manifest,
                    "rank_state_pattern": MODEL_ONLY_FILENAME,
                    "created_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
            _atomic_write_json(os.path.join(directory, "metadata.json"), meta)
            keep = spec.checkpointing.keep_last_n
            if keep and keep > 0:
                prune_checkpoints(directory, keep, protect=tag)
        except Exception as e:
            problem = f"{type(e).__name__}: {e}"
            shutil.rmtree(tmp_dir, ignore_errors=True)
            os.makedirs(final_dir, exist_ok=True)
            open(os.path.join(final_dir, "checkpoint.error"), "w").write(problem)
    _barrier(control_group)
    marker = os.path.join(final_dir, "checkpoint.error")
    if os.path.exists(marker):
        raise RuntimeError(f"model-only checkpoint {tag} failed: {open(marker).read()}")
    return tag


def validate_model_only_checkpoint(directory: str, tag: str = "latest") -> dict:
    """Checks the manifest against the state file (size, SHA-256, tensor inventory)."""
    tag = resolve_tag(directory, tag)
    tdir = os.path.join(directory, tag)
    man = json.load(open(os.path.join(tdir, MODEL_ONLY_MANIFEST)))
    problems = []
    if man.get("format") != MODEL_ONLY_FORMAT:
        problems.append(f"unexpected manifest format {man.get('format')!r}")
    spath = os.path.join(tdir, man.get("filename", MODEL_ONLY_FILENAME))
    if not os.path.exists(spath):
        problems.append("state file missing")
    else:
        if os.path.getsize(spath) != man.get("bytes"):
            problems.append("state file size differs from the manifest")
        if _file_sha256(spath) != man.get("sha256"):
            problems.append("state file SHA-256 differs from the manifest")
        else:
            st = torch.load(spath, map_location="cpu", weights_only=False)
            if sorted(st["module"]) != sorted(man["tensors"]):
                problems.append("tensor inventory differs from the manifest")
    return {"directory": directory, "tag": tag, "step": man.get("step"), "ok": not problems, "problems": problems}


def load_model_only_checkpoint(directory: str, tag: str, session) -> dict:
    """Loads adapter tensors into a session whose adapters have the same names and shapes. The optimizer's
    fp32 master copy of its shard is refreshed from the loaded values; its moments start from zero."""
    res = validate_model_only_checkpoint(directory, tag)
    if not res["ok"]:
        raise ValueError(f"model-only checkpoint {res['tag']} is damaged: {res['problems']}")
    lora = getattr(session, "lora", None)
    if lora is None:
        raise ValueError("the session has no adapters to load into (adapter.type: lora)")
    st = torch.load(os.path.join(directory, res["tag"], MODEL_ONLY_FILENAME), map_location="cpu", weights_only=False)
    module = dict(st["module"])
    for alias, src in st.get("shared_params", {}).items():
        module[alias] = module[src]
    have = lora.flat.params
    if sorted(module) != sorted(have):
        raise ValueError("adapter tensor names differ from the checkpoint's")
    with torch.no_grad():
        for n, t in module.items():
            if tuple(t.shape) != tuple(have[n].shape):
                raise ValueError(f"adapter tensor {n}: shape {tuple(have[n].shape)} here, {tuple(t.shape)} stored")
            have[n].copy_(t.to(have[n].device, have[n].dtype))
        opt = session.optimizer
        opt.master.copy_(lora.flat.data[opt.start:opt.stop].float())
    return {"step": st["step"], "tag": res["tag"]}


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
            "backbone_state": client_state["backbone_state"],
            "checkpoint_backend": client_state.get("checkpoint_backend", BACKEND),
            "model_state_scope": client_state.get("model_state_scope", "replicated_flat_parameters"),
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
    explicit = tag != "latest"
    tag = resolve_tag(directory, tag)
    if meta.get("checkpoint_backend") == "adapter_model_only" and tag == meta.get("latest_tag"):
        out = load_model_only_checkpoint(directory, tag, session)
        return {**out, "metadata": meta}
    if not explicit or tag == meta.get("latest_tag"):
        validate_topology(meta, session.spec, world_size, runtime)
    path = os.path.join(directory, tag, shard_name(rank, world_size))
    if not os.path.exists(path):
        raise FileNotFoundError(f"missing checkpoint shard {path}")
    payload = torch.load(path, map_location=session.device, weights_only=False)
    cs = payload["client_state"]
    if explicit and tag != meta.get("latest_tag"):
        # an older tag is checked against the topology recorded in its own shards, not the latest publication's
        validate_topology({"world_size": cs["world_size"], "topology": cs["topology"]}, session.spec, world_size,
                          runtime)
    session.load_state_dict({**{k: payload[k] for k in ("expert_model", "expert_optimizer", "adapter") if k in payload},
                             "model": payload["model"], "optimizer": payload["optimizer"],
                             "scheduler": cs["scheduler_state"], "objective": cs["objective_state"],
                             "data": cs["dataloader_state"], "steps_done": cs["step"]})
    if restore_rng:
        restore_rng_state(cs["rng_state"])
    return {"step": cs["step"], "tag": tag, "metadata": meta}


def load_model_weights(directory: str, tag: str, session) -> dict:
    """Weights (and adapters) only, on ONE process, from a checkpoint written by any number of ranks: for export and
    evaluation after a multi-GPU run. Works when the saved ranks together hold plain copies or plain slices of the
    weights: replicated parameters (data / context / block parallelism with a sharded optimizer: rank 0's file has
    them all) and parameter sharding (`optimizer.backend: fsdp`: every rank's slice of every unit is put back in
    place). Tensor- or expert-parallel checkpoints are exported by a job of the same shape instead (the export gathers
    over those groups). Optimizer, scheduler, data and RNG state are not restored."""
    meta = read_metadata(directory)
    tag = resolve_tag(directory, tag)
    if meta.get("checkpoint_backend") == "adapter_model_only" and tag == meta.get("latest_tag"):
        return {**load_model_only_checkpoint(directory, tag, session), "metadata": meta}
    world = int(meta["world_size"])
    topo = meta.get("topology", {})
    if int(topo.get("tensor_parallel_size", 1)) > 1 or int(topo.get("expert_parallel_size", 1)) > 1:
        raise ValueError("the checkpoint holds tensor- or expert-parallel shards: run the export as a job of the same "
                         f"shape ({world} ranks), which gathers them")

    def shard(r):
        path = os.path.join(directory, tag, shard_name(r, world))
        if not os.path.exists(path):
            raise FileNotFoundError(f"missing checkpoint shard {path}")
        return torch.load(path, map_location="cpu", weights_only=False)

    first = shard(0)
    flat = session.model.flat
    if first["model"].numel() == flat.data.numel():
        flat.data.copy_(first["model"].to(flat.data.device, flat.data.dtype))
    else:
        from ..parallel.fsdp import plan_units

        units = plan_units(flat, world)
        if first["model"].numel() != sum(u.shard for u in units):
            raise ValueError(f"rank 0 of the checkpoint holds {first['model'].numel()} parameter values; neither the whole "
                             f"model ({flat.data.numel()}) nor its 1/{world} parameter shard")
        for r in range(world):
            part = (first if r == 0 else shard(r))["model"]
            for u in units:
                lo = u.start + r * u.shard
                n = max(0, min(u.shard, u.stop - lo))
                if n:
                    flat.data[lo:lo + n].copy_(part[u.local:u.local + n].to(flat.data.device, flat.data.dtype))
    experts = getattr(session.model, "flat_experts", None)
    if experts is not None and "expert_model" in first:      # (expert_parallel_size 1: rank 0 holds every expert)
        experts.data.copy_(first["expert_model"].to(experts.data.device, experts.data.dtype))
    lora = getattr(session, "lora", None)
    if lora is not None and "adapter" in first:
        lora.flat.data.copy_(first["adapter"].to(lora.flat.data.device, lora.flat.data.dtype))
    return {"step": first["client_state"]["step"], "tag": tag, "metadata": meta}


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

"""Offline DFlash target features: capture with the frozen target, sharded record store, manifest.

`capture_features` runs the frozen target over batches of the run's data runtime and writes, per
shard file, the token ids, the concatenated hidden states of the selected target layers and the
final-norm hidden states, plus `manifest.json` (format `dllm.dflash_features.v1`, SHA-256 per shard).
`FeatureStore` reads records back in order for training with `data.target_features=offline`.

Counterparts: dllm_parallel/core/models/backbones/dflash/feature_capture.py:83-658 and
dllm_parallel/core/models/backbones/dflash/data.py:140-630, :764-899.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

FORMAT = "dllm.dflash_features.v1"


def _sha(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for c in iter(lambda: f.read(1 << 20), b""):
            h.update(c)
    return h.hexdigest()


@torch.no_grad()
def capture_features(spec, output: str, batches: int, *, rank: int = 0, world: int = 1, barrier=None,
                     device=None, resume: bool = False) -> dict:
    """Runs the frozen target over `batches` batches and writes one record per batch. With `world` > 1 every rank
    (its own data shard: the session's data runtime is seeded per data-parallel rank) writes the records
    rank, rank + world, ... under its own names, a barrier follows, and rank 0 merges the per-rank lists into
    `manifest.json` in record order. `resume` keeps records whose file already exists with the recorded hash (a capture
    that was interrupted continues; the data runtime is advanced past the kept records)."""
    from ..training.session import TrainingSession

    s = TrainingSession(spec, **({"device": device} if device is not None else {}))
    if s.task is None:
        raise ValueError("feature capture needs objective.name=dflash_distillation")
    if rank == 0:
        os.makedirs(output, exist_ok=resume)
    if barrier is not None:
        barrier()
    part_path = os.path.join(output, f"manifest.rank{rank:03d}.json")
    done = {}
    if resume and os.path.exists(part_path):
        done = {sh["index"]: sh for sh in json.load(open(part_path)) if os.path.exists(os.path.join(output, sh["name"]))
                and _sha(os.path.join(output, sh["name"])) == sh["sha256"]}
    shards = []
    for i in range(rank, batches, world):
        batch = s.data.next_batch()
        if i in done:
            shards.append(done[i])
            continue
        feats = s.task.target.features(batch.input_ids)
        name = f"shard_{i:05d}.pt"
        torch.save({"input_ids": batch.input_ids.cpu(), "hidden": feats.hidden.cpu(),
                    "final_hidden": feats.final_hidden.cpu()}, os.path.join(output, name))
        shards.append({"index": i, "name": name, "records": int(batch.input_ids.shape[0]),
                       "sha256": _sha(os.path.join(output, name))})
        json.dump(shards, open(part_path, "w"))          # progress survives an interruption
    json.dump(shards, open(part_path, "w"))
    if barrier is not None:
        barrier()
    if rank != 0:
        return {}
    merged = []
    for r in range(world):
        p = os.path.join(output, f"manifest.rank{r:03d}.json")
        merged += json.load(open(p))
        os.unlink(p)
    merged.sort(key=lambda sh: sh["index"])
    if [sh["index"] for sh in merged] != list(range(batches)):
        raise RuntimeError(f"feature capture is incomplete: records {sorted(set(range(batches)) - {sh['index'] for sh in merged})} are missing")
    man = {"format": FORMAT, "target": spec.model.verifier_id, "target_layer_ids": list(spec.model.target_layer_ids),
           "seq_len": spec.model.seq_len, "captured_by_ranks": world,
           "shards": [{k: v for k, v in sh.items() if k != "index"} for sh in merged]}
    json.dump(man, open(os.path.join(output, "manifest.json"), "w"), indent=1)
    return man


class FeatureStoreDataRuntime:
    """Data runtime over a feature store: a batch is one stored record (token ids plus the target's hidden
    states), shards dealt out round-robin over the data-parallel ranks, the next record read ahead into pinned
    memory while the current step runs. Counterpart of DFlashFeatureDataRuntime
    (dllm_parallel/core/models/backbones/dflash/data.py:248-630)."""

    def __init__(self, store: "FeatureStore", *, batch_size: int, device, dp_rank: int = 0, dp_size: int = 1,
                 context_rows=None):
        """context_rows(batch, seq_len) -> rows of the [batch * seq_len, ...] hidden states this rank attends to
        (a replica that spans several ranks shards the context): only those rows are read from the memory-mapped
        record and sent to the device, and the teacher states stay memory-mapped on the host until the step knows
        which positions its anchors need. A 256K-token record then costs a rank its shard, not the sequence."""
        from .runtimes import DataBatch  # noqa: F401

        self.store, self.device = store, torch.device(device)
        self.context_rows = context_rows
        self.batch_size, self.dp_rank, self.dp_size = batch_size, dp_rank, dp_size
        if len(store.manifest["shards"]) < dp_size:
            raise ValueError(f"feature store has {len(store.manifest['shards'])} records, fewer than the {dp_size} "
                             "data-parallel ranks")
        self.step = 0
        self._ahead = None

    def _load(self, step: int) -> dict:
        shards = self.store.manifest["shards"]
        sh = shards[(step * self.dp_size + self.dp_rank) % len(shards)]
        path = os.path.join(self.store.root, sh["name"])
        lazy = self.context_rows is not None
        try:
            rec = torch.load(path, map_location="cpu", mmap=lazy)
        except (RuntimeError, TypeError):       # a record written in a format that cannot be mapped
            rec = torch.load(path, map_location="cpu")
        if rec["input_ids"].shape[0] != self.batch_size:
            raise ValueError(f"feature records hold {rec['input_ids'].shape[0]} sequences, the run's batch size is "
                             f"{self.batch_size}")
        if lazy:
            b, l = rec["input_ids"].shape
            rows = self.context_rows(b, l).cpu()
            hidden = rec["hidden"].reshape(b * l, -1).index_select(0, rows)
            rec = {"input_ids": rec["input_ids"].clone(), "hidden": hidden, "final_hidden_host": rec["final_hidden"]}
        if self.device.type == "cuda":
            rec = {k: (v if k == "final_hidden_host" else v.pin_memory()) for k, v in rec.items()}
        return rec

    def next_batch(self):
        from .runtimes import DataBatch

        rec = self._ahead if self._ahead is not None else self._load(self.step)
        self.step += 1
        host = rec.pop("final_hidden_host", None)
        nbytes = sum(v.numel() * v.element_size() for v in rec.values()) if self.device.type == "cuda" else 0
        dev = {k: v.to(self.device, non_blocking=True) for k, v in rec.items()}
        self._ahead = self._load(self.step)
        b = DataBatch(dev["input_ids"], h2d_bytes=nbytes)
        if host is not None:
            b.features = {"hidden": dev["hidden"], "final_hidden": host, "hidden_is_shard": True}
        else:
            b.features = {"hidden": dev["hidden"], "final_hidden": dev["final_hidden"]}
        return b

    def next_optimizer_step_batches(self, micro_batches: int):
        return [self.next_batch() for _ in range(micro_batches)]

    def state_dict(self):
        return {"kind": "dflash_features", "step": self.step, "dp_size": self.dp_size}

    def load_state_dict(self, st):
        self.step = int(st["step"])
        self._ahead = None

    def close(self):
        self._ahead = None


class FeatureStore:
    def __init__(self, root: str, verify: bool = False):
        self.root = root
        self.manifest = json.load(open(os.path.join(root, "manifest.json")))
        if self.manifest.get("format") != FORMAT:
            raise ValueError(f"{root} is not a DFlash feature store")
        if verify:
            for sh in self.manifest["shards"]:
                if _sha(os.path.join(root, sh["name"])) != sh["sha256"]:
                    raise ValueError(f"{sh['name']}: sha256 mismatch")
        self.cursor = 0

    def next_record(self, device) -> dict:
        sh = self.manifest["shards"][self.cursor % len(self.manifest["shards"])]
        self.cursor += 1
        rec = torch.load(os.path.join(self.root, sh["name"]), map_location="cpu")
        return {k: v.to(device, non_blocking=True) for k, v in rec.items()}

    def state_dict(self):
        return {"cursor": self.cursor}

    def load_state_dict(self, st):
        self.cursor = int(st["cursor"])

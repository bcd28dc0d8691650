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
def capture_features(spec, output: str, batches: int) -> dict:
    from ..training.session import TrainingSession

    s = TrainingSession(spec)
    if s.task is None:
        raise ValueError("feature capture needs objective.name=dflash_distillation")
    os.makedirs(output, exist_ok=False)
    shards = []
    for i in range(batches):
        batch = s.data.next_batch()
        feats = s.task.target.features(batch.input_ids)
        name = f"shard_{i:05d}.pt"
        torch.save({"input_ids": batch.input_ids.cpu(), "hidden": feats.hidden.cpu(),
                    "final_hidden": feats.final_hidden.cpu()}, os.path.join(output, name))
        shards.append({"name": name, "records": int(batch.input_ids.shape[0]), "sha256": _sha(os.path.join(output, name))})
    man = {"format": FORMAT, "target": spec.model.verifier_id, "target_layer_ids": list(spec.model.target_layer_ids),
           "seq_len": spec.model.seq_len, "shards": shards}
    json.dump(man, open(os.path.join(output, "manifest.json"), "w"), indent=1)
    return man


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

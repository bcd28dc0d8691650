"""Data runtimes over prepared artifacts: packed, indexed-supervised and weighted blends.

All three read payload files through numpy memory maps, hand out `[B, L]` batches staged in
pinned memory and copied on a transfer stream one batch ahead, shard by data-parallel rank
(rank r takes batches r, r+DP, ...), and expose a resumable cursor in `state_dict()`.

* PackedTokenDataRuntime   – contiguous windows of `seq_len` tokens of tokens.i32, optional
  epoch-wise shuffle of the window order (seeded).
* IndexedSupervisedTokenDataRuntime – samples of index.i64 with their loss masks; a batch holds
  samples of one length (length buckets), padded up to the block size by the preparation step;
  samples shorter than `minimum_sequence_length` or not aligned to the block size are skipped.
  With `optimizer_step_unit="trajectory"` (artifacts with `groups.i64`) one optimizer step is one trajectory:
  its turns, in order, one sample per micro-batch, every data-parallel rank taking its own trajectory; the
  last turn carries `trajectory_terminal_turn_weight` for the `turn_mean` loss reduction.
* BlendedPackedTokenDataRuntime – several packed artifacts mixed by weight with a seeded
  multinomial choice per batch.

Counterparts: dllm_parallel/core/data.py:248-607 (packed), :610-1275 (indexed), :1277-1394
(blended), :1397-1530 (loaders).
"""
from __future__ import annotations

from pathlib import Path
from typing import Any

import numpy as np
import torch

from .artifacts import INDEXED_FORMAT, PACKED_TOKEN_FORMAT, ArtifactError, load_manifest
from .runtimes import DataBatch, DataRuntime


class _Stager:
    """Pinned double buffer + transfer stream (no-op on CPU)."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=self.device) if self.cuda else None

    def to_device(self, arr: np.ndarray, dtype=torch.int64) -> tuple[torch.Tensor, int]:
        host = torch.from_numpy(np.ascontiguousarray(arr)).to(dtype)
        if not self.cuda:
            return host, 0
        pinned = host.pin_memory()
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            dev = pinned.to(self.device, non_blocking=True)
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
        dev.record_stream(torch.cuda.current_stream(self.device))
        return dev, pinned.numel() * pinned.element_size()


SANITY_TEXT = ("Block diffusion language models denoise one block of tokens at a time, conditioned on the clean "
               "tokens before it. This sentence repeats so that a run can be checked without preparing a dataset. ")


class PackedTokenDataRuntime(DataRuntime):
    def __init__(self, root: str | Path | None, *, batch_size: int, seq_len: int, dp_rank: int = 0, dp_size: int = 1,
                 shuffle: bool = True, seed: int = 0, device="cpu", expected_fingerprint: str | None = None,
                 tokens: np.ndarray | None = None, fingerprint: str | None = None):
        """`root`: a packed-token artifact directory. Without one, `tokens` (a 1-D integer array, possibly
        memory-mapped) is the stream and `fingerprint` identifies it in checkpoints (`from_token_file`,
        `from_repeated_text`)."""
        if root is None:
            if tokens is None or fingerprint is None:
                raise ValueError("a packed runtime without an artifact directory needs tokens and a fingerprint")
            self.root, self.fingerprint, self.tokens = None, fingerprint, tokens
        else:
            self.root = Path(root)
            m = load_manifest(self.root)
            if m["format"] != PACKED_TOKEN_FORMAT:
                raise ArtifactError(f"{root} is not a packed-token artifact")
            self.fingerprint = m["metadata"]["dataset_fingerprint"]
            self.tokens = np.memmap(self.root / "tokens.i32", dtype="<i4", mode="r")
        if expected_fingerprint and expected_fingerprint != self.fingerprint:
            raise ArtifactError("dataset fingerprint differs from the one recorded in the checkpoint")
        self.batch_size, self.seq_len = batch_size, seq_len
        self.dp_rank, self.dp_size = dp_rank, dp_size
        self.windows = len(self.tokens) // seq_len
        if self.windows < batch_size * dp_size:
            raise ArtifactError(f"artifact has {self.windows} windows of {seq_len} tokens; one global batch needs "
                                f"{batch_size * dp_size}")
        self.shuffle, self.seed = shuffle, seed
        self.epoch, self.cursor = 0, 0      # cursor counts GLOBAL batches consumed in this epoch
        self.stager = _Stager(device)
        self._order = self._epoch_order(0)

    @classmethod
    def from_token_file(cls, path: str | Path, *, tokenizer=None, vocab_size: int | None = None, **kw):
        """A flat token file instead of a prepared artifact: raw little-endian `.i32 / .int32` and
        `.i64 / .int64 / .bin / .tokens` (memory-mapped), `.npy`, `.pt` (a tensor, or a mapping with `input_ids`,
        `tokens` or `data`), or any other file read as UTF-8 text and tokenised with `tokenizer`
        (dllm_parallel/core/data.py:1397-1440). The fingerprint is the SHA-256 of the file (plus the tokenizer name
        for text), so a resumed run refuses a different file."""
        from .artifacts import sha256_file

        path = Path(path)
        suffix = path.suffix.lower()
        ident = sha256_file(path)
        if suffix in (".i32", ".int32"):
            tokens = np.memmap(path, dtype="<i4", mode="r")
        elif suffix in (".i64", ".int64", ".bin", ".tokens"):
            if path.stat().st_size % 8:
                raise ArtifactError(f"{path}: an int64 token file has a size that divides by 8")
            tokens = np.memmap(path, dtype="<i8", mode="r")
        elif suffix == ".npy":
            tokens = np.load(path, mmap_mode="r").reshape(-1)
        elif suffix == ".pt":
            obj = torch.load(path, map_location="cpu", weights_only=True)
            if isinstance(obj, dict):
                key = next((k for k in ("input_ids", "tokens", "data") if k in obj), None)
                if key is None:
                    raise ArtifactError(f"{path}: expected a tensor or a mapping with input_ids / tokens / data")
                obj = obj[key]
            tokens = torch.as_tensor(obj).reshape(-1).numpy()
        else:
            if tokenizer is None:
                raise ArtifactError(f"{path} is read as text and needs a tokenizer (a model.id directory with one)")
            ids = tokenizer.encode(path.read_text(encoding="utf-8"), add_special_tokens=False)
            tokens = np.asarray(ids, dtype=np.int64)
            ident += ":" + str(getattr(tokenizer, "name_or_path", type(tokenizer).__name__))
        if tokens.size == 0:
            raise ArtifactError(f"{path} holds no tokens")
        if vocab_size is not None:
            # one pass over the stream: ids outside the vocabulary would index past the embedding table
            hi, lo = int(tokens.max()), int(tokens.min())
            if lo < 0 or hi >= vocab_size:
                raise ArtifactError(f"{path} holds token ids in [{lo}, {hi}], outside the model vocabulary of {vocab_size}")
        return cls(None, tokens=tokens, fingerprint="file:" + ident, **kw)

    @classmethod
    def from_repeated_text(cls, *, tokenizer, batch_size: int, seq_len: int, dp_size: int = 1, **kw):
        """`data.input_mode: text`: a built-in paragraph, tokenised and repeated until every rank has a batch; for
        checking a run end to end without a dataset (dllm_parallel/core/data.py:121-130)."""
        ids = np.asarray(tokenizer.encode(SANITY_TEXT, add_special_tokens=False), dtype=np.int64)
        need = seq_len * batch_size * dp_size * 4
        tokens = np.tile(ids, need // ids.size + 1)
        name = str(getattr(tokenizer, "name_or_path", type(tokenizer).__name__))
        return cls(None, tokens=tokens, fingerprint=f"repeated_text:{name}:{ids.size}", batch_size=batch_size,
                   seq_len=seq_len, dp_size=dp_size, **kw)

    def _epoch_order(self, epoch: int) -> np.ndarray:
        order = np.arange(self.windows)
        if self.shuffle:
            np.random.default_rng(self.seed + epoch).shuffle(order)
        return order

    def next_batch(self) -> DataBatch:
        per_global = self.batch_size * self.dp_size
        if (self.cursor + 1) * per_global > self.windows:
            self.epoch += 1
            self.cursor = 0
            self._order = self._epoch_order(self.epoch)
        base = self.cursor * per_global + self.dp_rank * self.batch_size
        idx = self._order[base: base + self.batch_size]
        rows = np.stack([self.tokens[i * self.seq_len:(i + 1) * self.seq_len] for i in idx])
        self.cursor += 1
        dev, nbytes = self.stager.to_device(rows)
        return DataBatch(dev, sample_ids=torch.from_numpy(idx.astype(np.int64)), h2d_bytes=nbytes)

    def state_dict(self) -> dict[str, Any]:
        return {"kind": "packed", "epoch": self.epoch, "cursor": self.cursor, "fingerprint": self.fingerprint,
                "seed": self.seed, "dp_size": self.dp_size}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        if state.get("fingerprint") != self.fingerprint:
            raise ArtifactError("checkpoint was written for a different dataset (fingerprint mismatch)")
        if state.get("dp_size") != self.dp_size:
            raise ArtifactError("data-parallel size changed since the checkpoint; the data cursor cannot be mapped")
        self.epoch, self.cursor = int(state["epoch"]), int(state["cursor"])
        self._order = self._epoch_order(self.epoch)


class IndexedSupervisedTokenDataRuntime(DataRuntime):
    def __init__(self, root: str | Path, *, batch_size: int, block_size: int, max_seq_len: int,
                 minimum_sequence_length: int | None = None, dp_rank: int = 0, dp_size: int = 1,
                 shuffle: bool = True, seed: int = 0, device="cpu", optimizer_step_unit: str = "microbatch",
                 terminal_turn_weight: float = 1.0, group_by_supervision_start: bool = False,
                 context_parallel_size: int = 1, block_parallel_size: int = 1):
        """Eligible samples fit `max_seq_len`, are whole blocks, give every block-parallel rank at least one block,
        and under pure context parallelism divide by the context-parallel degree
        (dllm_parallel/core/data.py:708-722)."""
        self.group_by_supervision_start = bool(group_by_supervision_start)
        self.root = Path(root)
        m = load_manifest(self.root)
        if m["format"] != INDEXED_FORMAT:
            raise ArtifactError(f"{root} is not an indexed supervised-token artifact")
        self.fingerprint = m["metadata"]["dataset_fingerprint"]
        self.tokens = np.memmap(self.root / "tokens.i32", dtype="<i4", mode="r")
        self.mask = np.memmap(self.root / "loss_mask.u8", dtype=np.uint8, mode="r")
        self.index = np.fromfile(self.root / "index.i64", dtype="<i8").reshape(-1, 4)
        lens = self.index[:, 1]
        shortest = max(int(block_parallel_size) * block_size, int(minimum_sequence_length or 1))
        ok = (lens % block_size == 0) & (lens <= max_seq_len) & (lens >= shortest)
        if context_parallel_size > 1 and block_parallel_size == 1:
            ok &= lens % int(context_parallel_size) == 0
        self.eligible = np.flatnonzero(ok)
        self.skipped = int((~ok).sum())
        if self.eligible.size == 0:
            raise ArtifactError("no sample is eligible: lengths must be multiples of the block size, fit seq_len and give "
                                "every block-parallel rank a block")
        self.batch_size, self.dp_rank, self.dp_size = batch_size, dp_rank, dp_size
        self.shuffle, self.seed = shuffle, seed
        self.epoch, self.cursor = 0, 0
        self.stager = _Stager(device)
        self.step_unit, self.terminal_turn_weight = optimizer_step_unit, float(terminal_turn_weight)
        self.groups = None
        if optimizer_step_unit == "trajectory":
            gpath = self.root / "groups.i64"
            if not gpath.exists():
                raise ArtifactError("data.optimizer_step_unit=trajectory needs an artifact with groups.i64 "
                                    "(prepare it with records.group_column)")
            self.groups = np.fromfile(gpath, dtype="<i8")
            self._trajectories = self._epoch_trajectories(0)
            self._batches = []
        else:
            self._batches = self._epoch_batches(0)

    def _epoch_trajectories(self, epoch: int) -> list[np.ndarray]:
        """Trajectories (samples of one group id, in file order), shuffled per epoch. A trajectory with a turn
        that is not eligible (length off the block grid, too long) is an error: turns are never dropped silently
        (dllm_parallel/core/data.py:966-1010)."""
        eligible = np.zeros(len(self.index), dtype=bool)
        eligible[self.eligible] = True
        order = np.argsort(self.groups, kind="stable")
        gids, starts = np.unique(self.groups[order], return_index=True)
        trajs = np.split(order, starts[1:])
        partial = [int(g) for g, t in zip(gids, trajs) if not eligible[t].all()]
        if partial:
            raise ArtifactError(f"trajectory steps cannot omit ineligible turns; {len(partial)} trajectories have "
                                f"one (first group id {partial[0]})")
        trajs = [np.sort(t) for t in trajs]
        if self.shuffle and len(trajs) > 1:
            perm = np.random.default_rng(self.seed + epoch).permutation(len(trajs))
            trajs = [trajs[i] for i in perm]
        if len(trajs) < self.dp_size:
            raise ArtifactError(f"{len(trajs)} trajectories cannot feed {self.dp_size} data-parallel ranks")
        return trajs

    def _sample_batch(self, ids: np.ndarray, turn_weight: float | None = None) -> DataBatch:
        toks = np.stack([self.tokens[o:o + n] for o, n in self.index[ids, :2]])
        msk = np.stack([self.mask[o:o + n] for o, n in self.index[ids, :2]])
        dev, nb = self.stager.to_device(toks)
        dmask, nb2 = self.stager.to_device(msk, torch.bool)
        return DataBatch(dev, supervision_mask=dmask, supervision_count=int(msk.sum()),
                         sample_ids=torch.from_numpy(self.index[ids, 3].copy()), h2d_bytes=nb + nb2,
                         turn_weight=turn_weight, supervision_count_shifted=int(msk[:, 1:].sum()))

    def next_optimizer_step_batches(self, micro_batches: int) -> list[DataBatch]:
        if self.step_unit != "trajectory":
            return super().next_optimizer_step_batches(micro_batches)
        per_global = self.dp_size
        if (self.cursor + 1) * per_global > len(self._trajectories):
            self.epoch += 1
            self.cursor = 0
            self._trajectories = self._epoch_trajectories(self.epoch)
        traj = self._trajectories[self.cursor * per_global + self.dp_rank]
        self.cursor += 1
        out = []
        for j, i in enumerate(traj):
            w = self.terminal_turn_weight if j == len(traj) - 1 else 1.0
            out.append(self._sample_batch(np.array([i]), turn_weight=w))
        return out

    def _epoch_batches(self, epoch: int) -> list[np.ndarray]:
        """Global batches of same-length samples; every DP rank takes a `batch_size` slice."""
        rng = np.random.default_rng(self.seed + epoch)
        per_global = self.batch_size * self.dp_size
        out = []
        lens = self.index[self.eligible, 1]
        if self.group_by_supervision_start:
            # one bucket per (length, first supervised position): a batch then shares its response start, which lets
            # the native-SFT objective pack the response suffix instead of masking
            key = lens * (int(self.index[:, 2].max()) + 1) + self.index[self.eligible, 2]
        else:
            key = lens
        for L in np.unique(key):
            ids = self.eligible[key == L]
            if self.shuffle:
                rng.shuffle(ids)
            for i in range(0, len(ids) - per_global + 1, per_global):
                out.append(ids[i:i + per_global])
        if not out:
            raise ArtifactError(f"no bucket of equal length{' and response start' if self.group_by_supervision_start else ''} "
                                f"holds a full global batch of {per_global} samples")
        if self.shuffle:
            rng.shuffle(out)
        return out

    def next_batch(self) -> DataBatch:
        if self.step_unit == "trajectory":
            raise ArtifactError("trajectory step units hand out whole optimizer steps (next_optimizer_step_batches)")
        if self.cursor >= len(self._batches):
            self.epoch += 1
            self.cursor = 0
            self._batches = self._epoch_batches(self.epoch)
        ids = self._batches[self.cursor][self.dp_rank * self.batch_size:(self.dp_rank + 1) * self.batch_size]
        self.cursor += 1
        return self._sample_batch(ids)

    def state_dict(self):
        return {"kind": "indexed", "epoch": self.epoch, "cursor": self.cursor, "fingerprint": self.fingerprint,
                "seed": self.seed, "dp_size": self.dp_size, "step_unit": self.step_unit}

    def load_state_dict(self, state):
        if state.get("fingerprint") != self.fingerprint:
            raise ArtifactError("checkpoint was written for a different dataset (fingerprint mismatch)")
        if state.get("step_unit", "microbatch") != self.step_unit:
            raise ArtifactError("data.optimizer_step_unit changed since the checkpoint")
        self.epoch, self.cursor = int(state["epoch"]), int(state["cursor"])
        if self.step_unit == "trajectory":
            self._trajectories = self._epoch_trajectories(self.epoch)
        else:
            self._batches = self._epoch_batches(self.epoch)


class BlendedPackedTokenDataRuntime(DataRuntime):
    """dataset_path = "w1:path1,w2:path2": each batch comes from one member chosen with probability ∝ weight."""

    def __init__(self, members: list[tuple[float, PackedTokenDataRuntime]], seed: int = 0):
        w = np.array([m[0] for m in members], dtype=np.float64)
        if (w <= 0).any():
            raise ArtifactError("blend weights must be positive")
        self.p = w / w.sum()
        self.members = [m[1] for m in members]
        self.seed, self.draws = seed, 0

    def next_batch(self) -> DataBatch:
        k = int(np.random.default_rng([self.seed, self.draws]).choice(len(self.members), p=self.p))
        self.draws += 1
        return self.members[k].next_batch()

    def state_dict(self):
        return {"kind": "blended", "draws": self.draws, "seed": self.seed,
                "members": [m.state_dict() for m in self.members]}

    def load_state_dict(self, state):
        self.draws = int(state["draws"])
        for m, s in zip(self.members, state["members"]):
            m.load_state_dict(s)


class _ByteTextTokenizer:
    """UTF-8 bytes as token ids: the stand-in when the run's model has no tokenizer on disk (synthetic presets)."""
    name_or_path = "utf8-bytes"

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return list(text.encode("utf-8"))


def _run_tokenizer(spec):
    """The tokenizer that ships with the run's model (or verifier) checkpoint directory; bytes otherwise."""
    from ..models.hf_loader import pretrained_directory

    for mid in (spec.model.id, spec.model.verifier_id):
        d = pretrained_directory(mid)
        if d is not None:
            try:
                from transformers import AutoTokenizer

                return AutoTokenizer.from_pretrained(d)
            except Exception:       # a checkpoint directory without tokenizer files
                continue
    return _ByteTextTokenizer()


def build_artifact_runtime(spec, *, device, dp_rank: int, dp_size: int) -> DataRuntime:
    """Chooses the runtime from the artifact's manifest (and the `w:path,...` blend syntax)."""
    path = spec.data.dataset_path
    common = dict(batch_size=spec.training.batch_size, dp_rank=dp_rank, dp_size=dp_size, shuffle=spec.data.shuffle,
                  device=device)
    if spec.data.input_mode == "text":
        return PackedTokenDataRuntime.from_repeated_text(tokenizer=_run_tokenizer(spec), seq_len=spec.model.seq_len,
                                                         seed=spec.launch.seed, **common)
    def member(p: Path, seed: int) -> PackedTokenDataRuntime:
        """One packed stream: a prepared artifact directory, a flat token file or a text file."""
        if p.is_dir():
            return PackedTokenDataRuntime(p, seq_len=spec.model.seq_len, seed=seed, **common)
        binary = p.suffix.lower() in (".i32", ".int32", ".i64", ".int64", ".bin", ".tokens", ".npy", ".pt")
        from ..models.config import model_config_from_run_spec

        return PackedTokenDataRuntime.from_token_file(
            p, tokenizer=None if binary else _run_tokenizer(spec), seq_len=spec.model.seq_len, seed=seed,
            vocab_size=model_config_from_run_spec(spec).vocab_size, **common)

    if Path(path).is_file() and Path(path).suffix.lower() == ".json":
        # a blend manifest: {"datasets": [{"path": ..., "weight": ...}, ...]} (or the bare list); relative member
        # paths are relative to the manifest (dllm_parallel/core/data.py:1302-1345)
        import json

        doc = json.loads(Path(path).read_text())
        entries = doc.get("datasets") if isinstance(doc, dict) else doc
        if not isinstance(entries, list) or not entries or not all(isinstance(e, dict) and e.get("path") for e in entries):
            raise ArtifactError(f"{path}: a blend manifest holds a non-empty `datasets` list of {{path, weight}} entries")
        members = []
        for e in entries:
            p = Path(str(e["path"]))
            p = p if p.is_absolute() else Path(path).parent / p
            members.append((float(e.get("weight", 1.0)), member(p, spec.data.blend_seed)))
        return BlendedPackedTokenDataRuntime(members, seed=spec.data.blend_seed)
    if Path(path).is_file():       # a flat token file or a text file instead of a prepared artifact
        return member(Path(path), spec.launch.seed)
    if "," in path or (":" in path and not Path(path).exists()):
        members = []
        for item in path.split(","):
            w, _, p = item.partition(":")
            members.append((float(w), PackedTokenDataRuntime(p, seq_len=spec.model.seq_len, seed=spec.data.blend_seed,
                                                             **common)))
        return BlendedPackedTokenDataRuntime(members, seed=spec.data.blend_seed)
    m = load_manifest(path)
    if m["format"] == PACKED_TOKEN_FORMAT:
        return PackedTokenDataRuntime(path, seq_len=spec.model.seq_len, seed=spec.launch.seed, **common)
    return IndexedSupervisedTokenDataRuntime(
        path, block_size=spec.objective.block_size or 1, max_seq_len=spec.model.seq_len,
        minimum_sequence_length=spec.data.minimum_sequence_length, seed=spec.launch.seed,
        optimizer_step_unit=spec.data.optimizer_step_unit,
        terminal_turn_weight=spec.data.trajectory_terminal_turn_weight,
        group_by_supervision_start=spec.objective.name == "diffusiongemma_native_sft",
        context_parallel_size=spec.topology.context_parallel_size, block_parallel_size=spec.topology.block_parallel_size,
        **common)

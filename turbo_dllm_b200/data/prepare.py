"""Offline data preparation (`dllm data prepare`): source records → formatted text / messages →
token ids + supervision mask → packed or indexed artifact, installed atomically.

`PreparationSpec` (format `dllm.data.prepare.v1`) has six strict sections:
  source      kind huggingface | jsonl | parquet | text | pretokenized (+ registered plug-ins), path(s), split
  records     type text | messages | prompt_completion | pretokenized and the column names
  tokenizer   model (HF id / local path) or the built-in `byte` tokenizer, add_eos, chat template
  supervision full | assistant_only | completion_only | provided
  packing     mode packed | indexed, sequence_length, overflow reject | split | truncate_left | truncate_right,
              alignment (pad sample lengths to a multiple, e.g. the diffusion block size)
  output      path, overwrite
Output is written to a staging directory next to the target and moved into place with
os.replace (the previous artifact is kept as a backup until the move succeeded).

Counterparts: dllm_parallel/data/schemas.py:23-208, prepare.py:52-267, sources.py:24-328,
formatting.py:24-262, tokenization.py:21-346, packing.py:44-164, registry.py:47-151.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterable, Iterator, Mapping

import numpy as np
import yaml

from .artifacts import ArtifactError, write_indexed_artifact, write_packed_artifact

PREPARE_FORMAT = "dllm.data.prepare.v1"
_SECTION_FIELDS = {
    "source": {"kind": "jsonl", "path": None, "paths": None, "split": "train", "name": None, "streaming": False,
               "limit": None},
    "records": {"type": "text", "text_column": "text", "messages_column": "messages", "prompt_column": "prompt",
                "completion_column": "completion", "tokens_column": "input_ids", "mask_column": "loss_mask",
                "group_column": None},
    "tokenizer": {"model": "byte", "revision": None, "add_bos": False, "add_eos": True, "chat_template": None,
                  "mask_token_id": None},
    "supervision": {"mode": "full"},
    "packing": {"mode": "packed", "sequence_length": None, "overflow": "split", "alignment": 1,
                "minimum_length": 1, "pad_token_id": None},
    "output": {"path": None, "overwrite": False},
}
_CHOICES = {
    ("source", "kind"): ("huggingface", "jsonl", "parquet", "text", "pretokenized"),
    ("records", "type"): ("text", "messages", "prompt_completion", "pretokenized"),
    ("supervision", "mode"): ("full", "assistant_only", "completion_only", "provided"),
    ("packing", "mode"): ("packed", "indexed"),
    ("packing", "overflow"): ("reject", "split", "truncate_left", "truncate_right"),
}


class PreparationError(ValueError):
    pass


@dataclass(frozen=True)
class PreparationSpec:
    source: dict
    records: dict
    tokenizer: dict
    supervision: dict
    packing: dict
    output: dict

    @classmethod
    def from_mapping(cls, m: Mapping[str, Any]) -> "PreparationSpec":
        m = dict(m or {})
        fmt = m.pop("format", PREPARE_FORMAT)
        if fmt != PREPARE_FORMAT:
            raise PreparationError(f"unsupported preparation format {fmt!r} (expected {PREPARE_FORMAT})")
        unknown = sorted(set(m) - set(_SECTION_FIELDS))
        if unknown:
            raise PreparationError(f"unknown section(s): {', '.join(unknown)}")
        secs = {}
        for sec, defaults in _SECTION_FIELDS.items():
            raw = dict(m.get(sec) or {})
            bad = sorted(set(raw) - set(defaults))
            if bad:
                raise PreparationError(f"unknown field(s) in section '{sec}': {', '.join(bad)}")
            secs[sec] = {**defaults, **raw}
        spec = cls(**secs)
        spec.validate()
        return spec

    def validate(self) -> None:
        for (sec, key), choices in _CHOICES.items():
            v = getattr(self, sec)[key]
            if v not in choices and not (sec == "source" and v in SOURCE_REGISTRY):
                raise PreparationError(f"{sec}.{key}={v!r} is not one of {choices}")
        if not (self.source["path"] or self.source["paths"] or self.source["name"]):
            raise PreparationError("source needs path, paths or name")
        if not self.output["path"]:
            raise PreparationError("output.path is required")
        p = self.packing
        if p["mode"] == "packed" and p["overflow"] == "reject" and not p["sequence_length"]:
            raise PreparationError("packing.overflow=reject needs packing.sequence_length")
        if p["alignment"] < 1:
            raise PreparationError("packing.alignment must be >= 1")
        if self.supervision["mode"] == "assistant_only" and self.records["type"] != "messages":
            raise PreparationError("supervision.mode=assistant_only needs records.type=messages")
        if self.supervision["mode"] == "completion_only" and self.records["type"] != "prompt_completion":
            raise PreparationError("supervision.mode=completion_only needs records.type=prompt_completion")
        if self.supervision["mode"] == "provided" and self.records["type"] != "pretokenized":
            raise PreparationError("supervision.mode=provided needs records.type=pretokenized")

    def sanitized(self) -> dict:
        d = {k: dict(getattr(self, k)) for k in _SECTION_FIELDS}
        d["format"] = PREPARE_FORMAT
        return d


def load_preparation_spec(path: str | Path) -> PreparationSpec:
    text = Path(path).read_text()
    data = json.loads(text) if str(path).endswith(".json") else yaml.safe_load(text)
    return PreparationSpec.from_mapping(data)


# ------------------------------------------------------------------ sources
SOURCE_REGISTRY: dict[str, Callable[[dict], Iterator[dict]]] = {}


def register_source(kind: str, fn: Callable[[dict], Iterator[dict]]) -> None:
    SOURCE_REGISTRY[kind] = fn


def _paths(src: dict) -> list[Path]:
    raw = [src["path"]] if src.get("path") else list(src.get("paths") or [])
    out: list[Path] = []
    for r in raw:
        p = Path(r)
        out += sorted(p.iterdir()) if p.is_dir() else [p]
    return out


def iter_source_records(src: dict) -> Iterator[dict]:
    kind = src["kind"]
    limit = src.get("limit")
    n = 0

    def gen():
        if kind in SOURCE_REGISTRY:
            yield from SOURCE_REGISTRY[kind](src)
        elif kind in ("jsonl", "pretokenized"):
            for p in _paths(src):
                with open(p) as f:
                    for line in f:
                        if line.strip():
                            yield json.loads(line)
        elif kind == "text":
            for p in _paths(src):
                yield {"text": Path(p).read_text()}
        elif kind == "parquet":
            import pyarrow.parquet as pq

            for p in _paths(src):
                for batch in pq.ParquetFile(p).iter_batches():
                    yield from batch.to_pylist()
        elif kind == "huggingface":
            try:
                import datasets
            except ImportError:
                raise PreparationError("source.kind=huggingface needs the `datasets` package") from None
            ds = datasets.load_dataset(src["name"] or src["path"], split=src["split"], streaming=src["streaming"])
            yield from ds
        else:
            raise PreparationError(f"unknown source kind {kind!r}")

    for rec in gen():
        yield rec
        n += 1
        if limit and n >= limit:
            return


def source_provenance(src: dict) -> dict:
    files = []
    if src["kind"] in ("jsonl", "pretokenized", "text", "parquet"):
        for p in _paths(src):
            h = hashlib.sha256()
            with open(p, "rb") as f:
                for chunk in iter(lambda: f.read(1 << 20), b""):
                    h.update(chunk)
            files.append({"name": p.name, "path": str(p), "bytes": p.stat().st_size, "sha256": h.hexdigest()})
    return {"kind": src["kind"], "split": src.get("split"), "name": src.get("name"), "files": files}


# --------------------------------------------------------------- tokenizers
class ByteTokenizer:
    """UTF-8 bytes 0..255, then <bos>=256, <eos>=257, <mask>=258, role markers 259.."""

    vocab_size = 264
    bos_token_id, eos_token_id, mask_token_id = 256, 257, 258
    name = "byte"
    ROLE = {"system": 259, "user": 260, "assistant": 261, "tool": 262}
    END_TURN = 263

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def vocab_sha256(self) -> str:
        return hashlib.sha256(b"turbo_dllm_b200.byte_tokenizer.v1").hexdigest()


class HFTokenizer:
    def __init__(self, model: str, revision: str | None):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(model, revision=revision)
        self.name = model
        self.vocab_size = len(self.tok)
        self.bos_token_id, self.eos_token_id = self.tok.bos_token_id, self.tok.eos_token_id
        self.mask_token_id = getattr(self.tok, "mask_token_id", None)

    def encode(self, text: str) -> list[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def vocab_sha256(self) -> str:
        return hashlib.sha256(json.dumps(self.tok.get_vocab(), sort_keys=True).encode()).hexdigest()


def build_tokenizer(tcfg: dict):
    return ByteTokenizer() if tcfg["model"] == "byte" else HFTokenizer(tcfg["model"], tcfg.get("revision"))


# ------------------------------------------------ formatting + tokenization
@dataclass
class TokenizedRecord:
    tokens: np.ndarray      # int32
    loss_mask: np.ndarray   # uint8, same length
    sample_id: int
    group: int | None = None


def tokenize_record(rec: Mapping[str, Any], spec: PreparationSpec, tok, sample_id: int) -> TokenizedRecord | None:
    r, tc, mode = spec.records, spec.tokenizer, spec.supervision["mode"]
    ids: list[int] = []
    mask: list[int] = []

    def add(piece: list[int], supervised: bool):
        ids.extend(piece)
        mask.extend([1 if supervised else 0] * len(piece))

    if tc["add_bos"] and tok.bos_token_id is not None:
        add([tok.bos_token_id], False)
    t = r["type"]
    if t == "text":
        text = rec.get(r["text_column"])
        if not isinstance(text, str) or not text:
            return None
        add(tok.encode(text), True)
    elif t == "prompt_completion":
        prompt, completion = rec.get(r["prompt_column"], ""), rec.get(r["completion_column"], "")
        if not completion:
            return None
        add(tok.encode(prompt), mode != "completion_only")
        add(tok.encode(completion), True)
    elif t == "messages":
        msgs = rec.get(r["messages_column"])
        if not msgs:
            return None
        for msg in msgs:
            role, content = msg.get("role", "user"), msg.get("content", "")
            sup = (role == "assistant") if mode == "assistant_only" else True
            if isinstance(tok, ByteTokenizer):
                add([tok.ROLE.get(role, tok.ROLE["user"])], False)
                add(tok.encode(content), sup)
                add([tok.END_TURN], sup)
            else:
                add(tok.encode(f"<|im_start|>{role}\n"), False)
                add(tok.encode(content + "<|im_end|>\n"), sup)
    elif t == "pretokenized":
        toks = rec.get(r["tokens_column"])
        if not toks:
            return None
        m = rec.get(r["mask_column"]) if mode == "provided" else None
        if m is not None and len(m) != len(toks):
            raise PreparationError(f"record {sample_id}: loss mask length differs from token length")
        ids.extend(int(x) for x in toks)
        mask.extend([int(bool(x)) for x in m] if m is not None else [1] * len(toks))
    if tc["add_eos"] and tok.eos_token_id is not None and t != "pretokenized":
        add([tok.eos_token_id], True)
    if not ids:
        return None
    grp = rec.get(r["group_column"]) if r.get("group_column") else None
    return TokenizedRecord(np.asarray(ids, dtype=np.int32), np.asarray(mask, dtype=np.uint8), sample_id,
                           int(grp) if grp is not None else None)


# ----------------------------------------------------------------- packing
def apply_overflow(rec: TokenizedRecord, limit: int | None, overflow: str) -> list[TokenizedRecord]:
    if not limit or rec.tokens.size <= limit:
        return [rec]
    if overflow == "reject":
        raise PreparationError(f"sample {rec.sample_id} has {rec.tokens.size} tokens > sequence_length {limit}")
    if overflow == "truncate_right":
        return [TokenizedRecord(rec.tokens[:limit], rec.loss_mask[:limit], rec.sample_id, rec.group)]
    if overflow == "truncate_left":
        return [TokenizedRecord(rec.tokens[-limit:], rec.loss_mask[-limit:], rec.sample_id, rec.group)]
    return [TokenizedRecord(rec.tokens[i:i + limit], rec.loss_mask[i:i + limit], rec.sample_id, rec.group)
            for i in range(0, rec.tokens.size, limit)]


def align_record(rec: TokenizedRecord, alignment: int, pad_id: int) -> TokenizedRecord:
    if alignment <= 1 or rec.tokens.size % alignment == 0:
        return rec
    pad = alignment - rec.tokens.size % alignment
    return TokenizedRecord(np.concatenate([rec.tokens, np.full(pad, pad_id, np.int32)]),
                           np.concatenate([rec.loss_mask, np.zeros(pad, np.uint8)]), rec.sample_id, rec.group)


# ----------------------------------------------------------------- driver
def prepare_dataset(spec: PreparationSpec) -> dict:
    """Runs the whole pipeline and returns the manifest of the installed artifact."""
    out = Path(spec.output["path"])
    if out.exists() and not spec.output["overwrite"]:
        raise PreparationError(f"{out} exists; set output.overwrite=true to replace it")
    tok = build_tokenizer(spec.tokenizer)
    pk = spec.packing
    pad_id = pk["pad_token_id"] if pk["pad_token_id"] is not None else (tok.eos_token_id or 0)
    mask_id = spec.tokenizer["mask_token_id"] if spec.tokenizer["mask_token_id"] is not None else tok.mask_token_id
    counters = {"source_records": 0, "empty_records": 0, "split_records": 0, "source_tokens": 0, "short_records": 0}
    saw_mask = {"v": False}

    def records() -> Iterator[TokenizedRecord]:
        for i, raw in enumerate(iter_source_records(spec.source)):
            counters["source_records"] += 1
            rec = tokenize_record(raw, spec, tok, i)
            if rec is None:
                counters["empty_records"] += 1
                continue
            counters["source_tokens"] += int(rec.tokens.size)
            if mask_id is not None and (rec.tokens == mask_id).any():
                saw_mask["v"] = True
            parts = apply_overflow(rec, pk["sequence_length"], pk["overflow"])
            counters["split_records"] += len(parts) > 1
            for part in parts:
                if part.tokens.size < pk["minimum_length"]:
                    counters["short_records"] += 1
                    continue
                yield align_record(part, pk["alignment"], pad_id) if pk["mode"] == "indexed" else part

    metadata = {
        "tokenizer": {"model": tok.name, "revision": spec.tokenizer.get("revision"), "vocab_size": tok.vocab_size,
                      "vocab_sha256": tok.vocab_sha256(),
                      "chat_template_sha256": hashlib.sha256((spec.tokenizer.get("chat_template") or "").encode()).hexdigest()},
        "mask_token_id": mask_id, "eos_token_id": tok.eos_token_id, "pad_token_id": pad_id,
        "block_size": pk["alignment"] if pk["alignment"] > 1 else None,
        "semantics": "full_sequence" if pk["mode"] == "packed" else "supervised_samples",
        "sampling_policy": "contiguous_windows" if pk["mode"] == "packed" else "one_sample_per_row",
        "sequence_layout": pk["mode"], "supervision_shape": spec.supervision["mode"],
        "preparation": spec.sanitized(), "source": source_provenance(spec.source),
    }
    staging = out.parent / f".{out.name}.staging-{os.getpid()}"
    if staging.exists():
        shutil.rmtree(staging)
    out.parent.mkdir(parents=True, exist_ok=True)
    try:
        if pk["mode"] == "packed":
            segs = (r.tokens for r in records())
            # contains_mask_token is only known after the stream ran: write, then patch through a rebuild
            manifest = write_packed_artifact(staging, segs, metadata={**metadata, "contains_mask_token": None},
                                             stats=counters)
        else:
            samples = ({"tokens": r.tokens, "loss_mask": r.loss_mask, "sample_id": r.sample_id,
                        "group": r.group if r.group is not None else r.sample_id} for r in records())
            manifest = write_indexed_artifact(staging, samples, metadata={**metadata, "contains_mask_token": None},
                                              with_groups=bool(spec.records.get("group_column")))
        # finalise fields that depend on the streamed content, then re-fingerprint
        from .artifacts import build_manifest, write_manifest

        md = dict(manifest["metadata"])
        md["contains_mask_token"] = bool(saw_mask["v"])
        stats = {**manifest["stats"], **counters}
        manifest = build_manifest(format_name=manifest["format"], metadata=md, files=manifest["files"], stats=stats,
                                  sample_count=manifest["sample_count"], token_count=manifest["token_count"])
        write_manifest(staging, manifest)
        backup = None
        if out.exists():
            backup = out.parent / f".{out.name}.backup-{os.getpid()}"
            os.replace(out, backup)
        try:
            os.replace(staging, out)
        except OSError:
            if backup is not None:
                os.replace(backup, out)
            raise
        if backup is not None:
            shutil.rmtree(backup, ignore_errors=True)
        return manifest
    except (ArtifactError, PreparationError):
        shutil.rmtree(staging, ignore_errors=True)
        raise
    except Exception:
        shutil.rmtree(staging, ignore_errors=True)
        raise

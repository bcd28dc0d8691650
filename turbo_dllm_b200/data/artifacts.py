"""Prepared-data artifact format: writers, manifest, fingerprint, validation.

An artifact is a directory with `manifest.json` and raw little-endian payload files:
  packed  (`dllm_parallel.packed_tokens`)             : tokens.i32
  indexed (`dllm_parallel.indexed_supervised_tokens`) : tokens.i32, index.i64 (columns token_offset,
            sequence_length, supervision_start, sample_id), loss_mask.u8 (uint8_per_token_v1), optional groups.i64
The manifest carries format, version 1, created_at, metadata (tokenizer identity, ids, block size,
preparation spec, provenance, `dataset_fingerprint`), sample_count, token_count, per-file
{dtype, elements, bytes, sha256[, columns]} and stats. The fingerprint is the SHA-256 of the
canonical JSON (sorted keys, compact separators, UTF-8) of format + version + metadata without
paths + the files' {columns, dtype, elements, sha256} + counts, so two preparations of the same
input agree byte for byte and with the reference's writer.

Format contract: dllm_parallel/data/indexed.py:50-234 (writers), :431-498 (manifest, fingerprint),
:257-428 (validation and run compatibility); dllm_parallel/data/provenance.py:15-36.
"""
from __future__ import annotations

import copy
import hashlib
import json
import os
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, Iterable, Mapping

import numpy as np

PACKED_TOKEN_FORMAT = "dllm_parallel.packed_tokens"
INDEXED_FORMAT = "dllm_parallel.indexed_supervised_tokens"
FORMAT_VERSION = 1
INDEX_COLUMNS = ["token_offset", "sequence_length", "supervision_start", "sample_id"]
LOSS_MASK_ENCODING = "uint8_per_token_v1"


class ArtifactError(ValueError):
    pass


def canonical_json_bytes(value: Any) -> bytes:
    return json.dumps(value, ensure_ascii=False, separators=(",", ":"), sort_keys=True).encode("utf-8")


def sha256_bytes(value: bytes) -> str:
    return hashlib.sha256(value).hexdigest()


def sha256_file(path: str | Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def file_metadata(path: Path, dtype: str, elements: int, columns: list[str] | None = None) -> dict:
    meta = {"dtype": dtype, "elements": int(elements), "bytes": path.stat().st_size, "sha256": sha256_file(path)}
    if columns is not None:
        meta["columns"] = list(columns)
    return meta


def dataset_fingerprint(*, format_name: str, version: int, metadata: Mapping[str, Any], files: Mapping[str, Any],
                        sample_count: int, token_count: int) -> str:
    stable = copy.deepcopy(dict(metadata))
    stable.pop("dataset_fingerprint", None)
    source = stable.get("source")
    if isinstance(source, dict) and isinstance(source.get("files"), list):
        for item in source["files"]:
            if isinstance(item, dict):
                item.pop("path", None)
    prep = stable.get("preparation")
    if isinstance(prep, dict) and isinstance(prep.get("source"), dict):
        prep["source"].pop("path", None)
        prep["source"].pop("paths", None)
    if isinstance(prep, dict) and isinstance(prep.get("output"), dict):
        prep["output"].pop("path", None)          # where the artifact was written says nothing about its contents
        prep["output"].pop("overwrite", None)
    payload = {"format": format_name, "version": version, "metadata": stable,
               "files": {name: {k: v for k, v in fm.items() if k in {"columns", "dtype", "elements", "sha256"}}
                         for name, fm in files.items()},
               "sample_count": sample_count, "token_count": token_count}
    return sha256_bytes(canonical_json_bytes(payload))


def build_manifest(*, format_name: str, metadata: dict, files: dict, stats: dict, sample_count: int,
                   token_count: int) -> dict:
    metadata = dict(metadata)
    metadata["dataset_fingerprint"] = dataset_fingerprint(
        format_name=format_name, version=FORMAT_VERSION, metadata=metadata, files=files,
        sample_count=sample_count, token_count=token_count)
    return {"format": format_name, "version": FORMAT_VERSION, "created_at": datetime.now(timezone.utc).isoformat(),
            "metadata": metadata, "sample_count": sample_count, "token_count": token_count, "files": files,
            "stats": stats}


def write_manifest(root: Path, manifest: dict) -> None:
    tmp = root / ".manifest.json.tmp"
    tmp.write_text(json.dumps(manifest, indent=2, sort_keys=True, ensure_ascii=False))
    os.replace(tmp, root / "manifest.json")


# ------------------------------------------------------------------ writers
def write_packed_artifact(root: str | Path, segments: Iterable[np.ndarray], *, metadata: Mapping[str, Any],
                          stats: Mapping[str, Any] | None = None, record_count: int | None = None) -> dict:
    """segments: int32 arrays appended to tokens.i32 in order (documents already joined / split)."""
    root = Path(root)
    root.mkdir(parents=True, exist_ok=False)
    total, nseg = 0, 0
    with open(root / "tokens.i32", "wb") as f:
        for seg in segments:
            arr = np.ascontiguousarray(seg, dtype="<i4")
            f.write(arr.tobytes())
            total += arr.size
            nseg += 1
    if total <= 0:
        raise ArtifactError("prepared packed dataset contains no tokens")
    files = {"tokens.i32": file_metadata(root / "tokens.i32", "int32", total)}
    st = {"records": record_count if record_count is not None else nseg, "stored_tokens": total}
    st.update(stats or {})
    manifest = build_manifest(format_name=PACKED_TOKEN_FORMAT, metadata=dict(metadata), files=files, stats=st,
                              sample_count=st["records"], token_count=total)
    write_manifest(root, manifest)
    return manifest


def write_indexed_artifact(root: str | Path, samples: Iterable[Mapping[str, Any]], *, metadata: Mapping[str, Any],
                           with_groups: bool = False) -> dict:
    """samples: {"tokens": int array, "loss_mask": bool/uint8 array (same length), "sample_id": int,
    "supervision_start": int (optional; default = first supervised position), "group": int (optional)}."""
    root = Path(root)
    root.mkdir(parents=True, exist_ok=False)
    offset, count, supervised = 0, 0, 0
    with open(root / "tokens.i32", "wb") as ft, open(root / "index.i64", "wb") as fi, \
            open(root / "loss_mask.u8", "wb") as fm:
        fg = open(root / "groups.i64", "wb") if with_groups else None
        try:
            for s in samples:
                tok = np.ascontiguousarray(s["tokens"], dtype="<i4")
                mask = np.ascontiguousarray(s["loss_mask"], dtype=np.uint8)
                if tok.ndim != 1 or mask.shape != tok.shape or tok.size == 0:
                    raise ArtifactError("each sample needs 1-D tokens and a loss mask of the same length")
                nz = np.flatnonzero(mask)
                start = int(s.get("supervision_start", nz[0] if nz.size else tok.size))
                ft.write(tok.tobytes())
                fm.write(mask.tobytes())
                fi.write(np.array([offset, tok.size, start, int(s.get("sample_id", count))], dtype="<i8").tobytes())
                if fg is not None:
                    fg.write(np.array([int(s.get("group", count))], dtype="<i8").tobytes())
                offset += tok.size
                supervised += int(mask.sum())
                count += 1
        finally:
            if fg is not None:
                fg.close()
    if count == 0:
        raise ArtifactError("prepared indexed dataset contains no samples")
    files = {"tokens.i32": file_metadata(root / "tokens.i32", "int32", offset),
             "index.i64": file_metadata(root / "index.i64", "int64", count * 4, INDEX_COLUMNS),
             "loss_mask.u8": file_metadata(root / "loss_mask.u8", "uint8", offset)}
    if with_groups:
        files["groups.i64"] = file_metadata(root / "groups.i64", "int64", count)
    md = dict(metadata)
    md.setdefault("loss_mask_encoding", LOSS_MASK_ENCODING)
    manifest = build_manifest(format_name=INDEXED_FORMAT, metadata=md, files=files,
                              stats={"samples": count, "stored_tokens": offset, "supervised_tokens": supervised},
                              sample_count=count, token_count=offset)
    write_manifest(root, manifest)
    return manifest


# --------------------------------------------------------------- validation
_DTYPES = {"int32": "<i4", "int64": "<i8", "uint8": "u1"}


def load_manifest(root: str | Path) -> dict:
    p = Path(root) / "manifest.json"
    if not p.exists():
        raise ArtifactError(f"{root} has no manifest.json")
    try:
        m = json.loads(p.read_text())
    except ValueError as e:
        raise ArtifactError(f"{p} is not valid JSON: {e}") from None
    if m.get("format") not in (PACKED_TOKEN_FORMAT, INDEXED_FORMAT):
        raise ArtifactError(f"unknown artifact format {m.get('format')!r}")
    if m.get("version") != FORMAT_VERSION:
        raise ArtifactError(f"unsupported artifact version {m.get('version')!r}")
    return m


def validate_artifact(root: str | Path, *, check_hashes: bool = True) -> dict:
    """Structural + integrity check. Raises ArtifactError with the first problem found."""
    root = Path(root)
    m = load_manifest(root)
    for name, fm in m["files"].items():
        path = root / name
        if not path.exists():
            raise ArtifactError(f"missing payload file {name}")
        item = np.dtype(_DTYPES[fm["dtype"]]).itemsize
        if path.stat().st_size != fm["bytes"] or fm["bytes"] != fm["elements"] * item:
            raise ArtifactError(f"{name}: size {path.stat().st_size} does not match manifest "
                                f"({fm['elements']} x {fm['dtype']})")
        if check_hashes and sha256_file(path) != fm["sha256"]:
            raise ArtifactError(f"{name}: sha256 mismatch (file was modified after preparation)")
    fp = dataset_fingerprint(format_name=m["format"], version=m["version"], metadata=m["metadata"], files=m["files"],
                             sample_count=m["sample_count"], token_count=m["token_count"])
    if fp != m["metadata"].get("dataset_fingerprint"):
        raise ArtifactError("dataset_fingerprint does not match the manifest contents")
    if m["format"] == INDEXED_FORMAT:
        idx = np.fromfile(root / "index.i64", dtype="<i8").reshape(-1, 4)
        if idx.shape[0] != m["sample_count"]:
            raise ArtifactError("index.i64 row count differs from sample_count")
        ends = idx[:, 0] + idx[:, 1]
        if (idx[:, 1] <= 0).any() or (idx[:, 0] < 0).any() or ends.max() > m["token_count"]:
            raise ArtifactError("index.i64 points outside tokens.i32")
        if (idx[1:, 0] != ends[:-1]).any() or idx[0, 0] != 0:
            raise ArtifactError("index.i64 offsets are not contiguous")
        if ((idx[:, 2] < 0) | (idx[:, 2] > idx[:, 1])).any():
            raise ArtifactError("index.i64 supervision_start outside its sample")
    return m


def validate_artifact_for_run(root: str | Path, *, vocab_size: int, mask_token_id: int | None,
                              block_size: int | None, seq_len: int | None = None,
                              tokenizer_vocab_sha256: str | None = None) -> dict:
    """Is this artifact usable by a run with these model/objective settings?"""
    m = load_manifest(root)
    md = m["metadata"]
    tv = md.get("tokenizer", {}).get("vocab_size")
    if tv is not None and tv > vocab_size:
        raise ArtifactError(f"artifact tokenizer has {tv} ids, model vocabulary only {vocab_size}")
    if md.get("contains_mask_token") and mask_token_id is not None and md.get("mask_token_id") == mask_token_id:
        raise ArtifactError("artifact contains the mask token id as data")
    if block_size and md.get("block_size") and md["block_size"] % block_size and block_size % md["block_size"]:
        raise ArtifactError(f"artifact was aligned to block size {md['block_size']}, run uses {block_size}")
    if tokenizer_vocab_sha256 and md.get("tokenizer", {}).get("vocab_sha256") not in (None, tokenizer_vocab_sha256):
        raise ArtifactError("artifact was tokenized with a different tokenizer vocabulary")
    if seq_len and m["format"] == PACKED_TOKEN_FORMAT and m["token_count"] < seq_len:
        raise ArtifactError(f"packed artifact has {m['token_count']} tokens, fewer than one sequence of {seq_len}")
    return {"compatible": True, "format": m["format"], "dataset_fingerprint": md["dataset_fingerprint"]}


def artifact_stats(root: str | Path) -> dict:
    m = load_manifest(root)
    out = {"format": m["format"], "samples": m["sample_count"], "tokens": m["token_count"], "stats": m["stats"]}
    if m["format"] == INDEXED_FORMAT:
        idx = np.fromfile(Path(root) / "index.i64", dtype="<i8").reshape(-1, 4)
        lens = idx[:, 1]
        out["length"] = {"min": int(lens.min()), "max": int(lens.max()), "mean": float(lens.mean())}
    return out

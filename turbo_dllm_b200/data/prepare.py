"""Offline data preparation (`dllm data prepare`): source records → formatted records → token ids + supervision
mask → packed or indexed artifact, installed atomically.

`PreparationSpec` (format `dllm.data.prepare.v1`) has six strict sections (unknown sections / fields are refused):

  source       type huggingface | jsonl | parquet | text | pretokenized (+ registered plug-ins); path / paths (files,
               directories, globs; sorted), id / name / revision / split / streaming / loader_kwargs (huggingface),
               text_mode document | line, encoding, limit
  records      type text | messages | prompt_completion | pretokenized (+ registered formatters) and the field names
               (dot-separated paths such as `document.body` reach into nested records)
  tokenizer    model (Hugging Face id / local directory) or the built-in `byte` tokenizer, revision,
               trust_remote_code, use_fast, chat_template (a template string, or `chatml` for the built-in
               turn markers), add_bos, add_eos, kwargs, chat_template_kwargs, mask_token_id
  supervision  policy full | assistant_only | completion_only | provided
  packing      maximum_length, overflow reject | split | truncate_left | truncate_right, alignment,
               alignment_policy reject | truncate_left | truncate_right | pad, minimum_length, pad_token_id,
               separator_token_id
  output       path, format auto | packed | indexed, overwrite

The spellings of earlier files of this package (`source.kind`, `records.*_column`, `supervision.mode`,
`packing.sequence_length`, `packing.mode`) are still read. Relative source and output paths in a file are resolved
against the file's directory. Output is written to a staging directory next to the target and moved into place with
os.replace (the previous artifact is kept as a backup until the move succeeded).

Extension points: `register_source(name, factory)` (factory(source section) → iterator of raw records) and
`register_formatter(name, fn)` (fn(raw record, records section) → `FormattedRecord` or None); both are also found
through the entry-point groups `turbo_dllm_b200.data_sources` / `turbo_dllm_b200.record_formatters`.

Counterparts: dllm_parallel/data/schemas.py:23-208, prepare.py:52-267, sources.py:24-328,
formatting.py:24-262, tokenization.py:21-346, packing.py:44-164, registry.py:47-151, provenance.py:15-36.
"""
from __future__ import annotations

import glob as _glob
import gzip
import hashlib
import json
import os
import shutil
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Iterator, Mapping, Sequence

import numpy as np
import yaml

from .artifacts import write_indexed_artifact, write_packed_artifact

PREPARE_FORMAT = "dllm.data.prepare.v1"
SOURCE_ENTRY_POINT_GROUP = "turbo_dllm_b200.data_sources"
FORMATTER_ENTRY_POINT_GROUP = "turbo_dllm_b200.record_formatters"
_SECTION_FIELDS = {
    "source": {"type": "jsonl", "path": None, "paths": None, "id": None, "name": None, "split": "train",
               "revision": None, "streaming": False, "text_mode": "document", "encoding": "utf-8",
               "loader_kwargs": {}, "limit": None},
    "records": {"type": "text", "text_field": "text", "messages_field": "messages", "role_field": "role",
                "content_field": "content", "prompt_field": "prompt", "completion_field": "completion",
                "input_ids_field": "input_ids", "labels_field": "labels", "loss_mask_field": "loss_mask",
                "assistant_mask_field": "assistant_masks", "completion_mask_field": "completion_mask",
                "sample_id_field": None, "group_id_field": None},
    "tokenizer": {"model": "byte", "revision": None, "trust_remote_code": False, "use_fast": True,
                  "chat_template": None, "add_bos": False, "add_eos": False, "kwargs": {}, "chat_template_kwargs": {},
                  "mask_token_id": None},
    "supervision": {"policy": "full"},
    "packing": {"maximum_length": None, "overflow": "reject", "alignment": 1, "alignment_policy": "truncate_right",
                "minimum_length": None, "pad_token_id": None, "separator_token_id": None},
    "output": {"path": None, "format": "auto", "overwrite": False},
}
# earlier spellings → (section, field) they now mean
_EARLIER_NAMES = {
    ("source", "kind"): ("source", "type"),
    ("records", "text_column"): ("records", "text_field"), ("records", "messages_column"): ("records", "messages_field"),
    ("records", "prompt_column"): ("records", "prompt_field"),
    ("records", "completion_column"): ("records", "completion_field"),
    ("records", "tokens_column"): ("records", "input_ids_field"), ("records", "mask_column"): ("records", "loss_mask_field"),
    ("records", "group_column"): ("records", "group_id_field"),
    ("supervision", "mode"): ("supervision", "policy"),
    ("packing", "sequence_length"): ("packing", "maximum_length"), ("packing", "mode"): ("output", "format"),
}
_SOURCE_TYPES = ("huggingface", "jsonl", "parquet", "text", "pretokenized")
_RECORD_TYPES = ("text", "messages", "prompt_completion", "pretokenized")
_CHOICES = {
    ("source", "text_mode"): ("document", "line"),
    ("supervision", "policy"): ("full", "assistant_only", "completion_only", "provided"),
    ("packing", "overflow"): ("reject", "split", "truncate_left", "truncate_right"),
    ("packing", "alignment_policy"): ("reject", "truncate_left", "truncate_right", "pad"),
    ("output", "format"): ("auto", "packed", "indexed"),
}
_POLICY_RECORD_TYPES = {"assistant_only": ("messages", "pretokenized"), "completion_only": ("prompt_completion", "pretokenized"),
                        "provided": ("pretokenized",)}


class PreparationError(ValueError):
    pass


# ------------------------------------------------------------- registries
SOURCE_REGISTRY: dict[str, Callable[[dict], Iterator[dict]]] = {}
FORMATTER_REGISTRY: dict[str, Callable[[Mapping[str, Any], dict], "FormattedRecord | None"]] = {}
_discovered: set[str] = set()


def _register(registry: dict, what: str, name: str, fn, replace: bool) -> None:
    key = str(name).strip().lower()
    if not key:
        raise ValueError(f"{what} name must not be empty")
    if not callable(fn):
        raise TypeError(f"{what} {key!r} must be callable")
    if key in registry and not replace:
        raise ValueError(f"{what} {key!r} is already registered (pass replace=True to override it)")
    registry[key] = fn


def register_source(name: str, factory: Callable[[dict], Iterator[dict]], *, replace: bool = False) -> None:
    """`factory(source_section)` yields raw records (mappings)."""
    _register(SOURCE_REGISTRY, "data source", name, factory, replace)


def register_formatter(name: str, fn: Callable[[Mapping[str, Any], dict], "FormattedRecord | None"], *,
                       replace: bool = False) -> None:
    """`fn(raw_record, records_section)` returns a `FormattedRecord`, or None to drop the record."""
    _register(FORMATTER_REGISTRY, "record formatter", name, fn, replace)


def _discover(group: str, registry: dict, what: str) -> None:
    """Loads plug-ins that installed distributions announce under `group` (once per process)."""
    if group in _discovered:
        return
    _discovered.add(group)
    from importlib import metadata

    eps = metadata.entry_points()
    found = eps.select(group=group) if hasattr(eps, "select") else eps.get(group, ())
    for ep in found:
        if ep.name.strip().lower() not in registry:
            _register(registry, what, ep.name, ep.load(), False)


def _known_source(name: str) -> bool:
    if name in _SOURCE_TYPES or name in SOURCE_REGISTRY:
        return True
    _discover(SOURCE_ENTRY_POINT_GROUP, SOURCE_REGISTRY, "data source")
    return name in SOURCE_REGISTRY


def _known_formatter(name: str) -> bool:
    if name in _RECORD_TYPES or name in FORMATTER_REGISTRY:
        return True
    _discover(FORMATTER_ENTRY_POINT_GROUP, FORMATTER_REGISTRY, "record formatter")
    return name in FORMATTER_REGISTRY


# ------------------------------------------------------------------- spec
@dataclass(frozen=True)
class PreparationSpec:
    source: dict
    records: dict
    tokenizer: dict
    supervision: dict
    packing: dict
    output: dict

    @classmethod
    def from_mapping(cls, m: Mapping[str, Any], *, base_dir: str | Path | None = None) -> "PreparationSpec":
        m = dict(m or {})
        fmt = m.pop("format", PREPARE_FORMAT)
        if fmt != PREPARE_FORMAT:
            raise PreparationError(f"unsupported preparation format {fmt!r} (expected {PREPARE_FORMAT})")
        unknown = sorted(set(m) - set(_SECTION_FIELDS))
        if unknown:
            raise PreparationError(f"unknown section(s): {', '.join(unknown)}")
        raw = {sec: dict(m.get(sec) or {}) for sec in _SECTION_FIELDS}
        for (sec, old), (nsec, new) in _EARLIER_NAMES.items():
            if old in raw[sec]:
                v = raw[sec].pop(old)
                if new in raw[nsec] and raw[nsec][new] != v:
                    raise PreparationError(f"{sec}.{old} and {nsec}.{new} are two names of one setting and disagree")
                raw[nsec][new] = v
        secs = {}
        for sec, defaults in _SECTION_FIELDS.items():
            bad = sorted(set(raw[sec]) - set(defaults))
            if bad:
                raise PreparationError(f"unknown field(s) in section '{sec}': {', '.join(bad)}")
            secs[sec] = {**{k: (dict(v) if isinstance(v, dict) else v) for k, v in defaults.items()}, **raw[sec]}
        if base_dir is not None:       # a file's relative paths are relative to the file
            base = Path(base_dir)

            def rel(p):
                return p if p is None or "://" in str(p) or os.path.isabs(str(p)) else str(base / str(p))

            secs["source"]["path"] = rel(secs["source"]["path"])
            if secs["source"]["paths"]:
                secs["source"]["paths"] = [rel(p) for p in secs["source"]["paths"]]
            secs["output"]["path"] = rel(secs["output"]["path"])
        spec = cls(**secs)
        spec.validate()
        return spec

    def with_output(self, path: str | None = None, overwrite: bool | None = None) -> "PreparationSpec":
        out = dict(self.output)
        if path is not None:
            out["path"] = path
        if overwrite is not None:
            out["overwrite"] = bool(overwrite)
        spec = PreparationSpec(self.source, self.records, self.tokenizer, self.supervision, self.packing, out)
        spec.validate()
        return spec

    @property
    def artifact_format(self) -> str:
        """`packed` (one token stream) or `indexed` (samples with a supervision mask)."""
        f = self.output["format"]
        return f if f != "auto" else ("packed" if self.supervision["policy"] == "full" else "indexed")

    def validate(self) -> None:
        for (sec, key), choices in _CHOICES.items():
            v = getattr(self, sec)[key]
            if v not in choices:
                raise PreparationError(f"{sec}.{key}={v!r} is not one of {choices}")
        if not _known_source(self.source["type"]):
            raise PreparationError(f"source.type={self.source['type']!r} is not one of {_SOURCE_TYPES} "
                                   f"or a registered source {sorted(SOURCE_REGISTRY)}")
        if not _known_formatter(self.records["type"]):
            raise PreparationError(f"records.type={self.records['type']!r} is not one of {_RECORD_TYPES} "
                                   f"or a registered formatter {sorted(FORMATTER_REGISTRY)}")
        s = self.source
        if not (s["path"] or s["paths"] or s["id"] or s["name"]):
            raise PreparationError("source needs path, paths or id")
        if s["type"] == "huggingface" and not (s["id"] or s["name"] or s["path"]):
            raise PreparationError("source.type=huggingface needs source.id")
        if not isinstance(s["loader_kwargs"], Mapping):
            raise PreparationError("source.loader_kwargs must be a mapping")
        if not self.output["path"]:
            raise PreparationError("output.path is required")
        policy, rtype = self.supervision["policy"], self.records["type"]
        if rtype in _RECORD_TYPES and policy in _POLICY_RECORD_TYPES and rtype not in _POLICY_RECORD_TYPES[policy]:
            raise PreparationError(f"supervision.policy={policy} needs records.type in {_POLICY_RECORD_TYPES[policy]}, "
                                   f"got {rtype!r}")
        p = self.packing
        for key in ("maximum_length", "minimum_length"):
            if p[key] is not None and (isinstance(p[key], bool) or int(p[key]) < 1):
                raise PreparationError(f"packing.{key} must be a positive integer")
        if isinstance(p["alignment"], bool) or int(p["alignment"]) < 1:
            raise PreparationError("packing.alignment must be >= 1")
        fmt = self.artifact_format
        if fmt == "packed" and policy != "full":
            raise PreparationError(f"output.format=packed stores no supervision mask: supervision.policy={policy} needs "
                                   "output.format auto or indexed")
        if p["overflow"] == "split" and fmt != "packed":
            raise PreparationError("packing.overflow=split keeps every token of a full-supervision packed stream; "
                                   "supervised samples use reject or truncate_*")
        if p["overflow"] == "split" and not p["maximum_length"]:
            raise PreparationError("packing.overflow=split needs packing.maximum_length")
        if p["separator_token_id"] is not None and fmt != "packed":
            raise PreparationError("packing.separator_token_id separates documents of a packed stream only")

    def sanitized(self) -> dict:
        """The spec as stored in the artifact's metadata: credentials in `loader_kwargs` are redacted."""
        d = {k: dict(getattr(self, k)) for k in _SECTION_FIELDS}
        d["source"]["loader_kwargs"] = redact_secrets(d["source"]["loader_kwargs"])
        d["tokenizer"]["kwargs"] = redact_secrets(d["tokenizer"]["kwargs"])
        d["format"] = PREPARE_FORMAT
        return d


_SECRET_WORDS = ("token", "key", "password", "secret", "credential")


def redact_secrets(value: Any) -> Any:
    """Mapping values whose key names a credential are replaced, at every nesting level."""
    if isinstance(value, Mapping):
        return {k: ("<redacted>" if any(w in str(k).lower() for w in _SECRET_WORDS) else redact_secrets(v))
                for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [redact_secrets(v) for v in value]
    return value


def load_preparation_spec(path: str | Path) -> PreparationSpec:
    text = Path(path).read_text()
    data = json.loads(text) if str(path).endswith(".json") else yaml.safe_load(text)
    return PreparationSpec.from_mapping(data, base_dir=Path(path).resolve().parent)


# ------------------------------------------------------------------ sources
def _paths(src: dict) -> list[Path]:
    """Files named by path / paths: a file, a directory (its files) or a glob; each group sorted."""
    raw = ([src["path"]] if src.get("path") else []) + list(src.get("paths") or [])
    out: list[Path] = []
    for r in raw:
        p = Path(r)
        if p.is_dir():
            out += sorted(q for q in p.iterdir() if q.is_file())
        elif any(c in str(r) for c in "*?["):
            hits = sorted(Path(h) for h in _glob.glob(str(r), recursive=True))
            if not hits:
                raise PreparationError(f"source path {r!r} matches no file")
            out += hits
        else:
            if not p.exists():
                raise PreparationError(f"source file {r!r} does not exist")
            out.append(p)
    return out


def _open_text(path: Path, encoding: str = "utf-8"):
    return gzip.open(path, "rt", encoding=encoding) if path.suffix == ".gz" else open(path, encoding=encoding)


def _jsonl_records(path: Path, encoding: str) -> Iterator[dict]:
    with _open_text(path, encoding) as f:
        for n, line in enumerate(f, 1):
            if not line.strip():
                continue
            rec = json.loads(line)
            if not isinstance(rec, dict):
                raise PreparationError(f"{path.name}:{n}: every JSONL line must be an object")
            yield rec


_RAW_TOKEN_DTYPES = {".i32": "<i4", ".int32": "<i4", ".bin": "<i4", ".tokens": "<i4", ".i64": "<i8", ".int64": "<i8"}


def _pretokenized_records(path: Path, src: dict, fields: dict | None = None) -> Iterator[dict]:
    """Token files: raw little-endian binaries and .npy are memory-mapped (a 1-D array is one record, a 2-D array one
    record per row, each a view); .pt, .json and .jsonl(.gz) carry records that may include masks and ids."""
    key = (fields or {}).get("input_ids_field", "input_ids")
    name = path.name[:-3] if path.suffix == ".gz" else path.name
    suffix = Path(name).suffix
    if suffix == ".jsonl":
        yield from _jsonl_records(path, src.get("encoding", "utf-8"))
        return
    if suffix == ".json":
        with _open_text(path, src.get("encoding", "utf-8")) as f:
            data = json.load(f)
        items = data if isinstance(data, list) else [data]
        for it in items:
            yield it if isinstance(it, dict) else {key: it}
        return
    if suffix in _RAW_TOKEN_DTYPES:
        arr = np.memmap(path, dtype=_RAW_TOKEN_DTYPES[suffix], mode="r")
    elif suffix == ".npy":
        arr = np.load(path, mmap_mode="r")
    elif suffix == ".pt":
        import torch

        obj = torch.load(path, map_location="cpu", weights_only=True)
        if isinstance(obj, (list, tuple)) and obj and isinstance(obj[0], Mapping):
            yield from ({k: (v.numpy() if hasattr(v, "numpy") else v) for k, v in o.items()} for o in obj)
            return
        if isinstance(obj, Mapping):
            obj = obj[key]
        arr = obj.numpy() if hasattr(obj, "numpy") else np.asarray(obj)
    else:
        raise PreparationError(f"pretokenized source {path.name}: unsupported file type {suffix!r}")
    if arr.ndim == 1:
        yield {key: arr}
    elif arr.ndim == 2:
        for row in arr:
            yield {key: row}
    else:
        raise PreparationError(f"pretokenized source {path.name}: expected a 1-D or 2-D token array, got {arr.ndim}-D")


def iter_source_records(src: dict, records: dict | None = None) -> Iterator[dict]:
    kind, limit, enc = src["type"], src.get("limit"), src.get("encoding", "utf-8")

    def gen():
        if kind in SOURCE_REGISTRY:
            yield from SOURCE_REGISTRY[kind](src)
        elif kind == "jsonl":
            for p in _paths(src):
                yield from _jsonl_records(p, enc)
        elif kind == "pretokenized":
            for p in _paths(src):
                yield from _pretokenized_records(p, src, records)
        elif kind == "text":
            for p in _paths(src):
                if src.get("text_mode", "document") == "line":
                    with _open_text(p, enc) as f:
                        for line in f:
                            if line.strip():
                                yield {"text": line.rstrip("\n")}
                else:
                    with _open_text(p, enc) as f:
                        yield {"text": f.read()}
        elif kind == "parquet":
            import pyarrow.parquet as pq

            for p in _paths(src):
                for batch in pq.ParquetFile(p).iter_batches():
                    yield from batch.to_pylist()
        elif kind == "huggingface":
            try:
                import datasets
            except ImportError:
                raise PreparationError("source.type=huggingface needs the `datasets` package") from None
            ds = datasets.load_dataset(src["id"] or src["path"] or src["name"], src["name"] if src["id"] else None,
                                       split=src["split"], revision=src["revision"], streaming=src["streaming"],
                                       **dict(src["loader_kwargs"]))
            yield from ds
        else:
            raise PreparationError(f"unknown source type {kind!r}")

    n = 0
    for rec in gen():
        yield rec
        n += 1
        if limit and n >= limit:
            return


def source_provenance(src: dict) -> dict:
    """What was read: every local file with size and SHA-256; remote sources by id / name / revision / split."""
    files = []
    if src["type"] in ("jsonl", "pretokenized", "text", "parquet"):
        for p in _paths(src):
            h = hashlib.sha256()
            with open(p, "rb") as f:
                for chunk in iter(lambda: f.read(1 << 20), b""):
                    h.update(chunk)
            files.append({"name": p.name, "path": str(p), "bytes": p.stat().st_size, "sha256": h.hexdigest()})
    return {"type": src["type"], "id": src.get("id"), "name": src.get("name"), "revision": src.get("revision"),
            "split": src.get("split"), "loader_kwargs": redact_secrets(src.get("loader_kwargs") or {}), "files": files}


# --------------------------------------------------------------- tokenizers
class ByteTokenizer:
    """UTF-8 bytes 0..255, then <bos>=256, <eos>=257, <mask>=258, role markers 259.."""

    vocab_size = 264
    bos_token_id, eos_token_id, mask_token_id = 256, 257, 258
    name = "byte"
    ROLE = {"system": 259, "user": 260, "assistant": 261, "tool": 262}
    END_TURN = 263
    chat_template = "byte-turn-markers"

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def vocab_sha256(self) -> str:
        return hashlib.sha256(b"turbo_dllm_b200.byte_tokenizer.v1").hexdigest()

    def encode_messages(self, messages: Sequence[Mapping[str, Any]], generation_prompt: bool = False):
        """(ids, assistant mask): one role marker, the content bytes, one end-of-turn marker per message."""
        ids: list[int] = []
        mask: list[int] = []
        for m in messages:
            role = m.get("role", "user")
            body = self.encode(str(m.get("content", ""))) + [self.END_TURN]
            ids += [self.ROLE.get(role, self.ROLE["user"])] + body
            mask += [0] + [int(role == "assistant")] * len(body)
        if generation_prompt:
            ids.append(self.ROLE["assistant"])
            mask.append(0)
        return ids, mask


class HFTokenizer:
    def __init__(self, tcfg: Mapping[str, Any]):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(tcfg["model"], revision=tcfg.get("revision"),
                                                 trust_remote_code=bool(tcfg.get("trust_remote_code")),
                                                 use_fast=bool(tcfg.get("use_fast", True)), **dict(tcfg.get("kwargs") or {}))
        self.name = tcfg["model"]
        self.vocab_size = len(self.tok)
        self.bos_token_id, self.eos_token_id = self.tok.bos_token_id, self.tok.eos_token_id
        self.mask_token_id = getattr(self.tok, "mask_token_id", None)
        tpl = tcfg.get("chat_template")
        self.chatml = tpl == "chatml"
        if tpl and not self.chatml:
            self.tok.chat_template = tpl
        self.chat_template = "chatml" if self.chatml else getattr(self.tok, "chat_template", None)
        self.template_kwargs = dict(tcfg.get("chat_template_kwargs") or {})

    def encode(self, text: str) -> list[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def vocab_sha256(self) -> str:
        return hashlib.sha256(json.dumps(self.tok.get_vocab(), sort_keys=True).encode()).hexdigest()

    def encode_messages(self, messages: Sequence[Mapping[str, Any]], generation_prompt: bool = False):
        """(ids, assistant mask or None). The mask comes from the template itself (generation markers); when the
        template does not mark assistant tokens it is None and assistant-only supervision is refused upstream.
        `chat_template: chatml` is the one built-in template: its turn boundaries are exact by construction."""
        if self.chatml:
            ids: list[int] = []
            mask: list[int] = []
            for m in messages:
                head = self.encode(f"<|im_start|>{m.get('role', 'user')}\n")
                body = self.encode(str(m.get("content", "")) + "<|im_end|>\n")
                ids += head + body
                mask += [0] * len(head) + [int(m.get("role") == "assistant")] * len(body)
            if generation_prompt:
                head = self.encode("<|im_start|>assistant\n")
                ids += head
                mask += [0] * len(head)
            return ids, mask
        if not self.chat_template:
            raise PreparationError(f"tokenizer {self.name!r} has no chat template; set tokenizer.chat_template "
                                   "(a template string, or 'chatml')")
        out = self.tok.apply_chat_template(list(messages), tokenize=True, return_dict=True,
                                           add_generation_prompt=generation_prompt,
                                           return_assistant_tokens_mask=not generation_prompt, **self.template_kwargs)
        ids = list(out["input_ids"])
        mask = out.get("assistant_masks")
        if mask is not None and (len(mask) != len(ids) or not any(mask)):
            mask = None
        return ids, (list(mask) if mask is not None else None)


def build_tokenizer(tcfg: dict):
    return ByteTokenizer() if tcfg["model"] == "byte" else HFTokenizer(tcfg)


# ------------------------------------------------ formatting + tokenization
@dataclass
class FormattedRecord:
    """One raw record in one of four shapes; exactly one of the payload fields is set."""
    text: str | None = None
    messages: list | None = None                 # [{"role": ..., "content": ..., ...}]
    prompt: Any = None                           # str or message list (with `completion` of the same kind)
    completion: Any = None
    input_ids: Any = None                        # token ids (array view or list)
    loss_mask: Any = None                        # with input_ids: the supervision mask, if the record carries one
    sample_id: Any = None
    group_id: Any = None


@dataclass
class TokenizedRecord:
    tokens: np.ndarray      # int32
    loss_mask: np.ndarray   # uint8, same length
    sample_id: int
    group: int | None = None


def field_value(rec: Mapping[str, Any], path: str | None, default=None):
    """`a.b.c` reaches into nested mappings; a literal key containing dots wins if it exists."""
    if path is None:
        return default
    if path in rec:
        return rec[path]
    cur: Any = rec
    for part in str(path).split("."):
        if not isinstance(cur, Mapping) or part not in cur:
            return default
        cur = cur[part]
    return cur


def stable_id(value: Any, fallback: int) -> int:
    """Sample / group ids are stored as int64: integers pass through, anything else is hashed (SHA-256, 63 bits)."""
    if value is None:
        return int(fallback)
    if isinstance(value, (int, np.integer)) and not isinstance(value, bool):
        return int(value)
    return int.from_bytes(hashlib.sha256(str(value).encode()).digest()[:8], "big") >> 1


def format_record(rec: Mapping[str, Any], r: dict, policy: str) -> FormattedRecord | None:
    """Raw record → FormattedRecord by `records.type` (None: nothing to train on)."""
    t = r["type"]
    if t in FORMATTER_REGISTRY:
        return FORMATTER_REGISTRY[t](rec, r)
    out = FormattedRecord(sample_id=field_value(rec, r["sample_id_field"]), group_id=field_value(rec, r["group_id_field"]))
    if t == "text":
        text = field_value(rec, r["text_field"])
        if not isinstance(text, str) or not text:
            return None
        out.text = text
    elif t == "messages":
        msgs = field_value(rec, r["messages_field"])
        if not msgs:
            return None
        # role / content are renamed to the template's names; every other key of a message is kept (tool calls ...)
        out.messages = [{**{k: v for k, v in m.items() if k not in (r["role_field"], r["content_field"])},
                         "role": m.get(r["role_field"], "user"), "content": m.get(r["content_field"], "")} for m in msgs]
    elif t == "prompt_completion":
        prompt, completion = field_value(rec, r["prompt_field"], ""), field_value(rec, r["completion_field"], "")
        if not completion:
            return None
        if isinstance(prompt, str) != isinstance(completion, str):
            raise PreparationError("prompt and completion must both be strings or both be message lists")
        out.prompt, out.completion = prompt, completion
    elif t == "pretokenized":
        ids = field_value(rec, r["input_ids_field"])
        if ids is None or len(ids) == 0:
            return None
        out.input_ids = ids
        if policy == "provided":
            m = field_value(rec, r["loss_mask_field"])
            if m is None:
                labels = field_value(rec, r["labels_field"])
                m = None if labels is None else (np.asarray(labels) != -100)
            if m is None:
                raise PreparationError("supervision.policy=provided needs a loss mask or labels in every record")
            out.loss_mask = m
        elif policy in ("assistant_only", "completion_only"):
            name = r["assistant_mask_field"] if policy == "assistant_only" else r["completion_mask_field"]
            m = field_value(rec, name)
            if m is None:
                raise PreparationError(f"supervision.policy={policy} needs the field {name!r} in every record")
            out.loss_mask = m
    return out


def tokenize_record(rec: Mapping[str, Any], spec: PreparationSpec, tok, sample_id: int) -> TokenizedRecord | None:
    tc, policy = spec.tokenizer, spec.supervision["policy"]
    fr = format_record(rec, spec.records, policy)
    if fr is None:
        return None
    ids: list[int] = []
    mask: list[int] = []

    def add(piece, supervised):
        ids.extend(piece)
        mask.extend(supervised if isinstance(supervised, list) else [1 if supervised else 0] * len(piece))

    if fr.input_ids is not None:
        toks = np.asarray(fr.input_ids)
        if fr.loss_mask is not None and len(fr.loss_mask) != toks.size:
            raise PreparationError(f"record {sample_id}: loss mask length differs from token length")
        m = np.ones(toks.size, np.uint8) if fr.loss_mask is None else np.asarray(fr.loss_mask).astype(bool).astype(np.uint8)
        if toks.size == 0:
            return None
        return TokenizedRecord(toks.astype(np.int32, copy=False), m, stable_id(fr.sample_id, sample_id),
                               None if fr.group_id is None else stable_id(fr.group_id, sample_id))
    if tc["add_bos"] and tok.bos_token_id is not None:
        add([tok.bos_token_id], False)
    if fr.text is not None:
        add(tok.encode(fr.text), True)
    elif fr.messages is not None:
        mids, mmask = tok.encode_messages(fr.messages)
        if policy == "assistant_only":
            if mmask is None:
                raise PreparationError("supervision.policy=assistant_only: the chat template does not mark assistant "
                                       "tokens (it needs generation markers); text boundaries are never guessed")
            add(mids, [int(x) for x in mmask])
        else:
            add(mids, True)
    elif isinstance(fr.completion, str):
        add(tok.encode(fr.prompt), policy != "completion_only")
        add(tok.encode(fr.completion), True)
    else:
        # message-shaped pair: the prompt rendered with a generation prompt must be an exact prefix of the whole
        pids, _ = tok.encode_messages(list(fr.prompt), generation_prompt=True)
        wids, _ = tok.encode_messages(list(fr.prompt) + list(fr.completion))
        if wids[:len(pids)] != pids:
            raise PreparationError(f"record {sample_id}: the chat template does not keep the prompt as a prefix of the "
                                   "conversation, so the completion boundary is unknown")
        add(pids, policy != "completion_only")
        add(wids[len(pids):], True)
    if tc["add_eos"] and tok.eos_token_id is not None:
        add([tok.eos_token_id], True)
    if not ids:
        return None
    return TokenizedRecord(np.asarray(ids, dtype=np.int32), np.asarray(mask, dtype=np.uint8),
                           stable_id(fr.sample_id, sample_id),
                           None if fr.group_id is None else stable_id(fr.group_id, sample_id))


# ----------------------------------------------------------------- packing
def _cut(rec: TokenizedRecord, sl: slice) -> TokenizedRecord:
    return TokenizedRecord(rec.tokens[sl], rec.loss_mask[sl], rec.sample_id, rec.group)


def apply_overflow(rec: TokenizedRecord, limit: int | None, overflow: str) -> list[TokenizedRecord]:
    if not limit or rec.tokens.size <= limit:
        return [rec]
    if overflow == "reject":
        raise PreparationError(f"sample {rec.sample_id} has {rec.tokens.size} tokens > maximum_length {limit} "
                               "(packing.overflow=reject)")
    if overflow == "truncate_right":
        return [_cut(rec, slice(0, limit))]
    if overflow == "truncate_left":
        return [_cut(rec, slice(rec.tokens.size - limit, None))]
    return [_cut(rec, slice(i, i + limit)) for i in range(0, rec.tokens.size, limit)]


def align_record(rec: TokenizedRecord, alignment: int, policy: str, pad_id: int) -> TokenizedRecord | None:
    """Supervised samples have lengths that divide by `alignment` (the diffusion block size): by truncation (the
    default; None when nothing is left), by refusal, or by unsupervised padding tokens (`pad`, which later attention
    can see: use it only where trailing padding is acceptable)."""
    extra = rec.tokens.size % alignment if alignment > 1 else 0
    if not extra:
        return rec
    if policy == "reject":
        raise PreparationError(f"sample {rec.sample_id} has {rec.tokens.size} tokens, not a multiple of "
                               f"packing.alignment={alignment} (alignment_policy=reject)")
    if policy == "pad":
        pad = alignment - extra
        return TokenizedRecord(np.concatenate([rec.tokens, np.full(pad, pad_id, np.int32)]),
                               np.concatenate([rec.loss_mask, np.zeros(pad, np.uint8)]), rec.sample_id, rec.group)
    keep = rec.tokens.size - extra
    if keep <= 0:
        return None
    return _cut(rec, slice(0, keep)) if policy == "truncate_right" else _cut(rec, slice(extra, None))


# ----------------------------------------------------------------- driver
def prepare_dataset(spec: PreparationSpec) -> dict:
    """Runs the whole pipeline and returns the manifest of the installed artifact."""
    out = Path(spec.output["path"])
    if out.exists() and not spec.output["overwrite"]:
        raise PreparationError(f"{out} exists; set output.overwrite=true to replace it")
    tok = build_tokenizer(spec.tokenizer)
    pk, fmt = spec.packing, spec.artifact_format
    pad_id = pk["pad_token_id"] if pk["pad_token_id"] is not None else (tok.eos_token_id or 0)
    mask_id = spec.tokenizer["mask_token_id"] if spec.tokenizer["mask_token_id"] is not None else tok.mask_token_id
    minimum = int(pk["minimum_length"] or 1)
    sep = pk["separator_token_id"]
    counters = {"source_records": 0, "empty_records": 0, "split_records": 0, "truncated_records": 0, "source_tokens": 0,
                "short_records": 0, "alignment_dropped_tokens": 0, "separator_tokens": 0}
    saw_mask = {"v": False}

    def records() -> Iterator[TokenizedRecord]:
        first = True
        for i, raw in enumerate(iter_source_records(spec.source, spec.records)):
            counters["source_records"] += 1
            rec = tokenize_record(raw, spec, tok, i)
            if rec is None:
                counters["empty_records"] += 1
                continue
            counters["source_tokens"] += int(rec.tokens.size)
            if mask_id is not None and (rec.tokens == mask_id).any():
                saw_mask["v"] = True
            parts = apply_overflow(rec, pk["maximum_length"], pk["overflow"])
            if len(parts) > 1:
                counters["split_records"] += 1
            elif parts[0].tokens.size < rec.tokens.size:
                counters["truncated_records"] += 1
            if fmt == "packed" and sep is not None and not first:
                # a separator marks a boundary between source documents, never between chunks of one document
                counters["separator_tokens"] += 1
                yield TokenizedRecord(np.asarray([sep], np.int32), np.ones(1, np.uint8), rec.sample_id, rec.group)
            first = False
            for part in parts:
                if fmt == "indexed":
                    before = part.tokens.size
                    part = align_record(part, int(pk["alignment"]), pk["alignment_policy"], pad_id)
                    if part is None:
                        counters["short_records"] += 1
                        counters["alignment_dropped_tokens"] += before
                        continue
                    counters["alignment_dropped_tokens"] += max(0, before - part.tokens.size)
                if part.tokens.size < minimum:
                    counters["short_records"] += 1
                    continue
                yield part

    tpl = getattr(tok, "chat_template", None) or ""
    metadata = {
        "tokenizer": {"model": tok.name, "revision": spec.tokenizer.get("revision"), "vocab_size": tok.vocab_size,
                      "vocab_sha256": tok.vocab_sha256(),
                      "chat_template_sha256": hashlib.sha256(str(tpl).encode()).hexdigest()},
        "mask_token_id": mask_id, "eos_token_id": tok.eos_token_id, "pad_token_id": pad_id,
        "block_size": int(pk["alignment"]) if int(pk["alignment"]) > 1 else None,
        "semantics": "full_sequence" if fmt == "packed" else "supervised_samples",
        "sampling_policy": "contiguous_windows" if fmt == "packed" else "one_sample_per_row",
        "sequence_layout": fmt, "supervision_shape": spec.supervision["policy"],
        "padding": "unsupervised_trailing_tokens" if (fmt == "indexed" and pk["alignment_policy"] == "pad") else "none",
        "preparation": spec.sanitized(), "source": source_provenance(spec.source),
    }
    staging = out.parent / f".{out.name}.staging-{os.getpid()}"
    if staging.exists():
        shutil.rmtree(staging)
    out.parent.mkdir(parents=True, exist_ok=True)
    try:
        if fmt == "packed":
            segs = (r.tokens for r in records())
            # contains_mask_token is only known after the stream ran: write, then patch through a rebuild
            manifest = write_packed_artifact(staging, segs, metadata={**metadata, "contains_mask_token": None},
                                             stats=counters)
        else:
            samples = ({"tokens": r.tokens, "loss_mask": r.loss_mask, "sample_id": r.sample_id,
                        "group": r.group if r.group is not None else r.sample_id} for r in records())
            manifest = write_indexed_artifact(staging, samples, metadata={**metadata, "contains_mask_token": None},
                                              with_groups=bool(spec.records.get("group_id_field")))
        # finalise fields that depend on the streamed content, then re-fingerprint
        from .artifacts import build_manifest, write_manifest

        md = dict(manifest["metadata"])
        md["contains_mask_token"] = bool(saw_mask["v"])
        stats = {**manifest["stats"], **counters}
        if fmt == "packed":
            stats["records"] = counters["source_records"] - counters["empty_records"]
        manifest = build_manifest(format_name=manifest["format"], metadata=md, files=manifest["files"], stats=stats,
                                  sample_count=stats["records"] if fmt == "packed" else manifest["sample_count"],
                                  token_count=manifest["token_count"])
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
    except BaseException:
        shutil.rmtree(staging, ignore_errors=True)
        raise

"""Command builders and verification for serving an exported DFlash drafter as the speculative
decoding draft model of SGLang or vLLM.

`build_sglang_command` / `build_vllm_command` return argv lists (no process is started here);
`verify_acceptance` talks to a running OpenAI-compatible endpoint, sends a few prompts and reads
the server's speculative-decoding metrics to check the mean acceptance length against a floor.

`ServerConfig` normalises what the two servers need from one mapping (ports, parallel sizes, memory share,
draft length from the drafter's block size); `validate_export_for_server` checks an exported drafter against the
contract of the chosen server before anything is started; `ServerProcess` starts the command, waits until the
endpoint answers, and stops exactly the process it started; `evaluate_response` / `verify_server` gate a running
server on ONE deterministic completion: the served model, the draft length the server reports, at least one fully
accepted draft block and a target-prefix match of at least one draft length.

Counterparts: dllm_parallel/serving/sglang_dflash.py:17-186, dllm_parallel/serving/vllm_dflash.py:21-328.
"""
from __future__ import annotations

import json
import os
import re
import subprocess
import time
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from typing import Any, Callable, Mapping, Sequence

QUALIFIED_SERVERS = {"vllm": "0.29.0", "sglang": None}     # None: any installed version is accepted


def draft_tokens(block_size: int) -> int:
    """Draft tokens per verification step of a drafter trained with `block_size`: the block's first token is
    the anchor the target already produced."""
    if not isinstance(block_size, int) or isinstance(block_size, bool) or block_size < 2:
        raise ValueError(f"block_size must be an integer >= 2, got {block_size!r}")
    return block_size - 1


def require_server_version(backend: str, installed_version: str | None = None) -> str | None:
    """The installed version of the server package; raises when the package is absent or (vLLM) not the
    qualified release."""
    from importlib import metadata

    if backend not in QUALIFIED_SERVERS:
        raise ValueError(f"unknown serving backend {backend!r} (sglang, vllm)")
    if installed_version is None:
        try:
            installed_version = metadata.version(backend)
        except metadata.PackageNotFoundError as e:
            raise RuntimeError(f"{backend} is not installed in this environment") from e
    want = QUALIFIED_SERVERS[backend]
    if want is not None and installed_version != want:
        raise RuntimeError(f"{backend} {want} is the qualified release; found {installed_version}")
    return installed_version


@dataclass
class ServerConfig:
    """One normalised description of a speculative-decoding server."""

    backend: str
    target_model: str
    draft_export: str
    block_size: int = 16
    host: str = "127.0.0.1"
    port: int | None = None
    tensor_parallel_size: int = 1
    memory_fraction: float | None = None
    max_model_len: int | None = None
    dtype: str = "bfloat16"
    extra: list[str] = field(default_factory=list)

    @classmethod
    def from_mapping(cls, m: Mapping[str, Any]) -> "ServerConfig":
        known = {f for f in cls.__dataclass_fields__}
        alias = {"tp": "tensor_parallel_size", "tensor_parallel": "tensor_parallel_size", "draft": "draft_export",
                 "model": "target_model", "gpu_memory_utilization": "memory_fraction",
                 "mem_fraction_static": "memory_fraction"}
        out: dict[str, Any] = {}
        for k, v in m.items():
            k = alias.get(k, k)
            if k not in known:
                raise ValueError(f"unknown server setting {k!r}")
            out[k] = v
        cfg = cls(**out)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.backend not in QUALIFIED_SERVERS:
            raise ValueError(f"backend must be sglang or vllm, got {self.backend!r}")
        draft_tokens(self.block_size)
        if self.port is None:
            self.port = 30000 if self.backend == "sglang" else 8000
        if not 0 < int(self.port) < 65536 or int(self.tensor_parallel_size) < 1:
            raise ValueError("port must be in 1..65535 and tensor_parallel_size >= 1")
        if self.memory_fraction is not None and not 0.05 <= float(self.memory_fraction) <= 1.0:
            raise ValueError("memory_fraction must lie in [0.05, 1]")
        self.extra = [str(x) for x in self.extra]

    @property
    def url(self) -> str:
        return f"http://{self.host}:{self.port}"

    def command(self) -> list[str]:
        n = draft_tokens(self.block_size)
        extra = list(self.extra)
        if self.backend == "sglang":
            if self.memory_fraction is not None:
                extra += ["--mem-fraction-static", str(self.memory_fraction)]
            if self.max_model_len is not None:
                extra += ["--context-length", str(self.max_model_len)]
            return build_sglang_command(target_model=self.target_model, draft_export=self.draft_export,
                                        port=self.port, tp=self.tensor_parallel_size, num_speculative_tokens=n,
                                        extra=["--host", self.host, "--dtype", self.dtype, *extra])
        if self.memory_fraction is not None:
            extra += ["--gpu-memory-utilization", str(self.memory_fraction)]
        if self.max_model_len is not None:
            extra += ["--max-model-len", str(self.max_model_len)]
        return build_vllm_command(target_model=self.target_model, draft_export=self.draft_export, port=self.port,
                                  tp=self.tensor_parallel_size, num_speculative_tokens=n,
                                  extra=["--host", self.host, "--dtype", self.dtype, *extra])


def validate_export_for_server(export_dir: str, backend: str, expected_block_size: int | None = None) -> dict:
    """Checks an exported drafter directory against what the server's loader reads: config.json with a `dflash_config`
    mapping, one consistent block size, the model type the loader supports, and the weight file."""
    cfg_path = os.path.join(export_dir, "config.json")
    if not os.path.exists(cfg_path):
        raise ValueError(f"{export_dir} has no config.json (not an exported drafter)")
    cfg = json.load(open(cfg_path))
    method = cfg.get("dflash_config")
    if not isinstance(method, Mapping):
        raise ValueError("the export's config.json has no dflash_config mapping")
    top, nested = cfg.get("block_size"), method.get("block_size")
    if top is not None and nested is not None and top != nested:
        raise ValueError(f"conflicting block sizes in the export: top-level {top!r}, dflash_config {nested!r}")
    block = top if top is not None else nested
    n = draft_tokens(block)
    if expected_block_size is not None and block != expected_block_size:
        raise ValueError(f"exported block_size {block!r}, expected {expected_block_size}")
    if backend == "vllm" and cfg.get("model_type") != "qwen3":
        raise ValueError(f"the vLLM drafter loader reads model_type 'qwen3' only, got {cfg.get('model_type')!r}")
    if not any(os.path.exists(os.path.join(export_dir, f)) for f in ("model.safetensors", "model.safetensors.index.json",
                                                                       "pytorch_model.bin")):
        raise ValueError(f"{export_dir} has no weight file")
    return {"backend": backend, "block_size": block, "num_speculative_tokens": n,
            "qualified_version": QUALIFIED_SERVERS.get(backend), "architectures": cfg.get("architectures")}


class ServerProcess:
    """Starts a server command, waits for its endpoint, stops the process it started (never by name)."""

    def __init__(self, command: Sequence[str], url: str, *, env: Mapping[str, str] | None = None, log_path: str | None = None):
        self.command, self.url = list(command), url.rstrip("/")
        self.env = dict(os.environ, **(env or {}))
        self.log_path = log_path
        self.proc: subprocess.Popen | None = None
        self._log = None

    def start(self) -> "ServerProcess":
        if self.proc is not None:
            raise RuntimeError("server already started")
        self._log = open(self.log_path, "ab") if self.log_path else subprocess.DEVNULL
        self.proc = subprocess.Popen(self.command, env=self.env, stdout=self._log, stderr=subprocess.STDOUT,
                                     start_new_session=True)
        return self

    def wait_ready(self, timeout: float = 1800.0, poll: float = 1.0, path: str = "/v1/models") -> dict:
        deadline = time.monotonic() + timeout
        last = "no answer yet"
        while time.monotonic() < deadline:
            if self.proc is not None and self.proc.poll() is not None:
                raise RuntimeError(f"server exited with code {self.proc.returncode} before it answered")
            try:
                with urllib.request.urlopen(self.url + path, timeout=5.0) as r:   # noqa: S310
                    return json.load(r)
            except (urllib.error.URLError, OSError, ValueError) as e:
                last = str(e)
            time.sleep(poll)
        raise TimeoutError(f"{self.url}{path} did not answer within {timeout:.0f} s ({last})")

    def stop(self, grace: float = 20.0) -> int | None:
        p, self.proc = self.proc, None
        if p is None:
            return None
        if p.poll() is None:
            p.terminate()
            try:
                p.wait(grace)
            except subprocess.TimeoutExpired:
                p.kill()
                p.wait(grace)
        if self._log not in (None, subprocess.DEVNULL):
            self._log.close()
        return p.returncode

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()


def _common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n


def _int_metric(m: Mapping[str, Any], name: str) -> int | None:
    v = m.get(name)
    return v if isinstance(v, int) and not isinstance(v, bool) else None


def evaluate_response(*, models: Mapping[str, Any], response: Mapping[str, Any], model: str, expected_text: str,
                      encode: Callable[[str], Sequence[int]], block_size: int) -> dict:
    """Gate on one deterministic completion of a server that reports its speculative-decoding counters in the
    response (`metrics.speculative_decoding` for vLLM, `meta_info` for SGLang)."""
    n = draft_tokens(block_size)
    served = {e.get("id") for e in models.get("data", []) if isinstance(e, Mapping)} if isinstance(models.get("data"), list) else set()
    choices = response.get("choices")
    choice = choices[0] if isinstance(choices, list) and choices and isinstance(choices[0], Mapping) else {}
    prefix = _common_prefix(list(encode(str(choice.get("text") or ""))), list(encode(expected_text)))
    spec = None
    if isinstance(response.get("metrics"), Mapping):
        spec = response["metrics"].get("speculative_decoding")
    if not isinstance(spec, Mapping) and isinstance(choice.get("meta_info"), Mapping):
        mi = choice["meta_info"]          # SGLang: counters sit beside the completion
        spec = {"num_spec_tokens": mi.get("spec_num_draft_tokens", mi.get("num_spec_tokens")),
                "num_spec_steps": mi.get("spec_verify_ct"),
                "num_accepted_draft_tokens": mi.get("spec_accepted_tokens", mi.get("num_accepted_draft_tokens")),
                "num_draft_tokens": mi.get("spec_draft_tokens", mi.get("num_draft_tokens")),
                "acceptance_histogram": mi.get("spec_accept_histogram", mi.get("acceptance_histogram"))}
    m = spec if isinstance(spec, Mapping) else {}
    reported, steps = _int_metric(m, "num_spec_tokens"), _int_metric(m, "num_spec_steps")
    accepted, drafted = _int_metric(m, "num_accepted_draft_tokens"), _int_metric(m, "num_draft_tokens")
    hist = m.get("acceptance_histogram")
    full = hist[n] if isinstance(hist, list) and len(hist) > n and isinstance(hist[n], int) and not isinstance(hist[n], bool) else 0
    errors = []
    if model not in served:
        errors.append(f"model {model!r} is not served")
    if response.get("model") != model:
        errors.append(f"response model {response.get('model')!r} != requested model {model!r}")
    if not isinstance(spec, Mapping):
        errors.append("the response carries no speculative-decoding counters")
    if reported != n:
        errors.append(f"server drafts {reported!r} tokens per step, the drafter was trained for {n}")
    if steps is None or steps <= 0:
        errors.append("num_spec_steps must be positive")
    if accepted is None or accepted < n:
        errors.append("accepted draft tokens do not cover one draft block")
    if drafted is None or drafted < n:
        errors.append("drafted tokens do not cover one draft block")
    if full < 1:
        errors.append("no complete draft block was accepted")
    if prefix < n:
        errors.append(f"target prefix match {prefix} < draft length {n}")
    return {"passed": not errors, "served_model": response.get("model"), "num_speculative_tokens": reported,
            "num_spec_steps": steps, "num_accepted_draft_tokens": accepted, "num_draft_tokens": drafted,
            "full_blocks_accepted": full, "target_prefix_match_tokens": prefix, "errors": errors}


def _request_json(url: str, payload: Mapping[str, Any] | None, timeout: float) -> dict:
    body = None if payload is None else json.dumps(payload).encode()
    req = urllib.request.Request(url, data=body, headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:   # noqa: S310 (user-supplied endpoint)
        return json.load(r)


def verify_server(*, server_url: str, model: str, prompt: str, expected_text: str,
                  encode: Callable[[str], Sequence[int]], block_size: int, max_tokens: int | None = None,
                  timeout: float = 1800.0, request=_request_json) -> dict:
    """One greedy completion of `prompt` against a running server, gated by `evaluate_response`."""
    n = draft_tokens(block_size)
    want = n if max_tokens is None else int(max_tokens)
    if want < n:
        raise ValueError("max_tokens must cover one draft block")
    root = server_url.rstrip("/")
    models = request(f"{root}/v1/models", None, 30.0)
    response = request(f"{root}/v1/completions", {"model": model, "prompt": prompt, "max_tokens": want,
                                                   "temperature": 0.0, "top_p": 1.0, "n": 1, "stream": False},
                       float(timeout))
    return evaluate_response(models=models, response=response, model=model, expected_text=expected_text, encode=encode,
                             block_size=block_size)


def build_sglang_command(*, target_model: str, draft_export: str, port: int = 30000, tp: int = 1,
                         num_speculative_tokens: int = 15, extra: list[str] | None = None) -> list[str]:
    return ["python", "-m", "sglang.launch_server", "--model-path", target_model, "--speculative-algorithm", "DFLASH",
            "--speculative-draft-model-path", draft_export, "--speculative-num-draft-tokens",
            str(num_speculative_tokens), "--tp", str(tp), "--port", str(port), *(extra or [])]


def build_vllm_command(*, target_model: str, draft_export: str, port: int = 8000, tp: int = 1,
                       num_speculative_tokens: int = 15, extra: list[str] | None = None) -> list[str]:
    spec = {"method": "dflash", "model": draft_export, "num_speculative_tokens": num_speculative_tokens}
    return ["vllm", "serve", target_model, "--speculative-config", json.dumps(spec), "--tensor-parallel-size", str(tp),
            "--port", str(port), *(extra or [])]


def _post(url: str, payload: dict, timeout: float = 120.0) -> dict:
    req = urllib.request.Request(url, data=json.dumps(payload).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:   # noqa: S310 (user-supplied local endpoint)
        return json.load(r)


def parse_acceptance_length(metrics_text: str) -> float | None:
    """Reads mean accepted tokens per verification step from Prometheus text of either server."""
    for pat in (r"spec_decode_mean_acceptance_length\S*\s+([0-9.eE+-]+)", r"sglang:spec_accept_length\S*\s+([0-9.eE+-]+)",
                r"avg_spec_accept_length\S*\s+([0-9.eE+-]+)"):
        m = re.search(pat, metrics_text)
        if m:
            return float(m.group(1))
    acc = re.search(r"spec_decode_num_accepted_tokens_total\S*\s+([0-9.eE+-]+)", metrics_text)
    drafts = re.search(r"spec_decode_num_drafts_total\S*\s+([0-9.eE+-]+)", metrics_text)
    if acc and drafts and float(drafts.group(1)) > 0:
        return 1.0 + float(acc.group(1)) / float(drafts.group(1))
    return None


def verify_acceptance(base_url: str, model: str, prompts: list[str], min_acceptance_length: float = 1.5,
                      max_tokens: int = 64, post=_post, fetch_metrics=None) -> dict:
    for p in prompts:
        post(f"{base_url}/v1/completions", {"model": model, "prompt": p, "max_tokens": max_tokens, "temperature": 0})
    if fetch_metrics is None:
        def fetch_metrics():
            with urllib.request.urlopen(f"{base_url}/metrics", timeout=30) as r:   # noqa: S310
                return r.read().decode()
    length = parse_acceptance_length(fetch_metrics())
    ok = length is not None and length >= min_acceptance_length
    return {"ok": ok, "acceptance_length": length, "min_acceptance_length": min_acceptance_length}

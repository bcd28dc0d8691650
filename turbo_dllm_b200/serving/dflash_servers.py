"""Command builders and verification for serving an exported DFlash drafter as the speculative
decoding draft model of SGLang or vLLM.

`build_sglang_command` / `build_vllm_command` return argv lists (no process is started here);
`verify_acceptance` talks to a running OpenAI-compatible endpoint, sends a few prompts and reads
the server's speculative-decoding metrics to check the mean acceptance length against a floor.

Counterparts: dllm_parallel/serving/sglang_dflash.py:17-186, dllm_parallel/serving/vllm_dflash.py:21-328.
"""
from __future__ import annotations

import json
import re
import urllib.request


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

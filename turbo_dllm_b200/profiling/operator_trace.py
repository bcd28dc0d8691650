"""Operator and communication annotations for system traces.

`operator_scope(name)` and `communication_scope(domain, phase, collective, input_bytes,
logical_bytes)` open a named range (NVTX under nsys, `record_function` under Kineto) with the label
grammar `dllm.communication.domain=…;phase=…;collective=…;input_bytes=…;logical_bytes=…`, which
`trace_analysis` parses back into bytes and exposed time per label. Outside a trace window they are
`nullcontext()`: the backend is read from `DLLM_INTERNAL_OPERATOR_TRACE_BACKEND`, which
`SystemTrace` sets while its window is open.

Counterpart of dllm_parallel/core/profiling/operator_trace.py:21-138.
"""
from __future__ import annotations

import contextlib
import functools
import os

BACKEND_ENV = "DLLM_INTERNAL_OPERATOR_TRACE_BACKEND"


def active_backend() -> str | None:
    v = os.environ.get(BACKEND_ENV)
    return v if v in ("kineto", "nsys") else None


def _range(label: str):
    backend = active_backend()
    if backend is None:
        return contextlib.nullcontext()
    import torch

    if backend == "nsys":
        return torch.cuda.nvtx.range(label)
    return torch.profiler.record_function(label)


def operator_label(name: str) -> str:
    return f"dllm.operator.{name}"


def communication_label(domain: str, phase: str, collective: str, input_bytes: int = 0,
                        logical_bytes: int | None = None) -> str:
    logical = input_bytes if logical_bytes is None else logical_bytes
    return (f"dllm.communication.domain={domain};phase={phase};collective={collective};"
            f"input_bytes={int(input_bytes)};logical_bytes={int(logical)}")


def parse_communication_label(label: str) -> dict | None:
    prefix = "dllm.communication."
    if not label.startswith(prefix):
        return None
    out = {}
    for part in label[len(prefix):].split(";"):
        k, _, v = part.partition("=")
        out[k] = int(v) if k.endswith("bytes") and v.lstrip("-").isdigit() else v
    return out


def operator_scope(name: str):
    return _range(operator_label(name))


def communication_scope(domain: str, phase: str, collective: str, input_bytes: int = 0,
                        logical_bytes: int | None = None):
    return _range(communication_label(domain, phase, collective, input_bytes, logical_bytes))


def traced_operator(name: str):
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **kw):
            with operator_scope(name):
                return fn(*a, **kw)

        return wrapper

    return deco

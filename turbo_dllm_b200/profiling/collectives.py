"""`torch.distributed` collectives wrapped in communication labels.

Call sites name their communication domain (the process-group axis: `tensor`, `expert`, `context_parallel`,
`optimizer_data_parallel`, `world`); the phase (`forward` / `backward`) is read from autograd, and the byte
counts from the tensors. Outside a trace window the label is a `nullcontext`, so the wrappers cost one
function call. `trace_analysis` turns the labels back into bytes and time per (domain, phase, collective).

The reference labels every collective site by hand with `communication_scope`
(dllm_parallel/core/profiling/operator_trace.py:80-138); here the sites share these wrappers.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .operator_trace import active_backend, communication_scope


def _phase() -> str:
    try:
        return "backward" if torch._C._current_graph_task_id() != -1 else "forward"
    except Exception:
        return "forward"


def _nbytes(t: torch.Tensor) -> int:
    return int(t.numel()) * int(t.element_size())


def _scope(domain: str, collective: str, input_bytes: int, logical_bytes: int | None = None):
    if active_backend() is None:
        import contextlib

        return contextlib.nullcontext()
    return communication_scope(domain, _phase(), collective, input_bytes, logical_bytes)


def all_reduce(t: torch.Tensor, domain: str, **kw):
    with _scope(domain, "all_reduce", _nbytes(t)):
        return dist.all_reduce(t, **kw)


def all_gather_into_tensor(out: torch.Tensor, x: torch.Tensor, domain: str, **kw):
    with _scope(domain, "all_gather", _nbytes(x), _nbytes(out)):
        return dist.all_gather_into_tensor(out, x, **kw)


def reduce_scatter_tensor(out: torch.Tensor, x: torch.Tensor, domain: str, **kw):
    with _scope(domain, "reduce_scatter", _nbytes(x), _nbytes(out)):
        return dist.reduce_scatter_tensor(out, x, **kw)


def all_to_all_single(out: torch.Tensor, x: torch.Tensor, *args, domain: str, **kw):
    with _scope(domain, "all_to_all", _nbytes(x), _nbytes(out)):
        return dist.all_to_all_single(out, x, *args, **kw)


def broadcast(t: torch.Tensor, domain: str, **kw):
    with _scope(domain, "broadcast", _nbytes(t)):
        return dist.broadcast(t, **kw)

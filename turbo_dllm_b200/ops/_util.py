"""Helpers shared by the op wrappers: pointers, streams, parameter gradient sinks."""
from __future__ import annotations

import torch

from ..kernels import native


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def use_native(*tensors: torch.Tensor) -> bool:
    """CUDA bf16 tensors run on the sm_100a kernels; anything else on the PyTorch reference.
    On a CUDA device a missing library raises instead of falling back."""
    t = tensors[0]
    if not t.is_cuda:
        return False
    if t.dtype != torch.bfloat16:
        return False
    native.lib()
    return True


def grad_sink(param: torch.Tensor):
    """Returns (buffer, accumulate) when `param` owns a slice of a flat gradient buffer
    (`param.main_grad`), else (None, False). The first write of a step overwrites, later
    writes accumulate, so the flat buffer never needs zeroing."""
    mg = getattr(param, "main_grad", None)
    if mg is None:
        return None, False
    acc = bool(getattr(param, "grad_acc", False))
    return mg, acc


def mark_grad_written(param: torch.Tensor) -> None:
    param.grad_acc = True


_scratch: dict = {}


def scratch(device: torch.device, nfloats: int, key: str = "f32") -> torch.Tensor:
    """A per-device fp32 scratch buffer that only grows (kernel partial sums and the like)."""
    k = (device, key)
    buf = _scratch.get(k)
    if buf is None or buf.numel() < nfloats:
        buf = torch.empty(max(nfloats, 1 << 16), dtype=torch.float32, device=device)
        _scratch[k] = buf
    return buf

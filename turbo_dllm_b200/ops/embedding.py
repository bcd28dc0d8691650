"""Token embedding whose gradient is scattered straight into the flat gradient buffer."""
from __future__ import annotations

import torch

from ._util import grad_sink, mark_grad_written


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, weight):
        ctx.save_for_backward(tokens)
        ctx.wref = weight
        return weight.index_select(0, tokens)

    @staticmethod
    def backward(ctx, dy):
        (tokens,) = ctx.saved_tensors
        sink, acc = grad_sink(ctx.wref)
        if sink is None:
            dw = torch.zeros_like(ctx.wref)
            dw.index_add_(0, tokens, dy.to(dw.dtype))
            return None, dw
        if not acc:
            sink.zero_()
        sink.index_add_(0, tokens, dy.to(sink.dtype))
        mark_grad_written(ctx.wref)
        return None, None


def embedding(tokens: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return _Embedding.apply(tokens, weight)

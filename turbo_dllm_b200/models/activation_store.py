"""Per-layer activation checkpointing with optional host offload.

Only the residual stream entering each layer is kept for the backward pass, plus (optionally) the
attention output and log-sum-exp of the layer so that the recomputation can skip the attention
forward kernel; everything else inside a layer is recomputed. With `offload=True` that tensor is copied to pinned host memory on a side
stream right after the layer ran and brought back (prefetched one layer ahead) during the
backward pass, so a long sequence costs one layer's activations of HBM instead of `num_layers`.
The copies run on their own CUDA stream and overlap the GEMMs; per-step PCIe traffic is
2 × rows × hidden × 2 bytes × layers.

The reference checkpoints each layer with torch.utils.checkpoint and keeps all layer inputs on
the device (dllm_parallel/core/models/backbones/nemotron/model.py:2373-2445).
"""
from __future__ import annotations

import torch


class ActivationStore:
    def __init__(self, device: torch.device, offload: bool = False, offload_attention: bool | None = None):
        self.device = torch.device(device)
        self.offload = bool(offload) and self.device.type == "cuda"            # layer inputs
        self.offload_attention = (self.offload if offload_attention is None
                                  else bool(offload_attention) and self.device.type == "cuda")
        self.kept: dict[int, torch.Tensor] = {}
        self.host: dict[int, torch.Tensor] = {}
        self.ready: dict[int, torch.cuda.Event] = {}
        self.inflight: dict[int, tuple[torch.Tensor, torch.cuda.Event]] = {}
        self.stream = (torch.cuda.Stream(device=self.device)
                       if (self.offload or self.offload_attention) else None)
        self.bytes_offloaded = 0
        self.recording = False      # True while a checkpointed layer runs its no-grad forward
        self.replaying = False      # True while a checkpointed layer is recomputed for backward
        self.keep_attention = True  # stash (out, lse) of the attention op across the boundary
        # attention outputs of layers >= this index stay on the device even when the others are offloaded
        # (the backward pass needs the last layers first, while earlier ones are still being fetched)
        self.attention_resident_from = 1 << 30
        # how many layers ahead the backward pass fetches offloaded tensors (TDLLM_PREFETCH_DEPTH; each layer in
        # flight holds its tensors in device memory until it is consumed)
        import os

        self.prefetch_depth = max(1, int(os.environ.get("TDLLM_PREFETCH_DEPTH", "1")))

    def has(self, idx) -> bool:
        return idx in self.kept or idx in self.ready

    def _to_host(self, idx) -> bool:
        if isinstance(idx, tuple):
            return self.offload_attention and idx[0] < self.attention_resident_from
        return self.offload

    def stash(self, idx, x: torch.Tensor) -> None:
        if not self._to_host(idx):
            self.kept[idx] = x
            return
        buf = self.host.get(idx)
        if buf is None or buf.shape != x.shape or buf.dtype != x.dtype:
            buf = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
            self.host[idx] = buf
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            buf.copy_(x, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        x.record_stream(self.stream)  # keep the device block alive until the copy has read it
        self.ready[idx] = ev
        self.bytes_offloaded += x.numel() * x.element_size()

    def prefetch(self, idx) -> None:
        if not self._to_host(idx) or idx in self.inflight or idx not in self.host or idx not in self.ready:
            return
        with torch.cuda.stream(self.stream):
            self.ready[idx].wait(self.stream)
            dev = torch.empty(self.host[idx].shape, dtype=self.host[idx].dtype, device=self.device)
            dev.copy_(self.host[idx], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.inflight[idx] = (dev, ev)

    def fetch(self, idx) -> torch.Tensor:
        if not self._to_host(idx):
            return self.kept.pop(idx)
        self.prefetch(idx)
        dev, ev = self.inflight.pop(idx)
        self.ready.pop(idx, None)
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(ev)
        dev.record_stream(cur)
        return dev


class _LayerCheckpoint(torch.autograd.Function):
    """Runs `layer(h, *args)` without building a graph; the backward pass re-runs it with grad and
    back-propagates. Parameter gradients are written by the ops themselves (flat gradient
    buffer), so only the gradient of `h` is returned."""

    @staticmethod
    def forward(ctx, h, layer, store, idx, args):
        ctx.layer, ctx.store, ctx.idx, ctx.args = layer, store, idx, args
        store.recording = True
        try:
            with torch.no_grad():
                out = layer(h, *args)
        finally:
            store.recording = False
        store.stash(idx, h)
        return out

    @staticmethod
    def backward(ctx, dout):
        store, idx = ctx.store, ctx.idx
        h = store.fetch(idx)
        for d in range(1, store.prefetch_depth + 1):   # host -> device copies of the layers the backward pass needs next
            for key in (idx - d, (idx - d, "attn_out"), (idx - d, "attn_lse"), (idx - d, "attn_kv_pulled")):
                store.prefetch(key)
        h = h.detach().requires_grad_(True)
        from ..ops.gemm import skip_last_output

        sharded = getattr(ctx.layer, "sharded", None)
        if sharded is not None:      # parameter sharding: bring the layer's weights back, point its gradients
            sharded.pre_layer(idx)
            sharded.begin_layer_backward(idx)
        store.replaying = True
        try:
            with torch.enable_grad(), skip_last_output():
                out = ctx.layer(h, *ctx.args)   # its value is not needed: only the graph behind it
        finally:
            store.replaying = False
        torch.autograd.backward(out, dout)
        if sharded is not None:      # the layer's gradients are complete: reduce them into the ranks' shards
            sharded.post_layer_backward(idx)
        return h.grad, None, None, None, None


def checkpointed_layer(layer, h, store: ActivationStore, idx: int, *args):
    return _LayerCheckpoint.apply(h, layer, store, idx, args)

"""AdamW over the flat parameter/gradient buffers, optionally sharded over a data-parallel group.

Each rank keeps fp32 master weights and Adam moments only for its contiguous shard of the flat
buffer (ZeRO-1/2 semantics: replicated low-precision parameters, sharded optimizer state):
  gradient sync  : reduce-scatter(sum) of the flat gradient -> this rank's shard
  clip           : global L2 norm = sqrt(all-reduce(Σ shard²)), folded into the update
  update         : one fused kernel per range (decayed / non-decayed), bf16 params rewritten
  parameter sync : all-gather of the updated shards
On one rank all collectives vanish. `sync_impl="nccl"` uses torch.distributed collectives (the
baseline twin); `"fused"` hands the whole sequence to the peer-memory kernel of
`parallel.symm` when the process group has one.

Reference counterparts: DeepSpeed ZeRO-2 + FusedAdam wiring (dllm_parallel/core/optim/zero.py:93-211, :402-462),
`FirstPartyDistributedAdamW` (dllm_parallel/core/optim/adamw.py:20-100) and gradient clipping
(dllm_parallel/training/optimizer_setup.py:311-372).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..kernels import native
from ..models.dense import ALIGN, FlatParams
from ..ops._util import ptr, stream
from ..profiling.operator_trace import communication_scope


def shard_bounds(numel: int, parts: int, index: int) -> tuple[int, int]:
    """Contiguous shards whose boundaries are multiples of ALIGN (the last one takes the tail)."""
    units = (numel + ALIGN - 1) // ALIGN
    base, rem = divmod(units, parts)
    start = index * base + min(index, rem)
    stop = start + base + (1 if index < rem else 0)
    return min(start * ALIGN, numel), min(stop * ALIGN, numel)


class FlatAdamW:
    def __init__(self, flat: FlatParams, *, lr: float, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, group=None, sync_impl: str = "nccl", fused_sync=None,
                 tp_group=None):
        self.flat = flat
        self.tp_group = tp_group   # matrices are sharded over it, norm weights replicated
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.group = group
        self.world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.sync_impl = sync_impl
        self.fused_sync = fused_sync
        # equal-sized shards make reduce-scatter / all-gather single collectives: pad the flat size
        per = (flat.numel + self.world * ALIGN - 1) // (self.world * ALIGN) * ALIGN
        self.shard_size = per
        self.start = min(self.rank * per, flat.numel)
        self.stop = min(self.start + per, flat.numel)
        n = self.stop - self.start
        dev = flat.data.device
        self.master = flat.data[self.start:self.stop].float().clone()
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.step_count = 0
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.last_grad_norm = None

    # ------------------------------------------------------------------ sync
    def _reduce_scatter_grads(self) -> torch.Tensor:
        """Returns the summed gradient of this rank's shard."""
        g = self.flat.grad
        if self.world == 1:
            return g[self.start:self.stop]
        per = self.shard_size
        if g.is_cuda:
            padded = g if g.numel() == per * self.world else torch.nn.functional.pad(g, (0, per * self.world - g.numel()))
            out = torch.empty(per, dtype=g.dtype, device=g.device)
            with communication_scope("optimizer_data_parallel", "gradient_sync", "reduce_scatter",
                                     padded.numel() * padded.element_size()):
                dist.reduce_scatter_tensor(out, padded, op=dist.ReduceOp.SUM, group=self.group)
            return out[: self.stop - self.start]
        with communication_scope("optimizer_data_parallel", "gradient_sync", "all_reduce", g.numel() * g.element_size()):
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group)  # gloo has no reduce_scatter
        return g[self.start:self.stop]

    def _all_gather_params(self) -> None:
        if self.world == 1:
            return
        p = self.flat.data
        per = self.shard_size
        mine = torch.zeros(per, dtype=p.dtype, device=p.device)
        mine[: self.stop - self.start] = p[self.start:self.stop]
        full = torch.empty(per * self.world, dtype=p.dtype, device=p.device)
        with communication_scope("optimizer_data_parallel", "optimizer", "all_gather", per * p.element_size(),
                                 per * self.world * p.element_size()):
            dist.all_gather_into_tensor(full, mine, group=self.group)
        p.copy_(full[: p.numel()])

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, *, lr: float | None = None, weight_decay: float | None = None,
             grad_scale: float = 1.0, max_grad_norm: float = 0.0) -> None:
        """One optimizer step on gradients already present in flat.grad."""
        if self.fused_sync is not None and self.world > 1:
            self.step_count += 1
            nbytes = (self.stop - self.start) * 2 * (self.world - 1)
            with communication_scope("optimizer_data_parallel", "optimizer", "fused_zero_pull_push", nbytes, 2 * nbytes):
                self.fused_sync.step(self, self.lr if lr is None else lr,
                                     self.weight_decay if weight_decay is None else weight_decay, grad_scale,
                                     max_grad_norm)
            return
        sumsq = self.reduce_gradients()
        self.apply_update(sumsq, lr=lr, weight_decay=weight_decay, grad_scale=grad_scale,
                          max_grad_norm=max_grad_norm)

    @torch.no_grad()
    def reduce_gradients(self) -> torch.Tensor:
        """Phase 1: gradient sync. Returns Σ g² of the synchronised gradient over this optimizer's
        whole buffer (already summed over the group's shards) as a 1-element device tensor."""
        self._gshard = self._reduce_scatter_grads()
        if self.tp_group is None:
            sumsq = self._grad_sumsq(self._gshard).clone()
        else:
            # tensor-parallel shards of the matrices add up over the TP group; replicated norm
            # weights (the non-decayed tail of the buffer) must be counted once
            n = self.stop - self.start
            # (a buffer may name the end of its sharded part itself: adapters decay all their matrices but
            # replicate some of them)
            sharded_end = getattr(self.flat, "tp_sharded_numel", self.flat.decay_numel)
            split = min(max(sharded_end - self.start, 0), n)
            sharded = self._grad_sumsq(self._gshard[:split]).clone() if split > 0 else torch.zeros(
                1, device=self._gshard.device)
            dist.all_reduce(sharded, op=dist.ReduceOp.SUM, group=self.tp_group)
            repl = self._grad_sumsq(self._gshard[split:]).clone() if n > split else torch.zeros_like(sharded)
            sumsq = sharded + repl
        if self.world > 1:
            with communication_scope("optimizer_data_parallel", "gradient_clip", "all_reduce", 4):
                dist.all_reduce(sumsq, op=dist.ReduceOp.SUM, group=self.group)
        return sumsq

    @torch.no_grad()
    def apply_update(self, sumsq: torch.Tensor, *, lr=None, weight_decay=None, grad_scale: float = 1.0,
                     max_grad_norm: float = 0.0) -> None:
        """Phase 2: clip against `sumsq` (which may include other optimizers' buffers), AdamW on the
        shard, parameter all-gather."""
        lr = self.lr if lr is None else lr
        wd = self.weight_decay if weight_decay is None else weight_decay
        self.step_count += 1
        gshard = self._gshard
        self.last_grad_norm = sumsq
        n = self.stop - self.start
        pshard = self.flat.data[self.start:self.stop]
        split = min(max(self.flat.decay_numel - self.start, 0), n)  # [0, split) decayed, rest not
        b1, b2 = self.betas
        for lo, hi, w in ((0, split, wd), (split, n, 0.0)):
            if hi <= lo:
                continue
            if gshard.is_cuda and gshard.dtype == torch.bfloat16:
                native.check(native.lib().tdllm_adamw(
                    ptr(self.master[lo:hi]), ptr(self.m[lo:hi]), ptr(self.v[lo:hi]), ptr(gshard[lo:hi]),
                    ptr(pshard[lo:hi]), hi - lo, lr, b1, b2, self.eps, w, self.step_count, grad_scale,
                    ptr(sumsq), max_grad_norm, stream()), "adamw")
            else:
                self._reference_update(lo, hi, gshard, pshard, lr, w, grad_scale, sumsq, max_grad_norm)
        self._gshard = None
        self._all_gather_params()

    def _grad_sumsq(self, gshard: torch.Tensor) -> torch.Tensor:
        if gshard.is_cuda and gshard.dtype == torch.bfloat16:
            self._sumsq.zero_()
            native.check(native.lib().tdllm_sumsq_bf16(ptr(gshard), gshard.numel(), ptr(self._sumsq), stream()),
                         "sumsq")
            return self._sumsq
        return gshard.float().pow(2).sum().reshape(1)

    def _reference_update(self, lo, hi, gshard, pshard, lr, wd, grad_scale, sumsq, max_norm):
        b1, b2 = self.betas
        gs = grad_scale
        if sumsq is not None and max_norm > 0:
            norm = float(sumsq.sqrt()) * grad_scale
            if norm > max_norm:
                gs *= max_norm / (norm + 1e-6)
        g = gshard[lo:hi].float() * gs
        m, v, p = self.m[lo:hi], self.v[lo:hi], self.master[lo:hi]
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        bias1 = 1 - b1 ** self.step_count
        bias2 = 1 - b2 ** self.step_count
        p.mul_(1 - lr * wd).addcdiv_(m / bias1, (v / bias2).sqrt().add_(self.eps), value=-lr)
        pshard[lo:hi].copy_(p)

    def grad_norm(self, grad_scale: float = 1.0) -> float:
        """Global gradient L2 norm of the last step (synchronises)."""
        if self.last_grad_norm is None:
            return float("nan")
        return math.sqrt(float(self.last_grad_norm)) * grad_scale

    # ------------------------------------------------------------- checkpoint
    def state_dict(self) -> dict:
        return {"step_count": self.step_count, "shard": (self.start, self.stop), "world": self.world,
                "master": self.master, "m": self.m, "v": self.v}

    def load_state_dict(self, state: dict) -> None:
        if tuple(state["shard"]) != (self.start, self.stop) or state["world"] != self.world:
            raise ValueError("optimizer shard layout differs from the checkpoint (resharding is not supported)")
        self.step_count = int(state["step_count"])
        self.master.copy_(state["master"])
        self.m.copy_(state["m"])
        self.v.copy_(state["v"])
        self.flat.data[self.start:self.stop].copy_(self.master)

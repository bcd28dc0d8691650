"""Parameter sharding (FSDP) over the optimizer data-parallel group.

Every rank keeps 1/W of the bf16 parameters, an fp32 gradient shard of the same size and the fp32 AdamW
state of that shard; full-size parameters and gradients exist only for the layer that is running.

Units. The flat parameter buffer (`FlatParams`) is cut into units: the matrices of one decoder layer (contiguous
in the buffer), every other matrix on its own (embedding, LM head) and the tail of non-decayed norm weights.
Each unit is split evenly over the W ranks (multiples of 128 elements), so every rank serves and receives the
same share of every unit.

Schedule of one step.
  forward   layer i      : gather unit i into one of two rotating full-size buffers (its parameters are views)
  backward  layer i      : gather again for the recomputation (activation checkpointing is required), run the
                           backward (weight gradients land in one of two rotating full-size gradient buffers),
                           barrier, reduce: this rank's piece of every rank's buffer, summed in fp32 into the
                           gradient shard (added to it for later micro-batches)
  end of the step        : the same reduce for the resident units (embedding, LM head, norm weights)
  optimizer              : Σg² of the shard (+ the other ranks') → clip → AdamW from the fp32 gradient shard,
                           new bf16 values into the parameter shard, barrier, resident units gathered again
One barrier per unit is enough with two gradient buffers: a rank passes the barrier of unit u+1 only after every
rank has finished reducing unit u, which is when the buffer of unit u may be overwritten by unit u+2.

Transports. On CUDA the gather and the reduce are peer-memory kernels over symmetric buffers (`csrc/comm.cu`:
plain peer loads, no NCCL); on CPU ranks, or with `kernel.impl: nccl_baseline`, they are `all_gather_into_tensor`
and `reduce_scatter` / `all_reduce` of torch.distributed, the twin the kernels are tested against.

Counterparts: `wrap_model_with_fsdp` and the FSDP2 `fully_shard` wiring of the reference
(dllm_parallel/core/optim/fsdp.py:56-114, :145-264), its sharded state-dict helpers (:267-317) and the
ZeRO partitioning of dllm_parallel/core/optim/zero.py:93-211.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..kernels import native
from ..profiling.operator_trace import communication_scope

ALIGN = 128

_V, _I, _LL, _F = native.c_void_p, native.c_int, native.c_ll, native.c_float
native.register_signatures({
    "tdllm_fsdp_gather": (_I, [_V, _LL, _LL, _LL, _I, _I, _V, _V]),
    "tdllm_fsdp_reduce": (_I, [_V, _LL, _LL, _I, _I, _V, _I, _V]),
    "tdllm_adamw_f32grad": (_I, [_V, _V, _V, _V, _V, _LL] + [_F] * 5 + [_I, _F, _V, _F, _V]),
})


@dataclass
class Unit:
    name: str
    start: int          # range of the flat buffer
    stop: int
    shard: int          # elements per rank (multiple of ALIGN); shard * world >= stop - start
    local: int          # offset of this rank's piece inside its shard buffers
    layer: int | None   # decoder layer index, None for resident units
    decay: bool

    @property
    def length(self) -> int:
        return self.stop - self.start


def plan_units(flat, world: int) -> list[Unit]:
    """Cuts the flat buffer into units (see the module docstring). Parameters of one layer must be contiguous,
    which `FlatParams` guarantees for the decayed matrices (stable order inside the decayed region)."""
    spans: dict[str, list[int]] = {}
    order: list[str] = []
    for name, (o, n, _shape, decay) in flat.offsets.items():
        end = (o + n + ALIGN - 1) // ALIGN * ALIGN
        if not decay:
            key = "norm_weights"
        else:
            m = re.match(r"layers\.(\d+)\.", name)
            key = f"layer.{int(m.group(1))}" if m else name
        if key not in spans:
            spans[key] = [o, end]
            order.append(key)
        else:
            spans[key][0] = min(spans[key][0], o)
            spans[key][1] = max(spans[key][1], end)
    order.sort(key=lambda k: spans[k][0])
    units, local, prev_end = [], 0, 0
    for key in order:
        a, b = spans[key]
        if a < prev_end:
            raise ValueError(f"parameters of unit {key} are not contiguous in the flat buffer")
        prev_end = b
        shard = (math.ceil((b - a) / world) + ALIGN - 1) // ALIGN * ALIGN
        layer = int(key.split(".")[1]) if key.startswith("layer.") else None
        units.append(Unit(key, a, b, shard, local, layer, key != "norm_weights"))
        local += shard
    # the non-decayed tail comes last in the shard so that weight decay covers one contiguous range
    units.sort(key=lambda u: (not u.decay, u.start))
    local = 0
    for u in units:
        u.local = local
        local += u.shard
    return units


class _LocalBuffer:
    """A buffer that only this rank touches; same surface as `SymmetricBuffer` where the code needs it."""

    def __init__(self, nbytes: int, device):
        self.t = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device=device)

    def as_tensor(self, dtype, numel=None, offset_bytes: int = 0):
        t = self.t[offset_bytes:].view(dtype)
        return t if numel is None else t[:numel]

    def close(self):
        self.t = None


class ShardedParameters:
    """Owns the shards, the rotating full-size buffers and the step schedule of one model's flat parameters."""

    def __init__(self, flat, group, device, *, use_peer_kernels: bool, num_layers: int):
        if flat.grad.numel() == 0:
            raise ValueError("parameter sharding needs a trainable model")
        self.flat, self.group, self.device = flat, group, torch.device(device)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.peer = bool(use_peer_kernels) and self.device.type == "cuda"
        self.dtype = flat.data.dtype
        self.itemsize = flat.data.element_size()
        self.units = plan_units(flat, self.world)
        self.by_layer = {u.layer: u for u in self.units if u.layer is not None}
        self.resident = [u for u in self.units if u.layer is None]
        if sorted(self.by_layer) != list(range(num_layers)):
            raise ValueError("every decoder layer must form one unit of the flat parameter buffer")
        self.n_local = sum(u.shard for u in self.units)
        self.decay_local = sum(u.shard for u in self.units if u.decay)
        max_layer = max(u.shard * self.world for u in self.by_layer.values())
        dev = self.device
        # ---- persistent shards
        self.param_buf = self._buffer(self.n_local * self.itemsize, symmetric=True)
        self.param_shard = self.param_buf.as_tensor(self.dtype, self.n_local)
        self.grad_shard = torch.zeros(self.n_local, dtype=torch.float32, device=dev)
        # ---- rotating full-size buffers of the layer units, dedicated ones for the resident units
        self.full = [torch.zeros(max_layer, dtype=self.dtype, device=dev) for _ in range(2)]
        self.grad_bufs = [self._buffer(max_layer * self.itemsize, symmetric=True) for _ in range(2)]
        self.grad_full = [b.as_tensor(self.dtype, max_layer) for b in self.grad_bufs]
        self.res_full, self.res_grad_buf, self.res_grad = {}, {}, {}
        for u in self.resident:
            n = u.shard * self.world
            self.res_full[u.name] = torch.zeros(n, dtype=self.dtype, device=dev)
            self.res_grad_buf[u.name] = self._buffer(n * self.itemsize, symmetric=True)
            self.res_grad[u.name] = self.res_grad_buf[u.name].as_tensor(self.dtype, n)
        self.barrier = None
        if self.peer:
            from .symm import SymmetricBarrier

            self.barrier = SymmetricBarrier(group, dev)
        # ---- scatter the initial values, re-point the parameters, drop the replicated buffers
        with torch.no_grad():
            for u in self.units:
                piece = flat.data[u.start + self.rank * u.shard: min(u.start + (self.rank + 1) * u.shard, u.stop)]
                self.param_shard[u.local: u.local + piece.numel()].copy_(piece)
        self.loaded = [None, None]                  # layer whose parameters sit in full[k]
        self.params_of: dict[str, list] = {u.name: [] for u in self.units}
        for name, (o, n, shape, decay) in flat.offsets.items():
            u = self._unit_of(o)
            p = flat.params[name]
            rel = o - u.start
            if u.layer is None:
                p.data = self.res_full[u.name][rel: rel + n].view(shape)
                p.main_grad = self.res_grad[u.name][rel: rel + n].view(shape)
            else:
                p.data = self.full[u.layer % 2][rel: rel + n].view(shape)
                p.main_grad = self.grad_full[u.layer % 2][rel: rel + n].view(shape)
            self.params_of[u.name].append(p)
        self.full_numel = flat.numel
        flat.data = torch.zeros(0, dtype=self.dtype, device=dev)     # nothing replicated is left
        flat.grad = torch.zeros(0, dtype=self.dtype, device=dev)
        flat.sharded = self
        self.micro = 0            # micro-batches reduced into the gradient shard in this step
        self._reduced: set[str] = set()
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
            torch.cuda.empty_cache()
        dist.barrier(group=group)
        self.gather_resident()

    # ------------------------------------------------------------------ plumbing
    def _buffer(self, nbytes: int, symmetric: bool):
        if self.peer and symmetric:
            from .symm import SymmetricBuffer

            return SymmetricBuffer(max(nbytes, 256), self.group, self.device)
        return _LocalBuffer(nbytes, self.device)

    def _unit_of(self, offset: int) -> Unit:
        for u in self.units:
            if u.start <= offset < u.stop:
                return u
        raise KeyError(offset)

    def _sync(self) -> None:
        """Every rank's earlier work on the stream is complete on every rank after this point."""
        if self.peer:
            self.barrier.sync()

    def _gather(self, u: Unit, out: torch.Tensor) -> None:
        n = u.shard * self.world
        nbytes = u.shard * self.itemsize
        with communication_scope("optimizer_data_parallel", "forward", "fsdp_gather", nbytes * (self.world - 1),
                                 nbytes * self.world):
            if self.peer:
                from ..ops._util import ptr, stream

                native.check(native.lib().tdllm_fsdp_gather(self.param_buf.ptr_array, u.local, u.shard, n, self.rank,
                                                            self.world, ptr(out), stream()), "fsdp_gather")
            else:
                dist.all_gather_into_tensor(out[:n], self.param_shard[u.local: u.local + u.shard].contiguous(),
                                            group=self.group)

    def _reduce(self, u: Unit, grad_buf, grad_full: torch.Tensor) -> None:
        """grad_full (every rank's, full unit) -> this rank's fp32 piece of the gradient shard."""
        out = self.grad_shard[u.local: u.local + u.shard]
        acc = self.micro > 0
        nbytes = u.shard * self.itemsize
        with communication_scope("optimizer_data_parallel", "backward", "fsdp_reduce_scatter",
                                 nbytes * (self.world - 1), nbytes):
            if self.peer:
                from ..ops._util import ptr, stream

                self._sync()
                native.check(native.lib().tdllm_fsdp_reduce(grad_buf.ptr_array, self.rank * u.shard, u.shard, self.rank,
                                                            self.world, ptr(out), 1 if acc else 0, stream()),
                             "fsdp_reduce")
            else:
                full = grad_full[: u.shard * self.world].float()
                dist.all_reduce(full, group=self.group)
                piece = full[self.rank * u.shard: (self.rank + 1) * u.shard]
                out.add_(piece) if acc else out.copy_(piece)

    # ------------------------------------------------------------------ schedule
    def gather_resident(self) -> None:
        for u in self.resident:
            self._gather(u, self.res_full[u.name])

    def pre_layer(self, i: int) -> None:
        """Parameters of layer i are in place after this call (forward, and again for the recomputation)."""
        k = i % 2
        if self.loaded[k] != i:
            self._gather(self.by_layer[i], self.full[k])
            self.loaded[k] = i

    def begin_layer_backward(self, i: int) -> None:
        for p in self.params_of[f"layer.{i}"]:
            p.grad_acc = False      # the rotating gradient buffer holds another layer's values

    def post_layer_backward(self, i: int) -> None:
        u = self.by_layer[i]
        for p in self.params_of[u.name]:
            if p.grad is not None:
                p.main_grad.copy_(p.grad) if not p.grad_acc else p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None
                p.grad_acc = True
            elif not p.grad_acc:
                p.main_grad.zero_()
        tail = u.shard * self.world - u.length
        if tail:
            self.grad_full[i % 2][u.length: u.length + tail].zero_()
        self._reduce(u, self.grad_bufs[i % 2], self.grad_full[i % 2])
        self._reduced.add(u.name)

    def end_micro_batch(self, before_reduce=None) -> None:
        """After the backward pass of one micro-batch: resident units' gradients, layers without a backward.
        `before_reduce()` runs once every resident gradient is complete in its buffer and before the buffers
        are reduced (the tensor-parallel sum of partially computed norm-weight gradients goes there)."""
        for u in self.resident:
            for p in self.params_of[u.name]:
                if p.grad is not None:
                    p.main_grad.copy_(p.grad) if not p.grad_acc else p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    p.grad = None
                    p.grad_acc = True
                elif not p.grad_acc:
                    p.main_grad.zero_()
        if before_reduce is not None:
            before_reduce()
        for u in self.resident:
            self._reduce(u, self.res_grad_buf[u.name], self.res_grad[u.name])
            for p in self.params_of[u.name]:
                p.grad_acc = False
        for i, u in self.by_layer.items():
            if u.name not in self._reduced and self.micro == 0:
                self.grad_shard[u.local: u.local + u.shard].zero_()
        self._reduced.clear()
        self.micro += 1

    def zero_grad(self) -> None:
        self.micro = 0
        self._reduced.clear()
        for ps in self.params_of.values():
            for p in ps:
                p.grad_acc = False
                p.grad = None

    def params_updated(self) -> None:
        """Called by the optimizer after it rewrote the parameter shard."""
        self._sync()
        self.loaded = [None, None]
        self.gather_resident()

    # ------------------------------------------------------------------ whole-model views (tests, export)
    @torch.no_grad()
    def gather_full(self) -> torch.Tensor:
        """The replicated flat parameter buffer, rebuilt from the shards (allocates the full size)."""
        out = torch.zeros(self.full_numel, dtype=self.dtype, device=self.device)
        for u in self.units:
            tmp = torch.zeros(u.shard * self.world, dtype=self.dtype, device=self.device)
            self._gather(u, tmp)
            out[u.start: u.stop].copy_(tmp[: u.length])
        return out

    @torch.no_grad()
    def load_full(self, full: torch.Tensor) -> None:
        for u in self.units:
            piece = full[u.start + self.rank * u.shard: min(u.start + (self.rank + 1) * u.shard, u.stop)]
            self.param_shard[u.local: u.local + piece.numel()].copy_(piece)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.params_updated()

    def memory_bytes(self) -> dict:
        it = self.itemsize
        return {"parameter_shard": self.n_local * it, "gradient_shard_fp32": self.n_local * 4,
                "rotating_parameters": sum(t.numel() for t in self.full) * it,
                "rotating_gradients": sum(t.numel() for t in self.grad_full) * it,
                "resident_units": sum(t.numel() for t in self.res_full.values()) * it * 2,
                "replicated_equivalent": self.full_numel * it * 2}

    def close(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for b in (self.param_buf, *self.grad_bufs, *self.res_grad_buf.values()):
            b.close()
        if self.barrier is not None:
            self.barrier.buf.close()


class ShardedAdamW:
    """AdamW on the fp32 master copy of this rank's parameter shard, fed by the fp32 gradient shard."""

    def __init__(self, sharded: ShardedParameters, *, lr: float, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, tp_group=None):
        self.sp = sharded
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.group, self.world, self.rank = sharded.group, sharded.world, sharded.rank
        self.tp_group = tp_group
        self.master = sharded.param_shard.float().clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.step_count = 0
        self.last_grad_norm = None
        self.fused_sync = None     # the trainer reports "zero_fused" when this is set; not this optimizer

    @torch.no_grad()
    def step(self, *, lr: float | None = None, weight_decay: float | None = None, grad_scale: float = 1.0,
             max_grad_norm: float = 0.0) -> None:
        self.apply_update(self.reduce_gradients(), lr=lr, weight_decay=weight_decay, grad_scale=grad_scale,
                          max_grad_norm=max_grad_norm)

    @torch.no_grad()
    def reduce_gradients(self) -> torch.Tensor:
        """Σ g² of the whole (unsharded) gradient of this optimizer's parameters, as a 1-element tensor: the
        gradient shards were reduced layer by layer during the backward pass, so only the norm is left to do.
        Same two-phase surface as `FlatAdamW` (a second optimizer's share can be added before `apply_update`)."""
        sp = self.sp
        g = sp.grad_shard
        split = sp.decay_local
        boundary = getattr(sp.flat, "tp_sharded_numel", None) if self.tp_group is not None else None
        if boundary is not None:
            # the buffer names the end of its tensor-parallel part itself (some non-decayed vectors are sharded too):
            # split every unit's local piece at that offset of the flat buffer
            sharded_sq = torch.zeros(1, dtype=torch.float32, device=g.device)
            repl_sq = torch.zeros_like(sharded_sq)
            for u in sp.units:
                lo = u.start + sp.rank * u.shard                    # flat offsets of this rank's piece of the unit
                hi = min(lo + u.shard, u.stop)
                if hi <= lo:
                    continue
                cut = min(max(boundary, lo), hi) - lo
                piece = g[u.local: u.local + (hi - lo)]
                if cut > 0:
                    sharded_sq += torch.linalg.vector_norm(piece[:cut]).square()
                if cut < hi - lo:
                    repl_sq += torch.linalg.vector_norm(piece[cut:]).square()
        else:
            # vector_norm reduces without a temporary and takes more than 2^31 elements (a dot product does not)
            sharded_sq = torch.linalg.vector_norm(g[:split]).square().reshape(1)
            repl_sq = torch.linalg.vector_norm(g[split:]).square().reshape(1)
        if self.tp_group is not None:
            # matrices are split over the tensor-parallel group, norm weights are replicated on it
            dist.all_reduce(sharded_sq, group=self.tp_group)
        sumsq = sharded_sq + repl_sq
        with communication_scope("optimizer_data_parallel", "gradient_clip", "all_reduce", 4):
            dist.all_reduce(sumsq, group=self.group)
        return sumsq

    @torch.no_grad()
    def apply_update(self, sumsq: torch.Tensor, *, lr: float | None = None, weight_decay: float | None = None,
                     grad_scale: float = 1.0, max_grad_norm: float = 0.0) -> None:
        sp = self.sp
        lr = self.lr if lr is None else lr
        wd = self.weight_decay if weight_decay is None else weight_decay
        g = sp.grad_shard
        split = sp.decay_local
        self.last_grad_norm = sumsq
        self.step_count += 1
        b1, b2 = self.betas
        for lo, hi, w in ((0, split, wd), (split, sp.n_local, 0.0)):
            if hi <= lo:
                continue
            if g.is_cuda and sp.dtype == torch.bfloat16:
                from ..ops._util import ptr, stream

                native.check(native.lib().tdllm_adamw_f32grad(
                    ptr(self.master[lo:hi]), ptr(self.m[lo:hi]), ptr(self.v[lo:hi]), ptr(g[lo:hi]),
                    ptr(sp.param_shard[lo:hi]), hi - lo, lr, b1, b2, self.eps, w, self.step_count, grad_scale,
                    ptr(sumsq), max_grad_norm, stream()), "adamw_f32grad")
            else:
                gs = grad_scale
                if max_grad_norm > 0:
                    norm = float(sumsq.sqrt()) * grad_scale
                    if norm > max_grad_norm:
                        gs *= max_grad_norm / (norm + 1e-6)
                gg = g[lo:hi] * gs
                m, v, p = self.m[lo:hi], self.v[lo:hi], self.master[lo:hi]
                m.mul_(b1).add_(gg, alpha=1 - b1)
                v.mul_(b2).addcmul_(gg, gg, value=1 - b2)
                bias1, bias2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
                p.mul_(1 - lr * w).addcdiv_(m / bias1, (v / bias2).sqrt().add_(self.eps), value=-lr)
                sp.param_shard[lo:hi].copy_(p)
        sp.params_updated()

    def grad_norm(self, grad_scale: float = 1.0) -> float:
        if self.last_grad_norm is None:
            return float("nan")
        return math.sqrt(float(self.last_grad_norm)) * grad_scale

    def _all_gather_params(self) -> None:     # same surface as FlatAdamW: parameters are gathered per unit here
        self.sp.params_updated()

    def state_dict(self) -> dict:
        return {"step_count": self.step_count, "world": self.world, "rank": self.rank, "n_local": self.sp.n_local,
                "master": self.master, "m": self.m, "v": self.v}

    def load_state_dict(self, state: dict) -> None:
        if state["world"] != self.world or state["n_local"] != self.sp.n_local or state["rank"] != self.rank:
            raise ValueError("optimizer shard layout differs from the checkpoint (resharding is not supported)")
        self.step_count = int(state["step_count"])
        self.master.copy_(state["master"])
        self.m.copy_(state["m"])
        self.v.copy_(state["v"])
        self.sp.param_shard.copy_(self.master.to(self.sp.dtype))

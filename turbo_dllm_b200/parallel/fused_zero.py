"""Fused ZeRO step over peer memory (see csrc/comm.cu): gradient reduce-scatter by pulling,
global-norm clipping, sharded AdamW and parameter all-gather by pushing, as two kernels between
three epoch barriers, with no NCCL call on the path.

The flat parameter and gradient buffers must live in symmetric memory, so `FusedZeroSync.create`
re-homes an existing `FlatParams` into `SymmetricBuffer`s (parameters keep their values; views are
re-pointed).
"""
from __future__ import annotations


import torch
import torch.distributed as dist

from ..kernels import native
from ..ops._util import ptr, stream
from .symm import SymmetricBarrier, SymmetricBuffer, peer_access_available

native.register_signatures({
    "tdllm_zero_fused_step": (native.c_int, [native.c_void_p] * 7 + [native.c_int, native.c_int, native.c_ll,
                                                                    native.c_ll, native.c_ll] + [native.c_float] * 5
                              + [native.c_int, native.c_float, native.c_float, native.c_void_p, native.c_int,
                                 native.c_void_p, native.c_void_p]),
})


class FusedZeroSync:
    def __init__(self, flat, group, params_buf, grads_buf, scalar_buf, barrier):
        self.flat, self.group = flat, group
        self.params_buf, self.grads_buf, self.scalar_buf, self.barrier = params_buf, grads_buf, scalar_buf, barrier
        self.norm = torch.zeros(1, dtype=torch.float32, device=flat.data.device)
        self.reduced = None       # fp32 rank sums of this rank's shard, between the norm pass and the update pass

    @classmethod
    def create(cls, flat, group) -> "FusedZeroSync":
        if flat.data.dtype != torch.bfloat16 or not flat.data.is_cuda:
            raise RuntimeError("fused ZeRO needs bf16 CUDA parameters")
        world = dist.get_world_size(group)
        if world < 2 or world > 16:
            raise RuntimeError(f"fused ZeRO supports 2..16 ranks per node, got {world}")
        if not peer_access_available(group):
            raise RuntimeError("GPUs of this group cannot address one another (no peer access)")
        dev = flat.data.device
        nbytes = flat.numel * 2
        params_buf = SymmetricBuffer(nbytes, group, dev)
        grads_buf = SymmetricBuffer(nbytes, group, dev)
        scalar_buf = SymmetricBuffer(256, group, dev)
        barrier = SymmetricBarrier(group, dev)
        new_data = params_buf.as_tensor(torch.bfloat16, flat.numel)
        new_grad = grads_buf.as_tensor(torch.bfloat16, flat.numel)
        new_data.copy_(flat.data)
        flat.data, flat.grad = new_data, new_grad
        for name, (o, n, shape, decay) in flat.offsets.items():
            p = flat.params[name]
            p.data = new_data[o:o + n].view(shape)
            p.main_grad = new_grad[o:o + n].view(shape)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()   # the buffers the parameters came from go back to the driver
        dist.barrier(group=group)
        return cls(flat, group, params_buf, grads_buf, scalar_buf, barrier)

    def step(self, opt, lr: float, wd: float, grad_scale: float, max_grad_norm: float):
        b1, b2 = opt.betas
        n = opt.stop - opt.start
        epoch = self.barrier.reserve(3)
        import os

        env = os.environ.get("TDLLM_ZERO_FP32_SUMS")
        if self.reduced is None and (opt.world > 2 or env == "1") and env != "0":
            # with more than one peer a second pull of the gradients costs more link time than 4 bytes per shard
            # element of memory; with one peer (or no room) the update pass pulls again instead
            # (TDLLM_ZERO_FP32_SUMS=1 / 0 forces either form)
            if env == "1" or 4 * n < 0.05 * torch.cuda.mem_get_info(self.flat.data.device)[0]:
                self.reduced = torch.empty(max(n, 8), dtype=torch.float32, device=self.flat.data.device)
            else:
                self.reduced = False
        reduced = ptr(self.reduced) if isinstance(self.reduced, torch.Tensor) else None
        rc = native.lib().tdllm_zero_fused_step(
            self.grads_buf.ptr_array, self.params_buf.ptr_array, self.scalar_buf.ptr_array,
            self.barrier.buf.ptr_array, ptr(opt.master), ptr(opt.m), ptr(opt.v), opt.rank, opt.world,
            opt.start, n, self.flat.decay_numel, lr, b1, b2, opt.eps, wd, opt.step_count, grad_scale,
            max_grad_norm, ptr(self.norm), epoch, reduced, stream())
        native.check(rc, "zero_fused_step")
        opt.last_grad_norm = self.norm * self.norm   # grad_norm() takes the square root
        return None

    def close(self) -> None:
        for b in (self.params_buf, self.grads_buf, self.scalar_buf, self.barrier.buf):
            b.close()

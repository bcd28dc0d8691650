"""Symmetric peer memory: buffers of equal size on every rank of a group, each mapped into every
other rank's address space, plus an epoch barrier living in such a buffer.

Allocation is `cudaMalloc` inside the kernel library (outside PyTorch's caching allocator, so the
IPC handle covers exactly the buffer), handles travel over the process group's object
collectives, and peers are opened with `cudaIpcOpenMemHandle`. Kernels then use ordinary loads
and stores on the peer pointers. `as_tensor` exposes the local buffer to PyTorch without a copy.

The reference has no first-party peer-memory layer (it relies on NCCL, TE Userbuffers and
DeepEP: dllm_parallel/core/parallel/transformer_engine.py:84-139,
dllm_parallel/core/parallel/expert/deepep.py:131-215).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..kernels import native

native.register_signatures({
    "tdllm_symm_alloc": (native.c_int, [native.c_ll, ctypes.POINTER(ctypes.c_void_p)]),
    "tdllm_symm_free": (native.c_int, [native.c_void_p]),
    "tdllm_ipc_get_handle": (native.c_int, [native.c_void_p, native.c_void_p]),
    "tdllm_ipc_open": (native.c_int, [native.c_void_p, ctypes.POINTER(ctypes.c_void_p)]),
    "tdllm_ipc_close": (native.c_int, [native.c_void_p]),
    "tdllm_symm_barrier": (native.c_int, [native.c_void_p, native.c_int, native.c_int, native.c_int,
                                          native.c_void_p]),
})

_TYPESTR = {torch.bfloat16: "<i2", torch.float16: "<f2", torch.float32: "<f4", torch.int32: "<i4",
            torch.uint8: "|u1"}


class _Raw:
    def __init__(self, ptr: int, nbytes: int, typestr: str, itemsize: int):
        self.__cuda_array_interface__ = {"shape": (nbytes // itemsize,), "typestr": typestr,
                                         "data": (ptr, False), "version": 3}


class SymmetricBuffer:
    """One buffer per rank; `ptrs[r]` is rank r's buffer as seen from this process."""

    def __init__(self, nbytes: int, group, device: torch.device):
        self.group, self.device, self.nbytes = group, device, int(nbytes)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        lib = native.lib()
        torch.cuda.set_device(device)
        local = ctypes.c_void_p()
        native.check(lib.tdllm_symm_alloc(self.nbytes, ctypes.byref(local)), "symm_alloc")
        self.local = local.value
        handle = ctypes.create_string_buffer(64)
        native.check(lib.tdllm_ipc_get_handle(self.local, handle), "ipc_get_handle")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs: list[int] = []
        self._opened: list[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local)
                continue
            out = ctypes.c_void_p()
            native.check(lib.tdllm_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(out)),
                         f"ipc_open(rank {r})")
            self.ptrs.append(out.value)
            self._opened.append(out.value)
        self.ptr_array = (ctypes.c_void_p * self.world)(*self.ptrs)

    def as_tensor(self, dtype: torch.dtype, numel: int | None = None, offset_bytes: int = 0) -> torch.Tensor:
        item = torch.empty(0, dtype=dtype).element_size()
        n = (self.nbytes - offset_bytes) // item if numel is None else numel
        raw = _Raw(self.local + offset_bytes, n * item, _TYPESTR[dtype], item)
        t = torch.as_tensor(raw, device=self.device)
        return t.view(dtype) if t.dtype != dtype else t

    def close(self) -> None:
        lib = native.lib()
        for p in self._opened:
            lib.tdllm_ipc_close(p)
        self._opened.clear()
        if self.local:
            lib.tdllm_symm_free(self.local)
            self.local = 0


class SymmetricBarrier:
    """Epoch barrier over a symmetric int32[world] array; waits are bounded on the device."""

    def __init__(self, group, device):
        self.buf = SymmetricBuffer(256, group, device)
        self.epoch = 0
        dist.barrier(group=group)

    def reserve(self, count: int) -> int:
        first = self.epoch + 1
        self.epoch += count
        return first

    def sync(self, stream: int | None = None) -> None:
        e = self.reserve(1)
        native.check(native.lib().tdllm_symm_barrier(self.buf.ptr_array, self.buf.rank, self.buf.world, e,
                                                     stream or torch.cuda.current_stream().cuda_stream),
                     "symm_barrier")


def peer_access_available(group) -> bool:
    """All ranks of the group sit on GPUs of this node that can address one another."""
    if not torch.cuda.is_available():
        return False
    n = torch.cuda.device_count()
    me = torch.cuda.current_device()
    ok = all(torch.cuda.can_device_access_peer(me, j) for j in range(n) if j != me)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(flag.item())

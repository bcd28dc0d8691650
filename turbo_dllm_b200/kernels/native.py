"""Runtime loading of the sm_100a kernel library and its ctypes signatures.

`lib()` returns the loaded `libtdllm_kernels.so` or raises `NativeKernelError`: there is no
silent PyTorch fallback on a CUDA device. `KernelRuntimePolicy.allow_runtime_jit` lets a
development checkout rebuild a stale library with nvcc; a packaged install must match its
manifest (source and binary hashes).

Reference counterpart: dllm_parallel/core/kernels/runtime.py:25-85 (policy + manifest check),
:189-223 (load_native_extension).
"""
from __future__ import annotations

import ctypes
import json
import os
import threading
from dataclasses import dataclass
from pathlib import Path

from . import build as _build

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float
c_ull = ctypes.c_ulonglong


class NativeKernelError(RuntimeError):
    pass


@dataclass(frozen=True)
class KernelRuntimePolicy:
    """allow_runtime_jit: rebuild with nvcc when the in-tree binary is missing or stale."""

    allow_runtime_jit: bool = True
    verify_manifest: bool = True


_policy = KernelRuntimePolicy(
    allow_runtime_jit=os.environ.get("TDLLM_RUNTIME_JIT", "1") != "0",
)
_lib = None
_lock = threading.Lock()


def configure(policy: KernelRuntimePolicy) -> None:
    global _policy
    _policy = policy


def library_path() -> Path:
    """The regular library, or the checked variant when DLLM_KERNEL_CHECKS=1."""
    return _build.OUT_DIR / (_build.CHECKED_LIB_NAME if _build.checks_requested() else _build.LIB_NAME)


def manifest() -> dict | None:
    p = _build.OUT_DIR / (_build.CHECKED_MANIFEST_NAME if _build.checks_requested() else _build.MANIFEST_NAME)
    if not p.exists():
        return None
    try:
        return json.loads(p.read_text())
    except Exception:
        return None


def verify_packaged_kernels() -> list[str]:
    """Returns a list of problems (empty = the in-tree binary matches its manifest)."""
    problems = []
    if not library_path().exists():
        problems.append(f"missing {library_path()}")
        return problems
    man = manifest()
    if man is None:
        problems.append("missing or unreadable native_kernels.json")
        return problems
    if man.get("arch") != "sm_100a":
        problems.append(f"library built for {man.get('arch')}, need sm_100a")
    if man.get("sources") != _build.source_hashes():
        problems.append("kernel sources changed since the library was built")
    if man.get("binary_sha256") != _build._sha256(library_path()):
        problems.append("library binary does not match its manifest hash")
    return problems


_SIGS = {
    "tdllm_last_error": (ctypes.c_char_p, []),
    "tdllm_num_sms": (c_int, []),
    "tdllm_get_error": (c_int, [c_void_p]),
    "tdllm_clear_error": (c_int, []),
    "tdllm_set_wait_timeout_ns": (c_int, [c_ull]),
    "tdllm_test_wait_timeout": (c_int, [c_void_p]),
    "tdllm_gemm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_ll,
                                c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_int, c_float, c_int, c_void_p, c_ll, c_void_p]),
    "tdllm_gemm_n_tiles": (c_int, [c_int]),
    "tdllm_rmsnorm_fwd": (c_int, [c_void_p] * 6 + [c_int, c_int, c_float, c_void_p]),
    "tdllm_rmsnorm_bwd_parts": (c_int, []),
    "tdllm_rmsnorm_bwd": (c_int, [c_void_p] * 7 + [c_int, c_int, c_void_p, c_int, c_int, c_void_p]),
    "tdllm_qk_norm_rope_fwd": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "tdllm_qk_bwd_parts": (c_int, []),
    "tdllm_qk_norm_rope_bwd": (c_int, [c_void_p] * 9 + [c_int, c_int, c_void_p, c_int, c_int, c_int,
                                                        c_int, c_float, c_void_p]),
    "tdllm_swiglu_fwd": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "tdllm_swiglu_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "tdllm_sumsq_bf16": (c_int, [c_void_p, c_ll, c_void_p, c_void_p]),
    "tdllm_adamw": (c_int, [c_void_p] * 5 + [c_ll] + [c_float] * 5 + [c_int, c_float, c_void_p,
                                                                   c_float, c_void_p]),
    "tdllm_ce_finalize": (c_int, [c_void_p, c_int, c_int] + [c_void_p] * 6),
    "tdllm_attn_merge": (c_int, [c_void_p] * 5 + [c_ll, c_int, c_int, c_void_p]),
    "tdllm_attn_merge_finalize": (c_int, [c_void_p] * 5 + [c_ll, c_int, c_void_p]),
    "tdllm_attn_merge_bwd": (c_int, [c_void_p] * 7 + [c_ll, c_int, c_void_p]),
}


def _bind(lib: ctypes.CDLL) -> None:
    for name, (res, args) in _SIGS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise NativeKernelError(f"{library_path()} lacks symbol {name}: rebuild with "
                                    "`python -m turbo_dllm_b200.kernels.build --force`") from e
        fn.restype = res
        fn.argtypes = args


def register_signatures(sigs: dict) -> None:
    """Lets sibling modules (attention, comm, ...) declare their entry points."""
    _SIGS.update(sigs)
    if _lib is not None:
        _bind(_lib)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        problems = verify_packaged_kernels() if _policy.verify_manifest else []
        if problems:
            if not _policy.allow_runtime_jit:
                raise NativeKernelError("native kernels unusable: " + "; ".join(problems))
            try:
                _build.build(checks=_build.checks_requested())
            except Exception as e:  # nvcc missing or compile error
                raise NativeKernelError(f"native kernels unusable ({'; '.join(problems)}) and "
                                        f"rebuild failed: {e}") from e
        try:
            loaded = ctypes.CDLL(str(library_path()))
        except OSError as e:
            raise NativeKernelError(f"cannot load {library_path()}: {e}") from e
        _bind(loaded)
        _lib = loaded
        return _lib


LAUNCHES = {"kernels": 0}
# device kernels launched by one successful call of each entry point
_KERNELS_PER_CALL = {"rmsnorm_bwd": 2, "qk_norm_rope_bwd": 4, "attn_bwd": 3, "attn_bwd_fused": 5}


def check(rc: int, what: str) -> None:
    LAUNCHES["kernels"] += _KERNELS_PER_CALL.get(what, 1)
    if rc != 0:
        msg = lib().tdllm_last_error()
        raise NativeKernelError(f"{what} failed (code {rc}): {msg.decode() if msg else ''}")


def device_error() -> dict:
    """Reads the device error record (synchronises). code 0 = no error."""
    buf = (ctypes.c_int * 8)()
    check(lib().tdllm_get_error(ctypes.cast(buf, c_void_p)), "get_error")
    names = {0: "none", 1: "wait_timeout", 2: "bad_index", 3: "capacity", 4: "peer_abort"}
    return {"code": buf[0], "name": names.get(buf[0], "unknown"), "kernel": buf[1],
            "block": buf[2], "detail": buf[3]}


def raise_on_device_error() -> None:
    err = device_error()
    if err["code"] != 0:
        lib().tdllm_clear_error()
        raise NativeKernelError(f"device-side error: {err}")

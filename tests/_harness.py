"""Spawn + deadline harness for multi-rank tests: runs `fn(rank, world, *args)` in `world` child
processes with a gloo (or nccl) process group on 127.0.0.1, collects ("ok" | "error", payload)
per rank through a queue, and terminates stragglers when the deadline passes — a hung or failed
rank becomes a test failure, never a hung test session."""
from __future__ import annotations

import os
import socket
import time
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _plain(obj):
    """Tensors cross the queue as numpy arrays: a torch tensor in a queue needs its sender alive
    until the receiver has mapped it, and ranks exit as soon as they are done."""
    import torch

    if torch.is_tensor(obj):
        return obj.detach().cpu().numpy()
    if isinstance(obj, (list, tuple)):
        return type(obj)(_plain(o) for o in obj)
    if isinstance(obj, dict):
        return {k: _plain(v) for k, v in obj.items()}
    return obj


def _child(rank, world, port, backend, fn, args, queue):
    try:
        import torch.distributed as dist

        os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank),
                           "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank)})
        if backend is not None:
            dist.init_process_group(backend, rank=rank, world_size=world)
        out = fn(rank, world, *args)
        if backend is not None and dist.is_initialized():
            dist.destroy_process_group()
        queue.put((rank, "ok", _plain(out)))
    except BaseException:
        queue.put((rank, "error", traceback.format_exc()))


_CONTEXT = None


def _context():
    """CPU ranks are forked from a fork server that has already imported torch and the package (a fresh interpreter
    per rank spends seconds on those imports; the server itself starts no threads and no process group, so forking it
    is safe). On a machine with GPUs, and for `nccl` ranks, every rank gets a fresh interpreter (`spawn`)."""
    global _CONTEXT
    if _CONTEXT is None:
        try:
            ctx = mp.get_context("forkserver")
            ctx.set_forkserver_preload(["torch", "numpy", "turbo_dllm_b200.training.session",
                                        "turbo_dllm_b200.parallel.runtime", "tests._harness"])
            _CONTEXT = ctx
        except ValueError:                      # no fork server on this platform
            _CONTEXT = mp.get_context("spawn")
    return _CONTEXT


def run_ranks(fn, world: int, args=(), backend: str | None = "gloo", deadline_s: float = 120.0):
    import torch

    # on a machine with GPUs every rank gets a fresh interpreter, whatever its backend (children may use CUDA)
    ctx = mp.get_context("spawn") if (backend == "nccl" or torch.cuda.is_available()) else _context()
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_child, args=(r, world, port, backend, fn, args, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results, t0 = {}, time.time()
    try:
        while len(results) < world and time.time() - t0 < deadline_s:
            try:
                rank, status, payload = queue.get(timeout=0.5)
                results[rank] = (status, payload)
                if status == "error":
                    break
            except Exception:
                if all(not p.is_alive() for p in procs) and queue.empty():
                    break
    finally:
        for p in procs:
            p.join(timeout=0.1 if len(results) < world else 10)
            if p.is_alive():
                p.terminate()
                p.join(timeout=5)
                if p.is_alive():
                    p.kill()
    errors = {r: pl for r, (st, pl) in results.items() if st == "error"}
    if errors:
        raise AssertionError("rank failure:\n" + "\n".join(f"[rank {r}]\n{tb}" for r, tb in errors.items()))
    if len(results) < world:
        missing = sorted(set(range(world)) - set(results))
        raise AssertionError(f"ranks {missing} did not finish within {deadline_s}s (terminated)")
    return [results[r][1] for r in range(world)]


def assert_params_close(got, want, *, rtol: float = 1e-3, atol: float = 2e-5, max_outliers: float = 1e-4,
                        max_abs: float = 5e-3) -> None:
    """Parameters after a few AdamW steps of two runs that compute the same function in a different summation order.
    AdamW divides by sqrt(v): an element whose gradient is at rounding level can move by a whole learning-rate step in
    either run, so elementwise closeness is required of all but a tiny share of the elements, and the vectors as a
    whole must agree to the tolerance."""
    import numpy as np
    import torch

    a = torch.from_numpy(got) if isinstance(got, np.ndarray) else got
    a, b = a.double().flatten(), want.double().flatten()
    diff = (a - b).abs()
    bad = diff > (atol + rtol * b.abs())
    rel = float(diff.norm() / b.norm().clamp_min(1e-30))
    share = float(bad.double().mean())
    if a.numel() >= 64 and int(bad.sum()) <= 1:       # one stray element of a small tensor
        share = 0.0
    assert rel < rtol and share <= max_outliers and float(diff.max()) < max_abs, (
        f"relative L2 error {rel:.3e}, {int(bad.sum())} of {a.numel()} elements outside tolerance "
        f"(share {share:.2e}), max abs difference {float(diff.max()):.3e}")

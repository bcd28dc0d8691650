"""Host-side failure visibility: stack dumps on signals and an atomic per-rank fatal marker.

Counterpart of dllm_parallel/training/fault_tolerance.py:17-45. Recovery itself is
restart-from-checkpoint (torchrun --max-restarts plus `checkpointing.auto_resume`).
"""
from __future__ import annotations

import faulthandler
import json
import os
import signal
import sys
import tempfile


def install_fault_handlers() -> None:
    """Dump all Python stacks on SIGUSR1 and on fatal signals (no effect on normal exits)."""
    try:
        faulthandler.enable(file=sys.stderr, all_threads=True)
        faulthandler.register(signal.SIGUSR1, file=sys.stderr, all_threads=True, chain=True)
    except (AttributeError, ValueError, RuntimeError):
        pass  # platforms / threads where signal registration is not possible


def fatal_marker_path(run_dir: str, rank: int) -> str:
    return os.path.join(run_dir, f"fatal_rank_{rank:05d}.json")


def write_fatal_marker(run_dir: str, rank: int, info: dict) -> str:
    """Writes `fatal_rank_{rank:05d}.json` atomically (tmp file + rename)."""
    os.makedirs(run_dir, exist_ok=True)
    path = fatal_marker_path(run_dir, rank)
    fd, tmp = tempfile.mkstemp(prefix=".fatal_", dir=run_dir)
    with os.fdopen(fd, "w") as f:
        json.dump(info, f, sort_keys=True, default=str)
    os.replace(tmp, path)
    return path

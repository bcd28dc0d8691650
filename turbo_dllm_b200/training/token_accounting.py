"""Token counts behind the throughput numbers: input (data) tokens, supervised (valid) tokens and
active (masked) tokens, per step and cumulative; and run metadata for logs and checkpoints.

Counterparts: dllm_parallel/training/token_accounting.py:15-48, dllm_parallel/training/run_metadata.py:32-113.
"""
from __future__ import annotations

import os
import platform
import subprocess
import sys
import time
from dataclasses import asdict, dataclass, field


@dataclass
class TokenCounters:
    input_tokens: int = 0
    supervised_tokens: float = 0.0
    active_tokens: float = 0.0
    steps: int = 0

    def add(self, *, input_tokens: int, supervised_tokens: float, active_tokens: float) -> None:
        self.input_tokens += int(input_tokens)
        self.supervised_tokens += float(supervised_tokens)
        self.active_tokens += float(active_tokens)
        self.steps += 1

    def throughput(self, elapsed_seconds: float, world_size: int) -> dict:
        if elapsed_seconds <= 0:
            return {}
        out = {}
        for name in ("input_tokens", "supervised_tokens", "active_tokens"):
            v = getattr(self, name) / elapsed_seconds
            out[f"{name}_per_second"] = v
            out[f"{name}_per_second_per_gpu"] = v / max(world_size, 1)
        return out


@dataclass
class RunContext:
    started_at: str = field(default_factory=lambda: time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()))
    hostname: str = field(default_factory=platform.node)
    python: str = field(default_factory=lambda: sys.version.split()[0])
    git_sha: str | None = None
    package_version: str | None = None
    torch_version: str | None = None
    cuda_version: str | None = None
    device_name: str | None = None
    world_size: int = 1
    run_dir: str | None = None

    def to_dict(self) -> dict:
        return asdict(self)


def _git_sha(cwd: str) -> str | None:
    try:
        out = subprocess.run(["git", "rev-parse", "HEAD"], cwd=cwd, capture_output=True, text=True, timeout=5)
        return out.stdout.strip() or None if out.returncode == 0 else None
    except (OSError, subprocess.SubprocessError):
        return None


def collect_run_context(world_size: int = 1) -> RunContext:
    import torch

    from .. import __version__

    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ctx = RunContext(git_sha=_git_sha(here), package_version=__version__, torch_version=torch.__version__,
                     cuda_version=torch.version.cuda, world_size=world_size, run_dir=os.environ.get("DLLM_RUN_DIR"))
    if torch.cuda.is_available():
        ctx.device_name = torch.cuda.get_device_name(torch.cuda.current_device())
    return ctx

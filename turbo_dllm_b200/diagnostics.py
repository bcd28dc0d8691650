"""`dllm doctor` and the runtime preflight: is this machine ready to train?

Portable checks (torch import, package version, virtual-env isolation) and training checks
(CUDA devices and their compute capability, the in-tree kernel library vs its manifest or an
nvcc toolchain to rebuild it, NCCL availability, peer access between GPUs, configured paths),
each with a remediation string. `require_ready()` raises with every failed check listed.

Counterpart of dllm_parallel/core/diagnostics.py:15-125 (check/report types), :128-252
(inspect_training_runtime), :255-418 (individual checks).
"""
from __future__ import annotations

import os
import shutil
import sys
from dataclasses import dataclass, field


@dataclass(frozen=True)
class RuntimeCheck:
    name: str
    ok: bool
    detail: str = ""
    remediation: str = ""
    required: bool = True


@dataclass
class RuntimeReadinessReport:
    checks: list[RuntimeCheck] = field(default_factory=list)

    @property
    def ready(self) -> bool:
        return all(c.ok or not c.required for c in self.checks)

    def failures(self) -> list[RuntimeCheck]:
        return [c for c in self.checks if not c.ok and c.required]

    def require_ready(self) -> None:
        bad = self.failures()
        if bad:
            from .config.run_spec import RunSpecError

            raise RunSpecError("runtime is not ready:\n" + "\n".join(
                f"  - {c.name}: {c.detail} ({c.remediation})" for c in bad))

    def to_dict(self) -> dict:
        return {"ready": self.ready, "checks": [c.__dict__ for c in self.checks]}


def portable_checks() -> list[RuntimeCheck]:
    out = []
    try:
        import torch

        out.append(RuntimeCheck("torch", True, torch.__version__))
    except Exception as e:  # pragma: no cover
        out.append(RuntimeCheck("torch", False, str(e), "install PyTorch >= 2.6"))
    out.append(RuntimeCheck("python", sys.version_info >= (3, 10), sys.version.split()[0], "use Python >= 3.10"))
    pp = os.environ.get("PYTHONPATH", "")
    out.append(RuntimeCheck("pythonpath", True, pp or "(unset)", required=False))
    in_venv = sys.prefix != getattr(sys, "base_prefix", sys.prefix)
    out.append(RuntimeCheck("virtual_env", in_venv, sys.prefix, "run inside a virtual environment", required=False))
    return out


def kernel_checks(allow_jit: bool) -> list[RuntimeCheck]:
    from .kernels import native

    problems = native.verify_packaged_kernels()
    if not problems:
        return [RuntimeCheck("native_kernels", True, str(native.library_path()))]
    nvcc = shutil.which("nvcc") or ("/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else None)
    if allow_jit and nvcc:
        return [RuntimeCheck("native_kernels", True, f"stale ({'; '.join(problems)}); will rebuild with {nvcc}")]
    return [RuntimeCheck("native_kernels", False, "; ".join(problems),
                         "run `dllm-build-kernels` (needs nvcc 12.8+ for sm_100a) or set kernel.runtime_jit=true")]


def cuda_checks(world_hint: int = 1) -> list[RuntimeCheck]:
    import torch

    out = []
    if not torch.cuda.is_available():
        return [RuntimeCheck("cuda", False, "no CUDA device visible",
                             "bf16 training needs a B200 (sm_100a); use model.dtype=fp32 for CPU runs")]
    n = torch.cuda.device_count()
    out.append(RuntimeCheck("cuda_devices", n >= 1, f"{n} device(s)"))
    caps = {torch.cuda.get_device_capability(i) for i in range(n)}
    ok = all(c[0] == 10 for c in caps)
    out.append(RuntimeCheck("compute_capability", ok, ", ".join(f"sm_{a}{b}" for a, b in sorted(caps)),
                            "the kernel library is built for sm_100a only"))
    import torch.distributed as dist

    out.append(RuntimeCheck("nccl", dist.is_nccl_available(), "torch.distributed NCCL backend", "install a CUDA build of PyTorch"))
    if n > 1:
        peer = all(torch.cuda.can_device_access_peer(0, j) for j in range(1, n))
        out.append(RuntimeCheck("peer_access", peer, "GPU0 ↔ others", "fused peer-memory kernels fall back to NCCL",
                                required=False))
    return out


def path_checks(spec) -> list[RuntimeCheck]:
    out = []
    for label, path, must_exist in (("data.dataset_path", spec.data.dataset_path, True),
                                    ("checkpointing.load_checkpoint_dir", spec.checkpointing.load_checkpoint_dir, True),
                                    ("data.target_feature_path", spec.data.target_feature_path, True)):
        if path:
            ok = os.path.exists(path)
            out.append(RuntimeCheck(label, ok or not must_exist, path, "path does not exist"))
    return out


def inspect_training_runtime(spec=None, portable_only: bool = False) -> RuntimeReadinessReport:
    rep = RuntimeReadinessReport(portable_checks())
    if portable_only:
        return rep
    allow_jit = bool(spec.kernel.runtime_jit) if spec is not None else True
    wants_cuda = spec is None or spec.model.dtype != "fp32"
    if wants_cuda:
        rep.checks += cuda_checks()
        rep.checks += kernel_checks(allow_jit)
    if spec is not None:
        rep.checks += path_checks(spec)
    return rep

"""Checks and environment policy applied before any process group or CUDA context exists.

* `prepare_parallel_environment(spec, env)`: the environment a worker needs for the parallel features its run
  spec turns on, and refusal of settings that contradict them.
    - peer-memory kernels (fused ZeRO, context-sharded attention, sequence-parallel GEMMs, expert exchange,
      parameter sharding) spin on flags written by other GPUs, so kernels of one rank must be able to run
      side by side: `CUDA_DEVICE_MAX_CONNECTIONS=1` (which serialises a process's streams onto one hardware queue,
      and which the reference REQUIRES for its NCCL overlap) is refused when such a feature is on;
    - rotating full-size buffers (parameter sharding, sequence parallelism) and long sequences fragment the
      caching allocator: `PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True` unless the user chose a setting;
    - tests and failure drills on this kind of machine switch NVLS off; nothing here changes `NCCL_NVLS_ENABLE`.
* `validate_supported_training_axes(spec)`: pipeline parallelism is an axis of size 1.
* `infer_parallel_mesh_sizes(world, spec)`: the size of every axis for a world size.
* `require_idle_assigned_gpus`: refuses to start on GPUs that already run compute processes.

Counterpart of dllm_parallel/core/parallel/preflight.py:38-65, :68-87, :122-183, :228-282.
"""
from __future__ import annotations

from ..config.run_spec import RunSpecError


def uses_peer_memory_kernels(spec, world_size: int | None = None) -> bool:
    t, o = spec.topology, spec.optimizer
    if spec.kernel.impl in ("cpu_reference", "nccl_baseline"):
        return False
    multi = world_size is None or world_size > 1
    return multi and (o.backend in ("auto", "zero_fused", "fsdp", "fsdp2") or t.tensor_parallel_size > 1
                      or t.expert_parallel_size > 1
                      or (t.context_parallel_size > 1 and spec.kernel.cp_bp_clean_kv_transport in ("peer_pull", "fused")))


def prepare_parallel_environment(spec, env: dict, world_size: int | None = None) -> dict:
    """Returns the updates to apply to `env` (does not modify it). Raises RunSpecError on a contradiction."""
    updates: dict[str, str] = {}
    if uses_peer_memory_kernels(spec, world_size) and env.get("CUDA_DEVICE_MAX_CONNECTIONS") == "1":
        raise RunSpecError("CUDA_DEVICE_MAX_CONNECTIONS=1 serialises this process's kernels on one queue; the "
                           "peer-memory kernels this run spec enables wait on other GPUs and need their neighbours "
                           "to keep running. Unset it, or choose kernel.impl=nccl_baseline.")
    alloc = env.get("PYTORCH_CUDA_ALLOC_CONF", "")
    wants_segments = (spec.topology.sequence_parallel or spec.optimizer.backend in ("fsdp", "fsdp2")
                      or spec.model.seq_len >= 65536)
    if wants_segments and "expandable_segments" not in alloc:
        updates["PYTORCH_CUDA_ALLOC_CONF"] = (alloc + "," if alloc else "") + "expandable_segments:True"
    if env.get("TORCH_NCCL_ASYNC_ERROR_HANDLING") is None:
        updates["TORCH_NCCL_ASYNC_ERROR_HANDLING"] = "1"
    return updates


def validate_supported_training_axes(spec) -> None:
    t = spec.topology
    if t.pipeline_parallel_size != 1:
        raise RunSpecError("pipeline parallelism is an axis of size 1 in this release (topology.pipeline_parallel_size)")
    if t.sequence_parallel and t.tensor_parallel_size < 2:
        raise RunSpecError("topology.sequence_parallel needs tensor_parallel_size > 1")
    if t.block_parallel_size > 1 and t.context_parallel_size > 1 and t.block_parallel_size % t.context_parallel_size:
        raise RunSpecError("fused context/block parallelism needs block_parallel_size to be a multiple of "
                           "context_parallel_size")


def infer_parallel_mesh_sizes(world_size: int, spec) -> dict[str, int]:
    from .topology import infer_data_parallel_size

    t = spec.topology
    return {"data": infer_data_parallel_size(world_size, spec), "pipeline": t.pipeline_parallel_size,
            "local": spec.local_parallel_size, "context": t.context_parallel_size, "block": t.block_parallel_size,
            "tensor": t.tensor_parallel_size, "expert": t.expert_parallel_size}


def require_idle_assigned_gpus(nproc: int, command_runner=None) -> None:
    from ..cli.launch import require_idle_assigned_gpus as impl

    impl(nproc, command_runner)

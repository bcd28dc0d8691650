"""Multi-GPU tests (2 ranks, NCCL, one process per GPU): the fused peer-memory ZeRO step against
its NCCL twin, data-parallel training sessions, and the bounded barrier wait (single GPU)."""
import pytest
import torch

from tests._harness import run_ranks

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _spec(backend):
    from turbo_dllm_b200.config.run_spec import RunSpec

    return RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-hd128", "seq_len": 512, "dtype": "bf16"},
        "objective": {"name": "fast_dllm_v2", "block_size": 32, "noise_schedule_epsilon": 0.1},
        "training": {"batch_size": 1, "steps": 3},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
        "kernel": {"impl": "nccl_baseline" if backend == "nccl" else "auto"},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0,
                      "backend": "zero_fused" if backend == "fused" else "auto"}}).validate()


def _train(rank, world, backend, steps):
    import os

    import torch.distributed as dist

    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.training.session import TrainingSession

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    s = TrainingSession(_spec(backend), device=f"cuda:{rank}")
    assert (s.optimizer.fused_sync is not None) == (backend == "fused")
    losses = []
    for _ in range(steps):
        r = s.step()
        t = r.loss_sum.double().clone()
        dist.all_reduce(t)
        losses.append(float(t) / r.denominator)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    return losses, s.model.flat.data.float().cpu(), s.optimizer.grad_norm()


@pytest.mark.distributed
def test_fused_zero_matches_nccl_twin():
    _need(2)
    a = run_ranks(_train, 2, args=("nccl", 3), backend="nccl", deadline_s=300)
    b = run_ranks(_train, 2, args=("fused", 3), backend="nccl", deadline_s=300)
    for (la, pa, na), (lb, pb, nb) in zip(a, b):
        assert la == pytest.approx(lb, rel=2e-2)
        assert na == pytest.approx(nb, rel=2e-2)
        pa, pb = torch.from_numpy(pa), torch.from_numpy(pb)
        assert (pa - pb).abs().max().item() < 2e-2
    # replicas hold identical parameters after the push all-gather
    assert (b[0][1] == b[1][1]).all()


def test_barrier_wait_runs_out_and_reports():
    """Host-made failure: the second slot of the flag array is never written (no peer exists), so
    the bounded wait must expire, record ERR_WAIT_TIMEOUT for the barrier kernel and return."""
    import ctypes

    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.parallel import symm  # registers the signatures  # noqa: F401

    lib = native.lib()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    other = torch.zeros(64, dtype=torch.int32, device="cuda")
    arr = (ctypes.c_void_p * 2)(flags.data_ptr(), other.data_ptr())
    lib.tdllm_clear_error()
    native.check(lib.tdllm_set_wait_timeout_ns(2_000_000), "timeout")
    try:
        native.check(lib.tdllm_symm_barrier(arr, 0, 2, 1, None), "symm_barrier")
        torch.cuda.synchronize()
        err = native.device_error()
        assert err["code"] == 1 and err["kernel"] == 10 and err["detail"] == 1
        assert int(other[0]) == 1  # our arrival was published before the wait gave up
    finally:
        lib.tdllm_clear_error()
        lib.tdllm_set_wait_timeout_ns(2_000_000_000)
    assert float(torch.ones(4, device="cuda").sum()) == 4.0

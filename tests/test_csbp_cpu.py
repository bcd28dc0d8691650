"""Context-sharded block parallelism over gloo ranks must reproduce the single-process run:
same loss curve and same parameters (CPU, fp32, tiny Qwen3-style model)."""
import pytest
import torch

from tests._harness import run_ranks

MAPPING = {
    "model": {"id": "synthetic:tiny-qwen3", "seq_len": 256, "dtype": "fp32", "num_layers": 2},
    "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
    "training": {"batch_size": 2, "steps": 3, "activation_checkpointing": True},
    "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
    "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0},
}


def _run(rank, world, cp, bp, steps, objective):
    import copy

    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    m = copy.deepcopy(MAPPING)
    m["topology"].update(context_parallel_size=cp, block_parallel_size=bp)
    m["objective"]["name"] = objective
    spec = RunSpec.from_mapping(m).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    losses = []
    for _ in range(steps):
        r = s.step()
        t = r.loss_sum.double().clone()
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t) / r.denominator)
    return losses, s.model.flat.data.clone()


@pytest.mark.distributed
@pytest.mark.parametrize("objective", ["standard_block_diffusion", "fast_dllm_v2"])
def test_csbp2_matches_single_process(objective):
    ref_losses, ref_params = _run(0, 1, 1, 1, 3, objective)
    outs = run_ranks(_run, 2, args=(2, 2, 3, objective), deadline_s=240)
    for losses, params in outs:
        assert losses == pytest.approx(ref_losses, rel=2e-4, abs=2e-4)
        assert torch.allclose(torch.from_numpy(params), ref_params, rtol=1e-3, atol=2e-5)


@pytest.mark.distributed
def test_data_parallel_two_ranks_runs_and_stays_in_sync():
    outs = run_ranks(_run, 2, args=(1, 1, 2, "standard_block_diffusion"), deadline_s=240)
    assert (outs[0][1] == outs[1][1]).all()
    assert outs[0][0] == outs[1][0]


def _boom(rank, world):
    if rank == 1:
        raise RuntimeError("injected failure on rank 1")
    import time

    time.sleep(30)


def _hang(rank, world):
    import time

    if rank == 0:
        time.sleep(60)


@pytest.mark.distributed
def test_harness_reports_failed_and_hung_ranks():
    with pytest.raises(AssertionError, match="injected failure"):
        run_ranks(_boom, 2, backend=None, deadline_s=20)
    with pytest.raises(AssertionError, match="did not finish"):
        run_ranks(_hang, 2, backend=None, deadline_s=3)


def _modes(rank, world):
    from turbo_dllm_b200.benchmarks.parallel_modes_bench import MODES, run_mode
    from turbo_dllm_b200.config.run_spec import RunSpec

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping(MAPPING)
    return [run_mode(spec, m, device="cpu", steps=1, warmup=0) for m in MODES]


@pytest.mark.distributed
def test_parallel_modes_benchmark_agrees_between_layouts():
    """Pure context parallelism, pure block parallelism with a replicated prefix and the fused layout
    compute the same loss on the same data; the benchmark reports one record per mode."""
    outs = run_ranks(_modes, 2, deadline_s=300)
    recs = outs[0]
    assert [r["mode"] for r in recs] == ["pure_cp", "pure_bp", "csbp"]
    losses = [r["loss"] for r in recs]
    assert losses[1] == pytest.approx(losses[0], rel=1e-4) and losses[2] == pytest.approx(losses[0], rel=1e-4)
    assert all(r["ms_per_step"] > 0 and r["world"] == 2 for r in recs)


@pytest.mark.distributed
def test_pure_context_parallel_matches_single_process():
    """CP 2 without block parallelism: both ranks compute every noisy block (the clean K/V are what is
    sharded), so the loss terms exist twice and the step must still equal the single-process one."""
    ref_losses, ref_params = _run(0, 1, 1, 1, 2, "standard_block_diffusion")
    outs = run_ranks(_run, 2, args=(2, 1, 2, "standard_block_diffusion"), deadline_s=240)
    for losses, params in outs:
        assert losses == pytest.approx(ref_losses, rel=2e-4, abs=2e-4)
        assert torch.allclose(torch.from_numpy(params), ref_params, rtol=1e-3, atol=2e-5)

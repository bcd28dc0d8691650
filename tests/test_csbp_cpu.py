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


def _run(rank, world, cp, bp, steps, objective, share=True, split=True):
    import copy

    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    m = copy.deepcopy(MAPPING)
    m["topology"].update(context_parallel_size=cp, block_parallel_size=bp)
    m["objective"]["name"] = objective
    m["kernel"] = {"cp_bp_share_clean_replicas": bool(share), "pure_cp_token_split": bool(split)}
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
    return losses, s.model.flat.data.clone(), (s.layout.n_clean if bp > 1 or cp == 1 else s.layout.n_noisy)


@pytest.mark.distributed
@pytest.mark.parametrize("share", [True, False])
def test_more_block_ranks_than_clean_shards(share):
    """CP 2 x BP 4 on four ranks. With clean-replica sharing the two ranks that would hold a second copy of a
    clean shard hold no clean rows: they attend to the owners' K/V and return dK/dV to them; without it they
    recompute the shard. Both reproduce the single-process run."""
    ref_losses, ref_params, _ = _run(0, 1, 1, 1, 2, "standard_block_diffusion")
    outs = run_ranks(_run, 4, args=(2, 4, 2, "standard_block_diffusion", share), deadline_s=300)
    clean_rows = [o[2] for o in outs]
    assert (clean_rows[2] == 0 and clean_rows[3] == 0) == share and clean_rows[0] > 0
    for losses, params, _ in outs:
        assert losses == pytest.approx(ref_losses, rel=2e-4, abs=2e-4)
        assert torch.allclose(torch.from_numpy(params), ref_params, rtol=1e-3, atol=2e-5)


@pytest.mark.distributed
@pytest.mark.parametrize("objective", ["standard_block_diffusion", "fast_dllm_v2"])
def test_csbp2_matches_single_process(objective):
    ref_losses, ref_params, _ = _run(0, 1, 1, 1, 3, objective)
    outs = run_ranks(_run, 2, args=(2, 2, 3, objective), deadline_s=240)
    for losses, params, _ in outs:
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
@pytest.mark.parametrize("split", [True, False])
def test_pure_context_parallel_matches_single_process(split):
    """CP 2 without block parallelism. Token split: each rank computes half of the offsets of every noisy block
    (two-ended) and all K/V rows are exchanged, so no row is computed twice. Without it both ranks compute every
    noisy block (only the clean K/V are sharded) and the loss terms exist twice. Both equal the single-process
    step."""
    ref_losses, ref_params, n_noisy_full = _run(0, 1, 1, 1, 2, "standard_block_diffusion")
    outs = run_ranks(_run, 2, args=(2, 1, 2, "standard_block_diffusion", True, split), deadline_s=240)
    for losses, params, n_noisy in outs:
        assert losses == pytest.approx(ref_losses, rel=2e-4, abs=2e-4)
        assert torch.allclose(torch.from_numpy(params), ref_params, rtol=1e-3, atol=2e-5)
        assert n_noisy == (n_noisy_full // 2 if split else n_noisy_full)


def test_pure_context_offsets_partition_the_block():
    from turbo_dllm_b200.parallel.layout import pure_context_offsets

    for bs, cp in ((32, 2), (32, 4), (32, 8), (16, 8), (8, 8), (12, 4)):
        got = [pure_context_offsets(bs, cp, r) for r in range(cp)]
        assert sorted(o for g in got for o in g) == list(range(bs))
        assert all(len(g) == bs // cp for g in got)
    assert pure_context_offsets(32, 4, 1) == [4, 5, 6, 7, 24, 25, 26, 27]     # two-ended
    assert pure_context_offsets(12, 4, 1) == [3, 4, 5]                        # odd share: one slice
    with pytest.raises(ValueError):
        pure_context_offsets(30, 4, 0)

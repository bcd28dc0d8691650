"""Context-sharded block parallelism over gloo ranks must reproduce the single-process run:
same loss curve and same parameters (CPU, fp32, tiny Qwen3-style model)."""
import pytest
import torch

from tests._harness import assert_params_close, run_ranks

MAPPING = {
    "model": {"id": "synthetic:tiny-qwen3", "seq_len": 256, "dtype": "fp32", "num_layers": 2},
    "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
    "training": {"batch_size": 2, "steps": 3, "activation_checkpointing": True},
    "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
    "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0},
}


def _run(rank, world, cp, bp, steps, objective, share=True, split=True, window=None):
    import copy

    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    m = copy.deepcopy(MAPPING)
    m["topology"].update(context_parallel_size=cp, block_parallel_size=bp)
    m["objective"]["name"] = objective
    if window:          # layer 0 slides, layer 1 attends to the full prefix
        m["model"].update(sliding_window=window, sliding_window_pattern=2)
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
        assert_params_close(params, ref_params)


@pytest.mark.distributed
@pytest.mark.parametrize("objective", ["standard_block_diffusion", "fast_dllm_v2"])
def test_csbp2_matches_single_process(objective):
    ref_losses, ref_params, _ = _run(0, 1, 1, 1, 3, objective)
    outs = run_ranks(_run, 2, args=(2, 2, 3, objective), deadline_s=240)
    for losses, params, _ in outs:
        assert losses == pytest.approx(ref_losses, rel=2e-4, abs=2e-4)
        assert_params_close(params, ref_params)


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
    """Pure context parallelism (token-split, and with every noisy block replicated), pure block parallelism
    with a replicated prefix and the fused layout compute the same loss on the same data; the benchmark reports
    one record per mode."""
    outs = run_ranks(_modes, 2, deadline_s=300)
    recs = outs[0]
    assert [r["mode"] for r in recs] == ["pure_cp", "pure_cp_replicated", "pure_bp", "csbp"]
    losses = [r["loss"] for r in recs]
    assert all(l == pytest.approx(losses[0], rel=1e-4) for l in losses[1:])
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
        assert_params_close(params, ref_params)
        assert n_noisy == (n_noisy_full // 2 if split else n_noisy_full)


@pytest.mark.distributed
@pytest.mark.parametrize("cp,bp", [(2, 2), (2, 1)])
def test_sliding_window_layers_exchange_only_the_window(cp, bp):
    """A model whose first layer has a 64-token window: under CP 2 x BP 2 that layer moves only the clean rows
    inside some local row's window (one all-to-all), the other layer moves all of them; under token-split pure
    CP only the mask narrows. The window changes the result, and every parallel form equals the single-process
    run with the same window."""
    ref_losses, ref_params, _ = _run(0, 1, 1, 1, 2, "standard_block_diffusion", True, True, 64)
    full_losses, _, _ = _run(0, 1, 1, 1, 2, "standard_block_diffusion")
    assert abs(ref_losses[-1] - full_losses[-1]) > 1e-4
    outs = run_ranks(_run, cp * max(bp // cp, 1), args=(cp, bp, 2, "standard_block_diffusion", True, True, 64),
                     deadline_s=300)
    for losses, params, _ in outs:
        assert losses == pytest.approx(ref_losses, rel=2e-4, abs=2e-4)
        assert_params_close(params, ref_params)


def test_windowed_exchange_plan_counts():
    """Single-process check of the plan arithmetic: a rank that owns clean [0, 128) and noisy blocks at
    [128, 256) with window 64 needs positions [64, 256) (own rows' windows); what it receives from the other
    owner are exactly the needed positions in [128, 256)."""
    import torch.distributed as dist

    from turbo_dllm_b200.parallel.context_attention import WindowedExchangePlan
    from turbo_dllm_b200.parallel.layout import build_packed_layout

    import os, socket
    with socket.socket() as so:
        so.bind(("127.0.0.1", 0))
        port = so.getsockname()[1]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        lay = build_packed_layout(seq_len=256, block_size=32, batch=2, owned_blocks=[4, 5, 6, 7],
                                  clean_pos=torch.arange(0, 128), window=64)
        kpos1 = [torch.arange(0, 128)]
        plan = WindowedExchangePlan(lay, 64, 256, 2, kpos1, dist.group.WORLD, 0)
        need = plan.needs[0]
        # clean rows at [0,128): windows cover [0,128); noisy blocks 4..7 start at 128..224: windows [64, 224)
        assert need[:224].all() and not need[224:].any()
        assert plan.recv_counts == [128 * 2] and plan.send_counts == [128 * 2]
    finally:
        dist.destroy_process_group()


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

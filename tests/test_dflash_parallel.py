"""DFlash drafter when one replica spans several ranks: anchors divided over the ranks, context rows sharded,
context K|V pulled or queries rotated. Every form must reproduce the single-process step."""
import pytest
import torch

from tests._harness import assert_params_close, run_ranks


def _run(rank, world, cp, bp, mode, steps=2, dflash2=False):
    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    model = {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "family": "dflash",
             "verifier_id": "synthetic:tiny-qwen3", "target_layer_ids": [0, 2], "max_layers": 2}
    objective = {"name": "dflash_distillation", "block_size": 8, "max_anchors": 4}
    if dflash2:
        model.update(dflash2_conv_kernel_size=3, dflash2_conv_group_size=16, dflash2_selector_rank=4,
                     dflash2_selector_top_k=4)
        objective.update(dflash_loss="dpace", decay_gamma=4.0)
    spec = RunSpec.from_mapping({
        "model": model, "objective": objective, "data": {"target_features": "online"},
        "training": {"batch_size": 2, "steps": steps},
        "topology": {"context_parallel_size": cp, "block_parallel_size": bp, "replicate_clean_prefix": cp == 1 and bp > 1},
        "kernel": {"dflash_context_exchange": mode},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    losses = []
    for _ in range(steps):
        t = s.step().loss_sum.double().clone()
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t))
    used = s.task.exchange.last_mode if s.task.exchange is not None else "single"
    return losses, s.model.flat.data.clone(), used


@pytest.mark.distributed
@pytest.mark.parametrize("cp,bp,mode", [(2, 2, "kv_pull"), (2, 2, "query_rotation"), (1, 2, "auto"), (2, 1, "auto")])
def test_dflash_replica_over_two_ranks_matches_single_process(cp, bp, mode):
    ref_losses, ref_params, _ = _run(0, 1, 1, 1, "auto")
    outs = run_ranks(_run, 2, args=(cp, bp, mode), deadline_s=240)
    for losses, params, used in outs:
        assert used == ("local" if cp == 1 else "kv_pull" if bp == 1 else mode)
        assert losses == pytest.approx(ref_losses, rel=2e-4, abs=2e-5)
        assert_params_close(params, ref_params)


@pytest.mark.distributed
def test_dflash2_replica_over_two_ranks_matches_single_process():
    ref_losses, ref_params, _ = _run(0, 1, 1, 1, "auto", 2, True)
    outs = run_ranks(_run, 2, args=(2, 2, "query_rotation", 2, True), deadline_s=240)
    for losses, params, _ in outs:
        assert losses == pytest.approx(ref_losses, rel=2e-4, abs=2e-5)
        assert_params_close(params, ref_params)


def test_bytes_model_prefers_queries_at_long_context():
    from turbo_dllm_b200.parallel.dflash_context import prefer_query_rotation

    kw = dict(ranks=2, q_heads=32, kv_heads=8, head_dim=128)
    assert prefer_query_rotation(draft_rows=512 * 16 // 2, context_rows_per_rank=262144 // 2, **kw)
    assert not prefer_query_rotation(draft_rows=2048 * 16 // 2, context_rows_per_rank=4096 // 2, **kw)
    assert not prefer_query_rotation(draft_rows=16, context_rows_per_rank=1 << 20, ranks=1, q_heads=32, kv_heads=8,
                                     head_dim=128)


def _run_offline(rank, world, cp, bp, mode, store, steps=2):
    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "family": "dflash",
                  "verifier_id": "synthetic:tiny-qwen3", "target_layer_ids": [0, 2], "max_layers": 2},
        "objective": {"name": "dflash_distillation", "block_size": 8, "max_anchors": 4},
        "data": {"target_features": "offline", "target_feature_path": store},
        "training": {"batch_size": 2, "steps": steps},
        "topology": {"context_parallel_size": cp, "block_parallel_size": bp},
        "kernel": {"dflash_context_exchange": mode},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device="cpu", runtime=rt)
    losses, shard_rows = [], None
    for _ in range(steps):
        t = s.step().loss_sum.double().clone()
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t))
    b = s.data.next_batch()
    shard_rows = (int(b.features["hidden"].shape[0]), bool(b.features.get("hidden_is_shard", False)),
                  type(b.features["final_hidden"]).__name__)
    return losses, s.model.flat.data.clone(), shard_rows


@pytest.mark.distributed
def test_offline_store_feeds_a_context_sharded_replica_its_shard_only(tmp_path):
    """Training from the feature store with the context divided over two ranks: each rank reads half of the hidden
    rows from the memory-mapped record, takes the teacher rows it needs from the host copy, and the step equals the
    single-process one."""
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.data.dflash_features import capture_features

    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "family": "dflash",
                  "verifier_id": "synthetic:tiny-qwen3", "target_layer_ids": [0, 2], "max_layers": 2},
        "objective": {"name": "dflash_distillation", "block_size": 8, "max_anchors": 4},
        "data": {"target_features": "online"}, "training": {"batch_size": 2, "steps": 3},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1}, "optimizer": {"lr": 1e-3}}).validate()
    store = str(tmp_path / "features")
    capture_features(spec, store, batches=4)
    ref_losses, ref_params, ref_rows = _run_offline(0, 1, 1, 1, "auto", store)
    assert ref_rows[0] == 2 * 64 and not ref_rows[1]
    outs = run_ranks(_run_offline, 2, args=(2, 2, "query_rotation", store), deadline_s=240)
    for losses, params, rows in outs:
        assert rows[0] == 64 and rows[1]                      # half of the 128 context rows of a record
        assert losses == pytest.approx(ref_losses, rel=2e-4, abs=2e-5)
        assert_params_close(params, ref_params)

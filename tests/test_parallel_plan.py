import pytest

from turbo_dllm_b200.parallel.layout import balanced_bounds, clean_shards_for_rank
from turbo_dllm_b200.parallel.schedule import build_block_schedule, dual_end_pairs
from turbo_dllm_b200.parallel.topology import build_parallel_plan


def test_dual_end_pairs_and_costs():
    assert dual_end_pairs(5) == [(0, 4), (1, 3), (2,)]
    assert build_block_schedule(32, 4).active_prefix_cost_by_worker == [124] * 4
    assert build_block_schedule(32, 8).active_prefix_cost_by_worker == [62] * 8
    s = build_block_schedule(32, 4)
    assert s.blocks_by_worker[0] == (0, 1, 2, 3, 28, 29, 30, 31)
    with pytest.raises(ValueError):
        build_block_schedule(3, 4)


@pytest.mark.parametrize("B,P", [(7, 3), (5, 4), (9, 2), (33, 8), (8, 8), (9, 8)])
def test_every_block_owned_once(B, P):
    for pol in ("dual_end", "contiguous"):
        s = build_block_schedule(B, P, pol)
        assert sorted(b for w in s.blocks_by_worker for b in w) == list(range(B))
        assert all(len(w) >= 1 for w in s.blocks_by_worker)
    assert build_block_schedule(B, P).imbalance() <= build_block_schedule(B, P, "contiguous").imbalance() + 1e-9


def test_policy_env_override(monkeypatch):
    monkeypatch.setenv("DLLM_BLOCK_SCHEDULE_POLICY", "contiguous")
    assert build_block_schedule(8, 2).blocks_by_worker == ((0, 1, 2, 3), (4, 5, 6, 7))


def test_plans_match_expected_groups():
    p = build_parallel_plan(num_blocks=32, world_size=4, context_parallel_size=4, block_parallel_size=4)
    assert p.layout == "dp_x_fused_cp_bp" and p.local_parallel_size == 4
    assert [r.context_block_parallel_group for r in p.rank_assignments] == [[0, 1, 2, 3]] * 4
    assert [r.data_parallel_group for r in p.rank_assignments] == [[0], [1], [2], [3]]
    p = build_parallel_plan(num_blocks=32, world_size=8, data_parallel_size=2, context_parallel_size=4,
                            block_parallel_size=4)
    assert p.rank_assignments[0].data_parallel_group == [0, 4]
    assert p.rank_assignments[4].context_block_parallel_group == [4, 5, 6, 7]
    p = build_parallel_plan(num_blocks=32, world_size=8, data_parallel_size=2, context_parallel_size=2,
                            block_parallel_size=2, tensor_parallel_size=2)
    assert p.layout == "dp_x_fused_cp_bp_x_tp" and p.model_parallel_size == 4
    assert p.rank_assignments[0].context_block_parallel_group == [0, 2]
    assert p.rank_assignments[0].tensor_parallel_group == [0, 1]
    assert p.rank_assignments[2].tensor_parallel_group == [2, 3]
    assert p.rank_assignments[4].model_parallel_group == [4, 5, 6, 7]
    assert [r.tensor_parallel_rank for r in p.rank_assignments[:4]] == [0, 1, 0, 1]
    p = build_parallel_plan(num_blocks=32, world_size=16, data_parallel_size=4, context_parallel_size=2,
                            block_parallel_size=2, tensor_parallel_size=2, node_size=4)
    assert p.placement == "node_local_model_parallel_tp_inner"


def test_clean_replica_groups_when_bp_exceeds_cp():
    p = build_parallel_plan(num_blocks=32, world_size=8, context_parallel_size=2, block_parallel_size=8)
    assert p.rank_assignments[0].clean_replica_group == [0, 2, 4, 6]
    assert p.rank_assignments[3].context_block_parallel_group == [2, 3]
    assert p.rank_assignments[5].context_parallel_rank == 1 and p.rank_assignments[5].block_parallel_rank == 5


def test_inter_node_cp_placement_is_a_permutation():
    p = build_parallel_plan(num_blocks=32, world_size=8, data_parallel_size=2, context_parallel_size=4,
                            block_parallel_size=4, node_size=4, placement_policy="inter_node_cp")
    assert sorted(p.logical_to_physical) == list(range(8))
    assert sorted(r.rank for r in p.rank_assignments) == list(range(8))


def test_clean_ownership_covers_each_token_once():
    for n, cp in ((512, 2), (1024, 4), (96, 3)):
        for lay in ("dual_chunk", "contiguous"):
            seen = []
            for r in range(cp):
                for s in clean_shards_for_rank(n, cp, r, lay, align=32):
                    seen += list(range(s.start, s.stop))
            assert sorted(seen) == list(range(n))
    assert balanced_bounds(10, 3, 0) == (0, 4) and balanced_bounds(10, 3, 2) == (7, 10)
    sh = clean_shards_for_rank(512, 2, 0, "dual_chunk", 32)
    assert [(s.start, s.stop) for s in sh] == [(0, 128), (384, 512)]


def test_parallel_preflight_environment_policy():
    import pytest

    from turbo_dllm_b200.config.run_spec import RunSpec, RunSpecError
    from turbo_dllm_b200.parallel.preflight import (infer_parallel_mesh_sizes, prepare_parallel_environment,
                                                    uses_peer_memory_kernels, validate_supported_training_axes)

    def spec(**topology):
        return RunSpec.from_mapping({"model": {"id": "synthetic:tiny-hd128", "seq_len": 512, "dtype": "bf16"},
                                     "objective": {"name": "fast_dllm_v2", "block_size": 32},
                                     "topology": {"context_parallel_size": 1, "block_parallel_size": 1, **topology}})

    s = spec(tensor_parallel_size=2, sequence_parallel=True)
    assert uses_peer_memory_kernels(s, 2) and not uses_peer_memory_kernels(s, 1)
    up = prepare_parallel_environment(s, {}, 2)
    assert up["PYTORCH_CUDA_ALLOC_CONF"] == "expandable_segments:True" and up["TORCH_NCCL_ASYNC_ERROR_HANDLING"] == "1"
    assert "PYTORCH_CUDA_ALLOC_CONF" not in prepare_parallel_environment(s, {"PYTORCH_CUDA_ALLOC_CONF": "expandable_segments:False"}, 2)
    with pytest.raises(RunSpecError, match="CUDA_DEVICE_MAX_CONNECTIONS"):
        prepare_parallel_environment(s, {"CUDA_DEVICE_MAX_CONNECTIONS": "1"}, 2)
    base = s.with_overrides({"kernel": {"impl": "nccl_baseline"}})
    assert prepare_parallel_environment(base, {"CUDA_DEVICE_MAX_CONNECTIONS": "1"}, 2) is not None
    assert infer_parallel_mesh_sizes(8, spec(tensor_parallel_size=2)) == {
        "data": 4, "pipeline": 1, "local": 1, "context": 1, "block": 1, "tensor": 2, "expert": 1}
    with pytest.raises(RunSpecError, match="pipeline"):
        validate_supported_training_axes(spec(pipeline_parallel_size=2))

"""Parameter sharding (optimizer.backend: fsdp) on gloo ranks must train exactly like the replicated-parameter
path on the same ranks: same losses, same parameters after the steps, bitwise resume from its sharded
checkpoint; the unit plan covers the flat buffer once."""
import pytest
import torch

from tests._harness import assert_params_close, run_ranks

MAPPING = {
    "model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32", "num_layers": 3},
    "objective": {"name": "fast_dllm_v2", "block_size": 32, "noise_schedule_epsilon": 0.1},
    "training": {"batch_size": 1, "steps": 4, "gradient_accumulation_steps": 2},
    "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
    "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0},
}


def _spec(backend, world, tp=1, tmp=None):
    import copy

    from turbo_dllm_b200.config.run_spec import RunSpec

    m = copy.deepcopy(MAPPING)
    m["optimizer"]["backend"] = backend
    m["topology"]["tensor_parallel_size"] = tp
    if tmp:
        m["checkpointing"] = {"save_checkpoint_dir": tmp}
    return RunSpec.from_mapping(m).validate(world_size=world)


def _run(rank, world, backend, tp, tmp):
    import torch.distributed as dist

    import turbo_dllm_b200.checkpoint as ck
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = _spec(backend, world, tp, tmp)

    def session():
        rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world) if tp > 1 else None
        return TrainingSession(spec, device="cpu", runtime=rt)

    def full(s):
        return s.sharded.gather_full().clone() if s.sharded is not None else s.model.flat.data.clone()

    a = session()
    assert (a.sharded is not None) == (backend == "fsdp")
    losses = []
    for _ in range(4):
        r = a.step()
        t = r.loss_sum.double().clone()
        dist.all_reduce(t)
        losses.append(float(t) / r.denominator / tp)
    out = {"losses": losses, "params": full(a), "norm": a.optimizer.grad_norm()}
    if backend == "fsdp" and tmp:
        mem = a.sharded.memory_bytes()
        out["shard_fraction"] = mem["parameter_shard"] * 2 / mem["replicated_equivalent"]
        b = session()
        for _ in range(2):
            b.step()
        ck.save_training_checkpoint(tmp, b, step=2, rank=rank, world_size=world, control_group=dist.group.WORLD)
        out["saved_params"] = full(b)
        c = session()
        meta = ck.load_training_checkpoint(tmp, "latest", c, rank=rank, world_size=world)
        for _ in range(2):
            c.step()
        out["resumed_equal"] = bool(torch.equal(full(c), out["params"]))
        out["backend"] = meta["metadata"]["checkpoint_backend"]
    return out


@pytest.mark.distributed
def test_fsdp2_matches_replicated_parameters_and_resumes(tmp_path):
    ref = run_ranks(_run, 2, args=("torch_adamw", 1, None), deadline_s=300)
    out = run_ranks(_run, 2, args=("fsdp", 1, str(tmp_path / "ck")), deadline_s=300)
    for r, o in zip(ref, out):
        assert o["losses"] == pytest.approx(r["losses"], rel=1e-4)
        assert o["norm"] == pytest.approx(r["norm"], rel=2e-3)    # Adam amplifies summation-order noise over steps
        assert_params_close(o["params"], torch.from_numpy(r["params"]), rtol=1e-3, atol=2e-5)
        assert o["resumed_equal"] and o["backend"] == "fsdp_sharded_rank_local"
        assert o["shard_fraction"] < 0.56          # about half of the parameters per rank (padding to 128)
    assert (out[0]["params"] == out[1]["params"]).all()
    # one process reads the two ranks' parameter slices back into a whole model and exports it
    from turbo_dllm_b200.models.export import export_training_checkpoint
    from turbo_dllm_b200.models.hf_loader import load_hf_config, load_hf_weights
    from turbo_dllm_b200.models.dense import BlockDiffusionTransformer

    export_training_checkpoint(_spec("fsdp", 2, 1, str(tmp_path / "ck")), str(tmp_path / "ck"), str(tmp_path / "hf"))
    model = BlockDiffusionTransformer(load_hf_config(str(tmp_path / "hf")), dtype=torch.float32, seed=0)
    load_hf_weights(model, str(tmp_path / "hf"))
    assert torch.equal(model.flat.data, torch.from_numpy(out[0]["saved_params"]))


@pytest.mark.distributed
def test_fsdp2_times_tp2_matches_tp2():
    """BASELINE config 2 in miniature: parameter sharding over the data-parallel ranks of each tensor-parallel
    coordinate (4 gloo ranks)."""
    ref = run_ranks(_run, 4, args=("torch_adamw", 2, None), deadline_s=400)
    out = run_ranks(_run, 4, args=("fsdp", 2, None), deadline_s=400)
    for r, o in zip(ref, out):
        assert o["losses"] == pytest.approx(r["losses"], rel=1e-4)
        assert_params_close(o["params"], torch.from_numpy(r["params"]), rtol=1e-3, atol=2e-5)


def test_unit_plan_covers_the_buffer_once():
    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.dense import BlockDiffusionTransformer
    from turbo_dllm_b200.parallel.fsdp import plan_units

    model = BlockDiffusionTransformer(PRESETS["synthetic:tiny-qwen3"], dtype=torch.float32, seed=1)
    for world in (2, 3, 8):
        units = plan_units(model.flat, world)
        names = [u.name for u in units]
        assert names[-1] == "norm_weights" and sum(n.startswith("layer.") for n in names) == 4
        spans = sorted((u.start, u.stop) for u in units)
        assert spans[0][0] == 0 and spans[-1][1] == model.flat.numel
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
        covered = sum(b - a for a, b in spans)
        assert covered >= sum(n for _, n, _, _ in model.flat.offsets.values())
        assert all(u.shard % 128 == 0 and u.shard * world >= u.length for u in units)
        locs = sorted((u.local, u.local + u.shard) for u in units)
        assert locs[0][0] == 0 and all(a[1] == b[0] for a, b in zip(locs, locs[1:]))


def test_fsdp_needs_activation_checkpointing_and_a_dense_model():
    import copy

    from turbo_dllm_b200.config.run_spec import RunSpec, RunSpecError

    m = copy.deepcopy(MAPPING)
    m["optimizer"]["backend"] = "fsdp"
    m["training"]["activation_checkpointing"] = False
    with pytest.raises(RunSpecError, match="activation_checkpointing"):
        RunSpec.from_mapping(m).validate()
    m["training"]["activation_checkpointing"] = True
    m["adapter"] = {"type": "lora", "rank": 4}
    with pytest.raises(RunSpecError, match="adapters"):
        RunSpec.from_mapping(m).validate()


def _moe_run(rank, world, backend, tmp):
    import torch.distributed as dist

    import turbo_dllm_b200.checkpoint as ck
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-moe", "seq_len": 128, "dtype": "fp32", "family": "diffusion_gemma", "num_layers": 2,
                  "moe_shared_intermediate_size": 64},
        "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
        "training": {"batch_size": 2, "steps": 4},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1, "expert_parallel_size": 2},
        "optimizer": {"backend": backend, "lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)

    def session():
        rt = build_parallel_runtime(spec, device="cpu", rank=rank, world_size=world)
        return TrainingSession(spec, device="cpu", runtime=rt), rt

    a, _ = session()
    assert (a.sharded is not None) == (backend == "fsdp")
    losses = []
    for _ in range(4):
        r = a.step()
        t = r.loss_sum.double().clone()
        dist.all_reduce(t)
        losses.append(float(t) / r.denominator)
    dense = a.sharded.gather_full().clone() if a.sharded is not None else a.model.flat.data.clone()
    out = {"losses": losses, "norm": a.optimizer.grad_norm(), "dense": dense, "experts": a.model.flat_experts.data.clone()}
    if tmp:
        b, rt = session()
        for _ in range(2):
            b.step()
        ck.save_training_checkpoint(tmp, b, step=2, rank=rank, world_size=world, control_group=dist.group.WORLD, runtime=rt)
        c, rt2 = session()
        ck.load_training_checkpoint(tmp, "latest", c, rank=rank, world_size=world, runtime=rt2)
        for _ in range(2):
            c.step()
        out["resumed_equal"] = bool(torch.equal(c.sharded.gather_full(), dense)
                                    and torch.equal(c.model.flat_experts.data, a.model.flat_experts.data))
    return out


@pytest.mark.distributed
def test_moe_parameter_sharding_beside_expert_parallelism(tmp_path):
    """The mixture-of-experts decoder with `optimizer.backend: fsdp`: the replicated part (attention, router, dense
    branch, embeddings) is sharded per layer over all ranks, the experts stay divided by expert parallelism with their own
    sharded optimizer, and one gradient norm covers both. Same step as the sharded optimizer; resumes bit for bit."""
    ref = run_ranks(_moe_run, 2, args=("torch_adamw", None), deadline_s=300)
    out = run_ranks(_moe_run, 2, args=("fsdp", str(tmp_path / "ck")), deadline_s=400)
    for r, o in zip(ref, out):
        assert o["losses"] == pytest.approx(r["losses"], rel=1e-4)
        assert o["norm"] == pytest.approx(r["norm"], rel=2e-3)
        assert_params_close(o["dense"], torch.from_numpy(r["dense"]), rtol=1e-3, atol=2e-5)
        assert_params_close(o["experts"], torch.from_numpy(r["experts"]), rtol=1e-3, atol=2e-5)
        assert o["resumed_equal"]

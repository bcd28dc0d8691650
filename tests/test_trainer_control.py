"""Decisions every rank must take together (save now, stop now), the checkpoint failure protocol, adapter-only
checkpoints, LoRA under data parallelism, phase timings and communication labels. All on CPU, gloo ranks."""
import json
import os

import pytest
import torch

from tests._harness import run_ranks

MAPPING = {
    "model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32", "num_layers": 2},
    "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
    "training": {"batch_size": 2, "steps": 4},
    "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
    "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0},
}


def _spec(extra=None, world=1):
    import copy

    from turbo_dllm_b200.config.run_spec import RunSpec

    m = copy.deepcopy(MAPPING)
    for k, v in (extra or {}).items():
        m.setdefault(k, {}).update(v)
    return RunSpec.from_mapping(m).validate(world_size=world)


# ---------------------------------------------------------------------------------- rank-0 driven control
def _skewed_clocks(rank, world, tmp):
    """Rank 1's clock runs far ahead of rank 0's: on its own it would stop after the first step and save the 50 %
    checkpoint at once. Both ranks must follow rank 0."""
    import torch.distributed as dist

    from turbo_dllm_b200.training.checkpointing import StepControl

    spec = _spec({"training": {"max_duration_seconds": 100.0},
                  "checkpointing": {"save_checkpoint_dir": tmp, "save_duration_fractions": [0.5], "save_final": True}}, world)
    now = {"t": 0.0}
    speed = 1.0 if rank == 0 else 1000.0
    ctl = StepControl(spec, total_steps=50, rank=rank, world=world, group=dist.group.WORLD, clock=lambda: now["t"] * speed)
    out = []
    for step in range(1, 8):
        now["t"] += 20.0                       # rank 0: 20 s per step -> 50 % after step 3, limit after step 5
        v = ctl.decide(step)
        out.append((step, v.save, v.tag, v.stop))
        if v.stop:
            break
    return out


@pytest.mark.distributed
def test_save_and_stop_follow_rank_zero_although_clocks_differ(tmp_path):
    a, b = run_ranks(_skewed_clocks, 2, args=(str(tmp_path),), deadline_s=120)
    assert a == b
    assert a == [(1, False, None, False), (2, False, None, False),
                 (3, True, "duration_050pct_step_00000003", False), (4, False, None, False),
                 (5, True, None, True)]


def test_fraction_state_belongs_to_the_run_object(tmp_path):
    from turbo_dllm_b200.training.checkpointing import StepControl

    spec = _spec({"training": {"max_duration_seconds": 10.0},
                  "checkpointing": {"save_checkpoint_dir": str(tmp_path), "save_duration_fractions": [0.5]}})
    for _ in range(2):      # a second run in the same process starts with a clean slate
        t = {"v": 0.0}
        ctl = StepControl(spec, 100, clock=lambda: t["v"])
        t["v"] = 6.0
        assert ctl.decide(1).tag == "duration_050pct_step_00000001"
        assert not ctl.decide(2).save


# ---------------------------------------------------------------------------------- checkpoint failure protocol
def _failing_save(rank, world, tmp):
    import torch.distributed as dist

    import turbo_dllm_b200.checkpoint as ck
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    s = TrainingSession(_spec(world=world), device="cpu")
    s.step()
    real = ck._atomic_torch_save
    if rank == 1:
        def broken(obj, path):
            raise OSError("disk full (injected)")
        ck._atomic_torch_save = broken
    raised = None
    try:
        ck.save_training_checkpoint(tmp, s, step=1, rank=rank, world_size=world, control_group=dist.group.WORLD,
                                    async_save=False)
    except RuntimeError as e:
        raised = str(e)
    ck._atomic_torch_save = real
    published = os.path.exists(os.path.join(tmp, "metadata.json"))
    # the same tag can be saved again: stale markers are cleared
    tag = ck.save_training_checkpoint(tmp, s, step=1, rank=rank, world_size=world, control_group=dist.group.WORLD,
                                      async_save=False)
    return raised, published, tag, ck.validate_checkpoint(tmp)["ok"]


@pytest.mark.distributed
def test_a_failed_shard_makes_every_rank_raise_and_the_tag_can_be_saved_again(tmp_path):
    outs = run_ranks(_failing_save, 2, args=(str(tmp_path / "ck"),), deadline_s=180)
    for raised, published, tag, ok in outs:
        assert raised is not None and "incomplete" in raised
        assert not published
        assert tag == "step_00000001" and ok


def _async_save(rank, world, tmp):
    import torch.distributed as dist

    import turbo_dllm_b200.checkpoint as ck
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    s = TrainingSession(_spec(world=world), device="cpu")
    s.step()
    before = s.model.flat.data.clone()
    tag = ck.save_training_checkpoint(tmp, s, step=1, rank=rank, world_size=world, control_group=dist.group.WORLD,
                                      async_save=True)
    s.step()                                  # training goes on while the writer thread works on the snapshot
    ck.wait_for_async_saves()
    dist.barrier()
    meta = ck.read_metadata(tmp)
    payload = torch.load(os.path.join(tmp, tag, ck.shard_name(rank, world)), weights_only=False)
    return meta["latest_tag"], bool(torch.equal(payload["model"], before))


@pytest.mark.distributed
def test_async_save_is_deferred_and_snapshots_the_state_of_its_step(tmp_path):
    for latest, same in run_ranks(_async_save, 2, args=(str(tmp_path / "ck"),), deadline_s=180):
        assert latest == "step_00000001" and same
    # one process reads the weights of the two-rank checkpoint (replicated parameters: rank 0's file has them all);
    # the full loader still refuses the other world size
    import turbo_dllm_b200.checkpoint as ck
    from turbo_dllm_b200.training.session import TrainingSession

    t = TrainingSession(_spec(), device="cpu")
    with pytest.raises(ValueError, match="written by 2 ranks"):
        ck.load_training_checkpoint(str(tmp_path / "ck"), "latest", t, rank=0, world_size=1)
    out = ck.load_model_weights(str(tmp_path / "ck"), "latest", t)
    payload = torch.load(os.path.join(str(tmp_path / "ck"), out["tag"], ck.shard_name(0, 2)), weights_only=False)
    assert out["step"] == 1 and torch.equal(t.model.flat.data, payload["model"])


def test_an_older_tag_is_checked_against_its_own_topology(tmp_path):
    import turbo_dllm_b200.checkpoint as ck
    from turbo_dllm_b200.training.session import TrainingSession

    d = str(tmp_path / "ck")
    s = TrainingSession(_spec(), device="cpu")
    s.step()
    ck.save_training_checkpoint(d, s, step=1, rank=0, world_size=1)
    s.step()
    ck.save_training_checkpoint(d, s, step=2, rank=0, world_size=1)
    meta = json.load(open(os.path.join(d, "metadata.json")))
    meta["topology"]["tensor_parallel_size"] = 2        # the LATEST publication claims another topology
    json.dump(meta, open(os.path.join(d, "metadata.json"), "w"))
    t = TrainingSession(_spec(), device="cpu")
    assert ck.load_training_checkpoint(d, "step_00000001", t, rank=0, world_size=1)["step"] == 1
    with pytest.raises(ValueError, match="topology mismatch"):
        ck.load_training_checkpoint(d, "latest", t, rank=0, world_size=1)


# ---------------------------------------------------------------------------------- LoRA on two data-parallel ranks
LORA = {"adapter": {"type": "lora", "rank": 4, "alpha": 8.0, "targets": ["attention", "mlp"]}}


def _lora_dp(rank, world, tmp, model_only):
    import torch.distributed as dist

    import turbo_dllm_b200.checkpoint as ck
    from turbo_dllm_b200.training.session import TrainingSession

    torch.set_num_threads(2)
    spec = _spec({**LORA, "checkpointing": {"save_checkpoint_dir": tmp, "model_only": model_only}}, world)
    a = TrainingSession(spec, device="cpu")
    base0 = a.model.flat.data.clone()
    full = [float(a.step().loss_sum) for _ in range(4)]
    moved = float(sum(p.abs().sum() for n, p in a.lora.flat.params.items() if n.endswith("lora_B")))
    base_same = bool(torch.equal(a.model.flat.data, base0))
    b = TrainingSession(spec, device="cpu")
    first = [float(b.step().loss_sum) for _ in range(2)]
    tag = ck.save_training_checkpoint(tmp, b, step=2, rank=rank, world_size=world, control_group=dist.group.WORLD)
    c = TrainingSession(spec, device="cpu")
    ck.load_training_checkpoint(tmp, "latest", c, rank=rank, world_size=world)
    adapters_equal = bool(torch.equal(c.lora.flat.data, b.lora.flat.data))
    rest = [float(c.step().loss_sum) for _ in range(2)] if not model_only else []
    files = sorted(os.listdir(os.path.join(tmp, tag)))
    return full, first + rest, moved, base_same, adapters_equal, files


@pytest.mark.distributed
def test_lora_on_two_ranks_trains_adapters_only_and_resumes_bitwise(tmp_path):
    for full, resumed, moved, base_same, adapters_equal, files in run_ranks(
            _lora_dp, 2, args=(str(tmp_path / "ck"), False), deadline_s=240):
        assert base_same and moved > 0 and adapters_equal
        assert resumed == full
        assert files == ["rank_00000_of_00002.pt", "rank_00001_of_00002.pt"]


@pytest.mark.distributed
def test_model_only_adapter_checkpoint(tmp_path):
    import turbo_dllm_b200.checkpoint as ck

    d = str(tmp_path / "ck")
    for full, resumed, moved, base_same, adapters_equal, files in run_ranks(_lora_dp, 2, args=(d, True), deadline_s=240):
        assert adapters_equal and base_same
        assert files == ["model_only_manifest.json", "mp_rank_00_model_states.pt"]
    meta = ck.read_metadata(d)
    assert meta["checkpoint_backend"] == "adapter_model_only" and meta["model_state_scope"] == "trainable_parameters"
    assert meta["objective_state"] == {} and meta["dataloader_state"] == {}      # no restart state is claimed
    man = json.load(open(os.path.join(d, meta["latest_tag"], "model_only_manifest.json")))
    assert man["format"] == "dllm_parallel.model_only_checkpoint.v1" and len(man["sha256"]) == 64
    assert ck.validate_model_only_checkpoint(d)["ok"]
    with open(os.path.join(d, meta["latest_tag"], "mp_rank_00_model_states.pt"), "ab") as f:
        f.write(b"x")
    assert not ck.validate_model_only_checkpoint(d)["ok"]


# ---------------------------------------------------------------------------------- phase timings, labels, TP loss
def _traced_run(rank, world, tmp, tp):
    import io
    from contextlib import redirect_stdout

    from turbo_dllm_b200.training.trainer import run_training

    torch.set_num_threads(2)
    os.environ["DLLM_RUN_DIR"] = tmp
    spec = _spec({"topology": {"tensor_parallel_size": tp},
                  "training": {"steps": 2},
                  "profiler": {"phase_timing": True, "system_trace": True, "system_trace_start_step": 2,
                               "system_trace_steps": 1, "system_trace_dir": os.path.join(tmp, "trace")}}, world)
    buf = io.StringIO()
    with redirect_stdout(buf):
        run_training(spec)
    events = [json.loads(l) for l in buf.getvalue().splitlines() if l.startswith("{")]
    return events


@pytest.mark.distributed
def test_step_events_carry_phase_ms_and_the_trace_reports_the_collectives(tmp_path):
    from turbo_dllm_b200.profiling.trace_analysis import analyze_kineto_trace

    events = run_ranks(_traced_run, 2, args=(str(tmp_path), 1), deadline_s=300)[0]
    steps = [e for e in events if e["event"] == "step"]
    assert len(steps) == 2
    for e in steps:
        assert {"zero_grad", "data", "forward", "loss", "backward", "gradient_sync", "optimizer"} <= set(e["phase_ms"])
        assert all(v >= 0 for v in e["phase_ms"].values())
    summary = analyze_kineto_trace(str(tmp_path / "trace" / "rank_0.trace.json.gz"))
    labels = summary["communication_labels"]
    assert "optimizer_data_parallel/gradient_sync/all_reduce" in labels
    assert labels["optimizer_data_parallel/gradient_sync/all_reduce"]["input_bytes"] > 0
    assert "optimizer_data_parallel/optimizer/all_gather" in labels
    assert any(k.startswith("dllm.phase.") for k in summary["operators"])


@pytest.mark.distributed
def test_logged_loss_under_tensor_parallelism_equals_the_single_rank_loss(tmp_path):
    one = _traced_run(0, 1, str(tmp_path / "a"), 1)
    two = run_ranks(_traced_run, 2, args=(str(tmp_path / "b"), 2), deadline_s=300)[0]
    l1 = [e["loss"] for e in one if e["event"] == "step"]
    l2 = [e["loss"] for e in two if e["event"] == "step"]
    a1 = [e["active_tokens"] for e in one if e["event"] == "step"]
    a2 = [e["active_tokens"] for e in two if e["event"] == "step"]
    assert l2 == pytest.approx(l1, rel=1e-3)
    assert a1 == a2


def test_evaluation_reads_its_own_dataset_and_leaves_the_training_stream_alone(tmp_path):
    import numpy as np

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.training.evaluation import evaluate_masked_token_accuracy
    from turbo_dllm_b200.training.session import TrainingSession

    (np.arange(8192) % 11 + 100).astype("<i4").tofile(tmp_path / "train.i32")
    (np.arange(8192) % 5 + 700).astype("<i4").tofile(tmp_path / "heldout.i32")
    base = {"model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "num_layers": 1},
            "objective": {"name": "standard_block_diffusion", "block_size": 16},
            "data": {"input_mode": "dataset", "dataset_path": str(tmp_path / "train.i32")},
            "training": {"batch_size": 2, "steps": 1}, "topology": {"context_parallel_size": 1, "block_parallel_size": 1}}
    s = TrainingSession(RunSpec.from_mapping({**base, "evaluation": {"dataset_path": str(tmp_path / "heldout.i32"),
                                                                      "batches": 2}}).validate(), device="cpu")
    cursor = s.data.state_dict()
    seen = []
    real = s.assemble_rows

    def spy(cb):
        seen.append(cb.clean_input_ids.clone())
        return real(cb)

    s.assemble_rows = spy
    out = evaluate_masked_token_accuracy(s, 2, 7)
    assert out["eval_masked_tokens"] > 0 and len(seen) == 2
    assert all(int(t.min()) >= 700 for t in seen)                 # the held-out ids, not the training ones
    assert s.data.state_dict() == cursor                          # the training stream did not move
    t = TrainingSession(RunSpec.from_mapping(base).validate(), device="cpu")
    before = t.data.state_dict()
    evaluate_masked_token_accuracy(t, 1, 7)
    assert t.data.state_dict() != before                          # without a held-out set the next training batches are used

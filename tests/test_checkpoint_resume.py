"""Save after step 2, reload in a fresh session, continue: must equal the uninterrupted run."""
import json
import os

import pytest
import torch

from turbo_dllm_b200.checkpoint import (list_tags, load_training_checkpoint, read_metadata, save_training_checkpoint,
                                        shard_name, validate_checkpoint)
from turbo_dllm_b200.config.run_spec import RunSpec
from turbo_dllm_b200.training.session import TrainingSession


def _spec(tmp, **ck):
    return RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-qwen3", "seq_len": 128, "dtype": "fp32", "num_layers": 2},
        "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
        "training": {"batch_size": 2, "steps": 4},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0},
        "scheduler": {"type": "cosine", "warmup_steps": 1, "decay_steps": 4},
        "checkpointing": {"save_checkpoint_dir": str(tmp), **ck}}).validate()


@pytest.mark.checkpoint_resume
def test_resume_is_bitwise_identical(tmp_path):
    spec = _spec(tmp_path / "ck")
    a = TrainingSession(spec, device="cpu")
    full = [float(a.step().loss_sum) for _ in range(4)]
    b = TrainingSession(spec, device="cpu")
    first = [float(b.step().loss_sum) for _ in range(2)]
    tag = save_training_checkpoint(str(tmp_path / "ck"), b, step=2, rank=0, world_size=1)
    assert tag == "step_00000002"
    c = TrainingSession(spec, device="cpu")
    meta = load_training_checkpoint(str(tmp_path / "ck"), "latest", c, rank=0, world_size=1)
    assert meta["step"] == 2
    rest = [float(c.step().loss_sum) for _ in range(2)]
    assert first + rest == full
    assert torch.equal(c.model.flat.data, a.model.flat.data)


def test_layout_metadata_pruning_and_validation(tmp_path):
    d = tmp_path / "ck"
    spec = _spec(d, keep_last_n=2)
    s = TrainingSession(spec, device="cpu")
    for step in (1, 2, 3):
        s.step()
        save_training_checkpoint(str(d), s, step=step, rank=0, world_size=1)
    assert list_tags(str(d)) == ["step_00000002", "step_00000003"]
    meta = read_metadata(str(d))
    assert meta["format"] == "dllm_parallel.distributed_checkpoint.v1"
    assert meta["latest_tag"] == "step_00000003" and meta["world_size"] == 1
    assert meta["rank_state_pattern"] == "rank_{rank:05d}_of_{world_size:05d}.pt"
    assert (d / "step_00000003" / shard_name(0, 1)).exists()
    assert validate_checkpoint(str(d))["ok"]
    os.unlink(d / "step_00000003" / shard_name(0, 1))
    assert not validate_checkpoint(str(d))["ok"]


def test_topology_mismatch_is_refused(tmp_path):
    d = tmp_path / "ck"
    s = TrainingSession(_spec(d), device="cpu")
    s.step()
    save_training_checkpoint(str(d), s, step=1, rank=0, world_size=1)
    meta = json.loads((d / "metadata.json").read_text())
    meta["world_size"] = 2
    (d / "metadata.json").write_text(json.dumps(meta))
    with pytest.raises(ValueError, match="resharding"):
        load_training_checkpoint(str(d), "latest", s, rank=0, world_size=1)


def test_incomplete_checkpoint_is_not_published(tmp_path):
    from turbo_dllm_b200.checkpoint import publish_metadata

    d = tmp_path / "ck"
    (d / "step_00000005").mkdir(parents=True)
    spec = _spec(d)
    with pytest.raises(RuntimeError, match="incomplete"):
        publish_metadata(str(d), "step_00000005", 5, 2, {"topology": {}, "config": {}, "objective_state": {},
                                                         "dataloader_state": {}, "scheduler_state": {},
                                                         "kernel_metadata": {}, "run_metadata": {},
                                                         "backbone_state": {}}, spec)
    assert not (d / "metadata.json").exists()
    assert (d / "step_00000005" / "checkpoint.error").exists()


def test_auto_resume_policy(tmp_path):
    from turbo_dllm_b200.training.checkpointing import resolve_load_checkpoint, should_save

    d = tmp_path / "ck"
    spec = _spec(d, auto_resume=True, save_checkpoint_interval=2, save_final=True)
    assert resolve_load_checkpoint(spec) == (None, "latest")
    s = TrainingSession(spec, device="cpu")
    s.step()
    save_training_checkpoint(str(d), s, step=1, rank=0, world_size=1)
    assert resolve_load_checkpoint(spec) == (str(d), "latest")
    assert [should_save(spec, st, 4, 0.0) for st in (1, 2, 3, 4)] == [False, True, False, True]


@pytest.mark.checkpoint_resume
@pytest.mark.parametrize("kind", ["hybrid", "dflash2"])
def test_resume_of_the_hybrid_family_and_the_dflash2_drafter(tmp_path, kind):
    """Same contract as above for the models with extra state: recurrence parameters and convolutions
    (hybrid), selector codebooks and the selector loss schedule (DFlash2)."""
    if kind == "hybrid":
        mapping = {"model": {"id": "synthetic:tiny-qwen3_8", "family": "qwen3_8", "seq_len": 64, "dtype": "fp32"},
                   "objective": {"name": "fast_dllm_v2", "block_size": 16}}
    else:
        mapping = {"model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "family": "dflash",
                             "verifier_id": "synthetic:tiny-qwen3", "target_layer_ids": [0, 2], "max_layers": 2,
                             "dflash2_conv_kernel_size": 2, "dflash2_conv_group_size": 64,
                             "dflash2_selector_rank": 4, "dflash2_selector_top_k": 2},
                   "objective": {"name": "dflash_distillation", "block_size": 8, "max_anchors": 4,
                                 "dflash_loss": "dpace", "selector_ramp_ratio": 0.5, "dflash_vocab_block_size": 512},
                   "data": {"target_features": "online"}}
    spec = RunSpec.from_mapping({
        **mapping, "training": {"batch_size": 1, "steps": 4},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0},
        "checkpointing": {"save_checkpoint_dir": str(tmp_path / "ck")}}).validate()
    a = TrainingSession(spec, device="cpu")
    full = [float(a.step().loss_sum) for _ in range(4)]
    b = TrainingSession(spec, device="cpu")
    first = [float(b.step().loss_sum) for _ in range(2)]
    save_training_checkpoint(str(tmp_path / "ck"), b, step=2, rank=0, world_size=1)
    c = TrainingSession(spec, device="cpu")
    load_training_checkpoint(str(tmp_path / "ck"), "latest", c, rank=0, world_size=1)
    rest = [float(c.step().loss_sum) for _ in range(2)]
    assert first + rest == full
    assert torch.equal(c.model.flat.data, a.model.flat.data)

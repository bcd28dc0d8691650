import json

import pytest
import yaml

from turbo_dllm_b200.config.run_spec import (RunSpec, RunSpecError, build_run_spec_arg_parser, load_run_spec,
                                             run_spec_from_args)
from turbo_dllm_b200.config.schema import SECTIONS


def base(**over):
    m = {"model": {"id": "synthetic:tiny-qwen3", "seq_len": 512, "dtype": "fp32"},
         "objective": {"name": "standard_block_diffusion", "block_size": 32},
         "topology": {"context_parallel_size": 1, "block_parallel_size": 1}}
    for k, v in over.items():
        m.setdefault(k, {}).update(v)
    return m


def test_sections_and_defaults_match_the_public_schema():
    assert list(SECTIONS) == ["model", "objective", "data", "training", "evaluation", "adapter", "topology",
                              "optimizer", "scheduler", "checkpointing", "profiler", "logging", "debug", "kernel",
                              "launch"]
    s = RunSpec.default()
    assert s.model.seq_len == 1024 and s.model.attention_backend == "flex"
    assert s.topology.context_parallel_size == 4 and s.topology.block_parallel_size == 4
    assert s.optimizer.lr == 1e-6 and s.optimizer.adam_eps == 1e-5 and s.launch.seed == 2026
    assert s.objective.noise_schedule == "loglinear" and s.objective.antithetic_sampling is True
    assert s.checkpointing.checkpoint_tag == "latest" and s.evaluation.seed == 314159


def test_unknown_section_and_field_are_rejected():
    with pytest.raises(RunSpecError, match="unknown run-spec section"):
        RunSpec.from_mapping({"modle": {}})
    with pytest.raises(RunSpecError, match="unknown field"):
        RunSpec.from_mapping({"model": {"sequence_length": 4}})
    with pytest.raises(RunSpecError, match="cannot interpret"):
        RunSpec.from_mapping({"model": {"seq_len": "many"}})


def test_validate_rules():
    RunSpec.from_mapping(base()).validate()
    with pytest.raises(RunSpecError, match="multiple of objective.block_size"):
        RunSpec.from_mapping(base(model={"seq_len": 500})).validate()
    with pytest.raises(RunSpecError, match="replicate_clean_prefix"):
        RunSpec.from_mapping(base(topology={"block_parallel_size": 2})).validate()
    with pytest.raises(RunSpecError, match="multiple of"):
        RunSpec.from_mapping(base(topology={"context_parallel_size": 4, "block_parallel_size": 6})).validate()
    with pytest.raises(RunSpecError, match="sequence_parallel needs"):
        RunSpec.from_mapping(base(topology={"sequence_parallel": True})).validate()
    with pytest.raises(RunSpecError, match="pipeline"):
        RunSpec.from_mapping(base(topology={"pipeline_parallel_size": 2})).validate()
    with pytest.raises(RunSpecError, match="not supported by family"):
        RunSpec.from_mapping(base(model={"family": "qwen3_8"})).validate()
    with pytest.raises(RunSpecError, match="production recipes"):
        RunSpec.from_mapping(base(launch={"recipe_kind": "prod"})).validate()
    with pytest.raises(RunSpecError, match="world size"):
        RunSpec.from_mapping(base(topology={"context_parallel_size": 2, "block_parallel_size": 2})).validate(world_size=3)


def test_yaml_roundtrip_and_cli_overrides(tmp_path):
    p = tmp_path / "train.yaml"
    p.write_text(yaml.safe_dump(base(optimizer={"lr": 3e-4})))
    spec = load_run_spec(p)
    assert spec.optimizer.lr == 3e-4
    again = RunSpec.from_mapping(yaml.safe_load(spec.to_yaml()))
    assert again == spec
    ap = build_run_spec_arg_parser()
    args = ap.parse_args(["--config", str(p), "--seq-len", "256", "--no-activation-checkpointing",
                          "--model-id", "synthetic:tiny-hd128", "--target-layer-ids", "1", "3", "--lr", "1e-3"])
    s2 = run_spec_from_args(args)
    assert s2.model.seq_len == 256 and s2.training.activation_checkpointing is False
    assert s2.model.id == "synthetic:tiny-hd128" and s2.model.target_layer_ids == (1, 3) and s2.optimizer.lr == 1e-3
    pj = tmp_path / "train.json"
    pj.write_text(json.dumps(base()))
    assert load_run_spec(pj).model.seq_len == 512


def test_every_field_has_a_cli_flag():
    ap = build_run_spec_arg_parser()
    dests = {a.dest for a in ap._actions}
    for section, rows in SECTIONS.items():
        for r in rows:
            assert f"{section}__{r.name}" in dests


def test_global_batch_rule():
    s = RunSpec.from_mapping(base(training={"batch_size": 2, "gradient_accumulation_steps": 3}))
    assert s.global_batch(4) == 24


def test_settings_without_effect_are_refused_and_debug_checks_fire():
    import torch

    from turbo_dllm_b200.config.run_spec import RunSpec, RunSpecError
    from turbo_dllm_b200.training.session import TrainingSession

    base = {"model": {"id": "synthetic:tiny-qwen3", "seq_len": 64, "dtype": "fp32", "num_layers": 1},
            "objective": {"name": "standard_block_diffusion", "block_size": 16},
            "training": {"batch_size": 1, "steps": 1},
            "topology": {"context_parallel_size": 1, "block_parallel_size": 1}}
    for section, field, value in (("optimizer", "zero_reduce_bucket_size", 1 << 20), ("optimizer", "fsdp_sharding_strategy", "no_shard"),
                                  ("kernel", "mlp_token_chunk_size", 100),
                                  ("model", "draft_vocab_path", "/x"), ("objective", "bp_loss_scale", 3.0)):
        m = {**base, section: {**base.get(section, {}), field: value}}
        with pytest.raises(RunSpecError, match=field):
            RunSpec.from_mapping(m).validate()
    RunSpec.from_mapping({**base, "objective": {**base["objective"], "bp_loss_scale": 1.0}}).validate()
    # the feed-forward over row chunks computes the same step
    runs = []
    for chunk in (0, 128):
        t = TrainingSession(RunSpec.from_mapping({**base, "model": {**base["model"], "seq_len": 256},
                                                  "kernel": {"mlp_token_chunk_size": chunk}}).validate(), device="cpu")
        runs.append((float(t.step().loss_sum), t.model.flat.data.clone()))
    assert runs[0][0] == pytest.approx(runs[1][0], rel=1e-6) and torch.allclose(runs[0][1], runs[1][1], atol=1e-5)
    # checkpointing only the feed-forward half computes the same step and keeps the residual stream between the halves
    t = TrainingSession(RunSpec.from_mapping({**base, "model": {**base["model"], "seq_len": 256},
                                              "training": {**base["training"], "activation_checkpointing_scope": "mlp"}}).validate(),
                        device="cpu")
    assert t.model.checkpoint_scope == "mlp"
    assert float(t.step().loss_sum) == pytest.approx(runs[0][0], rel=1e-6) and torch.allclose(t.model.flat.data, runs[0][1], atol=1e-5)
    with pytest.raises(RunSpecError, match="activation_checkpointing_scope"):
        RunSpec.from_mapping({**base, "training": {**base["training"], "activation_checkpointing_scope": "mlp",
                                                   "activation_checkpointing": False}}).validate()
    with pytest.raises(RunSpecError, match="activation_checkpointing_scope"):
        RunSpec.from_mapping({**base, "model": {**base["model"], "family": "qwen3_8", "id": "synthetic:tiny-qwen3-8"},
                              "training": {**base["training"], "activation_checkpointing_scope": "mlp"}}).validate()
    s = TrainingSession(RunSpec.from_mapping({**base, "debug": {"grad_finite": True, "optimizer_finite": True}}).validate(),
                        device="cpu")
    s.step()                                       # finite run: nothing raised
    orig = s.forward_backward

    def poisoned(batch, denom):
        out = orig(batch, denom)
        s.model.flat.params["layers.0.w_o"].main_grad[0, 0] = float("nan")
        return out

    s.forward_backward = poisoned
    with pytest.raises(FloatingPointError, match="layers.0.w_o"):
        s.step()


def test_run_files_of_the_large_recipe_shapes_validate():
    """Run files in the shape of the large multi-node recipes (hub model ids, DeepSpeed-style optimizer names, tensor +
    sequence parallelism times context-sharded block parallelism, expert parallelism with native SFT, a drafter with the
    context divided over two ranks) pass validation, including the model family's own checks."""
    from turbo_dllm_b200.config.run_spec import RunSpec

    common = {"training": {"batch_size": 1, "steps": 10, "activation_checkpointing": True,
                           "activation_checkpointing_scope": "full"},
              "optimizer": {"backend": "deepspeed_zero2", "allow_deepspeed_op_build": False, "lr": 1e-6, "gradient_clip_norm": 1.0},
              "scheduler": {"type": "cosine", "warmup_steps": 4, "decay_steps": 10, "min_lr": 1e-7},
              "kernel": {"runtime_jit": False}, "logging": {"wandb": False}}
    hybrid = {**common, "model": {"id": "Qwen/Qwen3.8-27B", "family": "qwen3_8", "seq_len": 262144, "mask_token": "<|mask|>",
                                  "dtype": "bf16"},
              "objective": {"name": "fast_dllm_v2", "block_size": 256, "noise_schedule": "linear_mask", "loss_weighting": "unit",
                            "antithetic_sampling": True},
              "topology": {"tensor_parallel_size": 2, "sequence_parallel": True, "tensor_parallel_overlap": False,
                           "context_parallel_size": 8, "block_parallel_size": 8, "placement_policy": "inter_node_cp"}}
    RunSpec.from_mapping(hybrid).validate(world_size=16)
    moe = {**common, "model": {"id": "google/diffusiongemma-26B-A4B-it", "family": "auto", "seq_len": 262144, "dtype": "bf16",
                               "trust_remote_code": True},
           "objective": {"name": "diffusiongemma_native_sft", "block_size": 256, "noise_schedule": "loglinear",
                         "loss_weighting": "unit", "self_conditioning_probability": 0.5},
           "topology": {"expert_parallel_size": 2, "context_parallel_size": 8, "block_parallel_size": 8}}
    RunSpec.from_mapping(moe).validate(world_size=16)
    moe_tp = {**moe, "objective": {"block_size": 256, "name": "standard_block_diffusion"},
              "topology": {"tensor_parallel_size": 2, "sequence_parallel": True, "context_parallel_size": 2, "block_parallel_size": 2}}
    RunSpec.from_mapping(moe_tp).validate(world_size=4)
    draft = {**common, "model": {"id": "z-lab/draft", "family": "dflash", "verifier_id": "org/verifier", "seq_len": 1048576,
                                 "target_layer_ids": [2, 11, 19], "dtype": "bf16"},
             "objective": {"name": "dflash_distillation", "block_size": 16, "max_anchors": 512, "decay_gamma": 4.0},
             "data": {"input_mode": "dataset", "target_features": "synthetic"},
             "topology": {"context_parallel_size": 2, "block_parallel_size": 1}}
    RunSpec.from_mapping(draft).validate(world_size=2)
    with pytest.raises(RunSpecError, match="tensor-parallel"):      # a drafter has no tensor-parallel form
        RunSpec.from_mapping({**draft, "topology": {"tensor_parallel_size": 2}}).validate(world_size=2)

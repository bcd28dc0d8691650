"""Declarative description of the train.yaml schema.

Each section is a table of (field, type, default, options) rows from which frozen dataclasses,
CLI flags and validation of enumerated values are generated. Section and field names, defaults
and CLI destinations follow the reference's RunSpec so existing train.yaml files load unchanged
(dllm_parallel/training/run_spec.py:25-252); fields marked `ext=True` are additions of this
framework (architecture overrides for random-init models, kernel implementation selector).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Any

OPT_INT = "int?"
OPT_FLOAT = "float?"
OPT_STR = "str?"
TUPLE_STR = "tuple[str]"
TUPLE_INT = "tuple[int]"
TUPLE_FLOAT = "tuple[float]"


@dataclass(frozen=True)
class F:
    """One schema row."""

    name: str
    kind: Any
    default: Any
    choices: tuple | None = None
    cli_dest: str | None = None
    metavar: str | None = None
    ext: bool = False
    help: str = ""


OPTIMIZER_BACKENDS = ("auto", "deepspeed_zero2", "torch_adamw", "torch_fused_adamw",
                      "torch_distributed_adamw", "fsdp", "fsdp2", "zero_fused")
OBJECTIVES = ("standard_block_diffusion", "diffusiongemma_native_sft", "fast_dllm_v2",
              "dflash_distillation")
FAMILIES = ("causal_lm", "dflash", "diffusion_gemma", "nemotron_labs_diffusion", "qwen3_8")

SECTIONS: dict[str, tuple[F, ...]] = {
    "model": (
        F("id", str, "nvidia/Nemotron-Labs-Diffusion-3B", cli_dest="model_id"),
        F("revision", OPT_STR, None),
        F("family", str, "auto", choices=("auto", "hf") + FAMILIES, cli_dest="model_family"),
        F("seq_len", int, 1024),
        F("hidden_size", OPT_INT, None),
        F("num_layers", OPT_INT, None),
        F("num_attention_heads", OPT_INT, None),
        F("conditioning_dim", OPT_INT, None),
        F("vocab_size", OPT_INT, None),
        F("mask_token_id", OPT_INT, None),
        F("mask_token", OPT_STR, None),
        F("attention_backend", str, "flex", choices=("sdpa", "flex", "sm100")),
        F("dtype", str, "bf16", choices=("bf16", "fp16", "fp32")),
        F("trust_remote_code", bool, False),
        F("max_position_embeddings", OPT_INT, None),
        F("max_layers", OPT_INT, None),
        F("verifier_id", OPT_STR, None),
        F("verifier_revision", OPT_STR, None),
        F("target_layer_ids", TUPLE_INT, (), metavar="LAYER"),
        F("draft_vocab_path", OPT_STR, None),
        F("num_key_value_heads", OPT_INT, None, ext=True),
        F("head_dim", OPT_INT, None, ext=True),
        F("intermediate_size", OPT_INT, None, ext=True),
        F("rope_theta", OPT_FLOAT, None, ext=True),
        F("partial_rotary_factor", OPT_FLOAT, None, ext=True,
          help="share of each head's dimensions that rotary embeddings touch (1.0 = all)"),
        F("qk_norm", bool, True, ext=True),
        F("num_experts", OPT_INT, None, ext=True),
        F("num_experts_per_token", OPT_INT, None, ext=True),
        F("moe_intermediate_size", OPT_INT, None, ext=True),
        F("moe_shared_intermediate_size", OPT_INT, None, ext=True,
          help="width of the dense feed-forward every token passes beside its routed experts"),
        F("dflash2_conv_kernel_size", OPT_INT, None),
        F("dflash2_conv_group_size", OPT_INT, None),
        F("dflash2_selector_rank", OPT_INT, None),
        F("dflash2_selector_top_k", OPT_INT, None),
        F("full_attention_interval", OPT_INT, None, ext=True,
          help="hybrid decoders: every n-th layer is softmax attention, the others are linear attention"),
        F("linear_num_key_heads", OPT_INT, None, ext=True),
        F("linear_num_value_heads", OPT_INT, None, ext=True),
        F("linear_key_head_dim", OPT_INT, None, ext=True),
        F("linear_value_head_dim", OPT_INT, None, ext=True),
        F("linear_conv_kernel", OPT_INT, None, ext=True),
        F("sliding_window", OPT_INT, None, ext=True,
          help="window (clean positions) of the sliding-window layers"),
        F("sliding_window_pattern", OPT_INT, None, ext=True,
          help="every n-th layer attends to the full prefix, the others slide (0: every layer slides)"),
        F("random_init", bool, False, ext=True, help="build from the shape fields, load no weights"),
    ),
    "objective": (
        F("name", str, "standard_block_diffusion", choices=OBJECTIVES, cli_dest="objective_name"),
        F("block_size", OPT_INT, None),
        F("bp_loss_scale", OPT_FLOAT, None),
        F("skip_rng_steps", int, 0),
        F("noise_schedule", str, "loglinear", choices=("loglinear", "linear_mask")),
        F("loss_weighting", str, "inverse_move_chance", choices=("inverse_move_chance", "unit")),
        F("noise_schedule_epsilon", float, 1.0e-3),
        F("sampling_epsilon_min", float, 1.0e-3),
        F("sampling_epsilon_max", float, 1.0),
        F("antithetic_sampling", bool, True),
        F("self_conditioning_probability", float, 0.5),
        F("encoder_loss_weight", float, 1.0),
        F("minimum_decoder_blocks", int, 1),
        F("pack_response_suffix", bool, True, ext=True,
          help="diffusiongemma_native_sft: decoder rows cover the supervised response only, blocks counted from its start"),
        F("self_conditioning_row_chunk_size", int, 256),
        F("self_conditioning_vocab_chunk_size", int, 32768),
        F("max_anchors", OPT_INT, None),
        F("anchor_sampling", str, "uniform", choices=("uniform", "locality")),
        F("anchor_group_size", int, 0),
        F("sample_from_anchor", bool, False),
        F("dflash_loss", str, "speculators_kl", choices=("speculators_kl", "paper_ce", "dflash", "dpace", "dpace-cumulative-confidence-only",
                   "dpace-continuation-value-only")),
        F("decay_gamma", OPT_FLOAT, None),
        F("dpace_alpha", float, 0.5),
        F("lk_loss_type", OPT_STR, None),
        F("kl_scale", float, 1.0),
        F("kl_decay", float, 1.0),
        F("selector_loss_alpha", float, 1.0),
        F("selector_warmup_ratio", float, 0.0),
        F("selector_ramp_ratio", float, 0.0),
        F("selector_stop_gradient", bool, False),
        F("dflash_vocab_block_size", int, 32768),
    ),
    "data": (
        F("input_mode", str, "random", choices=("random", "text", "dataset")),
        F("vocab_sample_size", OPT_INT, None),
        F("dataset_path", OPT_STR, None),
        F("minimum_sequence_length", OPT_INT, None),
        F("blend_seed", int, 0),
        F("shuffle", bool, True),
        F("optimizer_step_unit", str, "microbatch", choices=("microbatch", "trajectory")),
        F("trajectory_loss_reduction", str, "token_mean", choices=("token_mean", "turn_mean")),
        F("trajectory_terminal_turn_weight", float, 1.0),
        F("target_features", OPT_STR, None, choices=(None, "offline", "synthetic", "online")),
        F("target_feature_path", OPT_STR, None),
    ),
    "training": (
        F("batch_size", int, 1),
        F("steps", int, 3),
        F("max_duration_seconds", OPT_FLOAT, None),
        F("gradient_accumulation_steps", int, 1),
        F("activation_checkpointing", bool, True),
        F("activation_checkpointing_scope", str, "full", choices=("full", "mlp")),
        F("skip_optimizer_step", bool, False),
    ),
    "evaluation": (
        F("dataset_path", OPT_STR, None, cli_dest="evaluation_dataset_path"),
        F("batches", int, 0, cli_dest="evaluation_batches"),
        F("seed", int, 314159, cli_dest="evaluation_seed"),
    ),
    "adapter": (
        F("type", str, "none", choices=("none", "lora"), cli_dest="adapter_type"),
        F("rank", OPT_INT, None, cli_dest="adapter_rank"),
        F("alpha", OPT_FLOAT, None, cli_dest="adapter_alpha"),
        F("dropout", float, 0.0, cli_dest="adapter_dropout"),
        F("targets", TUPLE_STR, (), cli_dest="adapter_target", metavar="ROLE"),
    ),
    "topology": (
        F("context_parallel_size", int, 4),
        F("block_parallel_size", int, 4),
        F("replicate_clean_prefix", bool, False),
        F("tensor_parallel_size", int, 1),
        F("expert_parallel_size", int, 1),
        F("sequence_parallel", bool, False),
        F("tensor_parallel_overlap", bool, True),
        F("placement_policy", str, "auto", choices=("auto", "inter_node_cp")),
        F("process_group_timeout_seconds", OPT_FLOAT, None),
        F("process_group_timeout", TUPLE_STR, (), metavar="GROUP=SECONDS"),
        F("pipeline_parallel_size", int, 1, ext=True),
    ),
    "optimizer": (
        F("backend", str, "auto", choices=OPTIMIZER_BACKENDS, cli_dest="optimizer_backend"),
        F("zero_optimizer_impl", str, "auto"),
        F("lr", float, 1.0e-6),
        F("adam_eps", float, 1.0e-5),
        F("adam_beta1", float, 0.9),
        F("adam_beta2", float, 0.999),
        F("weight_decay", float, 0.01),
        F("zero_param_group_max_elements", int, 0),
        F("zero_reduce_bucket_size", int, 0),
        F("zero_contiguous_gradients", bool, True),
        F("zero_overlap_comm", bool, True),
        F("gradient_clip_norm", float, 0.0),
        F("allow_deepspeed_op_build", bool, False),
        F("fsdp_mixed_precision", OPT_STR, None),
        F("fsdp_sharding_strategy", str, "full_shard",
          choices=("full_shard", "shard_grad_op", "hybrid_shard", "no_shard")),
        F("fsdp_use_orig_params", bool, True),
    ),
    "scheduler": (
        F("type", str, "constant", choices=("constant", "linear", "cosine", "inverse_square_root"),
          cli_dest="scheduler_type"),
        F("warmup_steps", int, 0, cli_dest="lr_warmup_steps"),
        F("decay_steps", OPT_INT, None, cli_dest="lr_decay_steps"),
        F("min_lr", float, 0.0),
        F("weight_decay_style", str, "constant", choices=("constant", "linear", "cosine")),
        F("weight_decay_start", OPT_FLOAT, None),
        F("weight_decay_end", OPT_FLOAT, None),
        F("weight_decay_steps", OPT_INT, None),
    ),
    "checkpointing": (
        F("save_checkpoint_dir", OPT_STR, None),
        F("save_checkpoint_interval", int, 0),
        F("keep_last_n", int, 0),
        F("load_checkpoint_dir", OPT_STR, None),
        F("checkpoint_tag", str, "latest"),
        F("auto_resume", bool, False),
        F("save_first_step", bool, False),
        F("save_final", bool, False),
        F("async_checkpoint_save", bool, False),
        F("model_only", bool, False),
        F("save_duration_fractions", TUPLE_FLOAT, (), cli_dest="save_duration_fraction"),
    ),
    "profiler": (
        F("warmup_steps", int, 0, cli_dest="profile_warmup_steps"),
        F("phase_timing", bool, False),
        F("phase_timing_sync", bool, False),
        F("system_trace", bool, False),
        F("system_trace_backend", str, "kineto", choices=("kineto", "nsys")),
        F("system_trace_dir", OPT_STR, None),
        F("system_trace_start_step", int, 1),
        F("system_trace_steps", int, 1),
    ),
    "logging": (
        F("wandb", bool, False),
        F("wandb_project", OPT_STR, None),
        F("wandb_entity", OPT_STR, None),
        F("wandb_name", OPT_STR, None),
        F("wandb_group", OPT_STR, None),
        F("wandb_id", OPT_STR, None),
        F("wandb_mode", str, "online", choices=("online", "offline", "disabled")),
        F("wandb_dir", OPT_STR, None),
        F("wandb_tags", TUPLE_STR, (), metavar="TAG"),
    ),
    "debug": (
        F("grad_finite", bool, False, cli_dest="debug_grad_finite"),
        F("optimizer_finite", bool, False, cli_dest="debug_optimizer_finite"),
        F("trace", bool, False, cli_dest="debug_trace"),
    ),
    "kernel": (
        F("ring_attention_key_chunk_size", int, 0),
        F("mlp_token_chunk_size", int, 0),
        F("cp_bp_attention_policy", str, "production"),
        F("cp_bp_clean_kv_layout", str, "zigzag", choices=("zigzag", "contiguous")),
        F("cp_bp_clean_kv_transport", str, "collective", choices=("collective", "streaming", "peer_pull", "fused")),
        F("cp_bp_share_clean_replicas", bool, True),
        F("pure_cp_token_split", bool, True),
        F("dflash_context_exchange", str, "auto", choices=("auto", "kv_pull", "query_rotation")),
        F("cp_bp_debug_nonfinite_attention", bool, False),
        F("runtime_jit", bool, False),
        F("impl", str, "auto", choices=("auto", "cpu_reference", "nccl_baseline", "sm100_fused"), ext=True),
    ),
    "launch": (
        F("seed", int, 2026),
        F("recipe_kind", str, "smoke", choices=("smoke", "profile", "prod")),
    ),
}

_PY_TYPES = {int: int, float: float, str: str, bool: bool, OPT_INT: "int | None", OPT_FLOAT: "float | None",
             OPT_STR: "str | None", TUPLE_STR: tuple, TUPLE_INT: tuple, TUPLE_FLOAT: tuple}


def _section_class(name: str, rows: tuple[F, ...]):
    cls_name = "".join(p.capitalize() for p in name.split("_")) + "RunSpec"
    fields = [(r.name, _PY_TYPES[r.kind], field(default=r.default, metadata={"row": r})) for r in rows]
    return dataclasses.make_dataclass(cls_name, fields, frozen=True)


SECTION_CLASSES = {name: _section_class(name, rows) for name, rows in SECTIONS.items()}


def coerce(row: F, value: Any, where: str) -> Any:
    """Converts a YAML/CLI value to the row's type or raises ValueError with the field path."""
    k = row.kind
    if value is None:
        if k in (OPT_INT, OPT_FLOAT, OPT_STR):
            return None
        raise ValueError(f"{where}: null is not allowed")
    try:
        if k is bool:
            if isinstance(value, bool):
                return value
            if isinstance(value, str) and value.lower() in ("true", "false", "1", "0", "yes", "no"):
                return value.lower() in ("true", "1", "yes")
            raise ValueError
        if k in (int, OPT_INT):
            if isinstance(value, bool) or (isinstance(value, float) and value != int(value)):
                raise ValueError
            return int(value)
        if k in (float, OPT_FLOAT):
            if isinstance(value, bool):
                raise ValueError
            return float(value)
        if k in (str, OPT_STR):
            if not isinstance(value, str):
                raise ValueError
            return value
        if k in (TUPLE_STR, TUPLE_INT, TUPLE_FLOAT):
            if isinstance(value, (str, int, float)):
                value = [value]
            conv = {TUPLE_STR: str, TUPLE_INT: int, TUPLE_FLOAT: float}[k]
            return tuple(conv(v) for v in value)
    except (TypeError, ValueError):
        pass
    raise ValueError(f"{where}: cannot interpret {value!r} as {k if isinstance(k, str) else k.__name__}")

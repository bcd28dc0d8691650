"""RunSpec: the typed train.yaml contract.

Fifteen frozen sections make one immutable `RunSpec`. Loading rejects unknown sections and
fields, coerces scalars, and `validate()` applies the cross-field rules (objective ↔ family,
topology divisibility, pure-BP needs a replicated clean prefix, sequence parallel needs TP>1,
production-recipe rules). Every field is also a CLI flag (`--kebab-case`, booleans as
`--x / --no-x`), generated from the schema table.

Same public contract as the reference (dllm_parallel/training/run_spec.py:255-899 RunSpec,
:902 load_run_spec, :911 run_spec_from_args, :1008-1063 arg parser); the implementation here
is table-driven (see `schema.py`).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping

import yaml

from . import schema as S
from .schema import SECTION_CLASSES, SECTIONS, coerce


class RunSpecError(ValueError):
    """A configuration problem the user can fix (CLI exit code 2)."""


def _default_sections() -> dict:
    return {name: cls() for name, cls in SECTION_CLASSES.items()}


@dataclass(frozen=True)
class RunSpec:
    model: Any = field(default_factory=SECTION_CLASSES["model"])
    objective: Any = field(default_factory=SECTION_CLASSES["objective"])
    data: Any = field(default_factory=SECTION_CLASSES["data"])
    training: Any = field(default_factory=SECTION_CLASSES["training"])
    evaluation: Any = field(default_factory=SECTION_CLASSES["evaluation"])
    adapter: Any = field(default_factory=SECTION_CLASSES["adapter"])
    topology: Any = field(default_factory=SECTION_CLASSES["topology"])
    optimizer: Any = field(default_factory=SECTION_CLASSES["optimizer"])
    scheduler: Any = field(default_factory=SECTION_CLASSES["scheduler"])
    checkpointing: Any = field(default_factory=SECTION_CLASSES["checkpointing"])
    profiler: Any = field(default_factory=SECTION_CLASSES["profiler"])
    logging: Any = field(default_factory=SECTION_CLASSES["logging"])
    debug: Any = field(default_factory=SECTION_CLASSES["debug"])
    kernel: Any = field(default_factory=SECTION_CLASSES["kernel"])
    launch: Any = field(default_factory=SECTION_CLASSES["launch"])

    # ------------------------------------------------------------------ build
    @classmethod
    def default(cls) -> "RunSpec":
        return cls()

    @classmethod
    def from_mapping(cls, mapping: Mapping[str, Any] | None) -> "RunSpec":
        mapping = dict(mapping or {})
        unknown = sorted(set(mapping) - set(SECTIONS))
        if unknown:
            raise RunSpecError(f"unknown run-spec section(s): {', '.join(unknown)}; "
                               f"known sections: {', '.join(SECTIONS)}")
        sections = {}
        for name, rows in SECTIONS.items():
            raw = mapping.get(name) or {}
            if not isinstance(raw, Mapping):
                raise RunSpecError(f"section '{name}' must be a mapping, got {type(raw).__name__}")
            by_name = {r.name: r for r in rows}
            bad = sorted(set(raw) - set(by_name))
            if bad:
                raise RunSpecError(f"unknown field(s) in section '{name}': {', '.join(bad)}")
            values = {}
            for key, value in raw.items():
                try:
                    values[key] = coerce(by_name[key], value, f"{name}.{key}")
                except ValueError as e:
                    raise RunSpecError(str(e)) from None
            sections[name] = SECTION_CLASSES[name](**values)
        return cls(**sections)

    def with_overrides(self, overrides: Mapping[str, Mapping[str, Any]]) -> "RunSpec":
        """overrides = {section: {field: value}}; unknown names raise."""
        merged = self.to_dict()
        for sec, fields_ in overrides.items():
            if sec not in merged:
                raise RunSpecError(f"unknown run-spec section: {sec}")
            merged[sec].update(fields_)
        return RunSpec.from_mapping(merged)

    def to_dict(self) -> dict:
        out = {}
        for name in SECTIONS:
            sec = getattr(self, name)
            out[name] = {f.name: (list(v) if isinstance(v := getattr(sec, f.name), tuple) else v)
                         for f in dataclasses.fields(sec)}
        return out

    def to_yaml(self) -> str:
        return yaml.safe_dump(self.to_dict(), sort_keys=False)

    # --------------------------------------------------------------- validate
    def validate(self, world_size: int | None = None) -> "RunSpec":
        problems: list[str] = []

        def need(cond: bool, msg: str) -> None:
            if not cond:
                problems.append(msg)

        for name, rows in SECTIONS.items():
            sec = getattr(self, name)
            for r in rows:
                v = getattr(sec, r.name)
                if r.choices is not None and v not in r.choices:
                    problems.append(f"{name}.{r.name}={v!r} is not one of "
                                    f"{[c for c in r.choices if c is not None]}")
        m, o, t, tr, opt = self.model, self.objective, self.topology, self.training, self.optimizer
        need(m.seq_len > 0, "model.seq_len must be positive")
        for fname in ("context_parallel_size", "block_parallel_size", "tensor_parallel_size",
                      "expert_parallel_size", "pipeline_parallel_size"):
            need(getattr(t, fname) >= 1, f"topology.{fname} must be >= 1")
        need(t.pipeline_parallel_size == 1,
             "topology.pipeline_parallel_size must be 1: pipeline parallelism is an axis of the "
             "topology but has no schedule")
        cp, bp = t.context_parallel_size, t.block_parallel_size
        if bp > 1 and cp > 1:
            need(bp >= cp and bp % cp == 0,
                 f"fused CP+BP needs block_parallel_size ({bp}) to be a multiple of "
                 f"context_parallel_size ({cp})")
        if bp > 1 and cp == 1:
            need(t.replicate_clean_prefix,
                 "pure block parallelism (context_parallel_size=1) needs topology.replicate_clean_prefix=true")
        if t.replicate_clean_prefix:
            need(cp == 1, "topology.replicate_clean_prefix is only meaningful with context_parallel_size=1")
        need(not t.sequence_parallel or t.tensor_parallel_size > 1,
             "topology.sequence_parallel needs tensor_parallel_size > 1")
        if o.block_size is not None:
            need(o.block_size > 0, "objective.block_size must be positive")
            if o.block_size > 0 and o.name != "dflash_distillation":
                need(m.seq_len % o.block_size == 0,
                     f"model.seq_len ({m.seq_len}) must be a multiple of objective.block_size ({o.block_size})")
                if m.seq_len % o.block_size == 0 and bp > 1:
                    need(m.seq_len // o.block_size >= bp,
                         f"block_parallel_size ({bp}) exceeds the number of blocks "
                         f"({m.seq_len // o.block_size})")
        elif o.name in ("standard_block_diffusion", "fast_dllm_v2", "diffusiongemma_native_sft"):
            problems.append(f"objective.block_size is required for {o.name}")
        if o.name == "diffusiongemma_native_sft":
            need(o.noise_schedule == "loglinear", "diffusiongemma_native_sft requires objective.noise_schedule=loglinear")
            need(o.loss_weighting == "unit", "diffusiongemma_native_sft requires objective.loss_weighting=unit")
            need(0.0 <= o.self_conditioning_probability <= 1.0,
                 "objective.self_conditioning_probability must be in [0, 1]")
            need(o.self_conditioning_row_chunk_size > 0 and o.self_conditioning_vocab_chunk_size > 0,
                 "objective.self_conditioning_row_chunk_size / vocab_chunk_size must be positive")
        need(m.max_position_embeddings is None or m.seq_len <= m.max_position_embeddings,
             f"model.seq_len ({m.seq_len}) exceeds model.max_position_embeddings ({m.max_position_embeddings})")
        need(0.0 < o.sampling_epsilon_min <= o.sampling_epsilon_max <= 1.0,
             "objective.sampling_epsilon_min/max must satisfy 0 < min <= max <= 1")
        need(0.0 <= o.noise_schedule_epsilon < 1.0, "objective.noise_schedule_epsilon must be in [0, 1)")
        need(tr.batch_size >= 1 and tr.gradient_accumulation_steps >= 1 and tr.steps >= 0,
             "training.batch_size / gradient_accumulation_steps must be >= 1 and steps >= 0")
        need(opt.lr > 0 and 0 <= opt.adam_beta1 < 1 and 0 <= opt.adam_beta2 < 1 and opt.adam_eps > 0,
             "optimizer.lr, adam_beta1/2 and adam_eps out of range")
        need(opt.gradient_clip_norm >= 0, "optimizer.gradient_clip_norm must be >= 0")
        if opt.backend in ("fsdp", "fsdp2"):
            # parameter sharding: per-layer gather / reduce hooks sit on the checkpointed layer boundary
            need(tr.activation_checkpointing, "optimizer.backend=fsdp needs training.activation_checkpointing")
            need(self.adapter.type == "none", "optimizer.backend=fsdp shards the base model: adapters use the "
                                              "sharded-optimizer backends (auto, zero_fused, torch_*)")
            need(o.name != "dflash_distillation",
                 "optimizer.backend=fsdp is built for the dense decoder and the mixture-of-experts decoder (its "
                 "replicated part; the experts are divided by expert parallelism)")
        if self.data.optimizer_step_unit == "trajectory":
            need(self.data.input_mode == "dataset", "data.optimizer_step_unit=trajectory needs an indexed dataset "
                                                    "with trajectory groups (data.input_mode=dataset)")
        if self.data.trajectory_loss_reduction == "turn_mean":
            need(self.data.optimizer_step_unit == "trajectory",
                 "data.trajectory_loss_reduction=turn_mean applies to data.optimizer_step_unit=trajectory")
        if m.family not in ("auto", "hf"):
            from ..models.registry import objectives_for_family

            allowed = objectives_for_family(m.family)
            need(o.name in allowed, f"objective {o.name} is not supported by family {m.family} "
                                    f"(supported: {', '.join(allowed)})")
        # settings of other stacks' backends that nothing here reads: a value other than the default would be
        # silently ignored, so it is refused
        for section, name, default, why in (
                ("optimizer", "zero_optimizer_impl", "auto", "the sharded AdamW of this package is the only implementation"),
                ("optimizer", "zero_param_group_max_elements", 0, "the optimizer works on one flat buffer"),
                ("optimizer", "zero_reduce_bucket_size", 0, "gradients are reduced as one flat buffer (or per layer under fsdp)"),
                ("optimizer", "zero_contiguous_gradients", True, "gradients always live in one contiguous buffer"),
                ("optimizer", "zero_overlap_comm", True, "the fused step orders its own phases"),
                ("optimizer", "allow_deepspeed_op_build", False, "no DeepSpeed ops are built or used"),
                ("optimizer", "fsdp_sharding_strategy", "full_shard", "parameter sharding is always full sharding over the data-parallel group"),
                ("optimizer", "fsdp_use_orig_params", True, "parameters are views of flat buffers"),
                ("kernel", "ring_attention_key_chunk_size", 0, "key tiles are streamed by the attention kernel itself"),
                ("kernel", "cp_bp_attention_policy", "production", "one attention policy is built")):
            v = getattr(getattr(self, section), name)
            need(v == default, f"{section}.{name}={v!r} has no effect here ({why}); leave it at {default!r}")
        if tr.activation_checkpointing_scope == "mlp":
            # the attention half keeps its autograd graph, the feed-forward half is recomputed
            need(tr.activation_checkpointing, "training.activation_checkpointing_scope=mlp needs training.activation_checkpointing")
            need(m.family not in ("qwen3_8", "diffusion_gemma", "dflash") and t.tensor_parallel_size == 1
                 and opt.backend not in ("fsdp", "fsdp2") and self.adapter.type != "lora",
                 "training.activation_checkpointing_scope=mlp is built for the dense decoder without tensor parallelism, "
                 "parameter sharding or adapters; use 'full'")
        need(opt.fsdp_mixed_precision in (None, "bf16"),
             f"optimizer.fsdp_mixed_precision={opt.fsdp_mixed_precision!r}: parameter shards are bf16 with fp32 gradients "
             "and master weights (leave it unset, or 'bf16')")
        need(self.kernel.mlp_token_chunk_size >= 0 and self.kernel.mlp_token_chunk_size % 128 == 0,
             "kernel.mlp_token_chunk_size must be 0 (off) or a multiple of 128 rows")
        if self.kernel.mlp_token_chunk_size:
            need(t.tensor_parallel_size == 1 and m.family not in ("qwen3_8", "diffusion_gemma", "dflash"),
                 "kernel.mlp_token_chunk_size applies to the dense decoder on one tensor-parallel rank")
        if o.bp_loss_scale is not None:
            need(abs(float(o.bp_loss_scale) - float(bp if bp > 1 else 1)) < 1e-6,
                 f"objective.bp_loss_scale={o.bp_loss_scale} differs from the block-parallel degree {bp if bp > 1 else 1}: "
                 "gradients are summed over ranks and divided by the global token count, so no other scale applies")
        if m.draft_vocab_path:
            need(o.name == "dflash_distillation" and o.dflash_loss in ("speculators_kl", "paper_ce")
                 and not (m.dflash2_conv_kernel_size or m.dflash2_selector_rank),
                 "model.draft_vocab_path (a drafter over a subset of the verifier's vocabulary) is built for the DFlash "
                 "drafter with objective.dflash_loss speculators_kl or paper_ce")
        if o.name == "dflash_distillation":
            need(cp == 1 or bp == 1 or cp == bp,
                 "dflash_distillation divides anchors (block parallelism) and context rows (context parallelism) over the "
                 "ranks of one replica: context_parallel_size and block_parallel_size must be equal, or one of them 1")
            need(t.tensor_parallel_size == 1, "dflash_distillation has no tensor-parallel drafter")
            n_rep = bp
            if o.max_anchors:
                need(o.max_anchors % n_rep == 0, f"objective.max_anchors ({o.max_anchors}) must divide by the "
                                                 f"{n_rep} ranks of a replica")
            need(bool(m.target_layer_ids), "dflash_distillation needs model.target_layer_ids")
            need(self.data.target_features in ("offline", "synthetic", "online"),
                 "dflash_distillation needs data.target_features (offline, synthetic or online)")
            if self.data.target_features == "offline":
                need(bool(self.data.target_feature_path), "data.target_features=offline needs data.target_feature_path")
        if self.adapter.type == "lora":
            need((self.adapter.rank or 0) > 0, "adapter.rank must be positive for LoRA")
            bad = sorted(set(self.adapter.targets) - {"attention", "mlp", "experts"})
            need(not bad, f"adapter.targets has unknown roles: {bad}")
        if self.data.input_mode == "dataset" and not (o.name == "dflash_distillation"
                                                       and self.data.target_features in ("offline", "synthetic")):
            # (a drafter trained from stored or synthetic target features takes its token ids from there)
            need(bool(self.data.dataset_path), "data.input_mode=dataset needs data.dataset_path (a prepared artifact "
                                               "directory, a flat token file, or a text file)")
        ck = self.checkpointing
        need(ck.save_checkpoint_interval >= 0 and ck.keep_last_n >= 0, "checkpointing intervals must be >= 0")
        if ck.save_checkpoint_interval or ck.save_first_step or ck.save_final or ck.save_duration_fractions:
            need(bool(ck.save_checkpoint_dir), "checkpoint saving is enabled but checkpointing.save_checkpoint_dir is unset")
        for frac in ck.save_duration_fractions:
            need(0.0 < frac <= 1.0, f"checkpointing.save_duration_fractions entry {frac} not in (0, 1]")
        if ck.save_duration_fractions:
            need(tr.max_duration_seconds is not None,
                 "checkpointing.save_duration_fractions needs training.max_duration_seconds")
        for item in t.process_group_timeout:
            name, _, secs = item.partition("=")
            ok = bool(name) and bool(secs)
            try:
                ok = ok and float(secs) > 0
            except ValueError:
                ok = False
            need(ok, f"topology.process_group_timeout entry {item!r} is not GROUP=SECONDS")
        if self.launch.recipe_kind == "prod":
            need(not tr.skip_optimizer_step, "production recipes must not skip the optimizer step")
            need(not self.debug.trace, "production recipes must not enable debug.trace")
            need(self.data.input_mode != "random", "production recipes need real data (data.input_mode != random)")
            need(bool(ck.save_checkpoint_dir), "production recipes must configure checkpointing.save_checkpoint_dir")
        if world_size is not None:
            from ..parallel.topology import infer_data_parallel_size

            try:
                infer_data_parallel_size(world_size, self)
            except ValueError as e:
                problems.append(str(e))
        if not problems:
            # what the model family's executor cannot run (e.g. a parallel axis it does not build) is a problem of
            # the run spec too: `dllm config validate` reports it, not only the training start
            problems += self._family_problems(world_size)
        if problems:
            raise RunSpecError("invalid run spec:\n  - " + "\n  - ".join(problems))
        return self

    def _family_problems(self, world_size: int | None) -> list[str]:
        from ..models.config import PRESETS
        from ..models.registry import executor_for_family, infer_family

        m = self.model
        fam = m.family
        if fam in ("auto", "hf"):
            if self.objective.name == "dflash_distillation":
                fam = "dflash"
            else:
                cfg = PRESETS.get(m.id)
                if cfg is None and (m.num_experts or m.full_attention_interval):
                    fam = "diffusion_gemma" if m.num_experts else "qwen3_8"
                elif cfg is not None and (cfg.is_hybrid or m.full_attention_interval):
                    fam = "qwen3_8"
                elif cfg is not None and (cfg.is_moe or m.num_experts):
                    fam = "diffusion_gemma"
                else:
                    fam = (cfg.family if cfg is not None and cfg.family != "causal_lm" else None) or infer_family(m.id, self.objective.name)
        try:
            return list(executor_for_family(fam).validate_run_spec(self, world_size))
        except ValueError as e:
            return [str(e)]

    # ------------------------------------------------------------ conveniences
    @property
    def local_parallel_size(self) -> int:
        return max(self.topology.context_parallel_size, self.topology.block_parallel_size)

    def model_parallel_size(self) -> int:
        t = self.topology
        return (self.local_parallel_size * t.tensor_parallel_size * t.expert_parallel_size
                * t.pipeline_parallel_size)

    def global_batch(self, data_parallel_size: int) -> int:
        """global batch = batch_size × gradient accumulation × data-parallel size."""
        return self.training.batch_size * self.training.gradient_accumulation_steps * data_parallel_size


def load_run_spec(path: str | Path) -> RunSpec:
    p = Path(path)
    if not p.exists():
        raise RunSpecError(f"run spec not found: {p}")
    text = p.read_text()
    try:
        data = json.loads(text) if p.suffix == ".json" else yaml.safe_load(text)
    except Exception as e:
        raise RunSpecError(f"cannot parse {p}: {e}") from None
    if data is not None and not isinstance(data, Mapping):
        raise RunSpecError(f"{p}: top level must be a mapping of sections")
    return RunSpec.from_mapping(data)


# ---------------------------------------------------------------------- CLI
def _flag(row: S.F, section: str) -> tuple[str, str]:
    dest = row.cli_dest or row.name
    return "--" + dest.replace("_", "-"), f"{section}__{row.name}"


def build_run_spec_arg_parser(prog: str = "dllm-train") -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog=prog, description="Train a block-diffusion model from a RunSpec")
    ap.add_argument("--config", help="train.yaml / .json run spec")
    ap.add_argument("--validate-only", action="store_true", help="validate the merged spec and exit")
    ap.add_argument("--print-supported-configs", action="store_true")
    ap.add_argument("--print-config", action="store_true", help="print the merged spec as YAML and exit")
    seen: dict[str, str] = {}
    for section, rows in SECTIONS.items():
        grp = ap.add_argument_group(section)
        for r in rows:
            flag, dest = _flag(r, section)
            if flag in seen:  # same field name in two sections: prefix with the section
                flag = f"--{section}-{r.name}".replace("_", "-")
            seen[flag] = dest
            kw: dict[str, Any] = dict(dest=dest, default=None, help=r.help or None)
            if r.kind is bool:
                grp.add_argument(flag, action=argparse.BooleanOptionalAction, **kw)
            elif r.kind in (S.TUPLE_STR, S.TUPLE_INT, S.TUPLE_FLOAT):
                grp.add_argument(flag, nargs="*", metavar=r.metavar, **kw)
            else:
                grp.add_argument(flag, metavar=r.metavar, **kw)
    return ap


def run_spec_from_args(args: argparse.Namespace) -> RunSpec:
    spec = load_run_spec(args.config) if getattr(args, "config", None) else RunSpec.default()
    overrides: dict[str, dict[str, Any]] = {}
    for section, rows in SECTIONS.items():
        for r in rows:
            v = getattr(args, f"{section}__{r.name}", None)
            if v is None:
                continue
            if isinstance(v, str) and v.lower() in ("none", "null") and r.kind in (S.OPT_INT, S.OPT_FLOAT, S.OPT_STR):
                v = None
            overrides.setdefault(section, {})[r.name] = v
    return spec.with_overrides(overrides) if overrides else spec


def describe_supported_configs() -> dict:
    from ..models.registry import describe_supported_configs as d

    return d()

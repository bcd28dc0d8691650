"""Export CLIs: merged Hugging Face checkpoints from training checkpoints (dense and MoE models,
LoRA adapters folded in), and DFlash drafter exports for speculative-decoding servers.

`dllm-export-diffusiongemma --checkpoint DIR --config train.yaml --output OUT` rebuilds the model
from the run spec, loads rank 0's shard and writes `OUT/config.json` + safetensors plus an
`export_manifest.json` with SHA-256 of every file. The DFlash export adds `dflash_config.json`
(block size, target layer ids, mask token id, draft vocabulary) next to the drafter weights.

Counterparts: dllm_parallel/core/models/backbones/diffusiongemma/export.py:63-449, :1130 (CLI);
dllm_parallel/core/models/backbones/dflash/executor.py:412-566 (speculators / SGLang export + validation).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

import torch


def _sha(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for c in iter(lambda: f.read(1 << 20), b""):
            h.update(c)
    return h.hexdigest()


def write_export_manifest(out: str, extra: dict | None = None) -> dict:
    files = {f: {"bytes": os.path.getsize(os.path.join(out, f)), "sha256": _sha(os.path.join(out, f))}
             for f in sorted(os.listdir(out)) if f != "export_manifest.json"}
    man = {"format": "turbo_dllm_b200.export.v1", "files": files, **(extra or {})}
    json.dump(man, open(os.path.join(out, "export_manifest.json"), "w"), indent=1, sort_keys=True)
    return man


def export_training_checkpoint(spec, checkpoint_dir: str, output: str, tag: str = "latest") -> dict:
    """Training checkpoint -> Hugging Face layout (adapters merged by a checked plan), on one process."""
    from . import hf_loader

    device = "cpu" if spec.model.dtype == "fp32" or not torch.cuda.is_available() else "cuda"
    restore = hf_loader.EXPORT_DTYPE
    if device == "cpu" and spec.model.dtype != "fp32":
        # no GPU here: the model is rebuilt in fp32 (what the CPU path computes in) and written in the run's dtype
        hf_loader.EXPORT_DTYPE = {"bf16": torch.bfloat16, "fp16": torch.float16}[spec.model.dtype]
        spec = spec.with_overrides({"model": {"dtype": "fp32"}})
    try:
        return _export_training_checkpoint(spec, checkpoint_dir, output, tag, device)
    finally:
        hf_loader.EXPORT_DTYPE = restore


def _export_training_checkpoint(spec, checkpoint_dir: str, output: str, tag: str, device: str) -> dict:
    from ..checkpoint import load_model_weights, load_training_checkpoint, read_metadata
    from ..training.session import TrainingSession
    from .hf_loader import export_hf_checkpoint

    if int(read_metadata(checkpoint_dir)["world_size"]) > 1:
        # written by several ranks, exported by one process: the model is rebuilt on one rank (no parallel axes) and
        # only the weights are read, from rank 0's file or from every rank's parameter slices
        solo = spec.with_overrides({"topology": {"context_parallel_size": 1, "block_parallel_size": 1,
                                                 "tensor_parallel_size": 1, "expert_parallel_size": 1,
                                                 "sequence_parallel": False},
                                    "optimizer": {"backend": "auto"}})
        session = TrainingSession(solo, device=device)
        meta = load_model_weights(checkpoint_dir, tag, session)
    else:
        session = TrainingSession(spec, device=device)
        meta = load_training_checkpoint(checkpoint_dir, tag, session, rank=0, world_size=1, restore_rng=False)
    from ..adapters.lora import lora_merge_plan

    plan = lora_merge_plan(session.model)        # validated before anything is merged or written
    if session.cfg.is_moe:
        export_moe_checkpoint(session.model, output)
    else:
        export_hf_checkpoint(session.model, output)
    return write_export_manifest(output, {"step": meta["step"], "source_checkpoint": os.path.abspath(checkpoint_dir),
                                          "merged_adapters": plan})


@torch.no_grad()
def export_moe_checkpoint(model, path: str) -> str:
    """Dense parts in HF naming, experts as `model.layers.i.mlp.experts.{e}.{gate,up,down}_proj.weight`."""
    from safetensors.torch import save_file

    from .hf_loader import deinterleave_gate_up, hf_config_dict

    cfg = model.cfg
    if getattr(model, "lora", None) is not None:      # adapters (replicated and per-expert) go into the weights
        from ..adapters.lora import lora_merge_plan, merge_lora

        lora_merge_plan(model)
        merge_lora(model)
        for layer in model.layers:
            layer.lora = None
            layer.experts.lora = None
        model.lora = None
    from .hf_loader import _apply_partial_rotary_order

    bank0 = model.layers[0].experts
    experts = None
    if bank0.ep > 1:
        # expert parallelism: every rank of the expert group calls this; the experts are gathered in global order
        # (rank r owns experts [r * E_local, (r + 1) * E_local)) and the first rank of the group writes
        import torch.distributed as dist

        experts = []
        for layer in model.layers:
            b = layer.experts
            gu = [torch.empty_like(b.w_gu) for _ in range(b.ep)]
            dn = [torch.empty_like(b.w_down) for _ in range(b.ep)]
            dist.all_gather(gu, b.w_gu.detach().contiguous(), group=b.ep_group)
            dist.all_gather(dn, b.w_down.detach().contiguous(), group=b.ep_group)
            experts.append((torch.cat(gu).cpu(), torch.cat(dn).cpu()))
        if bank0.ep_rank != 0:
            dist.barrier(group=bank0.ep_group)
            return path
    os.makedirs(path, exist_ok=True)
    _apply_partial_rotary_order(model, inverse=True)
    try:
        return _write_moe_checkpoint(model, cfg, path, experts)
    finally:
        _apply_partial_rotary_order(model, inverse=False)
        if experts is not None:
            import torch.distributed as dist

            dist.barrier(group=bank0.ep_group)


@torch.no_grad()
def _write_moe_checkpoint(model, cfg, path: str, experts=None) -> str:
    """experts: per layer (gate_up [E, 2I, H], down [E, H, I]) gathered over the expert-parallel ranks, or None when this
    rank holds every expert."""
    from safetensors.torch import save_file

    from .hf_loader import deinterleave_gate_up, hf_config_dict

    out = {"model.embed_tokens.weight": model.embed, "model.norm.weight": model.final_norm}
    if not cfg.tie_word_embeddings:
        out["lm_head.weight"] = model.lm_head
    for i, layer in enumerate(model.layers):
        p = f"model.layers.{i}."
        qd, kd = cfg.q_dim, cfg.kv_dim
        if layer.w_gate_up is not None:      # the dense feed-forward beside the experts
            g, u = deinterleave_gate_up(layer.w_gate_up)
            out[p + "mlp.shared_expert.gate_proj.weight"], out[p + "mlp.shared_expert.up_proj.weight"] = g, u
            out[p + "mlp.shared_expert.down_proj.weight"] = layer.w_down
        out[p + "self_attn.q_proj.weight"], out[p + "self_attn.k_proj.weight"] = layer.w_qkv[:qd], layer.w_qkv[qd:qd + kd]
        out[p + "self_attn.v_proj.weight"], out[p + "self_attn.o_proj.weight"] = layer.w_qkv[qd + kd:], layer.w_o
        out[p + "input_layernorm.weight"], out[p + "post_attention_layernorm.weight"] = layer.input_norm, layer.post_norm
        if layer.q_norm is not None:
            out[p + "self_attn.q_norm.weight"], out[p + "self_attn.k_norm.weight"] = layer.q_norm, layer.k_norm
        out[p + "mlp.router.weight"] = layer.experts.router
        w_gu, w_down = experts[i] if experts is not None else (layer.experts.w_gu, layer.experts.w_down)
        for e in range(w_gu.shape[0]):
            g, u = deinterleave_gate_up(w_gu[e])
            q = p + f"mlp.experts.{e}."
            out[q + "gate_proj.weight"], out[q + "up_proj.weight"], out[q + "down_proj.weight"] = g, u, w_down[e]
    from .hf_loader import _stored

    save_file({k: _stored(v) for k, v in out.items()}, os.path.join(path, "model.safetensors"))
    c = hf_config_dict(cfg)
    c.update({"num_experts": cfg.num_experts, "num_experts_per_tok": cfg.num_experts_per_token,
              "moe_intermediate_size": cfg.moe_intermediate_size,
              "shared_expert_intermediate_size": cfg.moe_shared_intermediate_size, "model_type": "turbo_dllm_moe"})
    json.dump(c, open(os.path.join(path, "config.json"), "w"), indent=1)
    return path


@torch.no_grad()
def export_dflash_drafter(draft_model, spec, path: str) -> dict:
    """Drafter weights (flat parameter names) + dflash_config.json for SGLang / vLLM draft loading."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    from .hf_loader import _stored

    tensors = {name: _stored(p) for name, p in draft_model.flat.params.items()}
    if hasattr(draft_model, "candidate_selector"):
        return _export_dflash2_drafter(draft_model, spec, path, tensors)
    cfg = draft_model.cfg
    draft_vocab_size = cfg.vocab_size
    if spec.model.draft_vocab_path:      # the vocabulary subset travels with the drafter (t2d / d2t)
        from .dflash import DraftVocabulary

        dv = DraftVocabulary.load(spec.model.draft_vocab_path, cfg.vocab_size)
        tensors["t2d"], tensors["d2t"] = dv.t2d.contiguous(), dv.d2t.contiguous()
        draft_vocab_size = dv.size
    save_file(tensors, os.path.join(path, "model.safetensors"))
    json.dump({"architectures": ["DFlashDraftModel"], "model_type": "dflash", "hidden_size": cfg.hidden_size,
               "draft_vocab_size": draft_vocab_size,
               "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_attention_heads,
               "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
               "intermediate_size": cfg.intermediate_size, "vocab_size": cfg.vocab_size,
               "block_size": spec.objective.block_size, "target_layer_ids": list(spec.model.target_layer_ids),
               "conditioning_dim": draft_model.conditioning_dim, "mask_token_id": cfg.mask_token_id,
               "verifier": spec.model.verifier_id, "gate_up_layout": "interleaved", **_sliding_window_fields(cfg)},
              open(os.path.join(path, "dflash_config.json"), "w"), indent=1)
    return write_export_manifest(path, {"kind": "dflash_drafter"})


def _speculators_tensor_names(cfg) -> dict[str, tuple]:
    """Module-style tensor name -> (flat parameter name, how to cut it) for a DFlash drafter."""
    names = {"fc.weight": ("fc", None), "hidden_norm.weight": ("hidden_norm", None), "norm.weight": ("final_norm", None)}
    kd = cfg.kv_dim
    for i in range(cfg.num_layers):
        f, m = f"layers.{i}.", f"layers.{i}."
        names.update({
            m + "input_layernorm.weight": (f + "input_norm", None),
            m + "post_attention_layernorm.weight": (f + "post_norm", None),
            m + "self_attn.q_proj.weight": (f + "w_q", None), m + "self_attn.o_proj.weight": (f + "w_o", None),
            m + "self_attn.k_proj.weight": (f + "w_kv", ("rows", 0, kd)),
            m + "self_attn.v_proj.weight": (f + "w_kv", ("rows", kd, 2 * kd)),
            m + "mlp.gate_proj.weight": (f + "w_gate_up", ("stride", 0)),
            m + "mlp.up_proj.weight": (f + "w_gate_up", ("stride", 1)),
            m + "mlp.down_proj.weight": (f + "w_down", None)})
        if cfg.qk_norm:
            names[m + "self_attn.q_norm.weight"] = (f + "q_norm", None)
            names[m + "self_attn.k_norm.weight"] = (f + "k_norm", None)
    return names


def _cut(t: torch.Tensor, how):
    if how is None:
        return t
    if how[0] == "rows":
        return t[how[1]:how[2]]
    return t[how[1]::2]          # gate and up rows alternate in the fused weight


@torch.no_grad()
def export_speculators_checkpoint(draft_model, target, spec, path: str) -> dict:
    """A DFlash drafter as a self-contained speculative-decoding checkpoint: module-style tensor names
    (`layers.i.self_attn.q_proj.weight`, `fc.weight`, ...), the verifier's embedding and output head it drafts
    with (the head's rows of the draft vocabulary when `model.draft_vocab_path` is set, plus `t2d` / `d2t`), and a
    config.json with a `speculators_config` section naming the verifier and the proposal length
    (dllm_parallel/core/models/backbones/dflash/executor.py:412-455). `target`: the FrozenTarget of the run."""
    from safetensors.torch import save_file

    if hasattr(draft_model, "candidate_selector"):
        raise ValueError("the DFlash2 drafter has its own export (export_dflash_drafter)")
    cfg = draft_model.cfg
    os.makedirs(path, exist_ok=True)
    flat = draft_model.flat.params
    from .hf_loader import _stored

    tensors = {name: _stored(_cut(flat[src], how)) for name, (src, how) in _speculators_tensor_names(cfg).items()}
    head = _stored(target.lm_head)
    draft_vocab_size = int(head.shape[0])
    if spec.model.draft_vocab_path:
        from .dflash import DraftVocabulary

        dv = DraftVocabulary.load(spec.model.draft_vocab_path, head.shape[0])
        head, draft_vocab_size = dv.head_rows(head), dv.size
        tensors["t2d"], tensors["d2t"] = dv.t2d.contiguous(), dv.d2t.contiguous()
    tensors["embed_tokens.weight"] = _stored(target.embed)
    tensors["lm_head.weight"] = head.contiguous()
    tmp = os.path.join(path, ".model.safetensors.tmp")
    save_file(tensors, tmp)
    os.replace(tmp, os.path.join(path, "model.safetensors"))
    block = int(spec.objective.block_size or 16)
    # with sample_from_anchor the block's first slot is a prediction too; otherwise the anchor is the bonus token
    speculative = block if spec.objective.sample_from_anchor else block - 1
    config = {"architectures": ["DFlashDraftModel"], "model_type": "dflash", "hidden_size": cfg.hidden_size,
              "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_attention_heads,
              "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "qk_norm": cfg.qk_norm,
              "intermediate_size": cfg.intermediate_size, "vocab_size": int(target.lm_head.shape[0]),
              "draft_vocab_size": draft_vocab_size, "target_hidden_size": int(target.cfg.hidden_size),
              "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_norm_eps, "hidden_act": "silu",
              "block_size": block, "mask_token_id": cfg.mask_token_id, "sample_from_anchor": bool(spec.objective.sample_from_anchor),
              "aux_hidden_state_layer_ids": list(spec.model.target_layer_ids),
              "dflash_config": {"block_size": block, "target_layer_ids": list(spec.model.target_layer_ids),
                                "mask_token_id": cfg.mask_token_id},
              "speculators_model_type": "dflash",
              "speculators_config": {"algorithm": "dflash", "default_proposal_method": "greedy",
                                     "proposal_methods": [{"proposal_type": "greedy", "speculative_tokens": speculative}],
                                     "verifier": {"name_or_path": spec.model.verifier_id,
                                                  "architectures": ["Qwen3ForCausalLM"]}},
              **_sliding_window_fields(cfg)}
    tmp = os.path.join(path, ".config.json.tmp")
    with open(tmp, "w") as f:
        f.write(json.dumps(config, indent=2, sort_keys=True) + "\n")
    os.replace(tmp, os.path.join(path, "config.json"))
    return write_export_manifest(path, {"kind": "dflash_speculators", "tensor_count": len(tensors)})


@torch.no_grad()
def load_speculators_checkpoint(draft_model, path: str) -> dict:
    """Fills a DFlash drafter from a checkpoint in the layout `export_speculators_checkpoint` writes (to continue
    training a published drafter); returns its config. Shapes are checked tensor by tensor."""
    from safetensors import safe_open

    cfg = draft_model.cfg
    config = json.load(open(os.path.join(path, "config.json")))
    flat = draft_model.flat.params
    with safe_open(os.path.join(path, "model.safetensors"), framework="pt") as f:
        have = set(f.keys())
        for name, (dst, how) in _speculators_tensor_names(cfg).items():
            if name not in have:
                raise KeyError(f"{path} lacks {name}")
            t = f.get_tensor(name)
            view = _cut(flat[dst], how)
            if tuple(view.shape) != tuple(t.shape):
                raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)}, drafter expects {tuple(view.shape)}")
            view.copy_(t.to(view.device, view.dtype))
    return config


def _sliding_window_fields(cfg) -> dict:
    """Sliding-window settings of a drafter for the serving stack: window, per-layer kinds, and that a drafting
    block's own tokens see each other in both directions in every layer (as they do in training here)."""
    if not cfg.has_sliding_layers:
        return {}
    return {"sliding_window": int(cfg.sliding_window), "sliding_window_non_causal": True,
            "layer_types": ["sliding_attention" if cfg.layer_window(i) is not None else "full_attention"
                            for i in range(cfg.num_layers)]}


def dflash2_serving_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    """Tensor inventory a DFlash2 export must hold, from its config (no verifier tensors: embeddings and
    the output head are the target model's and are loaded by the serving stack)."""
    m = config["dflash_config"]
    h, L = config["hidden_size"], config["num_hidden_layers"]
    q = config["num_attention_heads"] * config["head_dim"]
    kv = config["num_key_value_heads"] * config["head_dim"]
    taps, groups = m["conv_kernel_size"], h // m["conv_group_size"]
    shapes = {"fc": (h, config["conditioning_dim"]), "hidden_norm": (h,), "final_norm": (h,),
              "selector_predecessor": (config["vocab_size"], m["selector_rank"]),
              "selector_successor": (config["vocab_size"], m["selector_rank"]),
              "selector_proj": (m["selector_rank"], h)}
    for i in range(L):
        p = f"layers.{i}."
        shapes.update({p + "input_norm": (h,), p + "post_norm": (h,), p + "w_q": (q, h), p + "w_kv": (2 * kv, h),
                       p + "w_o": (h, q), p + "w_gate_up": (2 * config["intermediate_size"], h),
                       p + "w_down": (h, config["intermediate_size"])})
        if config.get("qk_norm", True):
            shapes.update({p + "q_norm": (config["head_dim"],), p + "k_norm": (config["head_dim"],)})
        for c in ("attn_conv", "mlp_conv"):
            shapes.update({p + c + "_base": (2, taps, h), p + c + "_proj": (2 * taps * groups, h)})
    return shapes


def normalize_dflash2_config(config: dict, expected_block_size: int | None = None) -> dict:
    """Checks the fields a DFlash2 serving loader needs and returns a standalone copy
    (dllm_parallel/core/models/backbones/dflash/executor.py:465-514)."""
    cfg = json.loads(json.dumps(config))
    if cfg.get("architectures") != ["DFlash2DraftModel"]:
        raise ValueError("a DFlash2 export needs architectures=['DFlash2DraftModel']")
    m = cfg.get("dflash_config")
    if not isinstance(m, dict):
        raise ValueError("a DFlash2 export needs a dflash_config mapping")
    block = cfg.get("block_size", m.get("block_size"))
    if expected_block_size is not None and block != int(expected_block_size):
        raise ValueError(f"exported block_size={block!r}, expected {int(expected_block_size)}")
    for name in ("block_size", "conv_group_size", "conv_kernel_size", "selector_rank", "selector_top_k"):
        v = block if name == "block_size" else m.get(name)
        if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
            raise ValueError(f"DFlash2 requires positive integer {name}, got {v!r}")
    mode = str(m.get("attention_mode", "gqa")).lower()
    if mode not in ("gqa", "mha"):
        raise ValueError(f"DFlash2 serving supports GQA/MHA only, got attention_mode={mode!r}")
    m["attention_mode"] = mode
    cfg.pop("auto_map", None)
    return cfg


@torch.no_grad()
def _export_dflash2_drafter(draft_model, spec, path: str, tensors: dict) -> dict:
    from safetensors.torch import save_file

    cfg, sel = draft_model.cfg, draft_model.candidate_selector
    layer0 = draft_model.layers[0].attention_conv
    n_proj = 2 * layer0.taps * layer0.groups
    for name in list(tensors):           # drop the GEMM padding rows of the tap projections
        if name.endswith("_conv_proj"):
            tensors[name] = tensors[name][:n_proj].contiguous()
    save_file(tensors, os.path.join(path, "model.safetensors"))
    config = {"architectures": ["DFlash2DraftModel"], "model_type": "dflash2", "hidden_size": cfg.hidden_size,
              "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_attention_heads,
              "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "qk_norm": cfg.qk_norm,
              "intermediate_size": cfg.intermediate_size, "vocab_size": int(sel.predecessor.shape[0]),
              "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_norm_eps,
              "block_size": draft_model.block_size, "target_layer_ids": list(spec.model.target_layer_ids),
              "conditioning_dim": draft_model.conditioning_dim, "mask_token_id": cfg.mask_token_id,
              "verifier": spec.model.verifier_id, "gate_up_layout": "interleaved",
              "output_multiplier": draft_model.output_multiplier,
              "final_logit_softcapping": draft_model.final_logit_softcapping,
              "dflash_config": {"block_size": draft_model.block_size, "conv_kernel_size": layer0.taps,
                                "conv_group_size": cfg.hidden_size // layer0.groups,
                                "selector_rank": int(sel.predecessor.shape[1]), "selector_top_k": int(sel.top_k),
                                "attention_mode": "gqa" if cfg.num_key_value_heads < cfg.num_attention_heads else "mha",
                                "target_layer_ids": list(spec.model.target_layer_ids)}}
    config.update(_sliding_window_fields(cfg))
    normalize_dflash2_config(config)
    json.dump(config, open(os.path.join(path, "config.json"), "w"), indent=1)
    json.dump(config, open(os.path.join(path, "dflash_config.json"), "w"), indent=1)
    return write_export_manifest(path, {"kind": "dflash2_drafter", "tensor_count": len(tensors)})


def validate_dflash2_export(path: str, expected_block_size: int | None = None) -> list[str]:
    """Config, hashes and tensor inventory of a DFlash2 export
    (dllm_parallel/core/models/backbones/dflash/executor.py:516-566)."""
    problems = validate_dflash_export(path)
    if problems:
        return problems
    try:
        cfg = normalize_dflash2_config(json.load(open(os.path.join(path, "config.json"))), expected_block_size)
    except (OSError, ValueError) as e:
        return [str(e)]
    from safetensors import safe_open

    with safe_open(os.path.join(path, "model.safetensors"), framework="pt", device="cpu") as f:
        got = {k: tuple(f.get_slice(k).get_shape()) for k in f.keys()}
    want = dflash2_serving_shapes(cfg)
    forbidden = {"embed", "lm_head", "embed_tokens.weight", "lm_head.weight"} & set(got)
    if forbidden:
        problems.append(f"export contains verifier-only tensors: {sorted(forbidden)}")
    missing, extra = sorted(want.keys() - got.keys()), sorted(got.keys() - want.keys())
    wrong = sorted(k for k in want.keys() & got.keys() if want[k] != got[k])
    if missing or extra or wrong:
        problems.append(f"tensor inventory mismatch: missing={missing[:3]} extra={extra[:3]} wrong_shapes={wrong[:3]}")
    return problems


def validate_dflash_export(path: str) -> list[str]:
    problems = []
    for f in ("model.safetensors", "dflash_config.json", "export_manifest.json"):
        if not os.path.exists(os.path.join(path, f)):
            problems.append(f"missing {f}")
    if problems:
        return problems
    man = json.load(open(os.path.join(path, "export_manifest.json")))
    for f, meta in man["files"].items():
        if _sha(os.path.join(path, f)) != meta["sha256"]:
            problems.append(f"{f}: sha256 mismatch")
    cfg = json.load(open(os.path.join(path, "dflash_config.json")))
    for k in ("block_size", "target_layer_ids", "conditioning_dim", "mask_token_id"):
        if cfg.get(k) in (None, []):
            problems.append(f"dflash_config.json lacks {k}")
    return problems


def main(argv=None) -> int:
    from ..config.run_spec import RunSpecError, load_run_spec

    ap = argparse.ArgumentParser(prog="dllm-export-diffusiongemma")
    ap.add_argument("--config", required=True)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--tag", default="latest")
    a = ap.parse_args(argv)
    try:
        man = export_training_checkpoint(load_run_spec(a.config).validate(), a.checkpoint, a.output, a.tag)
    except (RunSpecError, FileNotFoundError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    print(json.dumps({"output": a.output, "files": sorted(man["files"])}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

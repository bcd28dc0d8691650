"""What this package makes of a model: family, objectives, shapes, parameter count, attention path per head width,
FLOPs per token. Reads built-in presets and local Hugging Face checkpoint directories (config.json only; no weights
are opened, nothing is downloaded).

    python -m turbo_dllm_b200.benchmarks.inspect_models synthetic:qwen3-8b /models/Qwen3-8B [--json] [--seq-len 32768]

Counterpart of the reference's benchmarks/tools/inspect_hf_dllm_models.py:21-62 (which fetches configs from the hub).
"""
from __future__ import annotations

import argparse
import json
import sys


def summarize(model_id: str, seq_len: int = 32768, block_size: int = 32) -> dict:
    from ..models.config import PRESETS
    from ..models.hf_loader import load_hf_config, pretrained_directory
    from ..models.registry import FAMILY_OBJECTIVES, infer_family

    local = pretrained_directory(model_id)
    if local is not None:
        cfg, source = load_hf_config(local), "checkpoint directory"
    elif model_id in PRESETS:
        cfg, source = PRESETS[model_id], "preset"
    else:
        raise ValueError(f"{model_id!r} is neither a preset ({', '.join(PRESETS)}) nor a local checkpoint directory")
    family = ("qwen3_8" if cfg.is_hybrid else "diffusion_gemma" if cfg.is_moe
              else cfg.family if cfg.family != "causal_lm" else infer_family(model_id))
    if cfg.head_dim == 128:
        attention = "fused tcgen05 kernel (scores and probabilities stay in TMEM / shared memory)"
    elif cfg.head_dim % 64 == 0:
        attention = "tensor-core products around masked-softmax kernels (scores pass through HBM)"
    else:
        attention = "fp32 reference only (head_dim must be a multiple of 64 for the CUDA path)"
    params = cfg.num_params()
    out = {"model_id": model_id, "source": source, "family": family, "objectives": list(FAMILY_OBJECTIVES.get(family, ())),
           "layers": cfg.num_layers, "hidden_size": cfg.hidden_size, "heads": cfg.num_attention_heads,
           "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate_size": cfg.intermediate_size,
           "vocab_size": cfg.vocab_size, "tie_word_embeddings": cfg.tie_word_embeddings, "parameters": params,
           "attention_path": attention}
    if cfg.is_moe:
        out.update(experts=cfg.num_experts, experts_per_token=cfg.num_experts_per_token,
                   expert_intermediate_size=cfg.moe_intermediate_size, shared_intermediate_size=cfg.moe_shared_intermediate_size)
    if cfg.is_hybrid:
        out.update(full_attention_interval=cfg.full_attention_interval, linear_key_heads=cfg.linear_num_key_heads,
                   linear_value_heads=cfg.linear_num_value_heads)
    if cfg.has_sliding_layers:
        out.update(sliding_window=cfg.sliding_window,
                   sliding_layers=sum(cfg.layer_window(i) is not None for i in range(cfg.num_layers)))
    # one training step on one sequence (two noisy views over one clean copy when the family's first objective is
    # Fast-dLLM v2, one view otherwise): rows = views·L noisy + L clean, visible pairs by the block-diffusion mask
    from ..profiling.perf import block_diffusion_pairs, transformer_step_flops

    views = 2 if (out["objectives"] and out["objectives"][0] == "fast_dllm_v2") else 1
    flops = transformer_step_flops(cfg, rows=(views + 1) * seq_len,
                                   pairs=block_diffusion_pairs(seq_len, block_size, views), vocab_rows=views * seq_len // 2)
    out["train_tflops_per_sequence"] = round(flops.total / 1e12, 3)
    out["attention_share_of_flops"] = round(flops.attention / flops.total, 3)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m turbo_dllm_b200.benchmarks.inspect_models")
    ap.add_argument("models", nargs="+")
    ap.add_argument("--json", action="store_true", help="one JSON object per line")
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--block-size", type=int, default=32)
    a = ap.parse_args(argv)
    rc = 0
    for mid in a.models:
        try:
            s = summarize(mid, a.seq_len, a.block_size)
        except (ValueError, FileNotFoundError, KeyError) as e:
            print(f"error: {e}", file=sys.stderr)
            rc = 2
            continue
        if a.json:
            print(json.dumps(s, sort_keys=True))
        else:
            print(s["model_id"])
            for k, v in s.items():
                if k != "model_id" and v is not None:
                    print(f"  {k}: {v}")
    return rc


if __name__ == "__main__":
    raise SystemExit(main())

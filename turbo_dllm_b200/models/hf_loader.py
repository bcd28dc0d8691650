"""Hugging Face interchange: read a local model directory into this package's decoder and write
one back (config.json + safetensors), for dense Qwen3-style and hybrid (Gated DeltaNet) checkpoints.

Name mapping (per layer i):
  self_attn.{q,k,v}_proj.weight → rows of `w_qkv` in that order     self_attn.o_proj.weight → `w_o`
  self_attn.{q,k}_norm.weight   → `q_norm` / `k_norm`               input_layernorm / post_attention_layernorm
  mlp.gate_proj / mlp.up_proj   → `w_gate_up`, rows interleaved (g0,u0,g1,u1,…) so the GEMM epilogue can
                                   apply SwiGLU;                     mlp.down_proj → `w_down`
  model.embed_tokens, lm_head, model.norm → `embed`, `lm_head`, `final_norm`
`max_layers` truncates; tensor-parallel ranks load their slice of each matrix.

Hybrid (qwen3_8) checkpoints: a linear-attention layer stores `linear_attn.in_proj_qkv|z|b|a` (stacked here
into `w_in` as q | k | v | z | b | a, zero-padded to a multiple of 64 rows), `linear_attn.conv1d.weight`
[channels, 1, taps] (+ optional bias) → `conv_w` / `conv_b`, `A_log`, `dt_bias`, `linear_attn.norm.weight` →
`gdn_norm`, `linear_attn.out_proj` → `w_out`; a gated attention layer stores per head the query rows followed by
the gate rows in `self_attn.q_proj` (split here into the q rows of `w_qkv` and `w_attn_gate`).

Counterparts: dllm_parallel/core/models/hf_loader.py:50-210 (config + weights through transformers) and the
export side of dllm_parallel/core/models/backbones/qwen3_8/export.py:70-512.
"""
from __future__ import annotations

import json
import os

import torch

from .config import ModelConfig


def load_hf_config(path: str, max_layers: int | None = None) -> ModelConfig:
    cfg_path = os.path.join(path, "config.json")
    if not os.path.exists(cfg_path):
        raise FileNotFoundError(f"{path} has no config.json (model loading works from local directories)")
    c = json.load(open(cfg_path))
    heads = c["num_attention_heads"]
    layers = c["num_hidden_layers"]
    if max_layers is not None:
        layers = min(layers, max_layers)
    arch = " ".join(c.get("architectures", []))
    hybrid = {}
    if c.get("full_attention_interval"):
        hybrid = dict(family="qwen3_8", full_attention_interval=int(c["full_attention_interval"]),
                      linear_num_key_heads=int(c["linear_num_key_heads"]),
                      linear_num_value_heads=int(c["linear_num_value_heads"]),
                      linear_key_head_dim=int(c["linear_key_head_dim"]),
                      linear_value_head_dim=int(c["linear_value_head_dim"]),
                      linear_conv_kernel=int(c.get("linear_conv_kernel_dim", 4)))
    sliding = {}
    if c.get("sliding_window") and c.get("use_sliding_window", True):
        types = c.get("layer_types")
        sliding = dict(sliding_window=int(c["sliding_window"]),
                       sliding_window_pattern=int(c.get("sliding_window_pattern", 0) or 0),
                       layer_types=tuple(types[:layers]) if types and not hybrid else None)
    return ModelConfig(**hybrid, **sliding,
        vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], num_layers=layers, num_attention_heads=heads,
        num_key_value_heads=c.get("num_key_value_heads", heads), head_dim=c.get("head_dim", c["hidden_size"] // heads),
        intermediate_size=c["intermediate_size"], rope_theta=float(c.get("rope_theta", 1e6)),
        partial_rotary_factor=float(c.get("partial_rotary_factor", 1.0) or 1.0),
        rms_norm_eps=float(c.get("rms_norm_eps", 1e-6)), qk_norm="Qwen3" in arch or bool(c.get("qk_norm", False)),
        tie_word_embeddings=bool(c.get("tie_word_embeddings", False)), mask_token_id=c.get("mask_token_id"))


def hf_config_dict(cfg: ModelConfig) -> dict:
    d = _hf_config_dict(cfg)
    if cfg.partial_rotary_factor != 1.0:
        d["partial_rotary_factor"] = cfg.partial_rotary_factor
    return d


def _hf_config_dict(cfg: ModelConfig) -> dict:
    if cfg.is_hybrid:
        kinds = [cfg.layer_kind(i) for i in range(cfg.num_layers)]
        return {"architectures": ["Qwen3NextForCausalLM"], "model_type": "qwen3_next", "vocab_size": cfg.vocab_size,
                "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
                "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "intermediate_size": cfg.intermediate_size, "rope_theta": cfg.rope_theta,
                "rms_norm_eps": cfg.rms_norm_eps, "tie_word_embeddings": cfg.tie_word_embeddings,
                "mask_token_id": cfg.mask_token_id, "hidden_act": "silu", "torch_dtype": "bfloat16", "qk_norm": cfg.qk_norm,
                "full_attention_interval": cfg.full_attention_interval, "layer_types": kinds,
                "linear_num_key_heads": cfg.linear_num_key_heads, "linear_num_value_heads": cfg.linear_num_value_heads,
                "linear_key_head_dim": cfg.linear_key_head_dim, "linear_value_head_dim": cfg.linear_value_head_dim,
                "linear_conv_kernel_dim": cfg.linear_conv_kernel}
    sliding = {}
    if cfg.has_sliding_layers:
        sliding = {"sliding_window": cfg.sliding_window, "use_sliding_window": True,
                   "layer_types": ["sliding_attention" if cfg.layer_window(i) else "full_attention"
                                   for i in range(cfg.num_layers)]}
    return {**sliding, "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": cfg.vocab_size,
            "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
            "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate_size": cfg.intermediate_size, "rope_theta": cfg.rope_theta,
            "rms_norm_eps": cfg.rms_norm_eps, "tie_word_embeddings": cfg.tie_word_embeddings,
            "mask_token_id": cfg.mask_token_id, "hidden_act": "silu", "torch_dtype": "bfloat16"}


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1])


def deinterleave_gate_up(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return w[0::2].contiguous(), w[1::2].contiguous()


def _open_weights(path: str) -> dict:
    from safetensors import safe_open

    index = os.path.join(path, "model.safetensors.index.json")
    files = sorted(set(json.load(open(index))["weight_map"].values())) if os.path.exists(index) else \
        [f for f in sorted(os.listdir(path)) if f.endswith(".safetensors")]
    if not files:
        raise FileNotFoundError(f"{path} has no .safetensors weights")
    handles = [safe_open(os.path.join(path, f), framework="pt", device="cpu") for f in files]
    table = {}
    for h in handles:
        for k in h.keys():
            table[k] = h
    return table


@torch.no_grad()
def load_hf_weights(model, path: str) -> None:
    """Fills `model` (a dense BlockDiffusionTransformer, possibly tensor-parallel) from `path`."""
    table = _open_weights(path)
    cfg, tp = model.cfg, model.tp

    def get(name):
        if name not in table:
            raise KeyError(f"checkpoint lacks {name}")
        return table[name].get_tensor(name)

    def put(param, tensor):
        param.copy_(tensor.to(param.device, param.dtype))

    def shard(t, dim):
        return tp.shard(t, dim) if tp is not None else t

    put(model.embed, shard(get("model.embed_tokens.weight"), 0))
    put(model.final_norm, get("model.norm.weight"))
    if not cfg.tie_word_embeddings:
        name = "lm_head.weight" if "lm_head.weight" in table else "model.embed_tokens.weight"
        put(model.lm_head, shard(get(name), 0))
    for i, layer in enumerate(model.layers):
        p = f"model.layers.{i}."
        if cfg.is_hybrid:
            if tp is not None:
                raise ValueError("hybrid checkpoints load on one tensor-parallel rank")
            _load_hybrid_layer(layer, cfg, p, get, put, table)
            continue
        q, k, v = (get(p + f"self_attn.{n}_proj.weight") for n in "qkv")
        put(layer.w_qkv, torch.cat([shard(q, 0), shard(k, 0), shard(v, 0)], dim=0))
        put(layer.w_o, shard(get(p + "self_attn.o_proj.weight"), 1))
        put(layer.input_norm, get(p + "input_layernorm.weight"))
        put(layer.post_norm, get(p + "post_attention_layernorm.weight"))
        if layer.q_norm is not None:
            put(layer.q_norm, get(p + "self_attn.q_norm.weight"))
            put(layer.k_norm, get(p + "self_attn.k_norm.weight"))
        put(layer.w_gate_up, interleave_gate_up(shard(get(p + "mlp.gate_proj.weight"), 0),
                                                shard(get(p + "mlp.up_proj.weight"), 0)))
        put(layer.w_down, shard(get(p + "mlp.down_proj.weight"), 1))
    _apply_partial_rotary_order(model, inverse=False)


def _apply_partial_rotary_order(model, inverse: bool) -> None:
    """Checkpoint order <-> kernel order of the q/k head dimensions under partial rotary embeddings (a no-op when the
    whole head rotates). Layers without q/k projections (linear attention) are left alone."""
    cfg = model.cfg
    if cfg.rotary_dim >= cfg.head_dim:
        return
    from ..ops.rope import partial_rotary_permutation

    perm = partial_rotary_permutation(cfg.head_dim, cfg.rotary_dim)
    if inverse:
        perm = torch.argsort(perm)
    for layer in model.layers:
        if getattr(layer, "w_qkv", None) is not None:
            _permute_qk_head_dims(layer, cfg, perm)


def _load_hybrid_layer(layer, cfg, p, get, put, table) -> None:
    put(layer.input_norm, get(p + "input_layernorm.weight"))
    put(layer.post_norm, get(p + "post_attention_layernorm.weight"))
    put(layer.w_gate_up, interleave_gate_up(get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")))
    put(layer.w_down, get(p + "mlp.down_proj.weight"))
    if cfg.layer_kind(layer.idx) == "linear_attention":
        m = p + "linear_attn."
        rows = torch.cat([get(m + f"in_proj_{n}.weight") for n in ("qkv", "z", "b", "a")], dim=0)
        w_in = torch.zeros(layer.w_in.shape, dtype=rows.dtype)
        w_in[: rows.shape[0]] = rows
        put(layer.w_in, w_in)
        put(layer.conv_w, get(m + "conv1d.weight").squeeze(1))
        if m + "conv1d.bias" in table:
            put(layer.conv_b, get(m + "conv1d.bias"))
        else:
            layer.conv_b.zero_()
        put(layer.A_log, get(m + "A_log"))
        put(layer.dt_bias, get(m + "dt_bias"))
        put(layer.gdn_norm, get(m + "norm.weight"))
        put(layer.w_out, get(m + "out_proj.weight"))
        return
    a = p + "self_attn."
    D = cfg.head_dim
    qg = get(a + "q_proj.weight").view(cfg.num_attention_heads, 2, D, cfg.hidden_size)
    put(layer.w_qkv, torch.cat([qg[:, 0].reshape(cfg.q_dim, -1), get(a + "k_proj.weight"), get(a + "v_proj.weight")]))
    put(layer.w_attn_gate, qg[:, 1].reshape(cfg.q_dim, -1))
    put(layer.w_o, get(a + "o_proj.weight"))
    if layer.q_norm is not None:
        put(layer.q_norm, get(a + "q_norm.weight"))
        put(layer.k_norm, get(a + "k_norm.weight"))


def _export_hybrid_layer(layer, cfg, p, out) -> None:
    out[p + "input_layernorm.weight"] = layer.input_norm
    out[p + "post_attention_layernorm.weight"] = layer.post_norm
    g, u = deinterleave_gate_up(layer.w_gate_up)
    out[p + "mlp.gate_proj.weight"], out[p + "mlp.up_proj.weight"] = g, u
    out[p + "mlp.down_proj.weight"] = layer.w_down
    if cfg.layer_kind(layer.idx) == "linear_attention":
        m = p + "linear_attn."
        cc, vd, hv = cfg.linear_conv_channels, cfg.linear_value_dim, cfg.linear_num_value_heads
        out[m + "in_proj_qkv.weight"] = layer.w_in[:cc]
        out[m + "in_proj_z.weight"] = layer.w_in[cc:cc + vd]
        out[m + "in_proj_b.weight"] = layer.w_in[cc + vd:cc + vd + hv]
        out[m + "in_proj_a.weight"] = layer.w_in[cc + vd + hv:cc + vd + 2 * hv]
        out[m + "conv1d.weight"] = layer.conv_w.unsqueeze(1)
        out[m + "conv1d.bias"] = layer.conv_b
        out[m + "A_log"], out[m + "dt_bias"] = layer.A_log, layer.dt_bias
        out[m + "norm.weight"] = layer.gdn_norm
        out[m + "out_proj.weight"] = layer.w_out
        return
    a = p + "self_attn."
    D, qd, kd = cfg.head_dim, cfg.q_dim, cfg.kv_dim
    q = layer.w_qkv[:qd].view(cfg.num_attention_heads, 1, D, -1)
    gate = layer.w_attn_gate.view(cfg.num_attention_heads, 1, D, -1)
    out[a + "q_proj.weight"] = torch.cat([q, gate], dim=1).reshape(2 * qd, -1)
    out[a + "k_proj.weight"] = layer.w_qkv[qd:qd + kd]
    out[a + "v_proj.weight"] = layer.w_qkv[qd + kd:]
    out[a + "o_proj.weight"] = layer.w_o
    if layer.q_norm is not None:
        out[a + "q_norm.weight"], out[a + "k_norm.weight"] = layer.q_norm, layer.k_norm


def _permute_qk_head_dims(layer, cfg: ModelConfig, perm: torch.Tensor) -> None:
    """Reorders the head dimensions of the q and k rows of `w_qkv` and of the q/k norm weights: new[d] = old[perm[d]]
    inside every head. q·k is unchanged; with partial rotary embeddings this moves a checkpoint's rotating pairs
    (j, j + rotary_dim/2) onto the pairs (i, i + head_dim/2) the rotary kernels use (ops/rope.py)."""
    D = cfg.head_dim
    w = layer.w_qkv
    hq = (w.shape[0] - 0) // D            # q, k and v heads of this rank, in that order
    n_q = layer.w_o.shape[1] // D
    n_kv = (hq - n_q) // 2
    perm = perm.to(w.device)
    for start, heads in ((0, n_q), (n_q * D, n_kv)):
        blk = w[start:start + heads * D].view(heads, D, -1)
        blk.copy_(blk[:, perm].clone())
    for t in (layer.q_norm, layer.k_norm):
        if t is not None:
            t.copy_(t[perm].clone())


@torch.no_grad()
def export_hf_checkpoint(model, path: str, merge_adapters: bool = True) -> str:
    """Writes config.json + model.safetensors in Hugging Face naming (single tensor-parallel rank)."""
    from safetensors.torch import save_file

    if model.tp is not None:
        raise ValueError("export from a tensor-parallel model: gather the shards first")
    if merge_adapters and getattr(model, "lora", None) is not None:
        from ..adapters.lora import merge_lora

        merge_lora(model)
    cfg = model.cfg
    os.makedirs(path, exist_ok=True)
    _apply_partial_rotary_order(model, inverse=True)        # the file keeps the checkpoint's head-dimension order
    try:
        return _write_hf_checkpoint(model, cfg, path)
    finally:
        _apply_partial_rotary_order(model, inverse=False)


@torch.no_grad()
def _write_hf_checkpoint(model, cfg, path: str) -> str:
    from safetensors.torch import save_file

    out = {"model.embed_tokens.weight": model.embed, "model.norm.weight": model.final_norm}
    if not cfg.tie_word_embeddings:
        out["lm_head.weight"] = model.lm_head
    for i, layer in enumerate(model.layers):
        p = f"model.layers.{i}."
        if cfg.is_hybrid:
            _export_hybrid_layer(layer, cfg, p, out)
            continue
        qd, kd = cfg.q_dim, cfg.kv_dim
        out[p + "self_attn.q_proj.weight"] = layer.w_qkv[:qd]
        out[p + "self_attn.k_proj.weight"] = layer.w_qkv[qd:qd + kd]
        out[p + "self_attn.v_proj.weight"] = layer.w_qkv[qd + kd:]
        out[p + "self_attn.o_proj.weight"] = layer.w_o
        out[p + "input_layernorm.weight"] = layer.input_norm
        out[p + "post_attention_layernorm.weight"] = layer.post_norm
        if layer.q_norm is not None:
            out[p + "self_attn.q_norm.weight"] = layer.q_norm
            out[p + "self_attn.k_norm.weight"] = layer.k_norm
        g, u = deinterleave_gate_up(layer.w_gate_up)
        out[p + "mlp.gate_proj.weight"], out[p + "mlp.up_proj.weight"] = g, u
        out[p + "mlp.down_proj.weight"] = layer.w_down
    save_file({k: v.detach().cpu().contiguous() for k, v in out.items()}, os.path.join(path, "model.safetensors"))
    json.dump(hf_config_dict(cfg), open(os.path.join(path, "config.json"), "w"), indent=1)
    return path

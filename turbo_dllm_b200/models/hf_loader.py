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


def pretrained_directory(model_id: str | None) -> str | None:
    """The local checkpoint directory `model_id` names (one with a config.json): the path itself, or the cached
    snapshot of a hub id; None otherwise. Nothing is downloaded."""
    if model_id and os.path.isdir(model_id) and os.path.exists(os.path.join(model_id, "config.json")):
        return model_id
    if model_id and model_id.count("/") == 1 and not model_id.startswith(("synthetic:", ".", "/")):
        # a hub id (`organization/model`): only a snapshot that is already in the local Hugging Face cache is used
        try:
            from huggingface_hub import snapshot_download

            path = snapshot_download(model_id, local_files_only=True)
        except Exception:
            return None
        if os.path.exists(os.path.join(path, "config.json")):
            return path
    return None


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
    moe = {}
    if c.get("num_experts"):
        moe = dict(family="diffusion_gemma", num_experts=int(c["num_experts"]),
                   num_experts_per_token=int(c.get("num_experts_per_tok", c.get("num_experts_per_token", 1))),
                   moe_intermediate_size=int(c["moe_intermediate_size"]),
                   moe_shared_intermediate_size=int(c.get("shared_expert_intermediate_size", 0) or 0))
    return ModelConfig(**hybrid, **sliding, **moe,
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
    """Fills `model` (dense, hybrid or mixture-of-experts decoder; tensor- or expert-parallel) from the Hugging Face
    checkpoint directory `path`. A tensor-parallel rank reads only its own rows / columns of every sharded matrix from
    the files (the role of a per-parameter tensor-parallel plan: dllm_parallel/core/parallel/hf_tensor_parallel.py:22-226)."""
    table = _open_weights(path)
    cfg, tp = model.cfg, model.tp

    def get(name):
        if name not in table:
            raise KeyError(f"checkpoint lacks {name}")
        return table[name].get_tensor(name)

    def put(param, tensor):
        if tuple(param.shape) != tuple(tensor.shape):
            raise ValueError(f"checkpoint tensor of shape {tuple(tensor.shape)} does not fit a parameter of shape "
                             f"{tuple(param.shape)}")
        param.copy_(tensor.to(param.device, param.dtype))

    def part(name, dim):
        """This rank's slice of a matrix that tensor parallelism divides along `dim` (read from the file as a slice)."""
        if tp is None:
            return get(name)
        if name not in table:
            raise KeyError(f"checkpoint lacks {name}")
        sl = table[name].get_slice(name)
        n = sl.get_shape()[dim] // tp.size
        lo = tp.rank * n
        return sl[lo:lo + n] if dim == 0 else sl[:, lo:lo + n]

    put(model.embed, part("model.embed_tokens.weight", 0))
    put(model.final_norm, get("model.norm.weight"))
    if not cfg.tie_word_embeddings:
        name = "lm_head.weight" if "lm_head.weight" in table else "model.embed_tokens.weight"
        put(model.lm_head, part(name, 0))
    for i, layer in enumerate(model.layers):
        p = f"model.layers.{i}."
        if cfg.is_hybrid:
            _load_hybrid_layer(layer, cfg, p, get, put, table, tp, part)
            continue
        put(layer.w_qkv, torch.cat([part(p + f"self_attn.{n}_proj.weight", 0) for n in "qkv"], dim=0))
        put(layer.w_o, part(p + "self_attn.o_proj.weight", 1))
        put(layer.input_norm, get(p + "input_layernorm.weight"))
        put(layer.post_norm, get(p + "post_attention_layernorm.weight"))
        if layer.q_norm is not None:
            put(layer.q_norm, get(p + "self_attn.q_norm.weight"))
            put(layer.k_norm, get(p + "self_attn.k_norm.weight"))
        if getattr(layer, "experts", None) is not None:
            _load_expert_layer(layer, p, get, put)
            continue
        put(layer.w_gate_up, interleave_gate_up(part(p + "mlp.gate_proj.weight", 0), part(p + "mlp.up_proj.weight", 0)))
        put(layer.w_down, part(p + "mlp.down_proj.weight", 1))
    _apply_partial_rotary_order(model, inverse=False)


def _load_expert_layer(layer, p, get, put) -> None:
    """Router, this rank's experts (global experts [ep_rank * E_local, (ep_rank + 1) * E_local)) and the dense
    feed-forward beside them, in the naming `models/export.py` writes."""
    bank = layer.experts
    put(bank.router, get(p + "mlp.router.weight"))
    first = bank.ep_rank * bank.e_local
    for e in range(bank.e_local):
        q = p + f"mlp.experts.{first + e}."
        put(bank.w_gu[e], interleave_gate_up(get(q + "gate_proj.weight"), get(q + "up_proj.weight")))
        put(bank.w_down[e], get(q + "down_proj.weight"))
    if layer.w_gate_up is not None:
        s = p + "mlp.shared_expert."
        put(layer.w_gate_up, interleave_gate_up(get(s + "gate_proj.weight"), get(s + "up_proj.weight")))
        put(layer.w_down, get(s + "down_proj.weight"))


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


def _load_hybrid_layer(layer, cfg, p, get, put, table, tp=None, part=None) -> None:
    """One layer of the hybrid family. Under tensor parallelism the rank takes its key / value heads of the
    linear-attention projections (`models/hybrid.py::fused_projection_rows`), its query / key / value heads and
    gate rows of the softmax layers, and its slice of the feed-forward."""
    part = part or (lambda name, dim: get(name))
    shard = (lambda t, dim: tp.shard(t, dim)) if tp is not None else (lambda t, dim: t)
    put(layer.input_norm, get(p + "input_layernorm.weight"))
    put(layer.post_norm, get(p + "post_attention_layernorm.weight"))
    put(layer.w_gate_up, interleave_gate_up(part(p + "mlp.gate_proj.weight", 0), part(p + "mlp.up_proj.weight", 0)))
    put(layer.w_down, part(p + "mlp.down_proj.weight", 1))
    if cfg.layer_kind(layer.idx) == "linear_attention":
        m = p + "linear_attn."
        rows = torch.cat([get(m + f"in_proj_{n}.weight") for n in ("qkv", "z", "b", "a")], dim=0)
        conv_w = get(m + "conv1d.weight").squeeze(1)
        conv_b = get(m + "conv1d.bias") if m + "conv1d.bias" in table else None
        a_log, dt_bias = get(m + "A_log"), get(m + "dt_bias")
        if tp is not None:
            from .hybrid import fused_projection_rows

            take, channels = fused_projection_rows(cfg, tp.rank, tp.size)
            rows, conv_w = rows[take], conv_w[channels]
            conv_b = conv_b[channels] if conv_b is not None else None
            a_log, dt_bias = shard(a_log, 0), shard(dt_bias, 0)
        w_in = torch.zeros(layer.w_in.shape, dtype=rows.dtype)     # rows past q | k | v | z | b | a pad the GEMM width
        w_in[: rows.shape[0]] = rows
        put(layer.w_in, w_in)
        put(layer.conv_w, conv_w)
        if conv_b is not None:
            put(layer.conv_b, conv_b)
        else:
            layer.conv_b.zero_()
        put(layer.A_log, a_log)
        put(layer.dt_bias, dt_bias)
        put(layer.gdn_norm, get(m + "norm.weight"))
        put(layer.w_out, part(m + "out_proj.weight", 1))
        return
    a = p + "self_attn."
    D = cfg.head_dim
    qg = get(a + "q_proj.weight").view(cfg.num_attention_heads, 2, D, cfg.hidden_size)
    q, gate = shard(qg[:, 0], 0), shard(qg[:, 1], 0)           # query and gate rows are interleaved per head in the file
    put(layer.w_qkv, torch.cat([q.reshape(-1, cfg.hidden_size), part(a + "k_proj.weight", 0), part(a + "v_proj.weight", 0)]))
    put(layer.w_attn_gate, gate.reshape(-1, cfg.hidden_size))
    put(layer.w_o, part(a + "o_proj.weight", 1))
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
def gather_tensor_parallel_model(model):
    """A stand-in for `model` whose layers hold FULL tensors assembled from the tensor-parallel ranks' shards (on the
    CPU, on every rank): what the checkpoint writers read. Column-parallel matrices are joined along rows, row-parallel
    ones along columns, the fused q | k | v projection section by section, the hybrid family's fused input projection
    and convolution by the head segments each rank owns."""
    import torch.distributed as dist
    from types import SimpleNamespace

    tp, cfg = model.tp, model.cfg
    n = tp.size

    def every(t):
        t = t.detach().contiguous()
        parts = [torch.empty_like(t) for _ in range(n)]
        dist.all_gather(parts, t, group=tp.group)
        return [x.cpu() for x in parts]

    def cat(t, dim):
        return torch.cat(every(t), dim=dim)

    def qkv(w, q_rows, kv_rows):
        parts = every(w)
        return torch.cat([torch.cat([x[:q_rows] for x in parts]), torch.cat([x[q_rows:q_rows + kv_rows] for x in parts]),
                          torch.cat([x[q_rows + kv_rows:] for x in parts])])

    lc = model.lcfg
    out = SimpleNamespace(cfg=cfg, tp=None, embed=cat(model.embed, 0), final_norm=model.final_norm.detach().cpu(), layers=[])
    out.lm_head = out.embed if cfg.tie_word_embeddings else cat(model.lm_head, 0)
    for layer in model.layers:
        full = SimpleNamespace(idx=layer.idx, input_norm=layer.input_norm.detach().cpu(),
                               post_norm=layer.post_norm.detach().cpu(), w_gate_up=cat(layer.w_gate_up, 0),
                               w_down=cat(layer.w_down, 1), q_norm=None, k_norm=None)
        if cfg.is_hybrid and cfg.layer_kind(layer.idx) == "linear_attention":
            from .hybrid import fused_projection_rows

            w_in = torch.zeros((cfg.linear_in_dim, layer.w_in.shape[1]), dtype=layer.w_in.dtype)
            conv_w = torch.zeros((cfg.linear_conv_channels, layer.conv_w.shape[1]), dtype=layer.conv_w.dtype)
            conv_b = torch.zeros((cfg.linear_conv_channels,), dtype=layer.conv_b.dtype)
            for r, (wi, cw, cb) in enumerate(zip(every(layer.w_in), every(layer.conv_w), every(layer.conv_b))):
                rows, channels = fused_projection_rows(cfg, r, n)
                w_in[rows] = wi[: rows.numel()]
                conv_w[channels], conv_b[channels] = cw, cb
            full.w_in, full.conv_w, full.conv_b = w_in, conv_w, conv_b
            full.A_log, full.dt_bias = cat(layer.A_log, 0), cat(layer.dt_bias, 0)
            full.gdn_norm, full.w_out = layer.gdn_norm.detach().cpu(), cat(layer.w_out, 1)
        else:
            full.w_qkv = qkv(layer.w_qkv, lc.q_dim, lc.kv_dim)
            full.w_o = cat(layer.w_o, 1)
            if layer.q_norm is not None:
                full.q_norm, full.k_norm = layer.q_norm.detach().cpu(), layer.k_norm.detach().cpu()
            if getattr(layer, "w_attn_gate", None) is not None:
                full.w_attn_gate = cat(layer.w_attn_gate, 0)
        out.layers.append(full)
    return out


@torch.no_grad()
def export_hf_checkpoint(model, path: str, merge_adapters: bool = True) -> str:
    """Writes config.json + model.safetensors in Hugging Face naming. A tensor-parallel model is assembled from its
    ranks' shards first (a collective over the tensor-parallel group: every rank calls this); rank 0 of the group
    writes the files."""
    if merge_adapters and getattr(model, "lora", None) is not None:
        from ..adapters.lora import merge_lora

        merge_lora(model)
    cfg = model.cfg
    if model.tp is not None:
        import torch.distributed as dist

        full = gather_tensor_parallel_model(model)
        if model.tp.rank == 0:
            os.makedirs(path, exist_ok=True)
            _apply_partial_rotary_order(full, inverse=True)
            _write_hf_checkpoint(full, cfg, path)
        dist.barrier(group=model.tp.group)
        return path
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
    save_file({k: _stored(v) for k, v in out.items()}, os.path.join(path, "model.safetensors"))
    json.dump(hf_config_dict(cfg), open(os.path.join(path, "config.json"), "w"), indent=1)
    return path


# dtype the exporters write floating-point tensors in (None: as they are). A bf16 run exported on a machine without a
# GPU is rebuilt in fp32 there (the CPU path computes in fp32) and written back in bf16.
EXPORT_DTYPE: torch.dtype | None = None


def _stored(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().cpu()
    if EXPORT_DTYPE is not None and t.is_floating_point():
        t = t.to(EXPORT_DTYPE)
    return t.contiguous()

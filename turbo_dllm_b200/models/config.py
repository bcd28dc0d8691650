"""Architecture description of the first-party decoder and named shape presets.

The reference reads architectures from Hugging Face configs
(dllm_parallel/core/models/hf_loader.py:50-78); here the same fields can also come from the
run spec (`model.random_init` with explicit sizes) or from a preset id such as
`synthetic:qwen3-8b`, because benchmarks and tests run without network access.
"""
from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass(frozen=True)
class ModelConfig:
    vocab_size: int
    hidden_size: int
    num_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float = 1.0e6
    partial_rotary_factor: float = 1.0     # share of each head's dimensions that rotary embeddings touch
    rms_norm_eps: float = 1.0e-6
    qk_norm: bool = True
    tie_word_embeddings: bool = False
    mask_token_id: int | None = None
    # mixture of experts (num_experts = 0 means dense FFN)
    num_experts: int = 0
    num_experts_per_token: int = 0
    moe_intermediate_size: int = 0
    # a dense SwiGLU feed-forward that every token passes beside its routed experts (0 = none)
    moe_shared_intermediate_size: int = 0
    # sliding-window layers: a layer whose window is set lets a row see only the last `sliding_window` clean
    # positions before its clean stop. Which layers slide: `layer_types` ("sliding_attention" / "full_attention"
    # per layer) when given, else every layer except each `sliding_window_pattern`-th one (0: all layers slide).
    sliding_window: int | None = None
    sliding_window_pattern: int = 0
    layer_types: tuple | None = None
    family: str = "causal_lm"
    # hybrid decoders (family qwen3_8): every `full_attention_interval`-th layer is gated softmax
    # attention, the others are Gated DeltaNet linear-attention layers (0 = no linear layers)
    full_attention_interval: int = 0
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel: int = 4

    @property
    def rotary_dim(self) -> int:
        r = int(self.head_dim * self.partial_rotary_factor)
        return max(r - r % 2, 2)

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_hybrid(self) -> bool:
        return self.full_attention_interval > 0

    def layer_window(self, i: int) -> int | None:
        """Window of layer i, or None when the layer attends to the whole clean prefix."""
        if not self.sliding_window:
            return None
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[i] == "sliding_attention" else None
        if self.sliding_window_pattern > 0 and (i + 1) % self.sliding_window_pattern == 0:
            return None
        return self.sliding_window

    @property
    def has_sliding_layers(self) -> bool:
        return any(self.layer_window(i) is not None for i in range(self.num_layers))

    def layer_kind(self, i: int) -> str:
        """"full_attention" or "linear_attention" for layer i (every interval-th layer is full)."""
        if not self.is_hybrid or (i + 1) % self.full_attention_interval == 0:
            return "full_attention"
        return "linear_attention"

    @property
    def linear_key_dim(self) -> int:
        return self.linear_num_key_heads * self.linear_key_head_dim

    @property
    def linear_value_dim(self) -> int:
        return self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def linear_conv_channels(self) -> int:
        return 2 * self.linear_key_dim + self.linear_value_dim

    @property
    def linear_in_dim(self) -> int:
        """Rows of the fused input projection of a linear-attention layer: q | k | v | z | b | a, padded to 64."""
        n = self.linear_conv_channels + self.linear_value_dim + 2 * self.linear_num_value_heads
        return (n + 63) // 64 * 64

    def layer_params(self) -> int:
        h = self.hidden_size
        attn = h * self.qkv_dim + self.q_dim * h + (2 * self.head_dim if self.qk_norm else 0)
        if self.is_hybrid:
            full = attn + h * self.q_dim   # output gate
            lin = (h * self.linear_in_dim + self.linear_value_dim * h
                   + self.linear_conv_channels * (self.linear_conv_kernel + 1)
                   + 2 * self.linear_num_value_heads + self.linear_value_head_dim)
            n_full = sum(self.layer_kind(i) == "full_attention" for i in range(self.num_layers))
            attn = (n_full * full + (self.num_layers - n_full) * lin) // max(self.num_layers, 1)
        if self.is_moe:
            ffn = (self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
                   + 3 * h * self.moe_shared_intermediate_size)
        else:
            ffn = 3 * h * self.intermediate_size
        return attn + ffn + 2 * h

    def num_params(self) -> int:
        emb = self.vocab_size * self.hidden_size
        head = 0 if self.tie_word_embeddings else emb
        return emb + head + self.num_layers * self.layer_params() + self.hidden_size


PRESETS: dict[str, ModelConfig] = {
    # BASELINE config 1 (CPU plumbing model)
    "synthetic:tiny-qwen3": ModelConfig(vocab_size=1024, hidden_size=256, num_layers=4, num_attention_heads=4,
                                        num_key_value_heads=2, head_dim=64, intermediate_size=704,
                                        mask_token_id=1023),
    # a small head_dim-128 model for GPU smoke tests
    "synthetic:tiny-hd128": ModelConfig(vocab_size=2048, hidden_size=512, num_layers=2, num_attention_heads=4,
                                        num_key_value_heads=2, head_dim=128, intermediate_size=1024,
                                        mask_token_id=2047),
    "synthetic:qwen3-1.7b": ModelConfig(vocab_size=151936, hidden_size=2048, num_layers=28, num_attention_heads=16,
                                        num_key_value_heads=8, head_dim=128, intermediate_size=6144,
                                        tie_word_embeddings=True, mask_token_id=151935),
    "synthetic:qwen3-8b": ModelConfig(vocab_size=151936, hidden_size=4096, num_layers=36, num_attention_heads=32,
                                      num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                                      mask_token_id=151935),
    "synthetic:moe-48l": ModelConfig(vocab_size=151936, hidden_size=2048, num_layers=48, num_attention_heads=32,
                                     num_key_value_heads=4, head_dim=128, intermediate_size=0, num_experts=128,
                                     num_experts_per_token=8, moe_intermediate_size=768, mask_token_id=151935,
                                     family="diffusion_gemma"),
    "synthetic:dflash-draft-5l": ModelConfig(vocab_size=151936, hidden_size=4096, num_layers=5,
                                             num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                                             intermediate_size=12288, mask_token_id=151935, family="dflash"),
}


def model_config_from_run_spec(spec) -> ModelConfig:
    """Preset named by `model.id` (when it is one) overridden by explicit shape fields."""
    m = spec.model
    base = PRESETS.get(m.id)
    if base is None:
        from .hf_loader import load_hf_config, pretrained_directory

        local = pretrained_directory(m.id)
        if local is not None:
            # a local Hugging Face checkpoint: its config.json gives the architecture (and, unless
            # model.random_init is set, the training session loads its weights)
            base = load_hf_config(local)
    if base is None:
        if not m.random_init:
            raise ValueError(
                f"model.id {m.id!r} is neither a built-in preset ({', '.join(PRESETS)}) nor a local checkpoint "
                "directory with a config.json; give a local path (nothing is downloaded), or set "
                "model.random_init=true with explicit shape fields")
        need = ("vocab_size", "hidden_size", "num_layers", "num_attention_heads")
        missing = [n for n in need if getattr(m, n) is None]
        if missing:
            raise ValueError(f"model.random_init needs model.{', model.'.join(missing)}")
        heads = m.num_attention_heads
        base = ModelConfig(vocab_size=m.vocab_size, hidden_size=m.hidden_size, num_layers=m.num_layers,
                           num_attention_heads=heads, num_key_value_heads=m.num_key_value_heads or heads,
                           head_dim=m.head_dim or m.hidden_size // heads,
                           intermediate_size=m.intermediate_size or 4 * m.hidden_size)
    over = {}
    for name in ("vocab_size", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                 "intermediate_size", "rope_theta", "partial_rotary_factor", "mask_token_id", "num_experts", "num_experts_per_token",
                 "moe_intermediate_size", "moe_shared_intermediate_size", "full_attention_interval", "linear_num_key_heads",
                 "linear_num_value_heads", "linear_key_head_dim", "linear_value_head_dim", "linear_conv_kernel",
                 "sliding_window", "sliding_window_pattern"):
        v = getattr(m, name)
        if v is not None:
            over[name] = v
    if m.num_layers is not None:
        over["num_layers"] = m.num_layers
    if m.max_layers is not None:
        over["num_layers"] = min(over.get("num_layers", base.num_layers), m.max_layers)
    over["qk_norm"] = m.qk_norm and base.qk_norm
    cfg = replace(base, **over)
    if cfg.mask_token_id is None and m.mask_token:
        # model.mask_token names the mask token; its id comes from the tokenizer that ships with the checkpoint
        import os

        if not os.path.isdir(m.id):
            raise ValueError(f"model.mask_token={m.mask_token!r} needs a local checkpoint directory with a tokenizer "
                             "(model.id); give model.mask_token_id instead")
        from transformers import AutoTokenizer

        tid = AutoTokenizer.from_pretrained(m.id).convert_tokens_to_ids(m.mask_token)
        if tid is None or tid < 0:
            raise ValueError(f"the tokenizer of {m.id} has no token {m.mask_token!r}")
        cfg = replace(cfg, mask_token_id=int(tid))
    if cfg.mask_token_id is None:
        cfg = replace(cfg, mask_token_id=cfg.vocab_size - 1)
    return cfg

PRESETS["synthetic:tiny-qwen3_8"] = ModelConfig(vocab_size=1024, hidden_size=128, num_layers=4, num_attention_heads=4,
                                                num_key_value_heads=2, head_dim=32, intermediate_size=256,
                                                mask_token_id=1023, family="qwen3_8", full_attention_interval=4,
                                                linear_num_key_heads=2, linear_num_value_heads=4,
                                                linear_key_head_dim=16, linear_value_head_dim=16)
PRESETS["synthetic:tiny-qwen3_8-hd128"] = ModelConfig(vocab_size=2048, hidden_size=256, num_layers=2,
                                                      num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                                                      intermediate_size=512, mask_token_id=2047, family="qwen3_8",
                                                      full_attention_interval=2, linear_num_key_heads=2,
                                                      linear_num_value_heads=4, linear_key_head_dim=64,
                                                      linear_value_head_dim=64)
PRESETS["synthetic:tiny-moe"] = ModelConfig(vocab_size=1024, hidden_size=128, num_layers=2, num_attention_heads=4,
                                            num_key_value_heads=2, head_dim=64, intermediate_size=0, num_experts=8,
                                            num_experts_per_token=2, moe_intermediate_size=96, mask_token_id=1023,
                                            family="diffusion_gemma")
PRESETS["synthetic:tiny-moe-hd128"] = ModelConfig(vocab_size=2048, hidden_size=256, num_layers=2, num_attention_heads=2,
                                                  num_key_value_heads=1, head_dim=128, intermediate_size=0,
                                                  num_experts=8, num_experts_per_token=2, moe_intermediate_size=128,
                                                  mask_token_id=2047, family="diffusion_gemma")

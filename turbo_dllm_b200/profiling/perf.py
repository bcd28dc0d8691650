"""FLOP models, hardware peaks and MFU.

Megatron-convention model FLOPs per optimizer step (no recompute counted):
    L·[6·rows·(h·(q+2kv) + q·h) + 12·pairs·q_dim_per_pair + 6·rows·3·h·i] + 6·vocab_rows·h·V
with `rows` the executed transformer rows (noisy + clean), `pairs` the exactly visible
query-key pairs and `vocab_rows` the rows that reach the LM head.

Counterparts: hardware presets and MegatronTransformerFlops / FastDLLMv2TransformerFlops
(dllm_parallel/core/profiling/perf.py:50-113, :161-381), exact pair counters (:872-878),
`model_flops_utilization_pct` (:855-869). The reference has no B200 preset; this module has,
plus the option to use peaks measured on the machine.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

from ..models.config import ModelConfig

HARDWARE_PEAK_TFLOPS_BF16 = {
    "B200": 2250.0, "H100 SXM": 989.0, "H100 PCIe": 756.0, "H200": 989.0, "A100": 312.0,
}


def hardware_peak_tflops(device_name: str) -> float:
    for key, v in HARDWARE_PEAK_TFLOPS_BF16.items():
        if key.split()[0] in device_name:
            return v
    raise ValueError(f"no bf16 peak preset for {device_name!r}; pass peak_tflops explicitly")


def measured_peaks(path: str | None = None) -> dict | None:
    """Peaks measured on this machine (JSON with bf16_tflops, bf16_tflops_sustained, hbm_gbs)."""
    cand = path or os.environ.get("TDLLM_MEASURED_PEAKS")
    if cand is None:
        here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        cand = os.path.join(here, "MEASURED_PEAKS.json")
    try:
        with open(cand) as f:
            return json.load(f)
    except OSError:
        return None


def block_diffusion_pairs(seq_len: int, block_size: int, noisy_views: int = 1, window: int | None = None) -> int:
    """Exactly visible (query, key) pairs of one sequence: every noisy row sees its own block plus the clean tokens
    before it, a clean row the clean tokens up to the end of its block. With `window` (sliding-window layers) the
    clean part of both is cut to the last `window` positions before that point (`ops/attention.py::block_diffusion_layout`)."""
    B = seq_len // block_size
    bs = block_size
    if window is None:
        noisy = bs * bs * B * (B + 1) // 2          # own block (B·bs²) + clean prefix (bs²·B(B-1)/2)
        clean = bs * bs * B * (B + 1) // 2
        return noisy_views * noisy + clean
    noisy = sum(bs * (bs + min(b * bs, window)) for b in range(B))
    clean = sum(bs * min((b + 1) * bs, window) for b in range(B))
    return noisy_views * noisy + clean


def model_attention_pairs(cfg: ModelConfig, seq_len: int, block_size: int, noisy_views: int = 1) -> float:
    """Visible pairs per layer, averaged over the layers (sliding-window layers see fewer): the `pairs` argument of
    `transformer_step_flops` for one sequence."""
    full = block_diffusion_pairs(seq_len, block_size, noisy_views)
    if not cfg.has_sliding_layers:
        return float(full)
    win = block_diffusion_pairs(seq_len, block_size, noisy_views, cfg.sliding_window)
    n_win = sum(cfg.layer_window(i) is not None for i in range(cfg.num_layers))
    return (n_win * win + (cfg.num_layers - n_win) * full) / cfg.num_layers


@dataclass(frozen=True)
class StepFlops:
    dense: float
    attention: float
    head: float

    @property
    def total(self) -> float:
        return self.dense + self.attention + self.head


def transformer_step_flops(cfg: ModelConfig, *, rows: int, pairs: int, vocab_rows: int) -> StepFlops:
    h = cfg.hidden_size
    if cfg.is_moe:
        ffn = (3 * h * cfg.moe_intermediate_size * cfg.num_experts_per_token + h * cfg.num_experts
               + 3 * h * cfg.moe_shared_intermediate_size)
    else:
        ffn = 3 * h * cfg.intermediate_size
    per_row = h * cfg.qkv_dim + cfg.q_dim * h + ffn
    if cfg.is_hybrid:
        # linear-attention layers: fused input projection + output projection + MLP per row, and per row
        # and value head the recurrence products (state read for u and o, state write, the intra-chunk
        # C x C terms are small next to them): about 3 · Dk · Dv multiply-adds forward
        n_full = sum(cfg.layer_kind(i) == "full_attention" for i in range(cfg.num_layers))
        n_lin = cfg.num_layers - n_full
        lin_row = h * cfg.linear_in_dim + cfg.linear_value_dim * h + ffn
        full_row = per_row + h * cfg.q_dim                       # output gate
        dense = 6.0 * rows * (n_full * full_row + n_lin * lin_row)
        recurrence = 6.0 * rows * n_lin * cfg.linear_num_value_heads * 3 * cfg.linear_key_head_dim * cfg.linear_value_head_dim
        attention = 12.0 * pairs * cfg.q_dim * n_full + recurrence
        return StepFlops(dense, attention, 6.0 * vocab_rows * h * cfg.vocab_size)
    dense = 6.0 * rows * per_row * cfg.num_layers
    attention = 12.0 * pairs * cfg.q_dim * cfg.num_layers      # 4·pairs·D per head fwd, ×3 fwd+bwd
    head = 6.0 * vocab_rows * h * cfg.vocab_size
    return StepFlops(dense, attention, head)


def model_flops_utilization_pct(flops_per_step: float, step_seconds: float, world_size: int,
                                peak_tflops: float) -> float:
    return 100.0 * flops_per_step / (step_seconds * world_size * peak_tflops * 1e12)


def causal_pairs(seq_len: int) -> int:
    return seq_len * (seq_len + 1) // 2


def dflash_step_flops(draft: ModelConfig, target: ModelConfig, *, seq_len: int, block_size: int, anchors: int,
                      num_target_layers: int, batch: int = 1, online_target: bool = True, supervised_rows: int | None = None,
                      mean_context: float | None = None, loss: str = "speculators_kl", context_rows: int | None = None,
                      draft_vocab_size: int | None = None) -> StepFlops:
    """Model FLOPs of one drafter-distillation step on `batch` sequences (Megatron convention: 2 per multiply-add,
    trainable matrices x3 for forward + both gradients, frozen ones x1 forward, or x2 where only the input gradient
    is taken). Parts: the frozen target's causal forward (online features only); the conditioning projection of the
    tapped target layers on the context rows; the drafter's layers on `anchors * block_size` draft rows with K|V
    projections on draft + context rows; attention of every draft row over its own block and its context
    (`mean_context` keys on average: half the sequence for uniform anchors); the frozen head on the supervised rows
    (student forward + input gradient, teacher forward for the KL loss).
    Counterpart of DFlashTransformerFlops (dllm_parallel/core/profiling/perf.py:630-852)."""
    L, bs = seq_len, block_size
    rows_d = anchors * bs
    rows_c = L if context_rows is None else context_rows
    sup = rows_d if supervised_rows is None else supervised_rows
    ctx = L / 2.0 if mean_context is None else mean_context
    V = draft_vocab_size or target.vocab_size
    h, ht = draft.hidden_size, target.hidden_size
    dense = 0.0
    attention = 0.0
    if online_target:
        per_row = ht * target.qkv_dim + target.q_dim * ht + 3 * ht * target.intermediate_size
        dense += 2.0 * L * per_row * target.num_layers
        attention += 4.0 * causal_pairs(L) * target.q_dim * target.num_layers
    dense += 6.0 * rows_c * (num_target_layers * ht) * h                       # conditioning projection
    per_draft_row = h * draft.q_dim + draft.q_dim * h + 3 * h * draft.intermediate_size
    per_key_row = h * 2 * draft.kv_dim
    dense += 6.0 * draft.num_layers * (rows_d * per_draft_row + (rows_d + rows_c) * per_key_row)
    attention += 12.0 * rows_d * (bs + ctx) * draft.q_dim * draft.num_layers
    head = 4.0 * sup * h * V                                                    # student logits and their input gradient
    if loss == "speculators_kl":
        head += 2.0 * sup * ht * V                                              # teacher logits
    return StepFlops(dense * batch, attention * batch, head * batch)


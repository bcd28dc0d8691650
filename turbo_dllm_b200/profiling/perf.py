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
    """Visible (query, key) pairs of one sequence: every noisy view sees its own block plus the clean
    blocks before it; the clean copy is block-causal."""
    B = seq_len // block_size
    bs2 = block_size * block_size
    noisy = bs2 * B * (B + 1) // 2          # own block (B·bs²) + clean prefix (bs²·B(B-1)/2)
    clean = bs2 * B * (B + 1) // 2
    return noisy_views * noisy + clean


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

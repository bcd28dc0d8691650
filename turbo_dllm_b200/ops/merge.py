"""Online-softmax merge of attention results computed over disjoint key shards.

State per (row, head): fp32 numerator N[D], running max m, denominator l.
  merge:    m' = max(m, lse_s);  N' = e^{m-m'}·N + e^{lse_s-m'}·o_s;  l' = e^{m-m'}·l + e^{lse_s-m'}
  finalize: out = N / l, lse = m + log l          (rows that saw no key: out = 0, lse = -inf)
  backward of one shard: go_s = go·w, dlse_s = w·Σ_d go_d (o_s,d − out_d), w = e^{lse_s − lse}
The merge is order-invariant in fp32. Kernels: csrc/optim_loss.cu; torch versions are the oracle.

Counterparts: dllm_parallel/core/csrc/cp_fusion/cp_fusion_cuda.cu:24-230, dflash_cp_fusion_cuda.cu:23-103,
`merge_attention_stats` (dllm_parallel/core/attention/cp_backend.py:226-273).
"""
from __future__ import annotations

import torch

from ..kernels import native
from ._util import ptr, stream, use_native


class MergeState:
    """out/lse layouts: o_s [rows, H, D], lse_s [H, rows_padded] (attention kernel layout)."""

    def __init__(self, rows: int, heads: int, dim: int, device):
        self.rows, self.heads, self.dim = rows, heads, dim
        self.num = torch.zeros(rows, heads, dim, dtype=torch.float32, device=device)
        self.m = torch.full((rows, heads), float("-inf"), dtype=torch.float32, device=device)
        self.l = torch.zeros(rows, heads, dtype=torch.float32, device=device)
        self.first = True

    def merge(self, o_s: torch.Tensor, lse_s: torch.Tensor) -> None:
        lse_rh = lse_s[:, : self.rows].t().contiguous()          # [rows, H]
        if use_native(o_s):
            native.check(native.lib().tdllm_attn_merge(ptr(self.num), ptr(self.m), ptr(self.l), ptr(o_s.contiguous()),
                                                       ptr(lse_rh), self.rows * self.heads, self.dim, int(self.first),
                                                       stream()), "attn_merge")
        else:
            m1 = torch.maximum(self.m, lse_rh)
            a = torch.where(torch.isinf(self.m), torch.zeros_like(m1), torch.exp(self.m - m1))
            b = torch.where(torch.isinf(lse_rh), torch.zeros_like(m1), torch.exp(lse_rh - m1))
            self.num = a[..., None] * self.num + b[..., None] * o_s.float()
            self.l = a * self.l + b
            self.m = m1
        self.first = False

    def finalize(self, dtype) -> tuple[torch.Tensor, torch.Tensor]:
        """Returns out [rows, H, D] and lse [H, rows]."""
        if self.num.is_cuda and dtype == torch.bfloat16:
            out = torch.empty(self.rows, self.heads, self.dim, dtype=dtype, device=self.num.device)
            lse = torch.empty(self.rows, self.heads, dtype=torch.float32, device=self.num.device)
            native.check(native.lib().tdllm_attn_merge_finalize(ptr(self.num), ptr(self.m), ptr(self.l), ptr(out),
                                                                ptr(lse), self.rows * self.heads, self.dim, stream()),
                         "attn_merge_finalize")
            return out, lse.t().contiguous()
        inv = torch.where(self.l > 0, 1.0 / self.l, torch.zeros_like(self.l))
        out = (self.num * inv[..., None]).to(dtype)
        lse = torch.where(self.l > 0, self.m + torch.log(self.l), torch.full_like(self.l, float("-inf")))
        return out, lse.t().contiguous()


def merge_backward(go, out, lse, o_s, lse_s):
    """Per-shard upstream gradients. go/out/o_s [rows,H,D]; lse/lse_s [H, rows]. Returns (go_s, dlse_s [H, rows])."""
    rows, H, D = go.shape
    lse_rh, lse_s_rh = lse[:, :rows].t().contiguous(), lse_s[:, :rows].t().contiguous()
    if use_native(go):
        go_s = torch.empty_like(go)
        dlse = torch.empty(rows, H, dtype=torch.float32, device=go.device)
        native.check(native.lib().tdllm_attn_merge_bwd(ptr(go.contiguous()), ptr(out.contiguous()), ptr(lse_rh),
                                                       ptr(o_s.contiguous()), ptr(lse_s_rh), ptr(go_s), ptr(dlse),
                                                       rows * H, D, stream()), "attn_merge_bwd")
        return go_s, dlse.t().contiguous()
    w = torch.where(torch.isinf(lse_s_rh) | torch.isinf(lse_rh), torch.zeros_like(lse_rh), torch.exp(lse_s_rh - lse_rh))
    go_s = (go.float() * w[..., None]).to(go.dtype)
    dlse = w * (go.float() * (o_s.float() - out.float())).sum(-1)
    return go_s, dlse.t().contiguous()

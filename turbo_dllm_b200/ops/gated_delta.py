"""Gated delta rule (Gated DeltaNet linear attention) with states at requested boundaries.

Per head, with a state S in R^{Dk x Dv}, one token does

    S <- exp(g_t) * S                      (g_t <= 0: log decay)
    u_t = beta_t * (v_t - S^T k_t)         (delta-rule correction of the value)
    S <- S + k_t u_t^T
    o_t = scale * S^T q_t

`gated_delta_reference` runs exactly this recurrence token by token in fp32: it is the oracle.
`gated_delta_chunked` is the form that trains: the sequence is cut into chunks of C tokens, all the
per-chunk quantities are batched matrix products, and only the state is carried from chunk to chunk.
With gamma_i the running sum of g inside a chunk and A_ij = beta_i exp(gamma_i - gamma_j) (k_i . k_j)
for j < i, the corrected values of a chunk that starts from state S0 are

    U = T (beta V) - [T (beta exp(gamma) K)] S0,          T = (I + A)^-1  (unit lower triangular)

so that S_C = exp(gamma_C) S0 + sum_i exp(gamma_C - gamma_i) k_i u_i^T and
o_i = scale (exp(gamma_i) q_i^T S0 + sum_{j<=i} exp(gamma_i - gamma_j) (q_i . k_j) u_j).
Every step is a differentiable torch op, so the states handed out at chunk boundaries carry gradients
back into the sequence that produced them: a noisy block of a block-diffusion batch starts from the
state of the clean prefix before it, and its loss reaches the clean tokens through that state.

Block-diffusion use (`models/hybrid.py`): the clean rows run once over the whole sequence with
`chunk = block size`, which yields the state in front of every block; the noisy blocks then run as
independent one-chunk sequences from those states.

Reference counterparts: dllm_parallel/core/kernels/gated_delta_boundaries.py:93-359 (autograd function
with differentiable boundary states, chunk 64), dllm_parallel/core/kernels/gated_delta_boundary.py:65
and :435 (the state recurrence and its backward), dllm_parallel/core/models/backbones/qwen3_8/model.py:2084-2125
(gate = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b), q and k L2-normalised, scale Dk^-1/2).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..kernels import native

MAX_CHUNK = 64

native.register_signatures({
    "tdllm_gdn_scan_fwd": (native.c_int, [native.c_void_p] * 11 + [native.c_int] * 5 + [native.c_void_p]),
    "tdllm_gdn_scan_bwd": (native.c_int, [native.c_void_p] * 17 + [native.c_int] * 5 + [native.c_void_p]),
})


def _native_scan_ok(t: torch.Tensor, C: int, Dk: int, Dv: int) -> bool:
    """The sm_100a scan kernel handles fp32 CUDA tensors with C <= 64, Dk <= 128 (multiple of 8) and Dv a
    multiple of 32; `TDLLM_GDN_SCAN=torch` keeps the batched-product loop (the oracle of the kernel)."""
    import os

    if not t.is_cuda or os.environ.get("TDLLM_GDN_SCAN", "native") == "torch":
        return False
    return C <= 64 and Dk <= 128 and Dk % 8 == 0 and Dv % 32 == 0


class _StateScan(torch.autograd.Function):
    """The sequential part of the chunked rule as one kernel per direction
    (`csrc/gated_delta_scan.cu`). Inputs are laid out [B, H, N, C, .]; returns
    (o [B, H, N, C, Dv], final state [B, H, Dk, Dv], states in front of every chunk [B, H, N, Dk, Dv])."""

    @staticmethod
    def forward(ctx, u_tilde, w, qk, q_in, k_out, total, s0):
        from ..kernels import native
        from ._util import ptr, stream

        u_tilde, w, qk, q_in, k_out, total = (t.contiguous() for t in (u_tilde, w, qk, q_in, k_out, total))
        B, H, N, C, Dv = u_tilde.shape
        Dk = w.shape[-1]
        s0c = None if s0 is None else s0.contiguous()
        o = torch.empty_like(u_tilde)
        u = torch.empty_like(u_tilde)
        states = torch.empty(B, H, N, Dk, Dv, dtype=torch.float32, device=w.device)
        s_final = torch.empty(B, H, Dk, Dv, dtype=torch.float32, device=w.device)
        rc = native.lib().tdllm_gdn_scan_fwd(ptr(u_tilde), ptr(w), ptr(qk), ptr(q_in), ptr(k_out), ptr(total), ptr(s0c),
                                             ptr(o), ptr(u), ptr(states), ptr(s_final), B * H, N, C, Dk, Dv, stream())
        native.check(rc, "gdn_scan_fwd")
        ctx.save_for_backward(w, qk, q_in, k_out, total, states, u)
        ctx.has_s0 = s0 is not None
        ctx.set_materialize_grads(False)
        return o, s_final, states

    @staticmethod
    def backward(ctx, d_o, d_sfinal, d_states):
        from ..kernels import native
        from ._util import ptr, stream

        w, qk, q_in, k_out, total, states, u = ctx.saved_tensors
        B, H, N, C, Dk = w.shape
        Dv = u.shape[-1]
        sl = Dv // 32
        dev = w.device
        d_o = torch.zeros_like(u) if d_o is None else d_o.contiguous().float()
        d_sfinal = None if d_sfinal is None else d_sfinal.contiguous().float()
        d_states = None if d_states is None else d_states.contiguous().float()
        d_ut = torch.empty_like(u)
        d_w = torch.empty(B, H, N, sl, C, Dk, dtype=torch.float32, device=dev)
        d_qi, d_ko = torch.empty_like(d_w), torch.empty_like(d_w)
        d_qk = torch.empty(B, H, N, sl, C, C, dtype=torch.float32, device=dev)
        d_total = torch.empty(B, H, N, sl, dtype=torch.float32, device=dev)
        d_s0 = torch.empty(B, H, Dk, Dv, dtype=torch.float32, device=dev)
        rc = native.lib().tdllm_gdn_scan_bwd(ptr(w), ptr(qk), ptr(q_in), ptr(k_out), ptr(total), ptr(states), ptr(u),
                                             ptr(d_o), ptr(d_states), ptr(d_sfinal), ptr(d_ut), ptr(d_w), ptr(d_qk),
                                             ptr(d_qi), ptr(d_ko), ptr(d_total), ptr(d_s0), B * H, N, C, Dk, Dv,
                                             stream())
        native.check(rc, "gdn_scan_bwd")
        return (d_ut, d_w.sum(3), d_qk.sum(3), d_qi.sum(3), d_ko.sum(3), d_total.sum(3),
                d_s0 if ctx.has_s0 else None)


def gdn_gate(a: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor) -> torch.Tensor:
    """Log decay per token and head: -exp(A_log) * softplus(a + dt_bias), always <= 0. fp32."""
    return -torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float())


def l2_normalize(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    x = x.float()
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def expand_key_heads(x: torch.Tensor, value_heads: int) -> torch.Tensor:
    """[B, T, Hk, D] -> [B, T, Hv, D]: every key head serves Hv / Hk consecutive value heads."""
    hk = x.shape[2]
    if hk == value_heads:
        return x
    if value_heads % hk:
        raise ValueError(f"value heads ({value_heads}) must be a multiple of key heads ({hk})")
    return x.repeat_interleave(value_heads // hk, dim=2)


def gated_delta_reference(q, k, v, g, beta, *, scale: float | None = None, initial_state=None,
                          boundaries: tuple[int, ...] = ()):
    """Token-by-token recurrence in fp32.

    q, k: [B, T, H, Dk] (already normalised), v: [B, T, H, Dv], g, beta: [B, T, H].
    Returns (o [B, T, H, Dv], final state [B, H, Dk, Dv], states in front of the tokens listed in
    `boundaries` stacked as [B, len(boundaries), H, Dk, Dv]; boundary T means the final state)."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    scale = 1.0 / math.sqrt(Dk) if scale is None else scale
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    S = q.new_zeros(B, H, Dk, Dv) if initial_state is None else initial_state.float()
    outs, kept = [], {}
    for t in range(T):
        if t in boundaries:
            kept[t] = S
        S = S * torch.exp(g[:, t])[..., None, None]
        u = beta[:, t][..., None] * (v[:, t] - torch.einsum("bhkv,bhk->bhv", S, k[:, t]))
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, t], u)
        outs.append(scale * torch.einsum("bhkv,bhk->bhv", S, q[:, t]))
    if T in boundaries:
        kept[T] = S
    states = (torch.stack([kept[t] for t in boundaries], dim=1) if boundaries
              else q.new_zeros(B, 0, H, Dk, Dv))
    return torch.stack(outs, dim=1), S, states


def chunk_size_for(block_size: int) -> int:
    """Largest chunk (<= 64 tokens) that puts a chunk boundary in front of every block."""
    if block_size <= MAX_CHUNK:
        return block_size
    for c in range(MAX_CHUNK, 0, -1):
        if block_size % c == 0:
            return c
    return 1


def _chunk_terms(q, k, v, g, beta, scale):
    """Everything that does not depend on the carried state, for all chunks at once.
    Inputs are [B, N, C, H, .] (N chunks of C tokens). Returns tensors laid out [B, H, N, C, .]."""
    q, k, v = (t.permute(0, 3, 1, 2, 4) for t in (q, k, v))          # [B, H, N, C, D]
    g, beta = (t.permute(0, 3, 1, 2) for t in (g, beta))              # [B, H, N, C]
    C = q.shape[3]
    gamma = g.cumsum(-1)
    diff = gamma[..., :, None] - gamma[..., None, :]                  # gamma_i - gamma_j
    idx = torch.arange(C, device=q.device)
    strict = idx[:, None] > idx[None, :]
    causal = idx[:, None] >= idx[None, :]
    neg = torch.finfo(torch.float32).min
    decay_strict = torch.exp(diff.masked_fill(~strict, neg)) * strict
    decay_causal = torch.exp(diff.masked_fill(~causal, neg)) * causal
    kk = k @ k.transpose(-1, -2)
    A = beta[..., None] * decay_strict * kk
    eye = torch.eye(C, device=q.device, dtype=q.dtype)
    rhs = torch.cat([beta[..., None] * v, (beta * torch.exp(gamma))[..., None] * k], dim=-1)
    # T = (I + A)^-1 once per chunk (a C x C solve), then one batched product with the wide right-hand side:
    # batched triangular solves with hundreds of right-hand-side columns are far slower than the product
    t_inv = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False, unitriangular=True)
    sol = t_inv @ rhs
    Dv = v.shape[-1]
    u_tilde, w = sol[..., :Dv], sol[..., Dv:]                         # [.., C, Dv], [.., C, Dk]
    qk = (q @ k.transpose(-1, -2)) * decay_causal * scale             # intra-chunk scores
    q_in = q * (torch.exp(gamma)[..., None] * scale)                  # reads the incoming state
    k_out = k * torch.exp(gamma[..., -1:, None] - gamma[..., None])   # writes into the outgoing state
    total = torch.exp(gamma[..., -1])                                 # decay of the incoming state
    return u_tilde, w, qk, q_in, k_out, total


def gated_delta_chunked(q, k, v, g, beta, *, scale: float | None = None, initial_state=None,
                        chunk: int = MAX_CHUNK, return_states: bool = False):
    """Chunked gated delta rule (see the module text). T must be a multiple of `chunk`.

    Returns (o [B, T, H, Dv] fp32, final state [B, H, Dk, Dv] fp32, states) where `states`
    ([B, T / chunk, H, Dk, Dv], the state in front of every chunk) is None unless `return_states`."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    if T % chunk:
        raise ValueError(f"sequence length {T} is not a multiple of the chunk size {chunk}")
    scale = 1.0 / math.sqrt(Dk) if scale is None else scale
    N = T // chunk
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    q, k, v = (t.reshape(B, N, chunk, H, t.shape[-1]) for t in (q, k, v))
    g, beta = (t.reshape(B, N, chunk, H) for t in (g, beta))
    u_tilde, w, qk, q_in, k_out, total = _chunk_terms(q, k, v, g, beta, scale)
    if _native_scan_ok(u_tilde, chunk, Dk, Dv):
        s0 = None if initial_state is None else initial_state.float()
        o, S, st = _StateScan.apply(u_tilde, w, qk, q_in, k_out, total, s0)
        o = o.permute(0, 2, 3, 1, 4).reshape(B, T, H, Dv)
        return o, S, (st.permute(0, 2, 1, 3, 4) if return_states else None)
    S = q.new_zeros(B, H, Dk, Dv) if initial_state is None else initial_state.float()
    outs, states = [], []
    for n in range(N):
        if return_states:
            states.append(S)
        u = u_tilde[:, :, n] - w[:, :, n] @ S                          # [B, H, C, Dv]
        outs.append(q_in[:, :, n] @ S + qk[:, :, n] @ u)
        S = S * total[:, :, n, None, None] + k_out[:, :, n].transpose(-1, -2) @ u
    o = torch.stack(outs, dim=2)                                       # [B, H, N, C, Dv]
    o = o.permute(0, 2, 3, 1, 4).reshape(B, T, H, Dv)
    return o, S, (torch.stack(states, dim=1) if return_states else None)


def causal_conv_reference(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                          history: torch.Tensor | None = None) -> torch.Tensor:
    """Depth-wise causal convolution followed by SiLU.

    x: [B, T, Ch], weight: [Ch, W] (tap W-1 multiplies the current token), history: [B, W-1, Ch]
    inputs in front of the first token (zeros when None). Returns [B, T, Ch] in x's dtype."""
    B, T, Ch = x.shape
    W = weight.shape[1]
    if history is None:
        history = x.new_zeros(B, W - 1, Ch)
    xp = torch.cat([history.to(x.dtype), x], dim=1).transpose(1, 2)    # [B, Ch, T + W - 1]
    y = F.conv1d(xp.float(), weight.float()[:, None, :], None if bias is None else bias.float(), groups=Ch)
    return F.silu(y).transpose(1, 2).to(x.dtype)


def conv_history_at(x: torch.Tensor, boundaries: torch.Tensor, width: int) -> torch.Tensor:
    """The `width - 1` inputs in front of every boundary token, zeros before the sequence start.

    x: [B, T, Ch]; boundaries: [n] token indices. Returns [B, n, width - 1, Ch]
    (dllm_parallel/core/models/backbones/qwen3_8/model.py:2127-2156 keeps `width` columns, of which the
    convolution reads the last width - 1)."""
    hist = torch.arange(-(width - 1), 0, device=x.device)
    idx = boundaries.to(x.device)[:, None] + hist[None, :]
    valid = (idx >= 0).to(x.dtype)
    got = x.index_select(1, idx.clamp_min(0).reshape(-1)).view(x.shape[0], idx.shape[0], width - 1, x.shape[2])
    return got * valid[None, :, :, None]


def gated_rmsnorm(o: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the value dimension of each head, gated by SiLU(z). o, z: [..., Dv]."""
    o = o.float()
    y = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * weight.float()
    return y * F.silu(z.float())

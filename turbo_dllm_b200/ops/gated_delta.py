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

MAX_CHUNK = 64


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
    sol = torch.linalg.solve_triangular(eye + A, rhs, upper=False, unitriangular=True)
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

"""Online-softmax merge: order invariance, equivalence with attention over the union of keys,
and the per-shard backward identities (CPU oracle; the GPU kernels are checked against it)."""
import math

import pytest
import torch

from turbo_dllm_b200.ops.attention import attention_reference, block_diffusion_layout
from turbo_dllm_b200.ops.merge import MergeState, merge_backward


def _shards(seed=0):
    torch.manual_seed(seed)
    L, bs, H, D = 96, 16, 2, 16
    pos = torch.arange(L)
    q = torch.randn(2 * L, H, D)
    full = block_diffusion_layout(pos, pos // bs, pos, bs)
    kn, vn = torch.randn(L, 1, D), torch.randn(L, 1, D)       # noisy keys
    kc, vc = torch.randn(L, 1, D), torch.randn(L, 1, D)       # clean keys
    ref, ref_lse = attention_reference(q, torch.cat([kn, kc]), torch.cat([vn, vc]), full)
    parts = []
    chunks = [pos[:40], pos[40:64], pos[64:]]
    for i, ch in enumerate(chunks):
        lay = block_diffusion_layout(pos, pos // bs, pos, bs, key_clean_pos=ch)
        if i == 0:
            k, v = torch.cat([kn, kc[ch]]), torch.cat([vn, vc[ch]])
        else:   # later shards carry clean keys only
            lay.k_code = lay.k_code[L:]
            k, v = kc[ch], vc[ch]
        parts.append(attention_reference(q, k, v, lay))
    return q, ref, ref_lse, parts


def test_merge_equals_attention_over_all_keys_in_any_order():
    q, ref, ref_lse, parts = _shards()
    for order in ([0, 1, 2], [2, 0, 1], [1, 2, 0]):
        st = MergeState(q.shape[0], q.shape[1], q.shape[2], "cpu")
        for i in order:
            st.merge(*parts[i])
        out, lse = st.finalize(torch.float32)
        assert torch.allclose(out, ref, atol=1e-5)
        assert torch.allclose(lse, ref_lse, atol=1e-5)


def test_merge_backward_matches_autograd():
    q, ref, ref_lse, parts = _shards(1)
    outs = [o.clone().requires_grad_() for o, _ in parts]
    lses = [l.clone().requires_grad_() for _, l in parts]
    rows = q.shape[0]
    m = torch.stack([l.t() for l in lses]).max(0).values
    ws = [torch.exp(l.t() - m) for l in lses]
    num = sum(w[..., None] * o for w, o in zip(ws, outs))
    den = sum(ws)
    out = num / den[..., None]
    go = torch.randn_like(out)
    (out * go).sum().backward()
    lse = (m + torch.log(den)).t().detach()
    for o, l in zip(outs, lses):
        go_s, dlse_s = merge_backward(go, out.detach(), lse, o.detach(), l.detach())
        assert torch.allclose(go_s, o.grad, atol=1e-5)
        assert torch.allclose(dlse_s, l.grad, atol=1e-5)

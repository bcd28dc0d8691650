"""Gated delta rule: the chunked form against the token-by-token recurrence, boundary states and
their gradients, the causal convolution with history.

Modelled on the reference's DeltaNet-vs-recurrence tests (tests/unit/models/, Qwen3.8 DeltaNet
against a reference recurrence)."""
import math

import pytest
import torch

from turbo_dllm_b200.ops.gated_delta import (causal_conv_reference, chunk_size_for, conv_history_at,
                                              expand_key_heads, gated_delta_chunked, gated_delta_reference,
                                              gdn_gate, l2_normalize)


def _inputs(B, T, H, Dk, Dv, seed=0, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    q = l2_normalize(torch.randn(B, T, H, Dk, generator=g)).to(dtype)
    k = l2_normalize(torch.randn(B, T, H, Dk, generator=g)).to(dtype)
    v = torch.randn(B, T, H, Dv, generator=g).to(dtype)
    a = torch.randn(B, T, H, generator=g)
    gate = gdn_gate(a, torch.zeros(H), torch.zeros(H)).to(dtype)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g)).to(dtype)
    return q, k, v, gate, beta


@pytest.mark.parametrize("chunk", [4, 8, 32])
def test_chunked_matches_recurrence(chunk):
    q, k, v, g, beta = _inputs(2, 64, 3, 16, 8, dtype=torch.float32)
    s0 = torch.randn(2, 3, 16, 8) * 0.1
    o_ref, s_ref, _ = gated_delta_reference(q, k, v, g, beta, initial_state=s0)
    o, s, _ = gated_delta_chunked(q, k, v, g, beta, initial_state=s0, chunk=chunk)
    assert torch.allclose(o, o_ref, atol=2e-5, rtol=1e-4)
    assert torch.allclose(s, s_ref, atol=2e-5, rtol=1e-4)


def test_boundary_states_match_recurrence():
    q, k, v, g, beta = _inputs(1, 48, 2, 8, 8, seed=1, dtype=torch.float32)
    bounds = (0, 8, 16, 24, 32, 40)
    _, _, st_ref = gated_delta_reference(q, k, v, g, beta, boundaries=bounds)
    _, _, st = gated_delta_chunked(q, k, v, g, beta, chunk=8, return_states=True)
    assert st.shape == st_ref.shape
    assert torch.allclose(st, st_ref, atol=2e-5, rtol=1e-4)
    assert torch.count_nonzero(st[:, 0]) == 0


def test_gradients_through_boundary_states():
    """A loss on a block that starts from a boundary state reaches the tokens in front of the
    boundary, and the chunked gradients equal those of the recurrence."""
    torch.manual_seed(2)
    base = _inputs(1, 32, 2, 8, 4, seed=3, dtype=torch.float64)
    blk = _inputs(1, 8, 2, 8, 4, seed=4, dtype=torch.float64)

    def run(fn_clean, fn_block):
        leaves = [t.clone().requires_grad_(True) for t in base]
        o, _, st = fn_clean(*leaves)
        ob, _, _ = fn_block(*blk, st[:, 2])     # block that starts after 16 clean tokens
        (o.square().sum() + ob.square().sum()).backward()
        return [t.grad for t in leaves]

    ref = run(lambda *a: gated_delta_reference(*a, boundaries=(0, 8, 16, 24)),
              lambda q, k, v, g, b, s: gated_delta_reference(q, k, v, g, b, initial_state=s))
    got = run(lambda *a: gated_delta_chunked(*a, chunk=8, return_states=True),
              lambda q, k, v, g, b, s: gated_delta_chunked(q, k, v, g, b, initial_state=s, chunk=8))
    for r, c in zip(ref, got):
        assert torch.allclose(r.float(), c.float(), atol=1e-4, rtol=1e-3)
    # tokens after the boundary (16..31) get no gradient from the block's output; tokens before it do
    only_block = [t.clone().requires_grad_(True) for t in base]
    _, _, st = gated_delta_chunked(*only_block, chunk=8, return_states=True)
    ob, _, _ = gated_delta_chunked(*blk, initial_state=st[:, 2], chunk=8)
    ob.sum().backward()
    gv = only_block[2].grad
    assert gv[:, :16].abs().sum() > 0 and gv[:, 16:].abs().sum() == 0


def test_key_head_expansion_and_chunk_choice():
    x = torch.arange(2 * 3 * 2 * 4, dtype=torch.float32).view(2, 3, 2, 4)
    y = expand_key_heads(x, 6)
    assert y.shape == (2, 3, 6, 4)
    assert torch.equal(y[:, :, 0], x[:, :, 0]) and torch.equal(y[:, :, 2], x[:, :, 0])
    assert torch.equal(y[:, :, 3], x[:, :, 1])
    with pytest.raises(ValueError):
        expand_key_heads(x, 5)
    assert chunk_size_for(32) == 32 and chunk_size_for(64) == 64 and chunk_size_for(128) == 64
    assert chunk_size_for(96) == 48


def test_causal_conv_history():
    torch.manual_seed(5)
    x = torch.randn(2, 24, 6)
    w, b = torch.randn(6, 4), torch.randn(6)
    full = causal_conv_reference(x, w, b)
    # direct definition at one token
    t = 10
    want = torch.nn.functional.silu((x[:, t - 3:t + 1] * w.t()[None]).sum(1) + b)
    assert torch.allclose(full[:, t], want, atol=1e-5)
    # a block that starts at token 8 with the clean history equals the tail of the full run
    hist = conv_history_at(x, torch.tensor([0, 8, 16]), 4)
    assert hist.shape == (2, 3, 3, 6)
    assert torch.count_nonzero(hist[:, 0]) == 0
    blk = causal_conv_reference(x[:, 8:16], w, b, history=hist[:, 1])
    assert torch.allclose(blk, full[:, 8:16], atol=1e-5)


def test_gate_is_a_decay():
    a = torch.randn(4, 5, 3)
    g = gdn_gate(a, torch.randn(3), torch.randn(3))
    assert (g <= 0).all() and g.dtype == torch.float32
    assert math.isfinite(float(g.min()))

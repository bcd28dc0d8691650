"""The sm_100a state-scan kernels of the gated delta rule against the batched-product loop in fp32
PyTorch (same chunked algebra, so the comparison isolates the kernels), and against the
token-by-token recurrence."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, Dk, Dv, seed):
    from turbo_dllm_b200.ops.gated_delta import gdn_gate, l2_normalize

    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    q, k, v = l2_normalize(r(B, T, H, Dk)), l2_normalize(r(B, T, H, Dk)), r(B, T, H, Dv)
    gate = gdn_gate(r(B, T, H), torch.zeros(H, device="cuda"), torch.zeros(H, device="cuda"))
    beta = torch.sigmoid(r(B, T, H))
    s0 = r(B, H, Dk, Dv) * 0.1
    return [q, k, v, gate, beta, s0]


@pytest.mark.parametrize("B,T,H,Dk,Dv,chunk", [(2, 128, 3, 64, 64, 32), (1, 192, 2, 128, 128, 64), (3, 32, 2, 16, 32, 16)])
def test_scan_kernels_match_the_torch_loop(monkeypatch, B, T, H, Dk, Dv, chunk):
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.ops.gated_delta import gated_delta_chunked, gated_delta_reference

    base = _inputs(B, T, H, Dk, Dv, seed=B * 100 + T)
    go = torch.randn(B, T, H, Dv, device="cuda")
    gs = torch.randn(B, H, Dk, Dv, device="cuda") * 0.1
    gst = torch.randn(B, T // chunk, H, Dk, Dv, device="cuda") * 0.1

    def run(mode):
        monkeypatch.setenv("TDLLM_GDN_SCAN", mode)
        leaves = [t.clone().requires_grad_(True) for t in base]
        o, s, st = gated_delta_chunked(*leaves[:5], initial_state=leaves[5], chunk=chunk, return_states=True)
        ((o * go).sum() + (s * gs).sum() + (st * gst).sum()).backward()
        return [o.detach(), s.detach(), st.detach()] + [t.grad for t in leaves]

    want = run("torch")
    got = run("native")
    torch.cuda.synchronize()
    native.raise_on_device_error()
    names = ["o", "final", "states", "dq", "dk", "dv", "dg", "dbeta", "ds0"]
    for n, a, b in zip(names, got, want):
        err = (a - b).abs().max().item()
        ref = b.abs().max().item()
        assert err <= 2e-4 * max(ref, 1.0), (n, err, ref)
    # and the chunked result is the recurrence
    with torch.no_grad():
        o_ref, s_ref, _ = gated_delta_reference(*base[:5], initial_state=base[5])
    assert torch.allclose(got[0], o_ref, atol=5e-4, rtol=1e-3)
    assert torch.allclose(got[1], s_ref, atol=5e-4, rtol=1e-3)


def test_scan_without_initial_state_or_state_gradients():
    from turbo_dllm_b200.ops.gated_delta import gated_delta_chunked

    q, k, v, g, beta, _ = _inputs(1, 64, 2, 32, 32, seed=7)
    v = v.requires_grad_(True)
    o, s, st = gated_delta_chunked(q, k, v, g, beta, chunk=32)
    assert st is None
    o.sum().backward()
    assert torch.isfinite(v.grad).all() and v.grad.abs().sum() > 0

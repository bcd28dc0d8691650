"""RMSNorm, q/k-norm+RoPE and SwiGLU kernels vs fp32 PyTorch references (forward and backward)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("H", [256, 2048, 4096])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(H, with_res):
    from turbo_dllm_b200.ops.norm import rmsnorm

    torch.manual_seed(0)
    rows = 333
    x = torch.randn(rows, H, device="cuda").bfloat16().requires_grad_()
    r = torch.randn(rows, H, device="cuda").bfloat16().requires_grad_() if with_res else None
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
    y, h = rmsnorm(x, w, 1e-6, r)
    gy, gh = torch.randn_like(y), torch.randn_like(y)
    (y.float() * gy.float()).sum().backward(retain_graph=True) if not with_res else \
        ((y.float() * gy.float()).sum() + (h.float() * gh.float()).sum()).backward()
    xr = x.detach().float().requires_grad_()
    rr = r.detach().float().requires_grad_() if with_res else None
    wr = w.detach().float().requires_grad_()
    hr = xr + rr if with_res else xr
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    loss = (yr * gy.float()).sum()
    if with_res:
        loss = loss + (hr * gh.float()).sum()
    loss.backward()
    assert torch.allclose(y.float(), yr, rtol=2e-2, atol=2e-2)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)
    if with_res:
        assert torch.allclose(r.grad.float(), rr.grad, rtol=3e-2, atol=3e-2)
    assert torch.allclose(w.grad.float(), wr.grad, rtol=3e-2, atol=0.3)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("with_norm", [True, False])
def test_qk_norm_rope(D, with_norm):
    from turbo_dllm_b200.ops.rope import qk_norm_rope, qk_norm_rope_reference, rope_inv_freq

    torch.manual_seed(0)
    rows, Hq, Hkv = 257, 4, 2
    qkv = torch.randn(rows, (Hq + 2 * Hkv) * D, device="cuda").bfloat16().requires_grad_()
    pos = torch.randint(0, 100000, (rows,), device="cuda", dtype=torch.int32)
    inv = rope_inv_freq(D, 1e6, "cuda")
    qw = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16().requires_grad_() if with_norm else None
    kw = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16().requires_grad_() if with_norm else None
    out = qk_norm_rope(qkv, pos, inv, qw, kw, Hq, Hkv, D, 1e-6)
    g = torch.randn_like(out)
    out.backward(g)
    q2 = qkv.detach().float().requires_grad_()
    qw2 = qw.detach().float().requires_grad_() if with_norm else None
    kw2 = kw.detach().float().requires_grad_() if with_norm else None
    ref = qk_norm_rope_reference(q2, pos, inv, qw2, kw2, Hq, Hkv, D, 1e-6)
    ref.backward(g.float())
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=3e-2)
    assert torch.allclose(qkv.grad.float(), q2.grad, rtol=3e-2, atol=3e-2)
    if with_norm:
        assert torch.allclose(qw.grad.float(), qw2.grad, rtol=3e-2, atol=0.5)
        assert torch.allclose(kw.grad.float(), kw2.grad, rtol=3e-2, atol=0.5)


def test_swiglu():
    from turbo_dllm_b200.ops.activation import swiglu

    torch.manual_seed(0)
    gu = torch.randn(300, 2 * 768, device="cuda").bfloat16().requires_grad_()
    out = swiglu(gu)
    g = torch.randn_like(out)
    out.backward(g)
    r = gu.detach().float().requires_grad_()
    ref = torch.nn.functional.silu(r[:, 0::2]) * r[:, 1::2]
    ref.backward(g.float())
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    assert torch.allclose(gu.grad.float(), r.grad, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("views,shift", [(1, False), (2, True)])
def test_noising_kernel_matches_host_twin(views, shift):
    from turbo_dllm_b200.objectives.runtime import fused_corrupt

    torch.manual_seed(0)
    B, L, bs = 3, 256, 32
    x0 = torch.randint(0, 1000, (B, L), device="cuda")
    t = torch.rand(B, L // bs, device="cuda") * 0.9 + 0.1
    el = torch.rand(B, L, device="cuda") > 0.2
    kw = dict(block_size=bs, views=views, shift=shift, mask_id=1023, seed=0x1234567890ABCDEF, offset=7)
    xt, lab = fused_corrupt(x0, t, el, **kw)
    xt_ref, lab_ref = fused_corrupt(x0.cpu(), t.cpu(), el.cpu(), **kw)
    assert torch.equal(xt.cpu(), xt_ref) and torch.equal(lab.cpu(), lab_ref)
    frac = (xt == 1023).float().mean().item()
    assert 0.2 < frac < 0.8

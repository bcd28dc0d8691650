"""tcgen05 GEMM vs an fp32 PyTorch reference, all operand major-ness combinations and epilogues."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return A @ B


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 768, 320), (1000, 520, 136),
                                   (4096, 4096, 1024)])
def test_gemm_majors(M, N, K, a_mn, b_mn):
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.ops.gemm import gemm

    torch.manual_seed(0)
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
    d = gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    ref = _ref(a, b, a_mn, b_mn)
    err = (d.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-3, (err, scale)


def test_gemm_fp32_out_and_accumulate():
    from turbo_dllm_b200.ops.gemm import gemm

    torch.manual_seed(1)
    M, N, K = 512, 768, 512
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    out = gemm(a, b, out_dtype=torch.float32)
    assert torch.allclose(out, ref, rtol=1e-3, atol=1e-2)
    gemm(a, b, out=out, accumulate=True)
    assert torch.allclose(out, 2 * ref, rtol=1e-3, atol=2e-2)
    ob = torch.ones(M, N, device="cuda", dtype=torch.bfloat16)
    gemm(a, b, out=ob, accumulate=True)
    assert torch.allclose(ob.float(), ref + 1, rtol=2e-2, atol=0.5)


def test_gemm_swiglu_epilogue():
    from turbo_dllm_b200.ops.gemm import gemm

    torch.manual_seed(2)
    M, N, K = 640, 1024, 256
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    acc = a.float() @ b.float().t()
    ref = torch.nn.functional.silu(acc[:, 0::2]) * acc[:, 1::2]
    out = gemm(a, b, swiglu=True)
    assert out.shape == (M, N // 2)
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)


def test_linear_autograd_matches_reference():
    from turbo_dllm_b200.ops.gemm import linear

    torch.manual_seed(3)
    x = torch.randn(4, 200, 256, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())
    assert torch.allclose(y.float(), yr, rtol=2e-2, atol=2e-2)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
    assert torch.allclose(w.grad.float(), wr.grad, rtol=2e-2, atol=1e-1)


def test_bounded_wait_returns_error_status():
    """A wait on a barrier nobody signals must give up, record ERR_WAIT_TIMEOUT and leave the
    context usable (host-made failure; nothing traps or hangs)."""
    from turbo_dllm_b200.kernels import native

    lib = native.lib()
    lib.tdllm_clear_error()
    native.check(lib.tdllm_set_wait_timeout_ns(2_000_000), "set timeout")  # 2 ms
    try:
        native.check(lib.tdllm_test_wait_timeout(None), "launch")
        torch.cuda.synchronize()
        err = native.device_error()
        assert err["code"] == 1 and err["kernel"] == 99 and err["detail"] == 7
    finally:
        lib.tdllm_clear_error()
        lib.tdllm_set_wait_timeout_ns(2_000_000_000)
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0


@pytest.mark.parametrize("counts", [[300, 0, 17, 512, 1], [0, 0, 40], [256, 256]])
def test_grouped_linear_matches_per_expert_reference(counts):
    """Forward, input gradient and stacked weight gradients of the grouped GEMM against fp32 matmuls per
    expert, with empty experts and segments that are not multiples of the tile."""
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.ops.grouped import build_grouped_rows, grouped_linear, grouped_supported

    torch.manual_seed(5)
    E, N, K = len(counts), 512, 192
    rows = sum(counts)
    x = (torch.randn(rows, K, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(E, N, K, device="cuda") * 0.1).bfloat16().requires_grad_()
    assert grouped_supported(x, w)
    g = build_grouped_rows(torch.tensor(counts, device="cuda"), rows)
    x_pad = x.new_zeros(g.capacity, K).index_copy(0, g.dest, x)
    y = grouped_linear(x_pad, w, g).index_select(0, g.dest)
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    outs, off = [], 0
    for e, n in enumerate(counts):
        outs.append(xr[off:off + n] @ wr[e].t())
        off += n
    yr = torch.cat(outs)
    yr.backward(dy.float())
    assert torch.allclose(y.float(), yr, rtol=2e-2, atol=2e-2)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
    scale = wr.grad.abs().max().item() + 1e-6
    assert (w.grad.float() - wr.grad).abs().max().item() < 2e-2 * scale + 1e-3


def test_kernels_with_a_fixed_reduction_order_repeat_bit_for_bit(monkeypatch):
    """Run twice, compare bitwise: the GEMM (no split-K), the attention forward, the split attention backward (one
    dQ kernel per query tile, one dK/dV kernel per key tile) and the RMSNorm backward (per-block partial sums, then
    an ordered column sum) have no atomics on their result paths."""
    import math

    from turbo_dllm_b200.ops.attention import (attention_backward_native, attention_forward_native,
                                               single_sequence_layout)
    from turbo_dllm_b200.ops.gemm import gemm
    from turbo_dllm_b200.ops.norm import rmsnorm

    torch.manual_seed(0)
    a = torch.randn(777, 520, device="cuda").bfloat16()
    w = torch.randn(392, 520, device="cuda").bfloat16()
    assert torch.equal(gemm(a, w), gemm(a, w))
    layout = single_sequence_layout(384, 32, "cuda", 2)
    n, Hq, Hkv, D = 3 * 384, 4, 2, 128
    qkv = (torch.randn(n, (Hq + 2 * Hkv) * D, device="cuda") * 0.5).bfloat16()
    q = qkv[:, : Hq * D].view(n, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(n, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(n, Hkv, D)
    scale = 1.0 / math.sqrt(D)
    o1, l1 = attention_forward_native(q, k, v, layout, scale)
    o2, l2 = attention_forward_native(q, k, v, layout, scale)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    monkeypatch.setenv("TDLLM_ATTN_BWD", "split")
    do = torch.randn_like(o1)
    g1 = [t.clone() for t in attention_backward_native(q, k, v, o1, do, l1, layout, scale)]
    g2 = attention_backward_native(q, k, v, o1, do, l1, layout, scale)
    assert all(torch.equal(x, y) for x, y in zip(g1, g2))
    x = torch.randn(1000, 512, device="cuda").bfloat16().requires_grad_()
    wn = torch.ones(512, device="cuda").bfloat16().requires_grad_()
    grads = []
    for _ in range(2):
        x.grad = wn.grad = None
        y, _ = rmsnorm(x, wn, 1e-6)
        y.backward(torch.ones_like(y))
        grads.append((x.grad.clone(), wn.grad.clone() if wn.grad is not None else None))
    assert torch.equal(grads[0][0], grads[1][0])
    if grads[0][1] is not None:
        assert torch.equal(grads[0][1], grads[1][1])


@pytest.mark.gpu
@pytest.mark.performance
def test_bf16_gemm_throughput_is_recorded():
    """Performance tier: records the tcgen05 GEMM's throughput beside the library GEMM's on the same shape; asserts only
    that the figures are sane (no hardware baseline is encoded: clocks and power caps differ between machines)."""
    import json

    from turbo_dllm_b200.ops.gemm import gemm

    M = N = K = 8192
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

    def time(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / iters * 1e-3

    ours = 2.0 * M * N * K / time(lambda: gemm(a, b, out=out)) / 1e12
    library = 2.0 * M * N * K / time(lambda: torch.matmul(a, b.t(), out=out)) / 1e12
    print(json.dumps({"event": "performance", "shape": [M, N, K], "tcgen05_gemm_tflops": round(ours, 1),
                      "library_gemm_tflops": round(library, 1)}))
    assert ours > 0 and library > 0

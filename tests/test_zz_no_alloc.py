"""The allocation-free RMSNorm backward (`tdllm_rmsnorm_bwd_noalloc`) must agree with the regular
entry point, which takes a caller-provided scratch buffer.

Some users of the kernel library cannot allocate device memory at the moment they need this
kernel (their memory pool is frozen, or their host application only hands them inputs and
outputs), so that variant keeps its partial sums in a fixed array inside the library. The test
calls it through its exported C symbol, several times in a row on different data and row counts,
because the array keeps the previous call's contents and a later call must not be affected by
them, checks the results against a plain fp32 PyTorch reference as well, and watches the driver's
free-memory figure across a call to see that nothing is allocated.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from turbo_dllm_b200.kernels import native

    lib = native.lib()
    fn = lib.tdllm_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    v = ctypes.c_void_p
    fn.argtypes = [v, v, v, v, v, v, v, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, v]
    return lib, fn


def _regular(lib, dy, h, w, rstd, dres, rows, H):
    from turbo_dllm_b200.kernels import native

    dx = torch.empty_like(h)
    dw = torch.empty(H, dtype=torch.float32, device="cuda")
    parts = lib.tdllm_rmsnorm_bwd_parts()
    scratch = torch.empty(parts * H, dtype=torch.float32, device="cuda")
    native.check(lib.tdllm_rmsnorm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                       dres.data_ptr() if dres is not None else None, dx.data_ptr(),
                                       dw.data_ptr(), 1, 0, scratch.data_ptr(), rows, H, None), "rmsnorm_bwd")
    return dx, dw


def _fp32_reference(dy, h, w, rstd, dres):
    """Plain PyTorch fp32 RMSNorm backward from the bf16 inputs."""
    g = dy.float() * w.float()
    xh = h.float() * rstd[:, None]
    dx = rstd[:, None] * (g - xh * (g * xh).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    return dx, (dy.float() * xh).sum(0)


@pytest.mark.parametrize("H", [512, 4096])
def test_noalloc_matches_regular_entry_point_on_calls_in_a_row(H):
    lib, fn = _symbol()
    torch.manual_seed(0)
    # three calls on different data: fewer rows than thread blocks after many rows (stale partial rows of the
    # first call stay in the array and must not be read), then MORE rows again (every partial row is rewritten)
    for call, rows in enumerate((700, 129, 1500)):
        h = torch.randn(rows, H, device="cuda").bfloat16()
        dy = torch.randn(rows, H, device="cuda").bfloat16()
        w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
        dres = torch.randn(rows, H, device="cuda").bfloat16() if call == 0 else None
        rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-6).contiguous()
        dx_ref, dw_ref = _regular(lib, dy, h, w, rstd, dres, rows, H)
        dx32, dw32 = _fp32_reference(dy, h, w, rstd, dres)
        dx = torch.empty_like(h)
        dw = torch.empty(H, dtype=torch.float32, device="cuda")
        args = (dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(), 1, 0, rows, H, None)
        assert fn(*args) == 0, lib.tdllm_last_error()      # warm call: the first one on a device resolves the address
        torch.cuda.synchronize()
        # the driver's view of free device memory (not just PyTorch's allocator): a cudaMalloc inside the
        # library would show here
        free_before = torch.cuda.mem_get_info()[0]
        torch_before = torch.cuda.memory_allocated()
        dx.zero_()
        dw.zero_()
        assert fn(*args) == 0, lib.tdllm_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.memory_allocated() == torch_before
        assert torch.equal(dx, dx_ref)                       # same kernel, same arithmetic per row
        assert torch.allclose(dw, dw_ref, rtol=1e-3, atol=1e-2)   # partial sums are grouped differently
        # against the fp32 reference: dw is an fp32 sum of exact products (order differs), dx is rounded to bf16
        assert torch.allclose(dw, dw32, rtol=1e-3, atol=1e-3 * float(dw32.abs().max()))
        assert torch.allclose(dx.float(), dx32, rtol=2e-2, atol=2e-2)


def test_noalloc_rejects_sizes_beyond_its_scratch_area():
    lib, fn = _symbol()
    x = torch.zeros(8, 8192, device="cuda", dtype=torch.bfloat16)
    r = torch.ones(8, device="cuda")
    dw = torch.zeros(8192, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), r.data_ptr(), None, x.data_ptr(), dw.data_ptr(), 1, 0, 8, 8192,
            None)
    assert rc != 0
    assert b"scratch" in lib.tdllm_last_error()

"""The allocation-free RMSNorm backward (`tdllm_rmsnorm_bwd_noalloc`) must agree with the regular
entry point, which takes a caller-provided scratch buffer.

Some users of the kernel library cannot allocate device memory at the moment they need this
kernel (their memory pool is frozen, or their host application only hands them inputs and
outputs), so that variant keeps its partial sums in a fixed array inside the library. The test
calls it through its exported C symbol, twice in a row on different data, because the array
keeps the previous call's contents and the second call must not be affected by them.
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


@pytest.mark.parametrize("H", [512, 4096])
def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row(H):
    lib, fn = _symbol()
    torch.manual_seed(0)
    for call, rows in enumerate((700, 129)):       # second call: other data, fewer rows than blocks
        h = torch.randn(rows, H, device="cuda").bfloat16()
        dy = torch.randn(rows, H, device="cuda").bfloat16()
        w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
        dres = torch.randn(rows, H, device="cuda").bfloat16() if call == 0 else None
        rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-6).contiguous()
        dx_ref, dw_ref = _regular(lib, dy, h, w, rstd, dres, rows, H)
        dx = torch.empty_like(h)
        dw = torch.empty(H, dtype=torch.float32, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(), 1, 0, rows, H, None)
        assert rc == 0, lib.tdllm_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(dx, dx_ref)                       # same kernel, same arithmetic per row
        assert torch.allclose(dw, dw_ref, rtol=3e-2, atol=0.3)  # partial sums are grouped differently


def test_noalloc_rejects_sizes_beyond_its_scratch_area():
    lib, fn = _symbol()
    x = torch.zeros(8, 8192, device="cuda", dtype=torch.bfloat16)
    r = torch.ones(8, device="cuda")
    dw = torch.zeros(8192, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), r.data_ptr(), None, x.data_ptr(), dw.data_ptr(), 1, 0, 8, 8192,
            None)
    assert rc != 0
    assert b"scratch" in lib.tdllm_last_error()

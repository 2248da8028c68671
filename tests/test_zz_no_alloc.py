"""The allocation-free batch-norm backward entry point against the regular one.

Some hosts of this library cannot call cudaMalloc where they call us (inside another framework's memory pool, inside a
region they are capturing, in a loop that must not take the allocator lock), so ``xb_bn_backward_static`` keeps its
scratch sums in a fixed array inside the library.  The test calls it through its exported C symbol, twice in a row (the
array keeps the first call's sums, so the second call proves they are cleared), and compares with ``xb_bn_backward``
fed with a fresh scratch vector.  It lives in a file of its own that is collected last.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(M, Cc, relu, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dev = "cuda"
    x = torch.randn(M, Cc, device=dev, generator=g)
    dy = torch.randn(M, Cc, device=dev, generator=g)
    mean, var = x.mean(0), x.var(0, unbiased=False)
    invstd = torch.rsqrt(var + 1e-5)
    gamma = torch.rand(Cc, device=dev, generator=g) + 0.5
    y = torch.relu((x - mean) * invstd * gamma) if relu else torch.empty(0, device=dev)
    return x, dy, y, mean.contiguous(), invstd.contiguous(), gamma


@pytest.mark.parametrize("M,Cc,relu", [(4096, 64, 1), (1000, 20, 0), (8192, 16, 1), (512, 4096, 1), (300, 4095, 0)])
def test_static_scratch_entry_point_matches_regular(M, Cc, relu):
    from crossbow_b200.ops import lib as L
    lib = L.load()
    fn = lib.xb_bn_backward_static                    # the exported C symbol
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 10 + [C.c_int] * 5 + [C.c_void_p]
    s = torch.cuda.current_stream().cuda_stream
    for call in range(2):                             # two calls in a row share the built-in scratch
        x, dy, y, mean, invstd, gamma = _args(M, Cc, relu, seed=7 + call)
        yp = y.data_ptr() if relu else 0
        dx_a, dg_a, db_a = torch.empty_like(x), torch.zeros(Cc, device="cuda"), torch.zeros(Cc, device="cuda")
        dx_b, dg_b, db_b = torch.empty_like(x), torch.zeros(Cc, device="cuda"), torch.zeros(Cc, device="cuda")
        scratch = torch.zeros(2 * Cc, device="cuda")
        L.check(lib.xb_bn_backward(dy.data_ptr(), x.data_ptr(), yp, mean.data_ptr(), invstd.data_ptr(), gamma.data_ptr(), scratch.data_ptr(),
                                   dx_a.data_ptr(), 0, dg_a.data_ptr(), db_a.data_ptr(), M, Cc, relu, 0, 0, s), "regular entry point")
        rc = fn(dy.data_ptr(), x.data_ptr(), yp, mean.data_ptr(), invstd.data_ptr(), gamma.data_ptr(),
                dx_b.data_ptr(), 0, dg_b.data_ptr(), db_b.data_ptr(), M, Cc, relu, 0, 0, s)
        assert rc == 0, rc
        torch.cuda.synchronize()
        scale = float(dx_a.abs().max())
        assert float((dx_a - dx_b).abs().max()) <= 1e-4 * scale, call
        assert torch.allclose(dg_a, dg_b, rtol=1e-4, atol=1e-4 * float(dg_a.abs().max()))
        assert torch.allclose(db_a, db_b, rtol=1e-4, atol=1e-4 * float(db_a.abs().max()))
        # and against plain PyTorch
        xr = x.clone().requires_grad_(True)
        gr = gamma.clone().requires_grad_(True)
        out = (xr - xr.mean(0)) * torch.rsqrt(xr.var(0, unbiased=False) + 1e-5) * gr
        if relu:
            out = torch.relu(out)
        out.backward(dy)
        assert float((dx_b - xr.grad).abs().max()) <= 2e-3 * float(xr.grad.abs().max())


def test_static_scratch_entry_point_rejects_too_many_channels():
    from crossbow_b200.ops import lib as L
    lib = L.load()
    fn = lib.xb_bn_backward_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 10 + [C.c_int] * 5 + [C.c_void_p]
    t = torch.zeros(8, device="cuda")
    rc = fn(t.data_ptr(), t.data_ptr(), 0, t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 0, t.data_ptr(), t.data_ptr(),
            1, 4097, 0, 0, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -1001

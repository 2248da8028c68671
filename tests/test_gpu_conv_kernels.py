"""Convolution / inner-product kernels in isolation against torch.nn.functional on the same device (fp32 reference,
TF32 disabled), for the CUDA-core (exact fp32) and tensor-core (tf32 operands) implementations."""
import ctypes as C

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

SHAPES = [
    # N, H, W, C, K, R, S, stride, pad
    (4, 32, 32, 16, 16, 3, 3, 1, 1),
    (4, 32, 32, 16, 32, 3, 3, 2, 1),
    (4, 16, 16, 32, 32, 3, 3, 1, 1),
    (4, 16, 16, 16, 32, 1, 1, 2, 0),
    (3, 9, 7, 8, 24, 3, 3, 1, 1),       # odd sizes, K not a multiple of 16
    (2, 14, 14, 64, 256, 1, 1, 1, 0),
    (2, 14, 14, 128, 320, 3, 3, 1, 1),  # more than 256 output channels (two N tiles)
    (2, 12, 12, 4, 20, 5, 5, 1, 2),
    (64, 1, 1, 256, 10, 1, 1, 1, 0),    # inner product
    (5, 1, 1, 1000, 520, 1, 1, 1, 0),
    (2, 23, 23, 12, 16, 7, 7, 2, 3),
    (8, 56, 56, 64, 256, 1, 1, 1, 0),   # 1x1 convolutions: TMA-fed GEMM
    (2, 7, 7, 512, 2048, 1, 1, 1, 0),
    (4, 28, 28, 256, 128, 1, 1, 2, 0),
    (2, 56, 56, 64, 96, 1, 1, 2, 0),
    (3, 14, 14, 64, 128, 1, 1, 2, 0),   # stride 2: reduction blocks of whole output rows, last block partial
    (2, 8, 8, 48, 40, 1, 1, 1, 0),      # reduction tail, N tile wider than the layer
    (3, 10, 10, 96, 64, 1, 1, 1, 0),
    (2, 56, 56, 64, 64, 3, 3, 1, 1),    # wide 3x3: implicit GEMM over 4-D TMA boxes
    (3, 14, 14, 256, 256, 3, 3, 1, 1),
    (5, 7, 7, 512, 96, 3, 3, 1, 1),     # two images per tile
    (1, 6, 150, 64, 32, 3, 3, 1, 1),    # rows wider than a tile
    (2, 9, 11, 64, 96, 5, 5, 1, 2),
]


def _geom(lib_mod, N, H, W, Cc, K, R, S, st, pad):
    g = lib_mod.XbConvGeom()
    P = (H + 2 * pad - R) // st + 1
    Q = (W + 2 * pad - S) // st + 1
    g.N, g.H, g.W, g.C, g.K, g.R, g.S, g.P, g.Q, g.sh, g.sw, g.ph, g.pw = N, H, W, Cc, K, R, S, P, Q, st, st, pad, pad
    return g, P, Q


@pytest.fixture(scope="module")
def env():
    from crossbow_b200.ops import lib as L
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    return L, L.init_device()


@pytest.mark.parametrize("impl", ["simt", "tc"])
@pytest.mark.parametrize("shape", SHAPES)
def test_fprop_dgrad_wgrad(env, impl, shape):
    L, lib = env
    N, H, W, Cc, K, R, S, st, pad = shape
    g, P, Q = _geom(L, *shape)
    if impl == "tc" and not lib.xb_tc_supported(C.byref(g), 0):
        pytest.skip("shape not covered by the tensor-core path")
    tol = 1e-4 if impl == "simt" else (4e-3 if R * S * Cc <= 1152 else 8e-3)   # tf32 operands: error grows with the reduction length
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(N, H, W, Cc, device=dev, generator=gen)
    w = torch.randn(K, R, S, Cc, device=dev, generator=gen) * (1.0 / (R * S * Cc) ** 0.5)
    b = torch.randn(K, device=dev, generator=gen)
    dy = torch.randn(N, P, Q, K, device=dev, generator=gen)
    # float64 reference: the library's fp32 convolution may itself pick a transform-domain algorithm with ~1e-3 error
    xr = x.double().permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    wr = w.double().permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    yr = F.conv2d(xr, wr, b.double(), stride=st, padding=pad)
    yr.backward(dy.double().permute(0, 3, 1, 2))
    y_ref = F.relu(yr.detach()).permute(0, 2, 3, 1).float()
    s = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(4, dtype=torch.int32, device=dev)

    # forward with bias + ReLU + statistics
    y = torch.full((N, P, Q, K), 7.0, device=dev)
    stats = torch.zeros(2 * K, device=dev)
    flags = 1 | 4
    if impl == "simt":
        L.check(lib.xb_conv_fprop_simt(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), stats.data_ptr(), C.byref(g), flags, s), "fprop")
    else:
        L.check(lib.xb_conv_fprop_tc(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), stats.data_ptr(), C.byref(g), flags, status.data_ptr(), s), "fprop")
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    scale = float(y_ref.abs().max()) + 1e-6
    assert float((y - y_ref).abs().max()) / scale < tol
    m = y_ref.reshape(-1, K)
    assert torch.allclose(stats[:K], m.sum(0), rtol=tol * 10, atol=tol * 10 * m.shape[0] ** 0.5)
    assert torch.allclose(stats[K:], (m * m).sum(0), rtol=tol * 10, atol=tol * 10 * m.shape[0] ** 0.5)

    # data gradient (with and without accumulation) through the transposed weight copy
    wt = w.permute(3, 1, 2, 0).contiguous()
    dx_ref = xr.grad.permute(0, 2, 3, 1).float()
    for accum in (0, 1):
        dx = torch.full((N, H, W, Cc), 0.5, device=dev)
        if impl == "simt" or not lib.xb_tc_supported(C.byref(g), 1):
            L.check(lib.xb_conv_dgrad_simt(dy.data_ptr(), wt.data_ptr(), dx.data_ptr(), C.byref(g), accum, s), "dgrad")
        else:
            L.check(lib.xb_conv_dgrad_tc(dy.data_ptr(), wt.data_ptr(), dx.data_ptr(), C.byref(g), accum, status.data_ptr(), s, None), "dgrad")
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        ref = dx_ref + (0.5 if accum else 0.0)
        assert float((dx - ref).abs().max()) / (float(dx_ref.abs().max()) + 1e-6) < tol

    # weight gradient
    dw = torch.zeros(K, R, S, Cc, device=dev)
    if impl == "simt" or not lib.xb_tc_supported(C.byref(g), 2):
        L.check(lib.xb_conv_wgrad_simt(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), C.byref(g), s), "wgrad")
    else:
        L.check(lib.xb_conv_wgrad_tc(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), C.byref(g), status.data_ptr(), s), "wgrad")
    torch.cuda.synchronize()
    dw_ref = wr.grad.permute(0, 2, 3, 1).float()
    assert float((dw - dw_ref).abs().max()) / (float(dw_ref.abs().max()) + 1e-6) < (tol if impl == "tc" else 2e-4)


def test_1x1_shapes_take_the_tma_path(env):
    L, lib = env
    for shape, which, want in [((8, 56, 56, 64, 256, 1, 1, 1, 0), 0, 1), ((8, 56, 56, 64, 256, 1, 1, 1, 0), 1, 1), ((8, 56, 56, 64, 256, 1, 1, 1, 0), 2, 1),
                               ((4, 28, 28, 256, 128, 1, 1, 2, 0), 0, 1), ((2, 8, 8, 48, 40, 1, 1, 1, 0), 2, 1), ((32, 1, 1, 2048, 1000, 1, 1, 1, 0), 2, 1),
                               ((4, 16, 16, 16, 32, 1, 1, 2, 0), 2, 0), ((4, 16, 16, 32, 32, 3, 3, 1, 1), 0, 0)]:
        g, _, _ = _geom(L, *shape)
        assert lib.xb_conv1x1_tma_supported(C.byref(g), which) == want


@pytest.mark.parametrize("shape", [(32, 1, 1, 2048, 1000, 1, 1, 1, 0), (128, 1, 1, 512, 512, 1, 1, 1, 0), (64, 1, 1, 800, 500, 1, 1, 1, 0),
                                   (7, 1, 1, 4096, 84, 1, 1, 1, 0), (200, 1, 1, 260, 1000, 1, 1, 1, 0)])
@pytest.mark.parametrize("accum", [0, 1])
def test_inner_products_at_batch_size(env, shape, accum):
    """Few output tiles and a long reduction: the forward pass and the data gradient split the reduction over CTAs that add
    their partial tiles, and the weight gradient of a layer whose widths are no multiples of 32 stays on the tensor cores."""
    L, lib = env
    N, _, _, Cc, K, _, _, _, _ = shape
    g, _, _ = _geom(L, *shape)
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(N, Cc, device=dev, generator=gen)
    w = torch.randn(K, Cc, device=dev, generator=gen) * (1.0 / Cc ** 0.5)
    b = torch.randn(K, device=dev, generator=gen)
    dy = torch.randn(N, K, device=dev, generator=gen)
    wt = w.t().contiguous()
    s = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    tol = 8e-3
    y_ref = (x.double() @ w.double().t() + b.double()).float()
    dx_ref = (dy.double() @ w.double()).float()
    dw_ref = (dy.double().t() @ x.double()).float()
    for split in (1, 0):                                       # the split form and the one-CTA-per-tile form agree with the reference
        lib.xb_gemm_set_split_k(split)
        y = torch.full((N, K), 0.25, device=dev)
        L.check(lib.xb_conv_fprop_tc(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), 0, C.byref(g), 2 if accum else 0, status.data_ptr(), s), "fprop")
        dx = torch.full((N, Cc), 0.5, device=dev)
        L.check(lib.xb_conv_dgrad_tc(dy.data_ptr(), wt.data_ptr(), dx.data_ptr(), C.byref(g), accum, status.data_ptr(), s, None), "dgrad")
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        assert float((y - (y_ref + (0.25 if accum else 0.0))).abs().max()) / float(y_ref.abs().max()) < tol, split
        assert float((dx - (dx_ref + (0.5 if accum else 0.0))).abs().max()) / float(dx_ref.abs().max()) < tol, split
    lib.xb_gemm_set_split_k(1)
    assert lib.xb_conv1x1_tma_supported(C.byref(g), 2) == 1
    dw = torch.zeros(K, Cc, device=dev)
    L.check(lib.xb_conv_wgrad_tc(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), C.byref(g), status.data_ptr(), s), "wgrad")
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert float((dw - dw_ref).abs().max()) / float(dw_ref.abs().max()) < tol


@pytest.mark.parametrize("shape", [(2, 64, 64, 3, 64, 7, 7, 2, 3), (4, 32, 32, 16, 32, 3, 3, 2, 1), (2, 12, 12, 4, 32, 5, 5, 1, 2),
                                   (3, 28, 28, 1, 20, 5, 5, 1, 0), (8, 32, 32, 3, 64, 3, 3, 1, 1), (8, 32, 32, 3, 16, 3, 3, 1, 1),
                                   (2, 17, 17, 8, 48, 5, 5, 2, 2), (2, 9, 9, 12, 208, 3, 3, 2, 1)])
def test_patch_matrix_gemm_path(env, shape):
    """Layers without a direct tensor-core kernel: gather to a patch matrix, then the TMA GEMM (forward, weight gradient)."""
    L, lib = env
    N, H, W, Cc, K, R, S, st, pad = shape
    g, P, Q = _geom(L, *shape)
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(N, H, W, Cc, device=dev, generator=gen)
    w = torch.randn(K, R, S, Cc, device=dev, generator=gen) * (1.0 / (R * S * Cc) ** 0.5)
    b = torch.randn(K, device=dev, generator=gen)
    dy = torch.randn(N, P, Q, K, device=dev, generator=gen)
    wr = w.permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    yr = F.conv2d(x.permute(0, 3, 1, 2), wr, b, stride=st, padding=pad)
    yr.backward(dy.permute(0, 3, 1, 2))
    y_ref = F.relu(yr.detach()).permute(0, 2, 3, 1)
    need = lib.xb_conv_im2col_scratch(C.byref(g), 0)
    assert need > 0 and lib.xb_conv_im2col_wanted(C.byref(g), 0) == need
    scratch = torch.empty(need // 4, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    s = torch.cuda.current_stream().cuda_stream
    y = torch.full((N, P, Q, K), 7.0, device=dev)
    stats = torch.zeros(2 * K, device=dev)
    L.check(lib.xb_conv_fprop_im2col(x.data_ptr(), w.data_ptr(), b.data_ptr(), y.data_ptr(), stats.data_ptr(), C.byref(g), 1 | 4, scratch.data_ptr(),
                                     status.data_ptr(), s), "fprop")
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert float((y - y_ref).abs().max()) / float(y_ref.abs().max()) < 4e-3
    m = y_ref.reshape(-1, K)
    assert torch.allclose(stats[:K], m.sum(0), rtol=4e-2, atol=4e-2 * m.shape[0] ** 0.5)
    # (output channel counts that are no multiples of 32: partial planes, the loads read zeros for the missing channels)
    assert lib.xb_conv_im2col_scratch(C.byref(g), 2) > 0
    dw = torch.zeros(K, R, S, Cc, device=dev)
    for reuse in (0, 1):          # 1: the patch matrix written by the forward call above is still in the scratch
        dw.zero_()
        L.check(lib.xb_conv_wgrad_im2col(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), C.byref(g), scratch.data_ptr(), reuse, status.data_ptr(), s), "wgrad")
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    dw_ref = wr.grad.permute(0, 2, 3, 1)
    assert float((dw - dw_ref).abs().max()) / float(dw_ref.abs().max()) < 4e-3


@pytest.mark.parametrize("shape", [(4, 32, 32, 16, 32, 3, 3, 2, 1), (3, 16, 16, 32, 64, 3, 3, 2, 1), (2, 8, 12, 8, 24, 3, 3, 2, 1)])
def test_stride2_dgrad_by_zero_insertion(env, shape):
    L, lib = env
    N, H, W, Cc, K, R, S, st, pad = shape
    g, P, Q = _geom(L, *shape)
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda").manual_seed(9)
    w = torch.randn(K, R, S, Cc, device=dev, generator=gen) * 0.1
    dy = torch.randn(N, P, Q, K, device=dev, generator=gen)
    xr = torch.zeros(N, Cc, H, W, device=dev, dtype=torch.float64, requires_grad=True)
    F.conv2d(xr, w.double().permute(0, 3, 1, 2), None, stride=2, padding=1).backward(dy.double().permute(0, 3, 1, 2))
    dx_ref = xr.grad.permute(0, 2, 3, 1).float()
    need = lib.xb_conv3x3_s2_dgrad_scratch(C.byref(g))
    assert need == N * H * W * K * 4
    scratch = torch.empty(need // 4, device=dev)
    wt = w.permute(3, 1, 2, 0).contiguous()
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    for accum in (0, 1):
        dx = torch.full((N, H, W, Cc), 0.25, device=dev)
        L.check(lib.xb_conv3x3_s2_dgrad(dy.data_ptr(), wt.data_ptr(), dx.data_ptr(), C.byref(g), accum, scratch.data_ptr(), status.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream, None), "dgrad")
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        ref = dx_ref + (0.25 if accum else 0.0)
        assert float((dx - ref).abs().max()) / float(dx_ref.abs().max()) < 4e-3


@pytest.mark.parametrize("shape", [(4, 32, 32, 16, 16, 3, 3, 1, 1), (4, 16, 16, 32, 32, 3, 3, 1, 1), (2, 14, 14, 64, 256, 1, 1, 1, 0),
                                   (2, 28, 28, 128, 128, 3, 3, 1, 1), (3, 8, 8, 64, 64, 3, 3, 1, 1)])
@pytest.mark.parametrize("relu,accum", [(1, 0), (0, 1)])
def test_dgrad_epilogue_produces_bn_backward_sums(env, shape, relu, accum):
    """The data-gradient kernel that completes dy of a normalisation layer also returns that layer's backward sums:
    sum dz and sum dz * xhat with dz = dy masked by the layer's ReLU."""
    L, lib = env
    N, H, W, Cc, K, R, S, st, pad = shape
    g, P, Q = _geom(L, *shape)
    assert lib.xb_conv_dgrad_fuses_bn(C.byref(g))
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda").manual_seed(11)
    w = torch.randn(K, R, S, Cc, device=dev, generator=gen) * (1.0 / (R * S * K) ** 0.5)
    dyo = torch.randn(N, P, Q, K, device=dev, generator=gen)              # gradient w.r.t. the convolution's output
    bn_x = torch.randn(N, H, W, Cc, device=dev, generator=gen)            # input of the normalisation layer in front of the convolution
    bn_y = torch.randn(N, H, W, Cc, device=dev, generator=gen)            # its output (sign = ReLU mask)
    mean = torch.randn(Cc, device=dev, generator=gen) * 0.1
    istd = torch.rand(Cc, device=dev, generator=gen) + 0.5
    base = torch.randn(N, H, W, Cc, device=dev, generator=gen) if accum else torch.zeros(N, H, W, Cc, device=dev)
    xr = torch.zeros(N, Cc, H, W, device=dev, dtype=torch.float64, requires_grad=True)
    F.conv2d(xr, w.double().permute(0, 3, 1, 2), None, stride=st, padding=pad).backward(dyo.double().permute(0, 3, 1, 2))
    dx_ref = xr.grad.permute(0, 2, 3, 1) + base.double()
    dz = dx_ref * (bn_y > 0) if relu else dx_ref
    s1 = dz.reshape(-1, Cc).sum(0)
    s2 = (dz * (bn_x.double() - mean.double()) * istd.double()).reshape(-1, Cc).sum(0)
    sums = torch.zeros(2 * Cc, device=dev)
    fuse = L.XbBnFuse()
    fuse.x, fuse.y, fuse.mean, fuse.istd, fuse.sums, fuse.relu = bn_x.data_ptr(), bn_y.data_ptr(), mean.data_ptr(), istd.data_ptr(), sums.data_ptr(), relu
    dx = base.clone()
    wt = w.permute(3, 1, 2, 0).contiguous()
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    L.check(lib.xb_conv_dgrad_tc(dyo.data_ptr(), wt.data_ptr(), dx.data_ptr(), C.byref(g), accum, status.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream, C.byref(fuse)), "dgrad")
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert float((dx.double() - dx_ref).abs().max()) / float(dx_ref.abs().max()) < 4e-3
    scale = float(dz.abs().sum(dim=(0, 1, 2)).max())
    assert float((sums[:Cc].double() - s1).abs().max()) / scale < 4e-3
    assert float((sums[Cc:].double() - s2).abs().max()) / (scale * 3) < 4e-3


def test_first_layer_three_channels(env):
    """C=3 takes the scalar CUDA-core path in every direction."""
    L, lib = env
    shape = (4, 32, 32, 3, 16, 3, 3, 1, 1)
    g, P, Q = _geom(L, *shape)
    assert not lib.xb_tc_supported(C.byref(g), 0)
    dev = torch.device("cuda")
    x = torch.randn(4, 32, 32, 3, device=dev)
    w = torch.randn(16, 3, 3, 3, device=dev)
    y = torch.empty(4, P, Q, 16, device=dev)
    s = torch.cuda.current_stream().cuda_stream
    L.check(lib.xb_conv_fprop_simt(x.data_ptr(), w.data_ptr(), 0, y.data_ptr(), 0, C.byref(g), 0, s), "fprop")
    ref = F.conv2d(x.permute(0, 3, 1, 2), w.permute(0, 3, 1, 2), padding=1).permute(0, 2, 3, 1)
    assert torch.allclose(y, ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("shape", [(4, 32, 32, 16, 16, 3, 3, 1, 1), (4, 16, 16, 32, 32, 3, 3, 1, 1), (8, 8, 8, 64, 64, 3, 3, 1, 1),
                                   (3, 9, 7, 16, 24, 3, 3, 1, 1), (2, 12, 12, 48, 20, 3, 3, 1, 1), (64, 32, 32, 16, 16, 3, 3, 1, 1),
                                   (2, 8, 8, 128, 256, 3, 3, 1, 1), (2, 6, 10, 20, 12, 3, 3, 1, 1), (1, 56, 56, 64, 64, 3, 3, 1, 1)])
def test_wgrad_tensor_core_slab(env, shape):
    """Weight gradient on tcgen05 with swizzled MN-major operands taken straight from the position-major tensors."""
    L, lib = env
    g, P, Q = _geom(L, *shape)
    lib.xb_tc_set_slab(3)
    try:
        assert lib.xb_tc_supported(C.byref(g), 2)
        N, H, W, Cc, K, R, S, st, pad = shape
        dev = torch.device("cuda")
        gen = torch.Generator(device="cuda").manual_seed(2)
        x = torch.randn(N, H, W, Cc, device=dev, generator=gen)
        dy = torch.randn(N, P, Q, K, device=dev, generator=gen)
        wr = torch.zeros(K, Cc, R, S, device=dev, requires_grad=True)
        F.conv2d(x.permute(0, 3, 1, 2), wr, None, stride=st, padding=pad).backward(dy.permute(0, 3, 1, 2))
        dw_ref = wr.grad.permute(0, 2, 3, 1)
        dw = torch.zeros(K, R, S, Cc, device=dev)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        L.check(lib.xb_conv_wgrad_tc(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), C.byref(g), status.data_ptr(), torch.cuda.current_stream().cuda_stream), "wgrad")
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        assert float((dw - dw_ref).abs().max()) / float(dw_ref.abs().max()) < 4e-3
    finally:
        lib.xb_tc_set_slab(3)


@pytest.mark.parametrize("M,C", [(4096, 64), (777, 256), (50, 1024), (3000, 16)])
def test_batch_norm_packed_sign_mask_equals_mask_from_output(M, C):
    """Residual + ReLU normalisation layers: the forward pass writes one byte per four channels with the signs of its
    output, and a backward pass that reads those bytes gives exactly what the one reading the output itself gives."""
    from crossbow_b200.ops import lib as L
    lib = L.load()
    g = torch.Generator(device="cuda").manual_seed(M + C)
    x, res, dy = (torch.randn(M, C, device="cuda", generator=g) for _ in range(3))
    gamma, beta = torch.rand(C, device="cuda", generator=g) + 0.5, torch.randn(C, device="cuda", generator=g) * 0.1
    sums = torch.stack([x.sum(0), (x * x).sum(0)]).contiguous()
    y = torch.empty_like(x)
    rm, rv, sm, si = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda"), torch.empty(C, device="cuda"), torch.empty(C, device="cuda")
    mask = torch.zeros(M * C // 4, dtype=torch.uint8, device="cuda")
    tp = torch.zeros(16, dtype=torch.int32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    L.check(lib.xb_bn_forward_mask(x.data_ptr(), res.data_ptr(), y.data_ptr(), sums.data_ptr(), gamma.data_ptr(), beta.data_ptr(), rm.data_ptr(),
                                   rv.data_ptr(), sm.data_ptr(), si.data_ptr(), tp.data_ptr(), M, C, 1e-5, 1, 1, 0, 0.1, mask.data_ptr(), s), "bn forward")
    torch.cuda.synchronize()
    bits = torch.stack([(mask >> e) & 1 for e in range(4)], -1).reshape(M, C).bool()
    assert torch.equal(bits, y > 0)
    outs = []
    for relu, ysrc in ((1, y), (3, mask)):
        dsums, dx, dres = torch.zeros(2 * C, device="cuda"), torch.empty_like(x), torch.empty_like(x)
        dg, db = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
        L.check(lib.xb_bn_backward(dy.data_ptr(), x.data_ptr(), ysrc.data_ptr(), sm.data_ptr(), si.data_ptr(), gamma.data_ptr(), dsums.data_ptr(),
                                   dx.data_ptr(), dres.data_ptr(), dg.data_ptr(), db.data_ptr(), M, C, relu, 0, 0, s), "bn backward")
        torch.cuda.synchronize()
        outs.append((dx, dres, dg, db))
    for a, b in zip(*outs):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-5 * float(a.abs().max()))      # (the sums are atomic: rounding only)
    assert torch.equal(outs[0][1], outs[1][1])                                            # dres = masked dy, no arithmetic

"""conv2d: the numpy oracle against the frozen ATen-CPU vectors (CPU tests), and the CUDA implicit-GEMM
path against the oracle through the C-ABI (GPU tests). Bar: relative Frobenius error <= 1e-2 for fp16 /
bf16 results against the float64 oracle evaluated on the same rounded inputs."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from conftest import rel_fro

GOLDEN_CASES = ["a", "b", "c", "d", "e"]


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_oracle_matches_golden(golden, name):
    st, pd = (int(v) for v in golden[f"conv_{name}_cfg"])
    x, w, gy = golden[f"conv_{name}_x"], golden[f"conv_{name}_w"], golden[f"conv_{name}_gy"]
    np.testing.assert_allclose(oracle.conv2d_forward(x, w, st, pd), golden[f"conv_{name}_y"], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(oracle.conv2d_backward_input(gy, w, x.shape, st, pd), golden[f"conv_{name}_gx"], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(oracle.conv2d_backward_weight(gy, x, w.shape, st, pd), golden[f"conv_{name}_gw"], rtol=1e-12, atol=1e-12)


def test_descriptor_validation():
    from torchvulkan_b200 import capi

    lib = capi.lib()
    n = C.c_uint64(0)
    ok = capi.Conv2dDesc(capi.F16, 2, 3, 8, 8, 4, 3, 3, 1, 1, 1, 1, 1, 1, 1)
    assert lib.tvk_conv2d_workspace_size(C.byref(ok), 0, C.byref(n)) == 0 and n.value > 0
    assert lib.tvk_conv2d_workspace_size(C.byref(ok), 3, C.byref(n)) == 0 and n.value > 0      # both gradients in one call
    assert lib.tvk_conv2d_workspace_size(C.byref(ok), 4, C.byref(n)) == 1
    for field, value in (("groups", 2), ("dtype", capi.I64)):
        d = capi.Conv2dDesc(capi.F16, 2, 3, 8, 8, 4, 3, 3, 1, 1, 1, 1, 1, 1, 1)
        setattr(d, field, value)
        assert lib.tvk_conv2d_workspace_size(C.byref(d), 0, C.byref(n)) == 2, field
        assert b"NOT IMPLEMENTED" in lib.tvk_last_error()
    # what the implicit-GEMM kernels do not take (dilation, strides above 2 or unequal, filters of many taps) goes through
    # unfold + GEMM like fp32
    for field, value in (("dilation_h", 2), ("stride_h", 3), ("kh", 9)):
        d = capi.Conv2dDesc(capi.F16, 2, 3, 8, 8, 4, 3, 3, 1, 1, 1, 1, 1, 1, 1)
        setattr(d, field, value)
        if field == "kh":
            d.kw, d.h, d.w = 9, 16, 16
        for mode in (0, 1, 2, 3):
            assert lib.tvk_conv2d_workspace_size(C.byref(d), mode, C.byref(n)) == 0 and n.value > 0, (field, mode)
    d = capi.Conv2dDesc(capi.F16, 2, 3, 2, 2, 4, 3, 3, 1, 1, 0, 0, 1, 1, 1)
    assert lib.tvk_conv2d_workspace_size(C.byref(d), 0, C.byref(n)) == 1  # filter larger than the input
    # fp32 goes through unfold + GEMM: any stride and dilation, no groups
    f = capi.Conv2dDesc(capi.F32, 2, 3, 9, 9, 4, 3, 3, 3, 3, 1, 1, 1, 1, 1)
    for mode in (0, 1, 2):
        assert lib.tvk_conv2d_workspace_size(C.byref(f), mode, C.byref(n)) == 0 and n.value > 0
    f.dilation_w = 2
    assert lib.tvk_conv2d_workspace_size(C.byref(f), 0, C.byref(n)) == 0 and n.value > 0
    f.groups = 3
    assert lib.tvk_conv2d_workspace_size(C.byref(f), 0, C.byref(n)) == 2 and b"NOT IMPLEMENTED" in lib.tvk_last_error()


# ------------------------------------------------------------------------------------ GPU
def f64(t):
    return t.detach().float().cpu().double().numpy()


def _case(n, ci, h, w, co, kh, kw, dtype, seed, stride, pad):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, ci, h, w, generator=g).to(dtype)
    wt = (torch.randn(co, ci, kh, kw, generator=g) / (ci * kh * kw) ** 0.5).to(dtype)
    ho, wo = (h + 2 * pad - kh) // stride + 1, (w + 2 * pad - kw) // stride + 1
    gy = torch.randn(n, co, ho, wo, generator=g).to(dtype)
    return x, wt, gy


# (n, cin, h, w, cout, kh, kw, stride, pad): ragged extents, channel counts off the 64 grid, both strides,
# 1x1 / 3x3 / 7x7 filters, and the shapes of the ResNet blocks
SHAPES = [
    (2, 3, 9, 7, 5, 3, 3, 1, 1),
    (2, 4, 8, 8, 6, 3, 3, 2, 1),
    (1, 5, 7, 9, 4, 1, 1, 2, 0),
    (2, 2, 6, 5, 3, 2, 3, 1, 0),
    (1, 3, 10, 10, 2, 7, 7, 2, 3),
    (3, 64, 16, 16, 64, 3, 3, 1, 1),
    (2, 64, 16, 16, 128, 3, 3, 2, 1),
    (2, 64, 15, 17, 128, 1, 1, 2, 0),
    (2, 128, 8, 8, 256, 3, 3, 2, 1),
    (2, 256, 4, 4, 512, 3, 3, 2, 1),
    (1, 512, 4, 4, 512, 3, 3, 1, 1),
    (5, 72, 11, 13, 200, 3, 3, 1, 1),
    (4, 3, 32, 32, 64, 3, 3, 1, 1),
    (1, 16, 150, 3, 24, 3, 3, 1, 1),
    (2, 40, 13, 11, 56, 3, 3, 1, 1),      # 3x3 / stride 1 / <= 64 channels: the resident-filter kernel, ragged tiles
    (3, 64, 33, 9, 64, 3, 3, 1, 1),
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_conv2d_against_oracle(cuda, shape, dtype):
    from torchvulkan_b200 import cuda_ops as ops

    n, ci, h, w, co, kh, kw, st, pd = shape
    x, wt, gy = _case(n, ci, h, w, co, kh, kw, dtype, 11, st, pd)
    xd, wd, gyd = x.cuda(), wt.cuda(), gy.cuda()
    y = ops.conv2d_forward(xd, wd, st, pd)
    gx = ops.conv2d_backward_input(gyd, wd, x.shape, st, pd)
    gw = ops.conv2d_backward_weight(gyd, xd, wt.shape, st, pd)
    ops.check_device_status()
    tol = 1e-2  # relative Frobenius error of a half-precision result against the float64 oracle
    assert rel_fro(f64(y), oracle.conv2d_forward(f64(x), f64(wt), st, pd)) < tol
    assert rel_fro(f64(gx), oracle.conv2d_backward_input(f64(gy), f64(wt), x.shape, st, pd)) < tol
    assert rel_fro(f64(gw), oracle.conv2d_backward_weight(f64(gy), f64(x), wt.shape, st, pd)) < tol
    # both gradients in one call (dy transposed once for the two products): the same bits, and each alone as well
    gx2, gw2 = ops.conv2d_backward(gyd, xd, wd, st, pd)
    assert torch.equal(gx2, gx) and torch.equal(gw2, gw)
    gx3, none = ops.conv2d_backward(gyd, xd, wd, st, pd, need_dw=False)
    none2, gw3 = ops.conv2d_backward(gyd, xd, wd, st, pd, need_dx=False)
    assert none is None and none2 is None and torch.equal(gx3, gx) and torch.equal(gw3, gw)
    # a channels-last dy with NCHW x (the layouts are independent)
    gx4, gw4 = ops.conv2d_backward(gyd.contiguous(memory_format=torch.channels_last), xd, wd, st, pd)
    assert not gx4.is_contiguous(memory_format=torch.channels_last) or gx4.is_contiguous()
    assert torch.equal(gx4, gx) and torch.equal(gw4, gw)
    ops.check_device_status()


@pytest.mark.gpu
@pytest.mark.parametrize("channels_last", [False, True])
@pytest.mark.parametrize("shape", SHAPES + [(3, 5, 11, 9, 7, 3, 2, 3, 1)])
def test_conv2d_fp32_against_oracle(cuda, shape, channels_last):
    """fp32 (unfold + 3xTF32 GEMM + fold): max relative error 1e-4 against the float64 oracle and the reference's own
    criterion for fp32 convolutions, atol=1e-4, rtol=1e-3 (tests/test_pytorch_ops.py:322-327); plain and channels-last
    tensors, stride 3 included."""
    from torchvulkan_b200 import cuda_ops as ops

    n, ci, h, w, co, kh, kw, st, pd = shape
    x, wt, gy = _case(n, ci, h, w, co, kh, kw, torch.float32, 13, st, pd)
    xd, wd, gyd = x.cuda(), wt.cuda(), gy.cuda()
    if channels_last:
        cl = torch.channels_last
        xd, wd, gyd = xd.contiguous(memory_format=cl), wd.contiguous(memory_format=cl), gyd.contiguous(memory_format=cl)
    y = ops.conv2d_forward(xd, wd, st, pd)
    gx = ops.conv2d_backward_input(gyd, wd, x.shape, st, pd)
    gw = ops.conv2d_backward_weight(gyd, xd, wt.shape, st, pd, channels_last_weight=channels_last)
    gx2, gw2 = ops.conv2d_backward(gyd, xd, wd, st, pd)          # both gradients in one call: the same bits
    assert torch.equal(gx2, gx) and torch.equal(gw2, gw)
    ops.check_device_status()
    if channels_last:
        assert all(t.is_contiguous(memory_format=torch.channels_last) for t in (y, gx, gw))
    refs = (oracle.conv2d_forward(f64(x), f64(wt), st, pd), oracle.conv2d_backward_input(f64(gy), f64(wt), x.shape, st, pd),
            oracle.conv2d_backward_weight(f64(gy), f64(x), wt.shape, st, pd))
    for name, got, ref in zip(("y", "gx", "gw"), (y, gx, gw), refs):
        g64 = f64(got)
        assert np.max(np.abs(g64 - ref)) <= 1e-4 * np.max(np.abs(ref)), name
        assert np.all(np.abs(g64 - ref) <= 1e-4 + 1e-3 * np.abs(ref)), name


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_conv2d_channels_last_against_oracle(cuda, shape, dtype):
    """The same cases with every tensor in channels-last memory: read and written in place when the channel count is
    a multiple of 8, through a padded copy otherwise; the results keep the format."""
    from torchvulkan_b200 import cuda_ops as ops

    n, ci, h, w, co, kh, kw, st, pd = shape
    x, wt, gy = _case(n, ci, h, w, co, kh, kw, dtype, 11, st, pd)
    cl = torch.channels_last
    xd, wd, gyd = x.cuda().contiguous(memory_format=cl), wt.cuda().contiguous(memory_format=cl), gy.cuda().contiguous(memory_format=cl)
    y = ops.conv2d_forward(xd, wd, st, pd)
    gx = ops.conv2d_backward_input(gyd, wd, x.shape, st, pd)
    gw = ops.conv2d_backward_weight(gyd, xd, wt.shape, st, pd, channels_last_weight=True)
    ops.check_device_status()
    for t in (y, gx, gw):
        assert t.is_contiguous(memory_format=cl)
    tol = 1e-2
    assert rel_fro(f64(y), oracle.conv2d_forward(f64(x), f64(wt), st, pd)) < tol
    assert rel_fro(f64(gx), oracle.conv2d_backward_input(f64(gy), f64(wt), x.shape, st, pd)) < tol
    assert rel_fro(f64(gw), oracle.conv2d_backward_weight(f64(gy), f64(x), wt.shape, st, pd)) < tol
    # mixed: channels-last activations with an OIHW filter must give the same bits
    y2 = ops.conv2d_forward(xd, wt.cuda(), st, pd)
    assert torch.equal(y2, y)


@pytest.mark.gpu
def test_conv2d_integer_valued_is_exact(cuda):
    """Small-integer inputs make every product and partial sum exact in fp16/fp32, so the result is bit-exact."""
    from torchvulkan_b200 import cuda_ops as ops

    g = torch.Generator().manual_seed(5)
    x = torch.randint(-2, 3, (4, 64, 12, 12), generator=g).half()
    wt = torch.randint(-1, 2, (96, 64, 3, 3), generator=g).half()
    for st in (1, 2):
        ho = (12 + 2 - 3) // st + 1
        gy = torch.randint(-1, 2, (4, 96, ho, ho), generator=g).half()
        y = ops.conv2d_forward(x.cuda(), wt.cuda(), st, 1)
        gx = ops.conv2d_backward_input(gy.cuda(), wt.cuda(), x.shape, st, 1)
        gw = ops.conv2d_backward_weight(gy.cuda(), x.cuda(), wt.shape, st, 1)
        np.testing.assert_array_equal(f64(y), oracle.conv2d_forward(f64(x), f64(wt), st, 1))
        np.testing.assert_array_equal(f64(gx), oracle.conv2d_backward_input(f64(gy), f64(wt), x.shape, st, 1))
        np.testing.assert_array_equal(f64(gw), oracle.conv2d_backward_weight(f64(gy), f64(x), wt.shape, st, 1))


@pytest.mark.gpu
def test_conv2d_full_size_linearity(cuda):
    """At the ResNet stage-1 size (256 x 64 x 32 x 32) the oracle is too slow; check conv(x1 + x2) = conv(x1) + conv(x2)
    on inputs whose sums are exact, and one output tile against the oracle on a cropped batch."""
    from torchvulkan_b200 import cuda_ops as ops

    g = torch.Generator().manual_seed(9)
    x1 = torch.randint(-2, 3, (256, 64, 32, 32), generator=g).half().cuda()
    x2 = torch.randint(-2, 3, (256, 64, 32, 32), generator=g).half().cuda()
    wt = torch.randint(-1, 2, (64, 64, 3, 3), generator=g).half().cuda()
    y1, y2, y12 = ops.conv2d_forward(x1, wt, 1, 1), ops.conv2d_forward(x2, wt, 1, 1), ops.conv2d_forward(x1 + x2, wt, 1, 1)
    assert torch.equal(y12, y1 + y2)
    ref = oracle.conv2d_forward(f64(x1[253:]), f64(wt), 1, 1)
    np.testing.assert_array_equal(f64(y1[253:]), ref)
    # the same size in channels-last memory (the in-place path) gives the same bits
    cl = torch.channels_last
    y1_cl = ops.conv2d_forward(x1.contiguous(memory_format=cl), wt.contiguous(memory_format=cl), 1, 1)
    assert y1_cl.is_contiguous(memory_format=cl) and torch.equal(y1_cl, y1)
    # input gradient: linear in dy; weight gradient: additive over the batch (all sums stay exact in fp16)
    g1 = torch.randint(-1, 2, (256, 64, 32, 32), generator=g).half().cuda()
    g2 = torch.randint(-1, 2, (256, 64, 32, 32), generator=g).half().cuda()
    d1, d2, d12 = (ops.conv2d_backward_input(t, wt, x1.shape, 1, 1) for t in (g1, g2, g1 + g2))
    assert torch.equal(d12, d1 + d2)
    np.testing.assert_array_equal(f64(d1[:2]), oracle.conv2d_backward_input(f64(g1[:2]), f64(wt), (2, 64, 32, 32), 1, 1))
    xs = (torch.rand(256, 64, 32, 32, generator=g) < 0.25).half().cuda()         # sparse 0/1 input keeps |dw| below 2048
    w_all = ops.conv2d_backward_weight(g1, xs, wt.shape, 1, 1)
    w_lo, w_hi = ops.conv2d_backward_weight(g1[:128], xs[:128], wt.shape, 1, 1), ops.conv2d_backward_weight(g1[128:], xs[128:], wt.shape, 1, 1)
    assert float(w_all.abs().max()) < 2048 and torch.equal(w_all, w_lo + w_hi)
    w_cl = ops.conv2d_backward_weight(g1.contiguous(memory_format=cl), xs.contiguous(memory_format=cl), wt.shape, 1, 1)
    assert torch.equal(w_cl, w_all)
    ops.check_device_status()

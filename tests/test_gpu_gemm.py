"""GPU parity of the dense contraction (tcgen05 path and CUDA-core path) through the C-ABI.

Bars (BASELINE north star): fp16/bf16 relative Frobenius error <= 1e-2 against the fp64 oracle on
the same seeded inputs; fp32 (3xTF32) max relative error 1e-4, measured as max|d| / max|ref| and
on the reduced scalar, plus the reference's own criterion atol=1e-4, rtol=1e-3
(tests/test_pytorch_ops.py:322-327).
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import rel_fro

pytestmark = pytest.mark.gpu

HALF_TOL = {torch.float16: 2e-3, torch.bfloat16: 1e-2}


def ops():
    from torchvulkan_b200 import cuda_ops
    return cuda_ops


def cpu_randn(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def f64(t):
    return t.detach().float().cpu().double().numpy()


def operand(rows, cols, dtype, seed, transposed, batch=None):
    """A [rows, cols] (or [batch, rows, cols]) tensor, stored transposed when asked."""
    shape = (cols, rows) if transposed else (rows, cols)
    if batch is not None:
        shape = (batch,) + shape
    t = cpu_randn(shape, dtype, seed)
    return t.transpose(-1, -2) if transposed else t


def check(out, ref, dtype):
    o = f64(out)
    assert not np.isnan(o).any(), "NaN in the output (unwritten tile?)"
    if dtype == torch.float32:
        scale = np.max(np.abs(ref))
        assert np.max(np.abs(o - ref)) / scale <= 1e-4
        assert np.all(np.abs(o - ref) <= 1e-4 + 1e-3 * np.abs(ref))
    else:
        err = rel_fro(o, ref)
        assert err <= HALF_TOL[dtype], f"relative Frobenius error {err:.3e}"


def run_case(cuda, dtype, m, n, k, ta, tb, path, batch=None, bias=None, alpha=1.0, beta=1.0, act=None, seed=0):
    a = operand(m, k, dtype, seed + 1, ta, batch)
    b = operand(k, n, dtype, seed + 2, tb, batch)
    bias_t = None
    if bias == "row":
        bias_t = cpu_randn(n, dtype, seed + 3)
    elif bias == "full":
        bias_t = cpu_randn((m, n), dtype, seed + 3)
    elif bias == "col":
        bias_t = cpu_randn((m, 1), dtype, seed + 3)
    ad, bd = a.to("cpu"), b.to("cpu")
    # .to(cuda) of a transposed view keeps its strides
    adev = torch.empty_strided(ad.shape, ad.stride(), dtype=dtype, device=cuda).copy_(ad)
    bdev = torch.empty_strided(bd.shape, bd.stride(), dtype=dtype, device=cuda).copy_(bd)
    shape = (m, n) if batch is None else (batch, m, n)
    out = torch.full(shape, float("nan"), dtype=dtype, device=cuda)  # NaN canary: every element must be written
    got_path = ops().gemm_path(adev, bdev, out, force_path=path)
    assert got_path == path
    ops().gemm(adev, bdev, bias=None if bias_t is None else bias_t.to(cuda), alpha=alpha, beta=beta, act=act, out=out, force_path=path)
    ops().check_device_status()
    ref = oracle.gemm(f64(a), f64(b), None if bias_t is None else f64(bias_t), alpha, beta, act)
    check(out, ref, dtype)
    return out


LAYOUTS = [(False, False), (False, True), (True, False), (True, True)]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("ta,tb", LAYOUTS)
def test_tc_layouts_aligned(cuda, dtype, ta, tb):
    run_case(cuda, dtype, 256, 384, 512, ta, tb, path=1)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k,ta,tb", [(512, 512, 8192, True, False), (128, 512, 8192, True, False), (520, 264, 4096, False, True),
                                         (2752, 512, 8192, True, False), (300, 200, 2048, False, False)])
def test_tc_split_k(cuda, dtype, m, n, k, ta, tb):
    """Weight-gradient shapes (few output tiles, long K): the K range runs as slices with fp32 partials; the full
    epilogue (alpha, bias, activation) is applied after the partials are summed."""
    run_case(cuda, dtype, m, n, k, ta, tb, path=1, seed=20)
    run_case(cuda, dtype, m, n, k, ta, tb, path=1, bias="row", alpha=0.5, beta=2.0, act="gelu", seed=21)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k,ta,tb", [(256, 10, 8192, False, True), (10, 8192, 256, True, False), (37, 7, 1000, False, True),
                                         (5, 1000, 77, True, False), (16, 2048, 130, False, False), (300, 16, 64, False, True)])
def test_skinny_shapes(cuda, dtype, m, n, k, ta, tb):
    """A classifier head (n of about ten) and its weight gradient (m of about ten): the CUDA-core kernels written
    for them, plain and with the full epilogue."""
    run_case(cuda, dtype, m, n, k, ta, tb, path=2, seed=30)
    run_case(cuda, dtype, m, n, k, ta, tb, path=2, bias="row", alpha=0.5, beta=2.0, act="relu", seed=31)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bn", [32, 64, 128, 256])
def test_tc_two_tiles_per_block(cuda, dtype, bn, monkeypatch):
    """A CTA that owns two vertically adjacent 128-row tiles sharing every B stage (chosen by the cost model for large
    products): forced here for every tile width, all operand layouts, ragged extents, an m whose last block has no
    lower tile, batches, and the epilogue."""
    monkeypatch.setenv("TORCHVULKAN_GEMM_MT", "2")
    monkeypatch.setenv("TORCHVULKAN_GEMM_BN", str(bn))
    for ta, tb in LAYOUTS:
        run_case(cuda, dtype, 520, 328, 264, ta, tb, path=1, seed=70)
    run_case(cuda, dtype, 300, 136, 72, False, True, path=1, batch=3, seed=71)                 # blocks 0..1, the second half empty below row 300
    run_case(cuda, dtype, 384, 200, 1024, True, False, path=1, bias="row", alpha=0.5, beta=2.0, act="gelu", seed=72)
    run_case(cuda, dtype, 1024, 512, 2048, False, False, path=1, seed=73)


def test_tc_block_choice_large_product(cuda):
    """4096 x 4096 x 1024 takes the two-tile blocks by itself; checked on a strided sample of rows."""
    a = cpu_randn((4096, 1024), torch.float16, 74)
    b = cpu_randn((1024, 4096), torch.float16, 75)
    out = ops().gemm(a.to(cuda), b.to(cuda))
    ops().check_device_status()
    rows = torch.arange(0, 4096, 61)
    assert rel_fro(f64(out[rows]), oracle.gemm(f64(a[rows]), f64(b))) <= 2e-3
    assert not torch.isnan(out).any()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k,ta,tb", [(256, 10, 8192, False, True),      # classifier head: split-K on the tensor cores
                                         (10, 8192, 256, True, False),      # its weight gradient: A^T is repacked
                                         (12, 4096, 250, True, True),       # both operands repacked
                                         (300, 7, 4096, False, True)])
def test_skinny_shapes_take_the_tensor_core_path(cuda, dtype, m, n, k, ta, tb):
    """Left to itself the library runs a large skinny product through the TMA pipeline, copying a small operand whose
    rows TMA cannot address into a K-major buffer first."""
    a = operand(m, k, dtype, 81, ta)
    b = operand(k, n, dtype, 82, tb)
    adev = torch.empty_strided(a.shape, a.stride(), dtype=dtype, device=cuda).copy_(a)
    bdev = torch.empty_strided(b.shape, b.stride(), dtype=dtype, device=cuda).copy_(b)
    out = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
    assert ops().gemm_path(adev, bdev, out) == 1
    bias = cpu_randn(n, dtype, 83)
    ops().gemm(adev, bdev, bias=bias.to(cuda), alpha=0.5, beta=2.0, act="relu", out=out)
    ops().check_device_status()
    check(out, oracle.gemm(f64(a), f64(b), f64(bias), 0.5, 2.0, "relu"), dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k,ta", [(256, 8192, 10, False),      # the input gradient of a classifier head
                                      (256, 8192, 10, True), (1, 512, 1, False), (5, 1032, 16, False), (300, 4096, 7, True), (9, 520, 3, False)])
def test_small_k_products_run_on_the_output_bound_kernel(cuda, dtype, m, n, k, ta):
    """k <= 16 against a wide B with contiguous rows: no contraction to speak of, the product is bound by writing C. One
    CUDA-core launch applies alpha, bias, the activation and the activation-gradient operand (the mm + gelu_backward
    pair of a classifier head's input gradient) in registers."""
    a, b = operand(m, k, dtype, 91, ta), operand(k, n, dtype, 92, False)
    bias = cpu_randn(n, dtype, 93)
    adev = torch.empty_strided(a.shape, a.stride(), dtype=dtype, device=cuda).copy_(a)
    bdev = b.to(cuda)
    out = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
    assert ops().gemm_path(adev, bdev, out) == 2
    ops().gemm(adev, bdev, bias=bias.to(cuda), alpha=0.5, beta=2.0, act="relu", out=out)
    ops().check_device_status()
    check(out, oracle.gemm(f64(a), f64(b), f64(bias), 0.5, 2.0, "relu"), dtype)
    x = cpu_randn((m, n), dtype, 94)
    for aux_op, back in (("gelu_backward", oracle.gelu_backward), ("relu_backward", lambda g, t: np.where(t > 0, g, 0.0))):
        out = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
        if dtype == torch.float32:
            continue                                     # the activation-gradient operand is a half-type feature of the product
        assert ops().gemm_path(adev, bdev, out, aux=x.to(cuda), aux_op=aux_op) == 2
        ops().gemm(adev, bdev, alpha=0.25, out=out, aux=x.to(cuda), aux_op=aux_op)
        ops().check_device_status()
        check(out, back(oracle.gemm(f64(a), f64(b), None, 0.25), f64(x)), dtype)
    # a column-major B is not this kernel's case
    bt = operand(k, n, dtype, 92, True)
    btdev = torch.empty_strided(bt.shape, bt.stride(), dtype=dtype, device=cuda).copy_(bt)
    out = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
    ops().gemm(adev, btdev, out=out)
    check(out, oracle.gemm(f64(a), f64(bt), None, 1.0), dtype)


def test_skinny_n_batched(cuda):
    run_case(cuda, torch.float16, 64, 12, 512, False, True, path=2, batch=3, seed=32)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("ta,tb", LAYOUTS)
def test_tc_ragged_edges(cuda, dtype, ta, tb):
    # none of m, n, k is a multiple of the tile; the strides stay 16-byte multiples
    run_case(cuda, dtype, 200, 328, 136, ta, tb, path=1, seed=10)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("m,n,k", [(128, 32, 64), (1024, 1024, 1024), (256, 8192, 784), (8192, 8192, 256), (4096, 64, 2048),
                                   (136, 4096, 8), (384, 640, 4096)])
def test_tc_shapes(cuda, dtype, m, n, k):
    if dtype == torch.float32 and m * n * k > 2 ** 31:
        pytest.skip("kept for the half types")
    run_case(cuda, dtype, m, n, k, False, True, path=1, seed=20)   # x @ W^T, the nn.Linear forward
    run_case(cuda, dtype, m, n, k, True, False, path=1, seed=21)   # g^T @ x, the weight gradient


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("path", [1, 2])
def test_epilogue_bias_alpha_beta_activation(cuda, dtype, path):
    for bias in ("row", "full", "col"):
        for act in (None, "relu", "gelu"):
            run_case(cuda, dtype, 160, 264, 192, False, True, path=path, bias=bias, alpha=0.5, beta=2.0, act=act, seed=30)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k,ta,tb", [(256, 8192, 512, False, True), (160, 264, 192, False, True), (300, 200, 136, False, False),
                                         (256, 1000, 320, True, False), (64, 72, 64, False, True)])
def test_fused_epilogue_two_outputs_and_activation_gradient(cuda, dtype, m, n, k, ta, tb):
    """The fused forms against the oracle's composition of the separate operators: (i) addmm with the pre-activation in
    C and gelu / relu of it in c2; (ii) mm followed by gelu_backward / threshold_backward with the saved pre-activation
    as the aux operand (src/shaders/core/dtype.slang:739-744). Same bars as the plain product."""
    a, b = operand(m, k, dtype, 61, ta), operand(k, n, dtype, 62, tb)
    bias = cpu_randn(n, dtype, 63)
    adev = torch.empty_strided(a.shape, a.stride(), dtype=dtype, device=cuda).copy_(a)
    bdev = torch.empty_strided(b.shape, b.stride(), dtype=dtype, device=cuda).copy_(b)
    for act in ("gelu", "relu"):
        z = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
        h = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
        ops().gemm(adev, bdev, bias=bias.to(cuda), alpha=0.25, beta=1.0, act=act, out=z, out2=h)
        ops().check_device_status()
        check(z, oracle.gemm(f64(a), f64(b), f64(bias), 0.25, 1.0, None), dtype)
        check(h, oracle.gemm(f64(a), f64(b), f64(bias), 0.25, 1.0, act), dtype)
        # c2 comes from the fp32 accumulator, not from the rounded value in C: it equals the one-output
        # addmm-activation result of the same kernel bit for bit
        h1 = ops().gemm(adev, bdev, bias=bias.to(cuda), alpha=0.25, beta=1.0, act=act, force_path=1)
        assert torch.equal(h, h1)
    x = cpu_randn((m, n), dtype, 64)                     # the saved pre-activation
    for aux_op, back in (("gelu_backward", oracle.gelu_backward), ("relu_backward", lambda g, t: np.where(t > 0, g, 0.0))):
        out = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
        ops().gemm(adev, bdev, alpha=0.25, out=out, aux=x.to(cuda), aux_op=aux_op)
        ops().check_device_status()
        check(out, back(oracle.gemm(f64(a), f64(b), None, 0.25), f64(x)), dtype)
    # a strided aux operand (a column slice of a wider buffer) and both fusions at once
    wide = cpu_randn((m, n + 24), dtype, 65)
    xs = wide.to(cuda)[:, 8:8 + n]
    z = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
    h = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
    ops().gemm(adev, bdev, alpha=0.25, act="relu", out=z, out2=h, aux=xs, aux_op="gelu_backward")
    ref = oracle.gelu_backward(oracle.gemm(f64(a), f64(b), None, 0.25), f64(wide[:, 8:8 + n]))
    check(z, ref, dtype)
    check(h, np.maximum(ref, 0.0), dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k,tb", [(256, 4096, 4096, True), (128, 2048, 8192, False), (200, 4096, 4096, False)])
def test_weight_streaming_product_runs_as_k_slices_with_fused_finishing_pass(cuda, dtype, m, n, k, tb):
    """One or two 128-row tiles against a large weight matrix run as K slices whose finishing pass applies the whole
    epilogue: bias + activation, the second output and the activation gradient, against the oracle's composition of
    the separate operators."""
    a, b = operand(m, k, dtype, 71, False), operand(k, n, dtype, 72, tb)
    bias = cpu_randn(n, dtype, 73)
    adev = a.to(cuda)
    bdev = torch.empty_strided(b.shape, b.stride(), dtype=dtype, device=cuda).copy_(b)
    z = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
    h = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
    d = ops().gemm_desc(adev, bdev, z, bias=bias.to(cuda), act="gelu", out2=h)
    assert ops().gemm_splits(d) > 1
    ops().gemm(adev, bdev, bias=bias.to(cuda), alpha=0.125, act="gelu", out=z, out2=h)
    ops().check_device_status()
    check(z, oracle.gemm(f64(a), f64(b), f64(bias), 0.125, 1.0, None), dtype)
    check(h, oracle.gemm(f64(a), f64(b), f64(bias), 0.125, 1.0, "gelu"), dtype)
    plain = ops().gemm(adev, bdev, bias=bias.to(cuda), alpha=0.125)
    assert torch.equal(plain, z)                              # the same slices, the same sums
    # two row tiles take the CTA-pair kernel (tcgen05 cta_group::2); the single-CTA kernel gives the same bits
    import os
    os.environ["TORCHVULKAN_GEMM_PAIR"] = "0"
    try:
        single = ops().gemm(adev, bdev, bias=bias.to(cuda), alpha=0.125)
    finally:
        del os.environ["TORCHVULKAN_GEMM_PAIR"]
    ops().check_device_status()
    assert torch.equal(single, plain)
    x = cpu_randn((m, n), dtype, 74)
    out = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
    ops().gemm(adev, bdev, alpha=0.125, out=out, aux=x.to(cuda), aux_op="gelu_backward")
    ops().check_device_status()
    check(out, oracle.gelu_backward(oracle.gemm(f64(a), f64(b), None, 0.125), f64(x)), dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("ta,tb", LAYOUTS)
@pytest.mark.parametrize("m,n,k", [(512, 512, 8192), (2752, 512, 4096), (328, 1376, 2048)])
def test_few_tiles_long_k_runs_on_cta_pairs(cuda, dtype, m, n, k, ta, tb):
    """Products with few 256 x 256 tiles and a long K (a decoder layer's weight gradients) run as K slices on CTA pairs
    (tcgen05 cta_group::2), for all four operand layouts and ragged last tiles; checked against the oracle and, bit for
    bit, against the single-CTA kernel on the same slices."""
    import os
    a, b = operand(m, k, dtype, 81, ta), operand(k, n, dtype, 82, tb)
    adev = torch.empty_strided(a.shape, a.stride(), dtype=dtype, device=cuda).copy_(a)
    bdev = torch.empty_strided(b.shape, b.stride(), dtype=dtype, device=cuda).copy_(b)
    out = torch.full((m, n), float("nan"), dtype=dtype, device=cuda)
    d = ops().gemm_desc(adev, bdev, out)
    splits = ops().gemm_splits(d)
    assert splits > 1
    ops().gemm(adev, bdev, out=out, alpha=0.5)
    ops().check_device_status()
    check(out, oracle.gemm(f64(a), f64(b), None, 0.5), dtype)
    os.environ["TORCHVULKAN_GEMM_PAIR"] = "0"
    try:
        same_slices = ops().gemm_splits(d) == splits
        single = ops().gemm(adev, bdev, alpha=0.5)
    finally:
        del os.environ["TORCHVULKAN_GEMM_PAIR"]
    ops().check_device_status()
    check(single, oracle.gemm(f64(a), f64(b), None, 0.5), dtype)
    if same_slices:
        assert torch.equal(single, out)


def test_fused_epilogue_is_refused_off_the_tensor_core_path(cuda):
    from torchvulkan_b200.capi import TvkError
    a, b = cpu_randn((64, 64), torch.float32, 1).to(cuda), cpu_randn((64, 64), torch.float32, 2).to(cuda)
    out, out2 = torch.empty(64, 64, device=cuda), torch.empty(64, 64, device=cuda)
    with pytest.raises(TvkError, match="NOT IMPLEMENTED"):
        ops().gemm(a, b, out=out, out2=out2, act="relu")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("path", [1, 2])
def test_batched(cuda, dtype, path):
    run_case(cuda, dtype, 136, 200, 264, False, False, path=path, batch=5, seed=40)
    run_case(cuda, dtype, 136, 200, 264, True, True, path=path, batch=3, seed=41)
    # batch broadcast of B (src/api/ops/matmul.cpp:27-78)
    a = cpu_randn((4, 128, 64), dtype, 42)
    b = cpu_randn((64, 96), dtype, 43)
    out = torch.full((4, 128, 96), float("nan"), dtype=dtype, device=cuda)
    ops().gemm(a.to(cuda), b.to(cuda), out=out, force_path=path)
    check(out, oracle.gemm(f64(a), f64(b)), dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_simt_path_odd_strides_and_shapes(cuda, dtype):
    for (m, n, k) in [(256, 10, 8192), (256, 8192, 10), (10, 8192, 256), (1, 1, 1), (3, 5, 7), (65, 63, 17), (1, 512, 300)]:
        for ta, tb in LAYOUTS:
            run_case(cuda, dtype, m, n, k, ta, tb, path=2, seed=50)


def test_auto_path_and_empty(cuda):
    a = cpu_randn((64, 10), torch.float16, 60).to(cuda)       # a small product: CUDA cores
    b = cpu_randn((10, 96), torch.float16, 61).to(cuda)
    assert ops().gemm_path(a, b, torch.empty((64, 96), dtype=torch.float16, device=cuda)) == 2
    out = torch.empty((256, 8192), dtype=torch.float16, device=cuda)
    a2 = cpu_randn((256, 784), torch.float16, 62).to(cuda)
    b2 = cpu_randn((8192, 784), torch.float16, 63).to(cuda)
    assert ops().gemm_path(a2, b2.t(), out) == 1
    # k == 0: out = act(beta * bias) (src/api/ops/matmul.cpp:284-288)
    bias = cpu_randn(8, torch.float32, 64)
    o = ops().gemm(torch.empty((4, 0), device=cuda), torch.empty((0, 8), device=cuda), bias=bias.to(cuda), beta=2.0)
    assert torch.allclose(o.cpu(), (2.0 * bias).expand(4, 8))
    assert ops().gemm(torch.empty((0, 5), device=cuda), torch.empty((5, 3), device=cuda)).shape == (0, 3)


def test_config1_fp32_mm_relu_sum(cuda):
    """BASELINE config 1: fp32 1024^3 mm -> relu -> sum on torch.manual_seed(0) N(0,1) inputs."""
    torch.manual_seed(0)
    x, y = torch.randn(1024, 1024), torch.randn(1024, 1024)
    z = ops().gemm(x.to(cuda), y.to(cuda))
    zr = ops().unary("relu", z)
    s = ops().reduce("sum", zr)
    ops().check_device_status()
    ref_z = np.maximum(x.double().numpy() @ y.double().numpy(), 0.0)
    ref_s = ref_z.sum()
    assert abs(float(s) - ref_s) / abs(ref_s) <= 1e-4
    assert np.max(np.abs(f64(zr) - ref_z)) / np.max(ref_z) <= 1e-4
    assert np.all(np.abs(f64(zr) - ref_z) <= 1e-4 + 1e-3 * np.abs(ref_z))
    # and against ATen CPU fp32 itself, the reference's fallback for this op
    cpu = (x @ y).relu()
    assert torch.allclose(zr.cpu(), cpu, atol=1e-4, rtol=1e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16])
def test_config5_bmm_slice(cuda, dtype):
    """BASELINE config 5 at 2 of its 64 batches: bf16 bmm of 4096^3 with N(0,1) inputs; checked on a
    strided sample of rows against the fp64 oracle (the full product takes the CPU minutes)."""
    torch.manual_seed(0)
    a = torch.randn(2, 4096, 4096).to(dtype)
    b = torch.randn(2, 4096, 4096).to(dtype)
    out = ops().gemm(a.to(cuda), b.to(cuda))
    ops().check_device_status()
    rows = torch.arange(0, 4096, 97)
    ref = oracle.gemm(f64(a[:, rows]), f64(b))
    err = rel_fro(f64(out[:, rows]), ref)
    assert err <= 1e-2, err
    assert not torch.isnan(out).any()


@pytest.mark.parametrize("a_dt,b_dt", [(torch.float8_e4m3fn, torch.float8_e4m3fn), (torch.float8_e5m2, torch.float8_e4m3fn)])
@pytest.mark.parametrize("m,n,k", [(256, 512, 128), (300, 520, 1040), (128, 64, 144), (1024, 1024, 2048)])
def test_scaled_mm_float8_kernel_through_the_c_abi(cuda, a_dt, b_dt, m, n, k):
    """tvk_scaled_mm on k-contiguous float8 operands (the tcgen05 kind::f8f6f4 kernel, scales / bias / cast in its epilogue)
    against the float64 product of the same float8 values: products of float8 numbers are exact in fp32, so only the order
    of the fp32 additions differs (1e-5 relative for an fp32 result; the 16-bit results to their rounding)."""
    g = torch.Generator().manual_seed(71)
    a = torch.randn(m, k, generator=g).to(a_dt)
    b = torch.randn(n, k, generator=g).to(b_dt).t()
    bias = torch.randn(n, generator=g)
    ref = f64(a.float()) @ f64(b.float())
    for rowwise in (False, True):
        sa = (torch.rand(m, 1, generator=g) + 0.5) if rowwise else torch.tensor(0.75)
        sb = (torch.rand(1, n, generator=g) + 0.5) if rowwise else torch.tensor(1.5)
        want = ref * f64(sa) * f64(sb)
        for out_dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2), (torch.float16, 1e-3)):
            bdev = bias.to(out_dtype).to(cuda)
            got = ops().scaled_mm(a.to(cuda), torch.empty_strided(b.shape, b.stride(), dtype=b_dt, device=cuda).copy_(b), sa.to(cuda), sb.to(cuda),
                                  out_dtype=out_dtype, bias=bdev)
            ops().check_device_status()
            assert rel_fro(f64(got), want + f64(bias.to(out_dtype))) <= tol
    # float8 output divided by scale_result (the accumulator route + finishing pass)
    sr = torch.tensor(4.0)
    got8 = ops().scaled_mm(a.to(cuda), torch.empty_strided(b.shape, b.stride(), dtype=b_dt, device=cuda).copy_(b), torch.tensor(0.75).to(cuda),
                           torch.tensor(1.5).to(cuda), out_dtype=torch.float8_e4m3fn, scale_result=sr.to(cuda))
    want8 = torch.from_numpy(ref * 0.75 * 1.5 / 4.0).float().to(torch.float8_e4m3fn).float()
    g8 = got8.cpu().float()
    same = (g8 == want8) | (g8.isnan() & want8.isnan())
    assert same.float().mean() >= 0.995

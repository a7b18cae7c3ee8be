"""GPU parity of the bandwidth kernels against the numpy oracle, through the C-ABI.

Tolerances (stated per test): index/byte results bit-exact; fp32 results max relative error
1e-4 (most are held to ~1e-6); fp16/bf16 results relative Frobenius error <= 1e-2 against the
float64 oracle evaluated on the same (already rounded) inputs.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import rel_fro

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
TOL = {torch.float32: 2e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}  # all far inside the 1e-4 / 1e-2 bars


def ops():
    from torchvulkan_b200 import cuda_ops
    return cuda_ops


def cpu_randn(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def f64(t):
    return t.detach().float().cpu().double().numpy()


def check_float(out, ref, dtype, tol=None):
    tol = TOL[dtype] if tol is None else tol
    o = f64(out)
    ref = np.asarray(ref, np.float64)
    # values beyond the range of the storage type become +-inf on both sides
    ref_rounded = torch.from_numpy(ref).to(dtype).double().numpy()
    finite = np.isfinite(ref_rounded)
    assert np.array_equal(np.isnan(o), np.isnan(ref))
    assert np.array_equal(o[~finite & ~np.isnan(ref)], ref_rounded[~finite & ~np.isnan(ref)])
    err = rel_fro(o[finite], ref[finite])
    assert err <= tol, f"relative Frobenius error {err:.3e} > {tol:.1e}"


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dtype", DTYPES)
def test_unary_all_ops(cuda, dtype):
    n = 100003  # not a multiple of the packet size: exercises the scalar tail
    x = cpu_randn(n, dtype, 1)
    for op in ops().UNARY:
        inp = x.abs() + 0.01 if op in ("log", "sqrt", "rsqrt") else x
        out = ops().unary(op, inp.to(cuda))
        check_float(out, oracle.unary(op, f64(inp)), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_unary_unaligned_pointer(cuda, dtype):
    x = cpu_randn(4099, dtype, 2)
    xd = x.to(cuda)
    out = torch.empty_like(xd)
    ops().unary("exp", xd[1:], out=out[1:])  # base pointers 2 or 4 bytes past a 16-byte boundary
    check_float(out[1:], oracle.unary("exp", f64(x[1:])), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_binary_ops_tensor_and_scalar(cuda, dtype):
    a, b = cpu_randn(70001, dtype, 3), cpu_randn(70001, dtype, 4)
    for op in ops().BINARY:
        alpha = 0.5 if op in ("add", "sub") else (0.1 if op == "threshold_backward" else 1.0)
        aa = a.abs() + 0.5 if op == "pow" else a
        out = ops().binary(op, aa.to(cuda), b.to(cuda), alpha=alpha)
        check_float(out, oracle.binary(op, f64(aa), f64(b), alpha), dtype)
    for op in ("add", "sub", "mul", "div", "maximum", "pow"):
        s = 2.0 if op == "pow" else 1.75
        out = ops().binary(op, a.to(cuda), s, alpha=1.0)
        check_float(out, oracle.binary(op, f64(a), np.float64(s)), dtype)


def test_compare_where_fill_cast(cuda):
    a, b = cpu_randn(5000, torch.float32, 5).round(decimals=1), cpu_randn(5000, torch.float32, 6).round(decimals=1)
    ad, bd = a.to(cuda), b.to(cuda)
    for op, fn in (("eq", torch.eq), ("ne", torch.ne), ("lt", torch.lt), ("le", torch.le), ("gt", torch.gt), ("ge", torch.ge)):
        assert torch.equal(ops().compare(op, ad, bd).cpu(), fn(a, b))          # bit-exact
        assert torch.equal(ops().compare(op, ad, 0.1).cpu(), fn(a, 0.1))
    cond = (a > 0)
    out = ops().ternary("where", ad, bd, cond.to(cuda))
    assert torch.equal(out.cpu(), torch.where(cond, a, b))
    for dtype in DTYPES + [torch.int64, torch.int32, torch.uint8]:
        t = torch.empty(1001, dtype=dtype, device=cuda)
        ops().fill(t, 3)
        assert torch.equal(t.cpu(), torch.full((1001,), 3, dtype=dtype))
    x = cpu_randn(4097, torch.float32, 7, 100.0)
    for src in DTYPES:
        for dst in DTYPES + [torch.int64]:
            xs = x.to(src)
            assert torch.equal(ops().cast(xs.to(cuda), dst).cpu(), xs.to(dst)), (src, dst)  # conversions are exact-rule
    idx = torch.arange(-500, 500)
    assert torch.equal(ops().cast(idx.to(cuda), torch.float16).cpu(), idx.to(torch.float16))


@pytest.mark.parametrize("dtype", DTYPES)
def test_ternary_ops(cuda, dtype):
    a, b, c = (cpu_randn(33333, dtype, s) for s in (8, 9, 10))
    c = c.abs() + 0.5
    fa, fb, fc = f64(a), f64(b), f64(c)
    check_float(ops().ternary("addcmul", a.to(cuda), b.to(cuda), c.to(cuda), value=0.3), fa + 0.3 * fb * fc, dtype)
    check_float(ops().ternary("addcdiv", a.to(cuda), b.to(cuda), c.to(cuda), value=-0.7), fa - 0.7 * fb / fc, dtype)
    check_float(ops().ternary("lerp", a.to(cuda), b.to(cuda), None, value=0.1), fa + 0.1 * (fb - fa), dtype)


def test_strided_and_broadcast(cuda):
    a = cpu_randn((7, 1, 33), torch.float32, 11)
    b = cpu_randn((5, 33), torch.float32, 12)
    out = ops().binary_strided("add", a.to(cuda), b.to(cuda), alpha=2.0)
    assert torch.allclose(out.cpu(), a + 2.0 * b, rtol=1e-6, atol=1e-6)
    t = cpu_randn((64, 48), torch.float16, 13)
    td = t.to(cuda)
    assert torch.equal(ops().unary_strided("neg", td.t()).cpu(), -t.t())
    assert torch.equal(ops().compare_strided("lt", td.t(), td.t().contiguous()).cpu(), torch.zeros(48, 64, dtype=torch.bool))
    # copies: transposing path, generic path, cast on the way
    for dtype in (torch.float16, torch.float32, torch.int64):
        m = (cpu_randn((130, 70), torch.float32, 14) * 10).to(dtype)
        md = m.to(cuda)
        assert torch.equal(ops().copy_strided(md.t()).cpu(), m.t().contiguous())
        assert torch.equal(ops().copy_strided(md[::2, 1::3]).cpu(), m[::2, 1::3].contiguous())
    b3 = cpu_randn((3, 40, 50), torch.bfloat16, 15)
    assert torch.equal(ops().copy_strided(b3.to(cuda).transpose(1, 2)).cpu(), b3.transpose(1, 2).contiguous())
    assert torch.equal(ops().copy_strided(b3.to(cuda).permute(2, 0, 1), torch.float32).cpu(), b3.permute(2, 0, 1).float().contiguous())
    w = ops().ternary_strided("addcmul", a.to(cuda), b.to(cuda), b.to(cuda), value=0.5)
    assert torch.allclose(w.cpu(), a + 0.5 * b * b, rtol=1e-6, atol=1e-6)


# ------------------------------------------------------------------ reductions
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,dim", [((1 << 21) + 3, None), ((2048, 512), 1), ((256, 4096), 0), ((32, 200, 48), 1),
                                        ((3, 5), 1), ((100000, 10), 1), ((7, 70000), 1)])
def test_reduce_sum_mean_amax(cuda, dtype, shape, dim):
    x = cpu_randn(shape, dtype, 20)
    xd = x.to(cuda)
    axis = dim
    ref_in = f64(x).reshape(1, -1) if dim is None else f64(x)
    axis = 1 if dim is None else dim
    for op in ("sum", "mean", "amax", "amin"):
        out = ops().reduce(op, xd, dim, out_dtype=torch.float32)
        ref = oracle.reduce(op, ref_in, axis).reshape(out.shape)
        # fp32 accumulation: compare against the float64 oracle relative to the scale of the data
        scale = np.sqrt(ref_in.shape[axis]) if op == "sum" else 1.0
        assert np.max(np.abs(f64(out) - ref)) <= 2e-5 * scale, op
    out = ops().reduce("sum", xd, dim)  # output in the input dtype: one rounding of the fp32 sum
    ref = torch.from_numpy(oracle.reduce("sum", ref_in, axis).reshape(out.shape)).to(dtype)
    assert torch.allclose(out.cpu().float(), ref.float(), rtol=2e-2 if dtype != torch.float32 else 1e-4, atol=1e-2)


def test_reduce_nan_and_empty(cuda):
    x = cpu_randn((64, 300), torch.float32, 21)
    x[3, 17] = float("nan")
    out = ops().reduce("amax", x.to(cuda), 1)
    np.testing.assert_array_equal(out.cpu().numpy(), x.amax(1).numpy())
    e = torch.empty((4, 0), device=cuda)
    assert torch.equal(ops().reduce("sum", e, 1).cpu(), torch.zeros(4))
    # over the leading axis of wide rows (the one-pass column kernel): NaN propagates, ragged last column tile
    y = cpu_randn((300, 1000), torch.float16, 22)
    y[299, 999] = float("nan"); y[0, 0] = float("nan")
    for op in ("amax", "amin", "sum"):
        got = ops().reduce(op, y.to(cuda), 0, out_dtype=torch.float32).cpu().numpy()
        want = getattr(y.float(), op)(0).numpy()
        assert np.array_equal(np.isnan(got), np.isnan(want)), op
        ok = ~np.isnan(want)
        assert np.allclose(got[ok], want[ok], rtol=1e-5, atol=1e-4), op


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,dim", [((1 << 22) + 5, None), ((256, 10), 1), ((300, 77, 5), 1), ((64, 50000), 1), ((5000, 33), 0)])
def test_argmax_argmin_bit_exact(cuda, dtype, shape, dim):
    g = torch.Generator().manual_seed(22)
    x = torch.randint(-50, 51, shape if isinstance(shape, tuple) else (shape,), generator=g).to(dtype)  # heavy ties
    flat = x.reshape(-1)
    flat[torch.randint(0, flat.numel(), (3,), generator=g)] = float("nan")
    xd = x.to(cuda)
    for is_max in (True, False):
        out = ops().argreduce(xd, dim, is_max)
        ref_in = x.float().numpy().reshape(1, -1) if dim is None else x.float().numpy()
        ref = oracle.argreduce(ref_in, 1 if dim is None else dim, is_max).reshape(out.shape)
        assert np.array_equal(out.cpu().numpy(), ref)
    # without NaN: the first maximal element wins
    y = torch.nan_to_num(x, nan=0.0)
    out = ops().argreduce(y.to(cuda), dim, True)
    ref_in = y.float().numpy().reshape(1, -1) if dim is None else y.float().numpy()
    assert np.array_equal(out.cpu().numpy(), oracle.argreduce(ref_in, 1 if dim is None else dim, True).reshape(out.shape))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("lines,n,k", [(256, 10, 3), (64, 128, 128), (7, 1000, 50), (3, 5000, 5000), (1, 70001, 16), (5, 1, 1)])
def test_topk_sort_bit_exact(cuda, dtype, lines, n, k):
    g = torch.Generator().manual_seed(23)
    x = (torch.randint(-30, 31, (lines, n), generator=g).float() / 4).to(dtype)
    if n > 8:
        x[0, 1] = float("nan"); x[0, n - 2] = float("nan"); x[-1, 3] = 0.0; x[-1, 5] = -0.0
    xd = x.to(cuda)
    for desc in (True, False):
        v, i = ops().topk(xd, k, descending=desc)
        rv, ri = oracle.stable_topk(x.float().numpy(), k, descending=desc)
        assert np.array_equal(i.cpu().numpy(), ri)
        np.testing.assert_array_equal(v.float().cpu().numpy(), rv)
        # the reference's own criterion: indices gather to the values (tests/test_pytorch_ops.py:277-290)
        np.testing.assert_array_equal(torch.gather(x, 1, i.cpu()).float().numpy(), v.float().cpu().numpy())


# ------------------------------------------------------------------ softmax / losses
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,cols", [(256, 10), (8192, 128), (33, 1000), (5, 3000), (1, 1)])
def test_softmax_family(cuda, dtype, rows, cols):
    x = cpu_randn((rows, cols), dtype, 30, 3.0)
    g = cpu_randn((rows, cols), dtype, 31)
    for log in (False, True):
        y = ops().softmax(x.to(cuda), log=log)
        ref = oracle.log_softmax(f64(x)) if log else oracle.softmax(f64(x))
        check_float(y, ref, dtype)
        y32 = ops().softmax(x.to(cuda), log=log, out_dtype=torch.float32)   # half_to_float
        check_float(y32, ref, torch.float32, 2e-6)
        gi = ops().softmax_backward(g.to(cuda), y, log=log)
        refg = oracle.log_softmax_backward(f64(g), f64(y)) if log else oracle.softmax_backward(f64(g), f64(y))
        check_float(gi, refg, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_nll_loss(cuda, dtype):
    n, c = 777, 13
    lp = torch.log_softmax(cpu_randn((n, c), torch.float32, 32), -1).to(dtype)
    g = torch.Generator().manual_seed(33)
    t = torch.randint(0, c, (n,), generator=g)
    t[5] = -100; t[9] = -100
    w = (torch.rand(c, generator=g) + 0.5).to(dtype)
    for red in ("mean", "sum", "none"):
        for wt in (None, w):
            out, total = ops().nll_loss_forward(lp.to(cuda), t.to(cuda), None if wt is None else wt.to(cuda), red)
            ref, rtotal = oracle.nll_loss_forward(f64(lp), t.numpy(), None if wt is None else f64(wt), red)
            check_float(out, np.asarray(ref), dtype, 4e-3 if dtype != torch.float32 else 1e-5)
            go = torch.ones((), dtype=dtype) if red != "none" else cpu_randn(n, dtype, 34)
            gi = ops().nll_loss_backward(go.to(cuda), t.to(cuda), c, None if wt is None else wt.to(cuda), red, total_weight=total)
            refg = oracle.nll_loss_backward(f64(go), t.numpy(), c, None if wt is None else f64(wt), red, total_weight=f64(total))
            check_float(gi, refg, dtype, 4e-3 if dtype != torch.float32 else 1e-6)


# ------------------------------------------------------------------ norms / embedding
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,cols", [(8192, 512), (37, 100), (3, 2048), (1000, 8)])
def test_rmsnorm(cuda, dtype, rows, cols):
    x, w, g = cpu_randn((rows, cols), dtype, 40), (cpu_randn(cols, dtype, 41) * 0.2 + 1), cpu_randn((rows, cols), dtype, 42)
    y, rstd = ops().rmsnorm_forward(x.to(cuda), w.to(cuda))
    ry, rrstd = oracle.rmsnorm_forward(f64(x), f64(w))
    check_float(y, ry, dtype)
    check_float(rstd, rrstd, torch.float32, 2e-6)
    gx, gw = ops().rmsnorm_backward(g.to(cuda), x.to(cuda), w.to(cuda), rstd)
    rgx, rgw = oracle.rmsnorm_backward(f64(g), f64(x), f64(w), f64(rstd))
    check_float(gx, rgx, dtype)
    check_float(gw, rgw, dtype, TOL[dtype] * 2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,c,h", [(256, 64, 32), (32, 128, 16), (5, 3, 7), (64, 256, 8)])
def test_batchnorm(cuda, dtype, n, c, h):
    if n * c * h * h > 8_000_000 and dtype == torch.float32:
        n //= 4
    x = (cpu_randn((n, c, h, h), torch.float32, 50) * 2 + 3).to(dtype)
    w, b = (cpu_randn(c, dtype, 51) * 0.1 + 1), cpu_randn(c, dtype, 52)
    g = cpu_randn((n, c, h, h), dtype, 53)
    rm, rv = torch.zeros(c, dtype=dtype), torch.ones(c, dtype=dtype)
    rmd, rvd = rm.to(cuda), rv.to(cuda)
    y, mean, invstd = ops().batchnorm_forward(x.to(cuda), w.to(cuda), b.to(cuda), rmd, rvd, 0.1, 1e-5)
    ry, rmean, rinv, rrm, rrv = oracle.batchnorm_forward(f64(x), f64(w), f64(b), f64(rm), f64(rv), 0.1, 1e-5)
    check_float(y, ry, dtype)
    check_float(mean, rmean, torch.float32, 1e-5)
    check_float(invstd, rinv, torch.float32, 1e-5)
    check_float(rmd, rrm, dtype)
    check_float(rvd, rrv, dtype)
    gx, gw, gb = ops().batchnorm_backward(g.to(cuda), x.to(cuda), w.to(cuda), mean, invstd)
    rgx, rgw, rgb = oracle.batchnorm_backward(f64(g), f64(x), f64(w), f64(mean), f64(invstd))
    check_float(gx, rgx, dtype)
    check_float(gw, rgw, dtype, TOL[dtype] * 2)
    check_float(gb, rgb, dtype, TOL[dtype] * 2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,c,h", [(256, 64, 32), (32, 128, 16), (5, 8, 7), (64, 256, 8), (3, 4104, 2)])
def test_batchnorm_channels_last(cuda, dtype, n, c, h):
    """The channels-last entry points on tensors of torch.channels_last memory format, against the same oracle."""
    if n * c * h * h > 8_000_000 and dtype == torch.float32:
        n //= 4
    cl = torch.channels_last
    x = (cpu_randn((n, c, h, h), torch.float32, 50) * 2 + 3).to(dtype)
    w, b = (cpu_randn(c, dtype, 51) * 0.1 + 1), cpu_randn(c, dtype, 52)
    g = cpu_randn((n, c, h, h), dtype, 53)
    rm, rv = torch.zeros(c, dtype=dtype), torch.ones(c, dtype=dtype)
    rmd, rvd = rm.to(cuda), rv.to(cuda)
    xd, gd = x.to(cuda).contiguous(memory_format=cl), g.to(cuda).contiguous(memory_format=cl)
    y, mean, invstd = ops().batchnorm_forward(xd, w.to(cuda), b.to(cuda), rmd, rvd, 0.1, 1e-5)
    assert y.is_contiguous(memory_format=cl)
    ry, rmean, rinv, rrm, rrv = oracle.batchnorm_forward(f64(x), f64(w), f64(b), f64(rm), f64(rv), 0.1, 1e-5)
    check_float(y, ry, dtype)
    check_float(mean, rmean, torch.float32, 1e-5)
    check_float(invstd, rinv, torch.float32, 1e-5)
    check_float(rmd, rrm, dtype)
    check_float(rvd, rrv, dtype)
    gx, gw, gb = ops().batchnorm_backward(gd, xd, w.to(cuda), mean, invstd)
    rgx, rgw, rgb = oracle.batchnorm_backward(f64(g), f64(x), f64(w), f64(mean), f64(invstd))
    check_float(gx, rgx, dtype)
    check_float(gw, rgw, dtype, TOL[dtype] * 2)
    check_float(gb, rgb, dtype, TOL[dtype] * 2)
    ops().check_device_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(cuda, dtype):
    table = cpu_randn((128, 512), dtype, 60)
    g = torch.Generator().manual_seed(61)
    idx = torch.randint(0, 128, (32, 256), generator=g)
    out = ops().embedding_forward(table.to(cuda), idx.to(cuda))
    assert torch.equal(out.cpu(), table[idx])                                  # bit-exact gather
    grad = cpu_randn((32 * 256, 512), dtype, 62)
    gt = ops().embedding_backward(grad.to(cuda), idx.to(cuda), 128)
    ref = torch.from_numpy(oracle.embedding_backward(grad.float().numpy(), idx.numpy(), 128)).to(dtype)
    assert torch.equal(gt.cpu(), ref)                                          # same fp32 summation order: bit-exact
    gt2 = ops().embedding_backward(grad.to(cuda), idx.to(cuda), 128, padding_idx=7)
    assert torch.count_nonzero(gt2[7]).item() == 0
    ops().check_device_status()


# ------------------------------------------------------------------ optimizers
@pytest.mark.parametrize("dtype", DTYPES)
def test_adam_and_sgd_steps(cuda, dtype):
    n = 100003
    p, g1, g2 = cpu_randn(n, dtype, 70), cpu_randn(n, dtype, 71), cpu_randn(n, dtype, 72)
    pd, md, vd = p.to(cuda), torch.zeros(n, dtype=dtype, device=cuda), torch.zeros(n, dtype=dtype, device=cuda)
    rp, rm, rv = p.float().numpy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    for step, g in ((1, g1), (2, g2)):
        ops().adam_step(pd, g.to(cuda), md, vd, step)
        rp, rm, rv = oracle.adam_step(rp, g.float().numpy(), rm, rv, step)
        # storage rounding: the oracle's fp32 values rounded to the storage dtype, as the device does
        rp, rm, rv = (torch.from_numpy(t).to(dtype).float().numpy() for t in (rp, rm, rv))
        tol = 1e-6 if dtype == torch.float32 else TOL[dtype]
        check_float(pd, rp.astype(np.float64), dtype, tol)
        check_float(md, rm.astype(np.float64), dtype, tol)
        check_float(vd, rv.astype(np.float64), dtype, tol)
    pd, bd = p.to(cuda), torch.zeros(n, dtype=dtype, device=cuda)
    rp, rb = p.float().numpy(), None
    for first, g in ((True, g1), (False, g2)):
        ops().sgd_step(pd, g.to(cuda), bd, 0.1, momentum=0.9, first_step=first)
        rp, rb = oracle.sgd_step(rp, g.float().numpy(), rb, 0.1, momentum=0.9, first_step=first)
        rp, rb = (torch.from_numpy(t).to(dtype).float().numpy() for t in (rp, rb))
        tol = 1e-6 if dtype == torch.float32 else TOL[dtype]
        check_float(pd, rp.astype(np.float64), dtype, tol)
        check_float(bd, rb.astype(np.float64), dtype, tol)


def test_bounded_wait_times_out_and_the_device_stays_usable(cuda):
    """The failure convention of every device-side wait (mbarrier waits of the tensor-core kernels): a wait that runs out
    raises the device status word, the kernel ends normally, tvk_check_device_status reports TVK_ERR_TIMEOUT once, and
    later work on the same context is unaffected. The wait here polls a flag nothing sets, 2000 times."""
    from torchvulkan_b200 import capi

    lib = capi.lib()
    ops().check_device_status()
    capi.call("tvk_debug_bounded_wait", 0, 2000, ops().stream())
    rc = lib.tvk_check_device_status(0)
    assert rc == capi.ERR_TIMEOUT
    msg = lib.tvk_last_error().decode()
    assert "bounded device-side wait ran out" in msg and "site 99" in msg
    assert lib.tvk_check_device_status(0) == capi.OK             # reported once, then cleared
    x = cpu_randn(4096, torch.float32, 77)
    assert torch.equal(ops().unary("neg", x.to(cuda)).cpu(), -x)  # the context still works
    ops().check_device_status()

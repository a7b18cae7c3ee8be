"""The rest of the elementwise / reduction surface on the "vulkan" device, each operator against ATen CPU on the same
inputs: the unary family (src/api/ops/unary.cpp), fmod / remainder / atan2 / floor_divide / clamp and the activations with
their gradients (src/api/ops/binary.cpp), logical and bitwise ops on masks and integer comparisons
(src/api/ops/compare.cpp), max / min / all / any / var / std / vector norm (src/api/ops/reduce.cpp), masked_fill, tril /
triu, arange / linspace / eye, mse_loss. fp32 within 1e-5 (transcendentals 1e-4 relative), fp16 within 1e-2."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vk():
    import torchvulkan  # noqa: F401

    return torch.device("vulkan:0")


def _close(got, want, tol):
    got = got.detach().cpu()
    want = want.detach()
    assert got.shape == want.shape and got.dtype == want.dtype, (got.shape, want.shape, got.dtype, want.dtype)
    if want.dtype == torch.bool or not want.dtype.is_floating_point:
        assert torch.equal(got, want)
        return
    g, w = got.double(), want.double()
    assert torch.equal(g.isnan(), w.isnan())
    fin = w.isfinite()
    assert torch.equal(g[~fin & ~w.isnan()], w[~fin & ~w.isnan()])
    err = (g[fin] - w[fin]).abs()
    assert bool((err <= tol * (1.0 + w[fin].abs())).all()), float(err.max())


UNARY = {
    "floor": (torch.floor, 4.0), "ceil": (torch.ceil, 4.0), "round": (torch.round, 4.0), "trunc": (torch.trunc, 4.0), "sign": (torch.sign, 4.0),
    "log2": (lambda t: torch.log2(t.abs() + 0.1), 4.0), "log10": (lambda t: torch.log10(t.abs() + 0.1), 4.0), "log1p": (lambda t: torch.log1p(t.abs()), 4.0),
    "expm1": (torch.expm1, 2.0), "exp2": (torch.exp2, 3.0), "tan": (torch.tan, 1.0), "sinh": (torch.sinh, 2.0), "cosh": (torch.cosh, 2.0),
    "asin": (lambda t: torch.asin(t.clamp(-0.99, 0.99)), 0.7), "acos": (lambda t: torch.acos(t.clamp(-0.99, 0.99)), 0.7), "atan": (torch.atan, 4.0),
    "erf": (torch.erf, 2.0), "erfc": (torch.erfc, 1.5), "hardsigmoid": (F.hardsigmoid, 4.0), "hardswish": (F.hardswish, 4.0), "mish": (F.mish, 4.0),
    "logsigmoid": (F.logsigmoid, 4.0), "isnan": (torch.isnan, 1.0), "isinf": (torch.isinf, 1.0), "isfinite": (torch.isfinite, 1.0),
    "isposinf": (torch.isposinf, 1.0), "isneginf": (torch.isneginf, 1.0),
    "asinh": (torch.asinh, 4.0), "acosh": (lambda t: torch.acosh(t.abs() + 1.0), 4.0), "atanh": (lambda t: torch.atanh(t.clamp(-0.95, 0.95)), 0.6),
    "erfinv": (lambda t: torch.erfinv(t.clamp(-0.98, 0.98)), 0.6), "lgamma": (lambda t: torch.lgamma(t.abs() + 0.5), 3.0), "frac": (torch.frac, 4.0), "sinc": (torch.sinc, 2.0),
    "nan_to_num": (lambda t: torch.nan_to_num(t, nan=0.5), 1.0), "nan_to_num_args": (lambda t: torch.nan_to_num(t, nan=0.0, posinf=9.0, neginf=-9.0), 1.0),
    "softshrink": (lambda t: F.softshrink(t, 0.4), 2.0), "count_nonzero": (lambda t: torch.count_nonzero(t.round(), dim=1), 1.0),
    "clamp": (lambda t: t.clamp(-1.0, 0.5), 2.0), "clamp_min": (lambda t: t.clamp_min(0.25), 2.0), "clamp_max": (lambda t: t.clamp(max=0.25), 2.0),
    "relu6": (F.relu6, 5.0), "hardtanh": (lambda t: F.hardtanh(t, -0.5, 1.5), 2.0), "leaky_relu": (lambda t: F.leaky_relu(t, 0.1), 2.0),
    "elu": (lambda t: F.elu(t, 1.3), 2.0), "softplus": (lambda t: F.softplus(t, 2.0), 6.0), "selu": (F.selu, 2.0), "celu": (lambda t: F.celu(t, 0.7), 2.0),
    "glu": (lambda t: F.glu(t[:, :-1]), 2.0), "prelu": (lambda t: F.prelu(t, torch.full((1,), 0.2, dtype=t.dtype, device=t.device)), 2.0),
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("name", sorted(UNARY))
def test_unary_surface(vk, name, dtype):
    fn, spread = UNARY[name]
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(37, 53, generator=g) * spread).to(dtype)
    if name.startswith("is") or name.startswith("clamp") or name.startswith("nan_to_num"):
        x[3, 5], x[4, 6], x[5, 7] = float("nan"), float("inf"), float("-inf")
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    _close(fn(x.to(vk)), fn(x), tol)
    # a transposed (strided) operand takes the strided kernels
    _close(fn(x.to(vk).t()), fn(x.t()), tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("name", ["clamp", "relu6", "hardtanh", "leaky_relu", "elu", "softplus", "hardsigmoid", "hardswish", "mish", "logsigmoid", "selu", "celu", "glu", "prelu"])
def test_activation_gradients(vk, name, dtype):
    fn, spread = UNARY[name]
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(41, 29, generator=g) * spread).to(dtype)
    xd, xc = x.to(vk).requires_grad_(), x.double().requires_grad_()
    yd, yc = fn(xd), fn(xc)
    gy = torch.randn(yc.shape, generator=g).to(dtype)
    yd.backward(gy.to(vk)); yc.backward(gy.double())
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    _close(xd.grad.double(), xc.grad, tol)


def test_elu_in_place_gradient_from_the_result(vk):
    x = torch.randn(64, 32)
    gy = torch.randn(64, 32)
    xd, xc = x.to(vk).requires_grad_(), x.clone().requires_grad_()
    F.elu(xd * 1.0, 0.7, inplace=True).backward(gy.to(vk)); F.elu(xc * 1.0, 0.7, inplace=True).backward(gy)
    _close(xd.grad, xc.grad, 2e-5)


BINARY = {
    "fmod": torch.fmod, "remainder": torch.remainder, "atan2": torch.atan2, "floor_divide": torch.floor_divide,
    "hypot": torch.hypot, "copysign": torch.copysign, "logaddexp": torch.logaddexp, "logaddexp2": torch.logaddexp2, "fmax": torch.fmax, "fmin": torch.fmin,
    "heaviside": lambda a, b: torch.heaviside(a.round(), b),
    "fmod_scalar": lambda a, b: a.fmod(1.5), "remainder_scalar": lambda a, b: a % -1.5, "floor_divide_scalar": lambda a, b: a // 0.75,
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("name", sorted(BINARY))
def test_binary_surface(vk, name, dtype):
    g = torch.Generator().manual_seed(5)
    a = (torch.randn(33, 47, generator=g) * 5).to(dtype)
    b = (torch.randn(33, 47, generator=g) * 2).to(dtype)
    b[b.abs() < 0.05] = 0.5
    fn = BINARY[name]
    got, want = fn(a.to(vk), b.to(vk)), fn(a, b)
    if dtype == torch.float16 and "floor_divide" in name:
        # the quotient is formed in fp32 on the device and in fp16 steps on the CPU: they may differ by one at an exact multiple
        assert float((got.cpu().float() - want.float()).abs().max()) <= 1.0
        assert float(((got.cpu() - want) != 0).float().mean()) < 0.01
        return
    _close(got, want, 2e-5 if dtype == torch.float32 else 1e-2)
    # broadcast second operand
    _close(fn(a.to(vk), b[:1].to(vk)), fn(a, b[:1]), 2e-5 if dtype == torch.float32 else 1e-2) if "scalar" not in name and "floor" not in name else None


def test_logical_and_bitwise_ops_on_masks(vk):
    g = torch.Generator().manual_seed(6)
    a, b = torch.rand(19, 23, generator=g) > 0.5, torch.rand(19, 23, generator=g) > 0.5
    x = torch.randn(19, 23, generator=g)
    x[x.abs() < 0.3] = 0
    ad, bd, xd = a.to(vk), b.to(vk), x.to(vk)
    for fn in (torch.logical_and, torch.logical_or, torch.logical_xor, lambda p, q: p & q, lambda p, q: p | q, lambda p, q: p ^ q, lambda p, q: p * q):
        _close(fn(ad, bd), fn(a, b), 0)
    _close(~ad, ~a, 0)
    _close(torch.logical_not(ad), torch.logical_not(a), 0)
    _close(torch.logical_not(xd), torch.logical_not(x), 0)                  # non-boolean input: x != 0 is true
    _close(torch.logical_and(xd, bd), torch.logical_and(x, b), 0)
    _close(torch.logical_or(ad, bd[:1]), torch.logical_or(a, b[:1]), 0)     # broadcast
    _close(ad.clone().logical_and_(bd), a.clone().logical_and_(b), 0)
    _close(xd * ad, x * a, 0)                                                # a mask times a tensor


def test_integer_comparisons_are_exact(vk):
    big = 2 ** 40
    a = torch.tensor([[0, 1, big, big + 1, -big, -5], [7, 7, 7, -7, big + 1, big]], dtype=torch.int64)
    b = torch.tensor([[0, 2, big + 1, big + 1, -big - 1, -5], [7, 8, 6, 7, big, big]], dtype=torch.int64)
    ad, bd = a.to(vk), b.to(vk)
    for fn in (torch.eq, torch.ne, torch.lt, torch.le, torch.gt, torch.ge):
        _close(fn(ad, bd), fn(a, b), 0)
        _close(fn(ad, 7), fn(a, 7), 0)
        _close(fn(ad.int(), bd.int()), fn(a.int(), b.int()), 0)
    m = torch.tensor([True, False, True])
    _close(m.to(vk) == torch.tensor([True, True, False]).to(vk), m == torch.tensor([True, True, False]), 0)
    # label smoothing compares the class indices with ignore_index
    logits, tgt = torch.randn(9, 5), torch.tensor([0, 4, 2, 1, 3, 3, 0, 2, 4])
    _close(F.cross_entropy(logits.to(vk), tgt.to(vk), label_smoothing=0.1), F.cross_entropy(logits, tgt, label_smoothing=0.1), 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_reductions_surface(vk, dtype):
    g = torch.Generator().manual_seed(7)
    x = torch.randn(6, 17, 11, generator=g).to(dtype)
    xd = x.to(vk)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    _close(xd.max(), x.max(), 0)
    _close(xd.min(), x.min(), 0)
    for dim, keep in ((1, False), (2, True), (0, False), (-1, False)):
        for fn in (torch.max, torch.min):
            (vd, idd), (vc, idc) = fn(xd, dim, keep), fn(x, dim, keep)
            _close(vd, vc, 0)
            _close(idd, idc, 0)
    _close(xd.var(), x.float().var().to(dtype), tol)
    _close(xd.std(), x.float().std().to(dtype), tol)
    _close(xd.var(1), x.float().var(1).to(dtype), tol)
    _close(xd.std(dim=(0, 2), keepdim=True), x.float().std(dim=(0, 2), keepdim=True).to(dtype), tol)
    _close(xd.var(2, unbiased=False), x.float().var(2, unbiased=False).to(dtype), tol)
    vm_d, vm_c = torch.var_mean(xd, 1), torch.var_mean(x.float(), 1)
    _close(vm_d[0], vm_c[0].to(dtype), tol)
    _close(vm_d[1], vm_c[1].to(dtype), tol)
    _close(xd.norm(), x.float().norm().to(dtype), tol)
    _close(xd.norm(dim=1), x.float().norm(dim=1).to(dtype), tol)
    _close(torch.linalg.vector_norm(xd, 1, dim=(0, 1)), torch.linalg.vector_norm(x.float(), 1, dim=(0, 1)).to(dtype), tol)
    _close(torch.linalg.vector_norm(xd, float("inf")), torch.linalg.vector_norm(x.float(), float("inf")).to(dtype), tol)
    _close(torch.linalg.vector_norm(xd, 3, dim=2, keepdim=True), torch.linalg.vector_norm(x.float(), 3, dim=2, keepdim=True).to(dtype), tol)
    _close(F.normalize(xd, dim=1), F.normalize(x.float(), dim=1).to(dtype), tol)
    _close(xd.logsumexp(1), x.float().logsumexp(1).to(dtype), tol)


def test_integer_and_boolean_sums_are_exact(vk):
    g = torch.Generator().manual_seed(11)
    a = torch.randint(-2 ** 40, 2 ** 40, (5, 7, 9), generator=g)
    ad = a.to(vk)
    _close(ad.sum(), a.sum(), 0)
    _close(ad.sum(1), a.sum(1), 0)
    _close(ad.sum((0, 2), keepdim=True), a.sum((0, 2), keepdim=True), 0)
    m = torch.rand(300, 70001, generator=g) > 0.5                             # a count above 2^24: not representable step by step in fp32
    _close(m.to(vk).sum(), m.sum(), 0)
    _close(m[:3].to(vk).sum(1), m[:3].sum(1), 0)
    _close(a.int().to(vk).sum(0), a.int().sum(0), 0)


def test_all_any(vk):
    g = torch.Generator().manual_seed(8)
    m = torch.rand(5, 7, 3, generator=g) > 0.2
    m[2] = True
    m[3] = False
    md = m.to(vk)
    _close(md.all(), m.all(), 0); _close(md.any(), m.any(), 0)
    _close(md[2].all(), m[2].all(), 0); _close(md[3].any(), m[3].any(), 0)
    for dim, keep in ((0, False), (1, True), (2, False)):
        _close(md.all(dim, keep), m.all(dim, keep), 0)
        _close(md.any(dim, keep), m.any(dim, keep), 0)
    x = torch.randn(4, 6, generator=g)
    x[1] = 0
    _close(x.to(vk).any(1), x.any(1), 0)
    _close(x.to(vk).all(), x.all(), 0)
    e = torch.empty(0, 3)
    _close(e.to(vk).all(), e.all(), 0); _close(e.to(vk).any(), e.any(), 0)
    assert torch.allclose(x.to(vk), x.to(vk)) and torch.isfinite(x.to(vk)).all().item()


def test_masked_fill_tril_triu_and_ranges(vk):
    g = torch.Generator().manual_seed(9)
    x = torch.randn(3, 6, 8, generator=g)
    m = torch.rand(6, 8, generator=g) > 0.5
    xd, md = x.to(vk), m.to(vk)
    _close(xd.masked_fill(md, -1.5), x.masked_fill(m, -1.5), 0)
    _close(xd.masked_fill(md, torch.tensor(2.0)), x.masked_fill(m, torch.tensor(2.0)), 0)
    _close(xd.clone().masked_fill_(md, float("-inf")), x.clone().masked_fill_(m, float("-inf")), 0)
    for k in (0, 1, -2):
        _close(xd.tril(k), x.tril(k), 0)
        _close(xd.triu(k), x.triu(k), 0)
    _close(torch.arange(7, device=vk), torch.arange(7), 0)
    _close(torch.arange(2, 11, 3, device=vk), torch.arange(2, 11, 3), 0)
    _close(torch.arange(0, 1, 0.125, device=vk), torch.arange(0, 1, 0.125), 0)
    _close(torch.linspace(-1, 1, 9, device=vk), torch.linspace(-1, 1, 9), 1e-6)
    _close(torch.eye(4, device=vk), torch.eye(4), 0)
    _close(torch.eye(3, 5, device=vk), torch.eye(3, 5), 0)
    # a causal mask built the way scripts do it
    L = 6
    causal_d = torch.ones(L, L, device=vk).tril().bool()
    s = torch.randn(2, L, L, generator=g)
    _close(s.to(vk).masked_fill(~causal_d, float("-inf")).softmax(-1), s.masked_fill(~torch.ones(L, L).tril().bool(), float("-inf")).softmax(-1), 1e-6)


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_mse_and_bce_losses(vk, reduction):
    g = torch.Generator().manual_seed(10)
    x, t = torch.randn(12, 9, generator=g), torch.randn(12, 9, generator=g)
    xd, xc = x.to(vk).requires_grad_(), x.clone().requires_grad_()
    ld, lc = F.mse_loss(xd, t.to(vk), reduction=reduction), F.mse_loss(xc, t, reduction=reduction)
    _close(ld, lc, 1e-5)
    gy = torch.randn(lc.shape, generator=g)
    ld.backward(gy.to(vk)); lc.backward(gy)
    _close(xd.grad, xc.grad, 1e-5)
    y = (t > 0).float()
    xd2, xc2 = x.to(vk).requires_grad_(), x.clone().requires_grad_()
    bd, bc = F.binary_cross_entropy_with_logits(xd2, y.to(vk), reduction=reduction), F.binary_cross_entropy_with_logits(xc2, y, reduction=reduction)
    _close(bd, bc, 1e-5)
    bd.backward(gy.to(vk)); bc.backward(gy)
    _close(xd2.grad, xc2.grad, 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_gather_family_with_gradients(vk, dtype):
    """index_select, gather, x[idx] and their adjoints (index_add, scatter_add, accumulate-put) on the row-gather kernel and
    its deterministic backward; flip, roll, one_hot, prod, equal."""
    g = torch.Generator().manual_seed(12)
    x = torch.randn(7, 9, 5, generator=g).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2

    def both(fn, *idx):
        xd, xc = x.to(vk).requires_grad_(), x.double().requires_grad_()
        yd, yc = fn(xd, *[i.to(vk) for i in idx]), fn(xc, *idx)
        _close(yd.double(), yc, tol)
        gy = torch.randn(yc.shape, generator=g).to(dtype)
        yd.backward(gy.to(vk)); yc.backward(gy.double())
        _close(xd.grad.double(), xc.grad, tol)

    i1 = torch.tensor([3, 0, 3, 6, 1])
    for dim in (0, 1, 2, -1):
        both(lambda t, i, dim=dim: t.index_select(dim, i), i1 % x.size(dim))
    both(lambda t, i: t[i], i1)                                              # rows by an index vector (repeats add up in the gradient)
    both(lambda t, i: t[i], torch.tensor([[0, 2], [6, -1]]))                 # an index matrix, a negative index
    both(lambda t, i: t[:, i], torch.tensor([8, 8, 1]))
    both(lambda t, i: t[..., i], torch.tensor([4, 0]))
    for dim in (0, 1, 2):
        idx = torch.randint(0, x.size(dim), (7, 9, 5), generator=g)
        both(lambda t, i, dim=dim: t.gather(dim, i), idx)
    both(lambda t, i: t.gather(1, i), torch.randint(0, 9, (4, 3, 5), generator=g))      # an index smaller than the input
    both(lambda t, i: t.log_softmax(-1).gather(-1, i), torch.randint(0, 5, (7, 9, 1), generator=g))   # picking token log-probabilities
    both(lambda t: t.flip(0))
    both(lambda t: t.flip((1, 2)))
    both(lambda t: t.roll(2, 1))
    both(lambda t: t.roll((-1, 3), (0, 2)))
    both(lambda t: t.roll(4))
    xd = x.to(vk)
    _close(torch.zeros(7, 9, 5, dtype=dtype).to(vk).scatter_add(1, torch.zeros(7, 2, 5, dtype=torch.long).to(vk), xd[:, :2]),
           torch.zeros(7, 9, 5, dtype=dtype).scatter_add(1, torch.zeros(7, 2, 5, dtype=torch.long), x[:, :2]), tol)
    _close(xd.index_add(1, torch.tensor([0, 0, 4]).to(vk), xd[:, :3], alpha=0.5), x.index_add(1, torch.tensor([0, 0, 4]), x[:, :3], alpha=0.5), tol)
    labels = torch.tensor([[1, 3, 0], [2, 2, 4]])
    _close(F.one_hot(labels.to(vk), 5), F.one_hot(labels, 5), 0)
    _close(xd.scatter(2, torch.randint(0, 5, (7, 9, 2), generator=torch.Generator().manual_seed(1)).to(vk), -2.0),
           x.scatter(2, torch.randint(0, 5, (7, 9, 2), generator=torch.Generator().manual_seed(1)), -2.0), 0)
    small = (torch.rand(4, 6, generator=g) + 0.5).to(dtype)
    _close(small.to(vk).prod(), small.float().prod().to(dtype), tol)
    _close(small.to(vk).prod(1), small.float().prod(1).to(dtype), tol)
    _close(small.to(vk).prod(0, keepdim=True), small.float().prod(0, keepdim=True).to(dtype), tol)
    assert torch.equal(xd, xd.clone()) and not torch.equal(xd, xd + 1) and not torch.equal(xd, xd[:3])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("kw", [
    dict(kernel_size=2), dict(kernel_size=3, stride=2, padding=1), dict(kernel_size=(3, 2), stride=(2, 1), padding=(1, 0)),
    dict(kernel_size=3, stride=2, padding=1, ceil_mode=True), dict(kernel_size=3, stride=1, padding=1, dilation=2),
])
def test_max_pool2d(vk, dtype, kw):
    """max_pool2d with indices and its gradient against ATen CPU: same values, same argmax positions (first maximum in
    row-major order), the gradient routed to exactly those positions."""
    g = torch.Generator().manual_seed(13)
    x = torch.randn(3, 5, 13, 11, generator=g).to(dtype)
    xd, xc = x.to(vk).requires_grad_(), x.float().requires_grad_()
    (yd, idd), (yc, idc) = F.max_pool2d(xd, return_indices=True, **kw), F.max_pool2d(xc, return_indices=True, **kw)
    _close(yd.float(), yc, 0)
    _close(idd, idc, 0)
    gy = torch.randn(yc.shape, generator=g).to(dtype)
    yd.backward(gy.to(vk)); yc.backward(gy.float())
    _close(xd.grad.float(), xc.grad, 1e-6 if dtype == torch.float32 else 2e-3)
    # 3-D input, and a channels-last input
    _close(F.max_pool2d(x[0].to(vk), **kw).float(), F.max_pool2d(x[0].float(), **kw), 0)
    _close(F.max_pool2d(x.to(vk).contiguous(memory_format=torch.channels_last), **kw).float(), F.max_pool2d(x.float(), **kw), 0)
    xn = x.clone(); xn[0, 0, 4, 4] = float("nan")
    _close(F.max_pool2d(xn.to(vk), **kw).float(), F.max_pool2d(xn.float(), **kw), 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("kw", [
    dict(kernel_size=2), dict(kernel_size=3, stride=2, padding=1), dict(kernel_size=3, stride=2, padding=1, count_include_pad=False),
    dict(kernel_size=(3, 2), stride=(2, 1), padding=(1, 1), ceil_mode=True), dict(kernel_size=3, stride=2, padding=1, ceil_mode=True, count_include_pad=False),
    dict(kernel_size=2, divisor_override=3),
])
def test_avg_pool2d(vk, dtype, kw):
    g = torch.Generator().manual_seed(14)
    x = torch.randn(2, 6, 12, 9, generator=g).to(dtype)
    xd, xc = x.to(vk).requires_grad_(), x.double().requires_grad_()
    yd, yc = F.avg_pool2d(xd, **kw), F.avg_pool2d(xc, **kw)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    _close(yd.double(), yc, tol)
    gy = torch.randn(yc.shape, generator=g).to(dtype)
    yd.backward(gy.to(vk)); yc.backward(gy.double())
    _close(xd.grad.double(), xc.grad, tol)


def test_random_fills_and_dropout(vk):
    """uniform / normal / Bernoulli fills and dropout (src/api/ops/random.cpp, dropout.cpp): the distributions' moments
    within a few standard errors, reproducible under a seed, advancing between calls; dropout's mask, scale and gradient."""
    import torchvulkan

    n = 1 << 20
    torchvulkan.manual_seed(1234)
    u = torch.rand(n, device=vk).cpu()
    assert 0.0 <= float(u.min()) and float(u.max()) < 1.0
    assert abs(float(u.mean()) - 0.5) < 2e-3 and abs(float(u.var()) - 1 / 12) < 2e-3
    z = torch.randn(n, device=vk).cpu()
    assert abs(float(z.mean())) < 5e-3 and abs(float(z.std()) - 1.0) < 5e-3
    assert abs(float((z.abs() < 1.0).float().mean()) - 0.6827) < 3e-3 and float(z.abs().max()) > 4.0
    assert abs(float(torch.corrcoef(torch.stack([z[:-1], z[1:]]))[0, 1])) < 5e-3
    w = torch.empty(300, 700, device=vk).uniform_(-2.0, 3.0).cpu()
    assert -2.0 <= float(w.min()) and float(w.max()) < 3.0 and abs(float(w.mean()) - 0.5) < 2e-2
    nrm = torch.empty(n, device=vk).normal_(3.0, 0.5).cpu()
    assert abs(float(nrm.mean()) - 3.0) < 3e-3 and abs(float(nrm.std()) - 0.5) < 3e-3
    h = torch.randn(n, device=vk, dtype=torch.float16).cpu().float()
    assert abs(float(h.mean())) < 5e-3 and abs(float(h.std()) - 1.0) < 5e-3
    b = torch.empty(n, device=vk).bernoulli_(0.3).cpu()
    assert set(b.unique().tolist()) == {0.0, 1.0} and abs(float(b.mean()) - 0.3) < 2e-3
    # the same seed replays the stream; the stream advances between calls; an odd length is filled to its end
    torchvulkan.manual_seed(7)
    a1, a2 = torch.randn(1001, device=vk).cpu(), torch.randn(1001, device=vk).cpu()
    torchvulkan.manual_seed(7)
    b1 = torch.randn(1001, device=vk).cpu()
    assert torch.equal(a1, b1) and not torch.equal(a1, a2) and bool(a1.isfinite().all())
    torch.manual_seed(7)                                                    # torch.manual_seed seeds every device's generator
    assert torch.equal(torch.randn(1001, device=vk).cpu(), a1)
    # nn.init and a strided target
    lin = torch.nn.Linear(64, 32).to(vk)
    torch.nn.init.kaiming_uniform_(lin.weight); torch.nn.init.normal_(lin.bias, std=0.02)
    assert float(lin.weight.detach().cpu().abs().max()) > 0 and abs(float(lin.bias.detach().cpu().std()) - 0.02) < 0.01
    t = torch.zeros(64, 64, device=vk)
    t.t()[:, :3].normal_()
    assert float(t.cpu()[:3].abs().sum()) > 0 and float(t.cpu()[3:].abs().sum()) == 0
    # dropout
    x = torch.randn(512, 1024)
    xd = x.to(vk).requires_grad_()
    y = F.dropout(xd, 0.25, training=True)
    yc = y.detach().cpu()
    kept = yc != 0
    assert abs(float(kept.float().mean()) - 0.75) < 3e-3
    assert torch.allclose(yc[kept], x[kept] / 0.75, rtol=1e-6, atol=1e-7)
    y.backward(torch.ones_like(y))
    assert torch.allclose(xd.grad.cpu(), kept.float() / 0.75, rtol=1e-6, atol=0)
    assert torch.equal(F.dropout(xd, 0.25, training=False).detach().cpu(), x)
    drop = torch.nn.Dropout(0.5)
    yh = drop(x.half().to(vk)).cpu()
    assert abs(float((yh != 0).float().mean()) - 0.5) < 3e-3 and torch.equal(yh[yh != 0], (x.half() * 2)[yh != 0])
    assert float(F.dropout(xd, 1.0, training=True).detach().abs().sum().cpu()) == 0.0


def test_random_launches_inside_a_graph_draw_new_numbers_on_every_replay(vk):
    """Dropout and random fills recorded into torchvulkan.Graph read the generator state from device memory that every
    launch of the graph refreshes: replays differ from each other, advance the generator, and repeat under the same seed."""
    import torchvulkan

    x = torch.ones(256, 512, device=vk)
    y, noise = torch.empty_like(x), torch.empty(1000, device=vk)

    def work():
        y.copy_(F.dropout(x, 0.5, training=True))
        noise.normal_()

    for _ in range(2):
        work()
    g = torchvulkan.Graph()
    with g.capture():
        work()

    def replays(seed, n=3):
        torchvulkan.manual_seed(seed)
        out = []
        for _ in range(n):
            g.replay()
            out.append((y.cpu().clone(), noise.cpu().clone()))
        return out

    a, b, c = replays(5), replays(5), replays(6)
    for i in range(3):
        assert torch.equal(a[i][0], b[i][0]) and torch.equal(a[i][1], b[i][1])           # the same seed replays the same sequence
        assert not torch.equal(a[i][0], c[i][0])
        assert abs(float((a[i][0] != 0).float().mean()) - 0.5) < 0.01 and abs(float(a[i][1].std()) - 1.0) < 0.1
    assert not torch.equal(a[0][0], a[1][0]) and not torch.equal(a[1][0], a[2][0]) and not torch.equal(a[0][1], a[1][1])
    # an eager launch after the replays continues the stream instead of repeating a replay's numbers
    torchvulkan.manual_seed(5)
    g.replay()
    eager = torch.empty(1000, device=vk).normal_().cpu()
    assert not torch.equal(eager, a[0][1]) and not torch.equal(eager, a[1][1])
    g.reset()


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_smooth_l1_huber_and_kl_div(vk, reduction):
    g = torch.Generator().manual_seed(15)
    x, t = torch.randn(14, 11, generator=g) * 2, torch.randn(14, 11, generator=g)
    for fn in (lambda a, b: F.smooth_l1_loss(a, b, reduction=reduction, beta=0.7), lambda a, b: F.smooth_l1_loss(a, b, reduction=reduction, beta=0.0),
               lambda a, b: F.huber_loss(a, b, reduction=reduction, delta=1.3)):
        xd, xc = x.to(vk).requires_grad_(), x.clone().requires_grad_()
        ld, lc = fn(xd, t.to(vk)), fn(xc, t)
        _close(ld, lc, 1e-5)
        gy = torch.randn(lc.shape, generator=g)
        ld.backward(gy.to(vk)); lc.backward(gy)
        _close(xd.grad, xc.grad, 1e-5)
    if reduction != "none":
        kr = "batchmean" if reduction == "mean" else reduction
        p, q = x.log_softmax(1), t.softmax(1)
        q[0, :3] = 0
        _close(F.kl_div(p.to(vk), q.to(vk), reduction=kr), F.kl_div(p, q, reduction=kr), 1e-5)
    a = torch.tensor([0.0, 0.0, 2.0, 1.5, 0.0]); b = torch.tensor([0.0, float("nan"), 3.0, 0.0, 5.0])
    _close(torch.xlogy(a.to(vk), b.to(vk)), torch.xlogy(a, b), 1e-6)


def test_masked_select_and_printing_a_device_tensor(vk):
    g = torch.Generator().manual_seed(16)
    x = torch.randn(7, 9, generator=g)
    m = torch.rand(7, 9, generator=g) > 0.6
    _close(x.to(vk).masked_select(m.to(vk)), x.masked_select(m), 0)
    _close(x.to(vk).masked_select(m[:1].to(vk)), x.masked_select(m[:1]), 0)            # a broadcast mask
    assert x.to(vk).masked_select(torch.zeros(7, 9, dtype=torch.bool).to(vk)).numel() == 0
    # repr of floating, half, integer, boolean and gradient-carrying tensors (the formatter runs its statistics on the device)
    for t in (x, x.half(), (x * 1e4), torch.arange(6), m, torch.tensor(3.5), torch.tensor([float("nan"), float("inf"), 1.0])):
        s = repr(t.to(vk))
        assert "vulkan" in s and s.startswith("tensor(")
    xr = x.to(vk).requires_grad_()
    assert "requires_grad=True" in repr(xr) and "grad_fn" in repr((xr * 2).sum())
    squeeze = lambda t: "".join(repr(t).split()).replace(",device='vulkan:0'", "")   # noqa: E731  (the suffix may wrap onto its own line)
    assert squeeze(x.to(vk)) == squeeze(x)


def test_multinomial(vk):
    """torch.multinomial on the device (the sampling step of the reference's language-model example,
    examples/llm.py:95-99): frequencies follow the probabilities, zero-probability classes are never drawn, sampling
    without replacement returns distinct classes, the seed reproduces the draw."""
    import torchvulkan

    torchvulkan.manual_seed(3)
    p = torch.tensor([[0.0, 0.1, 0.2, 0.0, 0.7, 0.0], [0.5, 0.0, 0.0, 0.5, 0.0, 0.0]])
    draws = torch.multinomial(p.to(vk), 20000, replacement=True).cpu()
    assert draws.shape == (2, 20000) and draws.dtype == torch.long
    for r in range(2):
        freq = torch.bincount(draws[r], minlength=6).float() / 20000
        assert float((freq - p[r]).abs().max()) < 0.015 and float(freq[p[r] == 0].sum()) == 0.0
    one = torch.stack([torch.multinomial(p.to(vk), 1).cpu() for _ in range(200)])
    assert one.shape == (200, 2, 1) and set(one[:, 1, 0].tolist()) <= {0, 3} and set(one[:, 0, 0].tolist()) <= {1, 2, 4}
    logits = torch.randn(4, 50)
    nr = torch.multinomial(logits.softmax(-1).to(vk), 10, replacement=False).cpu()
    assert nr.shape == (4, 10) and all(len(set(row.tolist())) == 10 for row in nr)
    assert torch.multinomial(p[0].to(vk), 3, replacement=True).shape == (3,)
    torchvulkan.manual_seed(11)
    a = torch.multinomial(logits.softmax(-1).half().to(vk), 5, replacement=True).cpu()
    torchvulkan.manual_seed(11)
    assert torch.equal(a, torch.multinomial(logits.softmax(-1).half().to(vk), 5, replacement=True).cpu())


def test_boolean_mask_indexing(vk):
    g = torch.Generator().manual_seed(18)
    x = torch.randn(6, 5, 4, generator=g)
    full, rows = torch.rand(6, 5, 4, generator=g) > 0.5, torch.tensor([True, False, True, True, False, False])
    mid = torch.rand(6, 5, generator=g) > 0.5
    for make in (lambda t, m: t[m], ):
        for m in (full, rows, mid):
            xd, xc = x.to(vk).requires_grad_(), x.clone().requires_grad_()
            yd, yc = make(xd, m.to(vk)), make(xc, m)
            _close(yd, yc, 0)
            gy = torch.randn(yc.shape, generator=g)
            yd.backward(gy.to(vk)); yc.backward(gy)
            _close(xd.grad, xc.grad, 0)
    _close(x.to(vk)[:, mid[0]], x[:, mid[0]], 0)                              # a mask on the second dimension
    a, b = x.to(vk).clone(), x.clone()
    a[a < 0] = 0.0; b[b < 0] = 0.0                                           # the usual in-place clean-up
    _close(a, b, 0)
    a[rows.to(vk)] = -1.0; b[rows] = -1.0
    _close(a, b, 0)
    assert x.to(vk)[torch.zeros(6, dtype=torch.bool).to(vk)].shape == (0, 5, 4)


def test_integer_arithmetic_is_exact(vk):
    big = 2 ** 40 + 3
    a = torch.tensor([[7, -7, big, -big, 0, 5], [1, 2, 3, -4, -5, 6]], dtype=torch.int64)
    b = torch.tensor([[2, 2, 3, 3, 5, -3], [1, -2, 7, 3, -2, 4]], dtype=torch.int64)
    ad, bd = a.to(vk), b.to(vk)
    for fn in (torch.floor_divide, torch.remainder, torch.fmod, torch.maximum, torch.minimum, torch.add, torch.sub, torch.mul):
        _close(fn(ad, bd), fn(a, b), 0)
        _close(fn(ad.int()[1:], bd.int()[1:]), fn(a.int()[1:], b.int()[1:]), 0)
    _close(ad // 3, a // 3, 0); _close(ad % 3, a % 3, 0); _close(ad % -3, a % -3, 0)
    _close(-ad, -a, 0); _close(ad.abs(), a.abs(), 0); _close(ad.clamp(-5, 5), a.clamp(-5, 5), 0); _close(ad.clamp(min=0), a.clamp(min=0), 0)
    _close(ad.clamp(min=bd), a.clamp(min=b), 0)
    emb = torch.nn.Embedding(10, 4, padding_idx=0)
    ids = torch.arange(24).reshape(4, 6)
    _close(emb.to(vk)(ids.to(vk) % 10), emb.cpu()(ids % 10), 0)
    x = torch.randn(5, 6)
    _close(x.to(vk).clamp(min=torch.zeros(6).to(vk), max=torch.ones(6).to(vk)), x.clamp(min=torch.zeros(6), max=torch.ones(6)), 0)
    _close(torch.lerp(x.to(vk), torch.ones(5, 6).to(vk), torch.rand(5, 6, generator=torch.Generator().manual_seed(1)).to(vk)),
           torch.lerp(x, torch.ones(5, 6), torch.rand(5, 6, generator=torch.Generator().manual_seed(1))), 1e-6)
    _close(F.threshold(x.to(vk), 0.1, -2.0), F.threshold(x, 0.1, -2.0), 0)
    _close(F.hardshrink(x.to(vk), 0.5), F.hardshrink(x, 0.5), 0)
    _close(F.cosine_similarity(x.to(vk), x.flip(0).to(vk)), F.cosine_similarity(x, x.flip(0)), 1e-6)


def test_autocast_and_gradient_scaler(vk):
    """torch.autocast("vulkan") with torch.amp.GradScaler, the mixed-precision recipe (reference: the AutocastPrivateUse1
    registration, src/api/registration.cpp:4-21, and the two scaler operators, src/api/decompositions.cpp:1625-1626): linear
    layers run in fp16 under autocast, the loss in fp32, the step matches the same recipe on ATen CPU in bf16/fp32 loosely and,
    exactly, the scaler's own rules: unscale, skip on overflow, back off, grow after the interval."""
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.GELU(), torch.nn.Linear(64, 10)).to(vk)
    ref = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.GELU(), torch.nn.Linear(64, 10))
    ref.load_state_dict({k: v.cpu() for k, v in model.state_dict().items()})
    x, y = torch.randn(16, 32), torch.randint(0, 10, (16,))
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    scaler = torch.amp.GradScaler("vulkan", init_scale=1024.0, growth_interval=2)
    with torch.autocast("vulkan", dtype=torch.float16):
        h = model[0](x.to(vk))
        assert h.dtype == torch.float16                                        # the matmul family runs in the lower precision
        logits = model(x.to(vk))
        loss = F.cross_entropy(logits, y.to(vk))
        assert loss.dtype == torch.float32                                     # the loss family runs in fp32
    loss_ref = F.cross_entropy(ref(x), y)
    assert abs(loss.item() - loss_ref.item()) < 5e-3
    opt.zero_grad()
    scaler.scale(loss).backward()
    assert float(model[0].weight.grad.abs().max().cpu()) > 1.0                 # gradients carry the scale
    scaler.unscale_(opt)
    loss_ref.backward()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert rel_fro_t(p.grad.cpu(), q.grad) < 2e-2
    before = [p.detach().cpu().clone() for p in model.parameters()]
    scaler.step(opt); scaler.update()
    assert any(not torch.equal(b, p.detach().cpu()) for b, p in zip(before, model.parameters())) and scaler.get_scale() == 1024.0
    # second clean step reaches the growth interval: the scale doubles
    opt.zero_grad()
    with torch.autocast("vulkan", dtype=torch.float16):
        loss = F.cross_entropy(model(x.to(vk)), y.to(vk))
    scaler.scale(loss).backward(); scaler.step(opt); scaler.update()
    assert scaler.get_scale() == 2048.0
    # an overflow: the step is skipped and the scale backs off
    opt.zero_grad()
    with torch.autocast("vulkan", dtype=torch.float16):
        loss = F.cross_entropy(model(x.to(vk)), y.to(vk))
    scaler.scale(loss).backward()
    model[0].weight.grad[0, 0] = float("inf")
    before = [p.detach().cpu().clone() for p in model.parameters()]
    scaler.step(opt); scaler.update()
    assert all(torch.equal(b, p.detach().cpu()) for b, p in zip(before, model.parameters())) and scaler.get_scale() == 1024.0
    # bf16 autocast, and ops outside the context are untouched
    with torch.autocast("vulkan", dtype=torch.bfloat16):
        assert model(x.to(vk)).dtype == torch.bfloat16
    assert model(x.to(vk)).dtype == torch.float32


def rel_fro_t(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_upsampling_adaptive_pools_bce_and_norms(vk, dtype):
    g = torch.Generator().manual_seed(19)
    x = torch.randn(2, 3, 6, 8, generator=g).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2

    def both(fn):
        xd, xc = x.to(vk).requires_grad_(), x.double().requires_grad_()
        yd, yc = fn(xd), fn(xc)
        _close(yd.double(), yc, tol)
        gy = torch.randn(yc.shape, generator=g).to(dtype)
        yd.backward(gy.to(vk)); yc.backward(gy.double())
        _close(xd.grad.double(), xc.grad, tol)

    both(lambda t: F.interpolate(t, scale_factor=2))
    both(lambda t: F.interpolate(t, size=(9, 13)))
    both(lambda t: F.interpolate(t, scale_factor=2, mode="bilinear"))
    both(lambda t: F.interpolate(t, size=(11, 5), mode="bilinear", align_corners=True))
    both(lambda t: F.interpolate(t, scale_factor=(1.5, 2.5), mode="bilinear", recompute_scale_factor=False))
    both(lambda t: F.adaptive_avg_pool2d(t, (3, 2)))
    both(lambda t: F.adaptive_max_pool2d(t, (2, 4)))
    both(lambda t: F.pixel_shuffle(t.repeat(1, 4, 1, 1)[:, :4], 2))
    both(lambda t: F.adaptive_avg_pool2d(t, (4, 3)))                 # windows of unequal size
    both(lambda t: F.adaptive_avg_pool2d(t, (5, 7)))
    both(lambda t: F.adaptive_max_pool2d(t, (4, 3)))
    both(lambda t: F.adaptive_max_pool2d(t[0], (5, 5)))
    idx_d = F.adaptive_max_pool2d(x.to(vk), (4, 5), return_indices=True)[1].cpu()
    assert torch.equal(idx_d, F.adaptive_max_pool2d(x.float(), (4, 5), return_indices=True)[1])
    p, t = torch.rand(7, 5, generator=g).clamp(0.02, 0.98), (torch.rand(7, 5, generator=g) > 0.5).float()
    pd, pc = p.to(vk).requires_grad_(), p.clone().requires_grad_()
    ld, lc = F.binary_cross_entropy(pd, t.to(vk)), F.binary_cross_entropy(pc, t)
    _close(ld, lc, 1e-6)
    ld.backward(); lc.backward()
    _close(pd.grad, pc.grad, 1e-5)
    a, b = torch.randn(6, 9, generator=g), torch.randn(6, 9, generator=g)
    _close(F.pairwise_distance(a.to(vk), b.to(vk)), F.pairwise_distance(a, b), 1e-6)
    _close(torch.norm(a.to(vk), p=3, dim=1), torch.norm(a, p=3, dim=1), 1e-6)
    _close(a.to(vk).norm(1), a.norm(1), 1e-6)
    _close(F.triplet_margin_loss(a.to(vk), b.to(vk), b.flip(0).to(vk)), F.triplet_margin_loss(a, b, b.flip(0)), 1e-6)


def test_integer_random_fills_and_permutations(vk):
    import torchvulkan

    torchvulkan.manual_seed(21)
    r = torch.randint(3, 11, (20000,), device=vk).cpu()
    assert r.dtype == torch.long and int(r.min()) == 3 and int(r.max()) == 10
    freq = torch.bincount(r - 3, minlength=8).float() / 20000
    assert float((freq - 0.125).abs().max()) < 0.01
    assert torch.randint(5, (4, 3), device=vk).shape == (4, 3)
    perm = torch.randperm(1000, device=vk).cpu()
    assert perm.dtype == torch.long and torch.equal(perm.sort().values, torch.arange(1000)) and not torch.equal(perm, torch.arange(1000))
    torchvulkan.manual_seed(21)
    assert torch.equal(torch.randint(3, 11, (20000,), device=vk).cpu(), r)


def test_nonzero_and_assignment_through_an_index(vk):
    g = torch.Generator().manual_seed(20)
    x = torch.randn(5, 4, 3, generator=g)
    x[x.abs() < 0.6] = 0
    _close(x.to(vk).nonzero(), x.nonzero(), 0)
    _close((x > 0).to(vk).nonzero(), (x > 0).nonzero(), 0)
    for got, want in zip(torch.where(x.to(vk) > 0), torch.where(x > 0)):
        _close(got, want, 0)
    assert torch.zeros(3, 2).to(vk).nonzero().shape == (0, 2)
    a, b = x.to(vk).clone(), x.clone()
    idx = torch.tensor([4, 0, 2])
    v = torch.randn(3, 4, 3, generator=g)
    a[idx.to(vk)] = v.to(vk); b[idx] = v
    _close(a, b, 0)
    cols = torch.tensor([3, 0])
    a[:, cols.to(vk)] = 7.0; b[:, cols] = 7.0
    _close(a, b, 0)
    w = torch.zeros(6, 3)
    wd = w.to(vk)
    wd[torch.tensor([1, 5]).to(vk)] = torch.ones(3).to(vk); w[torch.tensor([1, 5])] = torch.ones(3)
    _close(wd, w, 0)


def test_selections_on_integer_and_boolean_tensors_are_bit_exact(vk):
    g = torch.Generator().manual_seed(22)
    big = torch.randint(-2 ** 62, 2 ** 62, (7, 5, 3), generator=g)
    idx = torch.tensor([6, 0, 0, 3])
    for t in (big, big.int(), big > 0, (big % 200).to(torch.uint8)):
        td = t.to(vk)
        _close(td[idx.to(vk)], t[idx], 0)
        _close(td.index_select(1, idx[:3].to(vk) % 5), t.index_select(1, idx[:3] % 5), 0)
        _close(td[:, torch.tensor([True, False, True, True, False]).to(vk)], t[:, torch.tensor([True, False, True, True, False])], 0)
        _close(td.flip(0), t.flip(0), 0)
        _close(td.gather(2, torch.zeros(7, 5, 2, dtype=torch.long).to(vk)), t.gather(2, torch.zeros(7, 5, 2, dtype=torch.long)), 0)
    labels = torch.randint(0, 10, (64,), generator=g)
    perm = torch.randperm(64, generator=g)
    _close(labels.to(vk)[perm.to(vk)], labels[perm], 0)                      # shuffling a label vector
    _close(labels.to(vk).masked_select((labels > 4).to(vk)), labels.masked_select(labels > 4), 0)


def test_kthvalue_and_median(vk):
    g = torch.Generator().manual_seed(23)
    x = torch.randn(6, 9, generator=g)
    for k, dim, keep in ((1, 1, False), (4, 1, True), (6, 0, False)):
        (vd, idd), (vc, idc) = x.to(vk).kthvalue(k, dim, keep), x.kthvalue(k, dim, keep)
        _close(vd, vc, 0); _close(idd, idc, 0)
    (vd, idd), (vc, idc) = x.to(vk).median(1), x.median(1)
    _close(vd, vc, 0); _close(idd, idc, 0)
    _close(x.to(vk).median(), x.median(), 0)
    _close(x[:, :8].to(vk).median(1).values, x[:, :8].median(1).values, 0)     # even count: the lower middle value


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_dropout_packet_and_scalar_kernels_draw_the_same_mask(vk, dtype):
    """The dropout stream is a function of (seed, offset, element index) alone: an aligned tensor (eight elements per thread)
    and the same values at an odd address (one block of four per thread) are dropped at the same positions."""
    import torchvulkan

    n = 8 * 1000 + 5
    data = torch.randn(n + 1).to(dtype)
    aligned, shifted = data[1:].clone().to(vk), data.to(vk)[1:]
    torchvulkan.manual_seed(9)
    ya = F.dropout(aligned, 0.3, training=True).cpu()
    torchvulkan.manual_seed(9)
    ys = F.dropout(shifted, 0.3, training=True).cpu()
    assert torch.equal(ya, ys) and abs(float((ya != 0).float().mean()) - 0.7) < 0.02


def test_new_operators_on_empty_tensors(vk):
    e = torch.empty(0, 5)
    none = torch.empty(0, dtype=torch.long)
    for fn in (lambda t: t.clamp(0, 1), lambda t: F.leaky_relu(t), lambda t: (t > 0) & (t < 1), lambda t: t.sum(0), lambda t: (t > 0).all(1), lambda t: t.masked_fill(t > 0, 1.0),
               lambda t: t.index_select(0, none.to(t.device)), lambda t: t[none.to(t.device)], lambda t: t[t[:, 0] > 0], lambda t: t.masked_select(t > 0), lambda t: t.nonzero(),
               lambda t: t.flip(0), lambda t: F.dropout(t, 0.5, training=True), lambda t: t.clone().normal_(), lambda t: t.prod(0), lambda t: t @ t.t()):
        got, want = fn(e.to(vk)), fn(e)
        assert got.shape == want.shape and got.dtype == want.dtype
    assert float(e.to(vk).sum().cpu()) == 0.0 and int((e.to(vk) > 0).sum().cpu()) == 0 and not bool((e.to(vk) > 0).any().cpu())
    assert torch.ones(3, 4).to(vk)[none.to(vk)].shape == (0, 4)


def test_index_fill_and_nan_aware_extrema(vk):
    x = torch.randn(5, 7)
    idx = torch.tensor([6, 0, 0])
    _close(x.to(vk).index_fill(1, idx.to(vk), -3.0), x.index_fill(1, idx, -3.0), 0)
    a = torch.tensor([1.0, float("nan"), 3.0, float("nan")]); b = torch.tensor([2.0, 5.0, float("nan"), float("nan")])
    _close(torch.fmax(a.to(vk), b.to(vk)), torch.fmax(a, b), 0)
    _close(torch.fmin(a.to(vk), b.to(vk)), torch.fmin(a, b), 0)
    _close(torch.logaddexp(torch.tensor([float("-inf"), 1.0]).to(vk), torch.tensor([float("-inf"), float("inf")]).to(vk)),
           torch.logaddexp(torch.tensor([float("-inf"), 1.0]), torch.tensor([float("-inf"), float("inf")])), 0)


def test_upsampling_in_one_and_three_dimensions(vk):
    g = torch.Generator().manual_seed(24)
    x1, x3 = torch.randn(2, 3, 9, generator=g), torch.randn(2, 3, 4, 5, 6, generator=g)

    def both(x, **kw):
        xd, xc = x.to(vk).requires_grad_(), x.double().requires_grad_()
        yd, yc = F.interpolate(xd, **kw), F.interpolate(xc, **kw)
        _close(yd.double(), yc, 1e-5)
        gy = torch.randn(yc.shape, generator=g)
        yd.backward(gy.to(vk)); yc.backward(gy.double())
        _close(xd.grad.double(), xc.grad, 1e-5)

    both(x1, scale_factor=2); both(x1, size=14, mode="nearest-exact"); both(x1, scale_factor=1.5, mode="linear"); both(x1, size=17, mode="linear", align_corners=True)
    both(x3, scale_factor=2); both(x3, size=(7, 9, 8), mode="nearest-exact"); both(x3, scale_factor=(2, 1.5, 2), mode="trilinear"); both(x3, size=(6, 7, 11), mode="trilinear", align_corners=True)
    both(torch.randn(1, 2, 5, 7, generator=g), size=(8, 9), mode="nearest-exact")


def test_running_extremes_unique_and_bincount(vk):
    g = torch.Generator().manual_seed(41)
    x = torch.randint(0, 5, (4, 37, 3), generator=g).float()          # many ties: the later position must win
    for dim in (0, 1, -1):
        for fn in (torch.cummax, torch.cummin):
            d, c = fn(x.to(vk), dim), fn(x, dim)
            assert torch.equal(d.values.cpu(), c.values) and torch.equal(d.indices.cpu(), c.indices), (dim, fn)
    y = torch.randn(3, 50, generator=g)
    y[0, 7] = float("nan"); y[1, 20] = float("nan"); y[1, 30] = float("nan"); y[2, 3] = float("inf")
    for fn in (torch.cummax, torch.cummin):
        d, c = fn(y.to(vk), 1), fn(y, 1)
        assert torch.equal(d.indices.cpu(), c.indices)
        assert torch.allclose(d.values.cpu(), c.values, equal_nan=True)
    li = torch.randint(-1000, 1000, (5, 9), generator=g)
    d, c = torch.cummin(li.to(vk), 1), torch.cummin(li, 1)
    assert torch.equal(d.values.cpu(), c.values) and torch.equal(d.indices.cpu(), c.indices)
    h = torch.randn(6, 20, generator=g).half()
    d, c = torch.cummax(h.to(vk), 1), torch.cummax(h, 1)
    assert torch.equal(d.values.cpu(), c.values) and torch.equal(d.indices.cpu(), c.indices)
    xd, xc = y[2:].to(vk).requires_grad_(), y[2:].clone().requires_grad_()
    torch.cummax(xd, 1).values.sum().backward(); torch.cummax(xc, 1).values.sum().backward()
    _close(xd.grad, xc.grad, 1e-6)

    for t in (torch.randint(-5, 9, (7, 11), generator=g), torch.randn(50, generator=g).round(), torch.tensor([3.0]),
              torch.tensor([2, 2, 2]), torch.zeros(0)):
        d = torch.unique(t.to(vk), return_inverse=True, return_counts=True)
        c = torch.unique(t, return_inverse=True, return_counts=True)
        for a, b in zip(d, c):
            assert a.dtype == b.dtype and torch.equal(a.cpu(), b), t
    assert torch.equal(torch.unique(li.to(vk)).cpu(), torch.unique(li))

    b = torch.randint(0, 13, (500,), generator=g)
    w = torch.rand(500, generator=g)
    assert torch.equal(torch.bincount(b.to(vk)).cpu(), torch.bincount(b))
    assert torch.equal(torch.bincount(b.to(vk), minlength=20).cpu(), torch.bincount(b, minlength=20))
    _close(torch.bincount(b.to(vk), weights=w.to(vk)), torch.bincount(b, weights=w), 1e-5)
    with pytest.raises(RuntimeError, match="non-negative"):
        torch.bincount(torch.tensor([1, -1]).to(vk))


def test_cross_product(vk):
    g = torch.Generator().manual_seed(43)
    a, b = torch.randn(5, 3, 4, generator=g), torch.randn(1, 3, 1, generator=g)
    ad, ac = a.to(vk).requires_grad_(), a.clone().requires_grad_()
    yd, yc = torch.linalg.cross(ad, b.to(vk), dim=1), torch.linalg.cross(ac, b, dim=1)
    _close(yd, yc, 1e-6)
    gy = torch.randn(yc.shape, generator=g)
    yd.backward(gy.to(vk)); yc.backward(gy)
    _close(ad.grad, ac.grad, 1e-6)
    u, v = torch.randn(7, 3, generator=g), torch.randn(7, 3, generator=g)
    _close(torch.cross(u.to(vk), v.to(vk), dim=-1), torch.cross(u, v, dim=-1), 1e-6)


def _pooling_of_volumes(dev):
    g = torch.Generator().manual_seed(47)
    x = torch.randint(0, 4, (2, 3, 9, 10, 11), generator=g).float()          # ties: the first maximum must win
    for k, s, p, d, ceil in (((2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1), False), ((3, 2, 3), (2, 1, 2), (1, 1, 1), (1, 1, 1), True),
                             ((2, 3, 2), (1, 2, 2), (0, 1, 1), (2, 1, 2), False)):
        vd, idd = F.max_pool3d(x.to(dev), k, s, p, d, ceil, return_indices=True)
        vc, idc = F.max_pool3d(x, k, s, p, d, ceil, return_indices=True)
        assert torch.equal(vd.cpu(), vc) and torch.equal(idd.cpu(), idc), (k, s, p, d, ceil)
    y = torch.randn(2, 3, 9, 10, 11, generator=g)
    cases = [lambda t: F.max_pool3d(t, 2), lambda t: F.max_pool3d(t, (3, 2, 3), (2, 1, 2), (1, 1, 1), ceil_mode=True),
             lambda t: F.avg_pool3d(t, 2), lambda t: F.avg_pool3d(t, (3, 2, 3), (2, 1, 2), (1, 1, 1), True, True),
             lambda t: F.avg_pool3d(t, (3, 2, 3), (2, 1, 2), (1, 1, 1), True, False),
             lambda t: F.avg_pool3d(t, (2, 3, 2), (1, 2, 2), (0, 1, 1), False, False, 5),
             lambda t: F.adaptive_avg_pool3d(t, 1), lambda t: F.adaptive_avg_pool3d(t, (3, 5, 11)), lambda t: F.adaptive_avg_pool3d(t[0], (4, 3, 2))]
    for fn in cases:
        yd, yc = y.clone().to(dev).requires_grad_(), y.clone().requires_grad_()
        od, oc = fn(yd), fn(yc)
        _close(od, oc, 1e-5)
        gy = torch.randn(oc.shape, generator=g)
        od.backward(gy.to(dev)); oc.backward(gy)
        _close(yd.grad, yc.grad, 1e-5)


def _assorted_small_operators(dev):
    g = torch.Generator().manual_seed(53)
    a = torch.randn(6, 9, generator=g)
    _close(2.0 ** a.to(dev), 2.0 ** a, 1e-5)
    _close(torch.pow(0.5, a.to(dev)), torch.pow(0.5, a), 1e-5)
    nan = a.clone(); nan[1, 2] = float("nan"); nan[4, 0] = float("nan")
    _close(torch.nansum(nan.to(dev)), torch.nansum(nan), 1e-5)
    _close(torch.nansum(nan.to(dev), dim=1, keepdim=True), torch.nansum(nan, dim=1, keepdim=True), 1e-5)
    pr = torch.rand(6, 9, generator=g).clamp(0.01, 0.99)
    for eps in (None, 0.2):
        pd, pc = pr.clone().to(dev).requires_grad_(), pr.clone().requires_grad_()
        ld, lc = torch.logit(pd, eps), torch.logit(pc, eps)
        _close(ld, lc, 1e-5)
        ld.sum().backward(); lc.sum().backward()
        _close(pd.grad, pc.grad, 1e-5)
    for kw in ({}, {"dim": 1}, {"dim": 0, "keepdim": True}):
        d, c = torch.aminmax(a.to(dev), **kw), torch.aminmax(a, **kw)
        assert torch.equal(d.min.cpu(), c.min) and torch.equal(d.max.cpu(), c.max)
    img = torch.randn(2, 12, 5, 4, generator=g)
    assert torch.equal(F.channel_shuffle(img.to(dev), 3).cpu(), F.channel_shuffle(img, 3))
    ints = torch.randint(0, 20, (7, 5), generator=g)
    cand = torch.tensor([3, 7, 19, 40])
    assert torch.equal(torch.isin(ints.to(dev), cand.to(dev)).cpu(), torch.isin(ints, cand))
    assert torch.equal(torch.isin(ints.to(dev), cand.to(dev), invert=True).cpu(), torch.isin(ints, cand, invert=True))
    assert torch.equal(torch.isin(ints.to(dev), 7).cpu(), torch.isin(ints, 7))
    assert torch.equal(torch.isin(a.to(dev), a[2].to(dev)).cpu(), torch.isin(a, a[2]))
    reps = torch.tensor([2, 0, 3, 1])
    assert torch.equal(torch.repeat_interleave(reps.to(dev)).cpu(), torch.repeat_interleave(reps))
    rows = torch.randn(4, 3, generator=g)
    assert torch.equal(torch.repeat_interleave(rows.to(dev), reps.to(dev), dim=0).cpu(), torch.repeat_interleave(rows, reps, dim=0))
    assert torch.equal(torch.repeat_interleave(rows.to(dev), 2, dim=1).cpu(), torch.repeat_interleave(rows, 2, dim=1))
    pooled, where = F.max_pool2d(img, 2, return_indices=True, ceil_mode=True)
    ud = F.max_unpool2d(pooled.to(dev), where.to(dev), 2, output_size=(5, 4))
    assert torch.equal(ud.cpu(), F.max_unpool2d(pooled, where, 2, output_size=(5, 4)))
    index = torch.stack([torch.randperm(9, generator=g)[:4] for _ in range(6)])           # unique along the scattered dimension
    src = torch.randn(6, 7, generator=g)
    assert torch.equal(a.to(dev).scatter(1, index.to(dev), src.to(dev)).cpu(), a.scatter(1, index, src))
    col = torch.stack([torch.randperm(6, generator=g)[:3] for _ in range(9)], 1)
    src_rows = torch.randn(3, 9, generator=g)
    b = a.clone().to(dev)
    b.scatter_(0, col.to(dev), src_rows.to(dev))
    assert torch.equal(b.cpu(), a.clone().scatter_(0, col, src_rows))
    mean, std = torch.full((20000,), 3.0), torch.full((20000,), 0.5)
    for draw in (torch.normal(mean.to(dev), std.to(dev)), torch.normal(mean.to(dev), 0.5), torch.normal(3.0, std.to(dev))):
        draw = draw.cpu()
        assert draw.shape == (20000,) and abs(float(draw.mean()) - 3.0) < 0.02 and abs(float(draw.std()) - 0.5) < 0.02


def test_pooling_of_volumes(vk):
    _pooling_of_volumes(vk)
    h = torch.randn(2, 3, 8, 10, 6, generator=torch.Generator().manual_seed(48)).half()
    _close(F.max_pool3d(h.to(vk), 2).float(), F.max_pool3d(h.float(), 2), 1e-3)
    _close(F.avg_pool3d(h.to(vk), 2).float(), F.avg_pool3d(h.float(), 2), 2e-3)


def test_assorted_small_operators(vk):
    _assorted_small_operators(vk)


def _bicubic_and_embedding_bags(dev):
    g = torch.Generator().manual_seed(59)
    x = torch.randn(2, 3, 7, 9, generator=g)
    for kw in ({"size": (14, 18)}, {"size": (11, 5), "align_corners": True}, {"size": (5, 13)}, {"size": (1, 1), "align_corners": True},
               {"scale_factor": (1.5, 2.5), "recompute_scale_factor": False}, {"size": (20, 3)}):
        xd, xc = x.clone().to(dev).requires_grad_(), x.clone().requires_grad_()
        yd, yc = F.interpolate(xd, mode="bicubic", **kw), F.interpolate(xc, mode="bicubic", **kw)
        _close(yd, yc, 2e-5)
        gy = torch.randn(yc.shape, generator=g)
        yd.backward(gy.to(dev)); yc.backward(gy)
        _close(xd.grad, xc.grad, 2e-5)

    V, D = 20, 6
    idx = torch.randint(0, V, (17,), generator=g)
    offs = torch.tensor([0, 3, 3, 9, 15])
    psw = torch.rand(17, generator=g)
    table = torch.randn(V, D, generator=g)
    for mode, weights in (("sum", None), ("sum", psw), ("mean", None)):
        for include_last in (False, True):
            for pad in (None, 4):
                o = torch.cat([offs, torch.tensor([17])]) if include_last else offs
                wd, wc = table.clone().to(dev).requires_grad_(), table.clone().requires_grad_()
                pd = None if weights is None else weights.clone().to(dev).requires_grad_()
                pc = None if weights is None else weights.clone().requires_grad_()
                yd = F.embedding_bag(idx.to(dev), wd, o.to(dev), mode=mode, per_sample_weights=pd, include_last_offset=include_last, padding_idx=pad)
                yc = F.embedding_bag(idx, wc, o, mode=mode, per_sample_weights=pc, include_last_offset=include_last, padding_idx=pad)
                _close(yd, yc, 1e-5)
                gy = torch.randn(yc.shape, generator=g)
                yd.backward(gy.to(dev)); yc.backward(gy)
                _close(wd.grad, wc.grad, 1e-5)
                if pc is not None:
                    _close(pd.grad, pc.grad, 1e-5)
    torch.manual_seed(3)
    ref = torch.nn.EmbeddingBag(V, D)                                   # mean over the rows of a 2-D input
    bag = torch.nn.EmbeddingBag(V, D)
    bag.load_state_dict(ref.state_dict())
    bag = bag.to(dev)
    two_d = torch.randint(0, V, (4, 5), generator=g)
    _close(bag(two_d.to(dev)), ref(two_d), 1e-5)
    with torch.no_grad():
        _close(bag(idx.to(dev), offs.to(dev)), ref(idx, offs), 1e-5)


def test_bicubic_upsampling_and_embedding_bags(vk):
    _bicubic_and_embedding_bags(vk)


def _volume_padding_and_index_copy(dev):
    g = torch.Generator().manual_seed(61)
    v = torch.randn(2, 3, 5, 6, 7, generator=g)
    for mode in ("reflect", "replicate"):
        vd, vc = v.clone().to(dev).requires_grad_(), v.clone().requires_grad_()
        yd, yc = F.pad(vd, (1, 2, 0, 3, 2, 1), mode=mode), F.pad(vc, (1, 2, 0, 3, 2, 1), mode=mode)
        assert torch.equal(yd.detach().cpu(), yc.detach())
        gy = torch.randn(yc.shape, generator=g)
        yd.backward(gy.to(dev)); yc.backward(gy)
        _close(vd.grad, vc.grad, 1e-5)
    a = torch.randn(6, 9, generator=g)
    rows, src = torch.tensor([4, 0, 2]), torch.randn(3, 9, generator=g)
    assert torch.equal(a.clone().to(dev).index_copy(0, rows.to(dev), src.to(dev)).cpu(), a.index_copy(0, rows, src))
    cols, src_c = torch.tensor([8, 1]), torch.randn(6, 2, generator=g)
    b = a.clone().to(dev)
    b.index_copy_(1, cols.to(dev), src_c.to(dev))
    assert torch.equal(b.cpu(), a.clone().index_copy_(1, cols, src_c))


def test_volume_padding_and_index_copy(vk):
    _volume_padding_and_index_copy(vk)

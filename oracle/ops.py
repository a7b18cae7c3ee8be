"""numpy restatements of the hot-path algorithms (test infrastructure, see oracle/__init__.py).

Inputs are numpy arrays; floating inputs are taken as the exact values the device sees (a
half/bf16 tensor is passed after widening to float32). Results are float64 or float32 "ideal"
values unless a function says it rounds; the tests apply the stated tolerance or round with the
same rule as the device before a bit-exact comparison.
"""
from __future__ import annotations

import math

import numpy as np

try:  # scipy is in the image; fall back to math.erf element-wise if it is not
    from scipy.special import erf as _erf
except Exception:  # pragma: no cover
    _erf = np.vectorize(math.erf)

__all__ = [
    "gelu", "gelu_backward", "gemm", "argreduce", "stable_topk", "reduce", "softmax", "log_softmax",
    "softmax_backward", "log_softmax_backward", "nll_loss_forward", "nll_loss_backward", "rmsnorm_forward",
    "rmsnorm_backward", "batchnorm_forward", "batchnorm_backward", "embedding_forward", "embedding_backward",
    "adam_step", "sgd_step", "unary", "binary", "mlp_step", "attention_forward", "attention_backward",
    "conv2d_forward", "conv2d_backward_input", "conv2d_backward_weight", "layernorm_forward", "layernorm_backward",
    "groupnorm_forward", "groupnorm_backward", "cross_entropy_forward", "cross_entropy_backward", "scan",
    "gelu_tanh", "gelu_tanh_backward",
]


# ----------------------------------------------------------------------------- activations
def gelu(x):
    """Exact (erf) GELU: 0.5*x*(1+erf(x/sqrt 2)) — src/shaders/core/dtype.slang:736-737."""
    x = np.asarray(x, dtype=np.float64)
    return 0.5 * x * (1.0 + _erf(x * 0.7071067811865476))


def gelu_backward(grad, x):
    """grad*(cdf + x*pdf) — src/shaders/core/dtype.slang:739-744."""
    grad = np.asarray(grad, dtype=np.float64)
    x = np.asarray(x, dtype=np.float64)
    cdf = 0.5 * (1.0 + _erf(x * 0.7071067811865476))
    pdf = np.exp(-0.5 * x * x) * 0.3989422804014327
    return grad * (cdf + x * pdf)


def _act(v, activation):
    if activation in (None, 0, "none"):
        return v
    if activation in (1, "relu"):
        return np.where(np.isnan(v), v, np.maximum(v, 0.0))
    if activation in (2, "gelu"):
        return gelu(v)
    raise ValueError(activation)


# ----------------------------------------------------------------------------- contraction
def gemm(a, b, bias=None, alpha=1.0, beta=1.0, activation=None):
    """act(alpha * a @ b + beta * bias) in float64.

    Epilogue order of src/shaders/ops/matmul_coop.slang:401-408 (scale, add bias, activate);
    a: [..., m, k], b: [..., k, n], bias broadcastable to the result (src/api/ops/matmul.cpp:49-53).
    """
    v = alpha * np.matmul(np.asarray(a, np.float64), np.asarray(b, np.float64))
    if bias is not None:
        v = v + beta * np.asarray(bias, np.float64)
    return _act(v, activation)


# ----------------------------------------------------------------------------- reductions
def reduce(op, x, axis):
    """sum / mean / amax / amin along one axis; fp64 accumulation stands in for the reference's
    fp32 accumulate (src/api/ops/reduce.cpp:266-274); amax/amin propagate NaN
    (src/shaders/ops/reduce_subgroup.slang:39-53)."""
    x = np.asarray(x, np.float64)
    if op == "sum":
        return x.sum(axis=axis)
    if op == "mean":
        return x.mean(axis=axis) if x.shape[axis] else np.full(np.delete(x.shape, axis), np.nan)
    if op == "amax":
        return np.max(x, axis=axis)  # np.max propagates NaN
    if op == "amin":
        return np.min(x, axis=axis)
    raise ValueError(op)


def argreduce(x, axis, is_max=True):
    """Index of the first extreme element along `axis`; NaN counts as the extreme and the first
    NaN wins — the serial scan of src/shaders/ops/arg_reduce.slang:49-65, vectorised."""
    x = np.asarray(x)
    xm = np.moveaxis(x, axis, -1)
    nan = np.isnan(xm)
    has_nan = nan.any(axis=-1)
    first_nan = nan.argmax(axis=-1)
    filled = np.where(nan, -np.inf if is_max else np.inf, xm)
    # np.argmax / np.argmin return the first occurrence of the extreme
    best = filled.argmax(axis=-1) if is_max else filled.argmin(axis=-1)
    return np.where(has_nan, first_nan, best).astype(np.int64)


def stable_topk(x, k, descending=True):
    """Full stable sort of each last-axis line, then the first k — src/api/ops/sort.cpp:118-140 with
    the comparator of src/shaders/ops/sort.slang:24-49: by value, NaN largest, ties by ascending
    original position. Returns (values, int64 indices)."""
    x = np.asarray(x)
    n = x.shape[-1]
    nan = np.isnan(x)
    # Rank key: NaN is the largest value; -0.0 == +0.0.
    key = np.where(nan, np.inf, x.astype(np.float64)) + 0.0
    pos = np.broadcast_to(np.arange(n), x.shape)
    if descending:
        # primary: NaN first, then value descending; secondary: position ascending
        order = np.lexsort((pos, -key, ~nan), axis=-1)
    else:
        order = np.lexsort((pos, key, nan), axis=-1)
    idx = order[..., :k].astype(np.int64)
    return np.take_along_axis(x, idx, axis=-1), idx


# ----------------------------------------------------------------------------- softmax family
def softmax(x):
    """Last-axis softmax on float32-widened input, one rounding at the end
    (src/api/decompositions.cpp:506-571)."""
    x = np.asarray(x, np.float64)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def log_softmax(x):
    """(x - max) - log(sum(exp(x - max))) — src/api/decompositions.cpp:506-520."""
    x = np.asarray(x, np.float64)
    s = x - x.max(axis=-1, keepdims=True)
    return s - np.log(np.exp(s).sum(axis=-1, keepdims=True))


def softmax_backward(grad, y):
    grad, y = np.asarray(grad, np.float64), np.asarray(y, np.float64)
    return y * (grad - (grad * y).sum(axis=-1, keepdims=True))


def log_softmax_backward(grad, y):
    grad, y = np.asarray(grad, np.float64), np.asarray(y, np.float64)
    return grad - np.exp(y) * grad.sum(axis=-1, keepdims=True)


def nll_loss_forward(logp, target, weight=None, reduction="mean", ignore_index=-100):
    """Gather -logp[i, t_i]; ignored or out-of-range targets contribute 0
    (src/shaders/ops/nllloss.slang:20-39); mean divides by the summed weights
    (src/api/ops/nllloss.cpp:79-130). Returns (loss, total_weight)."""
    logp = np.asarray(logp, np.float64)
    target = np.asarray(target, np.int64)
    n, c = logp.shape
    valid = (target != ignore_index) & (target >= 0) & (target < c)
    t = np.where(valid, target, 0)
    w = np.ones(c) if weight is None else np.asarray(weight, np.float64)
    wi = np.where(valid, w[t], 0.0)
    per = -logp[np.arange(n), t] * wi
    total = wi.sum()
    if reduction == "none":
        return per, 0.0
    if reduction == "sum":
        return per.sum(), total
    return per.sum() / total, total


def nll_loss_backward(grad_out, target, c, weight=None, reduction="mean", ignore_index=-100, total_weight=None):
    """Scatter of -grad*w into zeros [n, c] (src/shaders/ops/nllloss.slang:42-52)."""
    target = np.asarray(target, np.int64)
    n = target.shape[0]
    w = np.ones(c) if weight is None else np.asarray(weight, np.float64)
    g = np.zeros((n, c))
    valid = (target != ignore_index) & (target >= 0) & (target < c)
    go = np.asarray(grad_out, np.float64)
    for i in np.nonzero(valid)[0]:
        gi = go[i] if reduction == "none" else float(go)
        v = -gi * w[target[i]]
        if reduction == "mean":
            v /= total_weight
        g[i, target[i]] = v
    return g


# ----------------------------------------------------------------------------- norms
def rmsnorm_forward(x, weight=None, eps=None):
    """y = x * rsqrt(mean(x^2) + eps) * w; eps defaults to float32 epsilon
    (src/api/ops/norm.cpp:177); returns (y, rstd) — norm.slang:193-240."""
    x = np.asarray(x, np.float64)
    if eps is None:
        eps = float(np.finfo(np.float32).eps)
    rstd = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    y = x * rstd
    if weight is not None:
        y = y * np.asarray(weight, np.float64)
    return y, rstd[..., 0]


def rmsnorm_backward(grad_y, x, weight, rstd):
    """grad_x = rstd*(g*w - xhat*mean(g*w*xhat)), grad_w = sum_rows g*xhat — norm.slang:242-317."""
    g, x = np.asarray(grad_y, np.float64), np.asarray(x, np.float64)
    rstd = np.asarray(rstd, np.float64)[..., None]
    w = 1.0 if weight is None else np.asarray(weight, np.float64)
    xhat = x * rstd
    gw = g * w
    gx = rstd * (gw - xhat * (gw * xhat).mean(axis=-1, keepdims=True))
    gwt = (g * xhat).reshape(-1, x.shape[-1]).sum(axis=0)
    return gx, gwt


def batchnorm_forward(x, weight, bias, running_mean, running_var, momentum=0.1, eps=1e-5):
    """Training batch norm over [n, c, ...]: biased variance for normalisation, unbiased for the
    running estimate (src/shaders/ops/norm.slang:72-131). Returns
    (y, save_mean, save_invstd, new_running_mean, new_running_var)."""
    x = np.asarray(x, np.float64)
    axes = (0,) + tuple(range(2, x.ndim))
    cnt = x.size / x.shape[1]
    mean = x.mean(axis=axes)
    var = x.var(axis=axes)
    invstd = 1.0 / np.sqrt(var + eps)
    shp = (1, -1) + (1,) * (x.ndim - 2)
    w = np.ones_like(mean) if weight is None else np.asarray(weight, np.float64)
    b = np.zeros_like(mean) if bias is None else np.asarray(bias, np.float64)
    y = (x - mean.reshape(shp)) * (invstd * w).reshape(shp) + b.reshape(shp)
    unbiased = var * cnt / (cnt - 1.0) if cnt > 1 else var
    rm = None if running_mean is None else (1 - momentum) * np.asarray(running_mean, np.float64) + momentum * mean
    rv = None if running_var is None else (1 - momentum) * np.asarray(running_var, np.float64) + momentum * unbiased
    return y, mean, invstd, rm, rv


def batchnorm_backward(grad_y, x, weight, save_mean, save_invstd):
    """src/shaders/ops/norm.slang:133-191: grad_x, grad_weight, grad_bias."""
    g, x = np.asarray(grad_y, np.float64), np.asarray(x, np.float64)
    axes = (0,) + tuple(range(2, x.ndim))
    shp = (1, -1) + (1,) * (x.ndim - 2)
    cnt = x.size / x.shape[1]
    mean = np.asarray(save_mean, np.float64).reshape(shp)
    invstd = np.asarray(save_invstd, np.float64).reshape(shp)
    w = np.ones(x.shape[1]) if weight is None else np.asarray(weight, np.float64)
    xmu = x - mean
    sum_dy = g.sum(axis=axes)
    sum_dy_xmu = (g * xmu).sum(axis=axes)
    gx = (g - sum_dy.reshape(shp) / cnt - xmu * invstd * invstd * sum_dy_xmu.reshape(shp) / cnt) * (w.reshape(shp) * invstd)
    return gx, sum_dy_xmu * invstd.reshape(-1), sum_dy


# ----------------------------------------------------------------------------- conv2d
def _conv_taps(x, kh, kw, stride, padding, ho, wo):
    """Padded input and, per tap, the strided window that meets output pixel (ho, wo)."""
    n, c, h, w = x.shape
    xp = np.zeros((n, c, h + 2 * padding, w + 2 * padding), np.float64)
    xp[:, :, padding:padding + h, padding:padding + w] = x
    for i in range(kh):
        for j in range(kw):
            yield i, j, xp[:, :, i:i + (ho - 1) * stride + 1:stride, j:j + (wo - 1) * stride + 1:stride]


def conv2d_forward(x, w, stride=1, padding=0):
    """y[n,o,p,q] = sum_{c,i,j} x[n,c,p*s-pad+i,q*s-pad+j] * w[o,c,i,j], zero outside the input:
    the FORWARD mode's implicit-GEMM index map (src/shaders/helpers/conv.slang, mode 0; host side
    src/api/ops/conv.cpp:1088-1117). float64 accumulation."""
    x = np.asarray(x, np.float64)
    w = np.asarray(w, np.float64)
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    ho = (h + 2 * padding - kh) // stride + 1
    wo = (wd + 2 * padding - kw) // stride + 1
    y = np.zeros((n, o, ho, wo), np.float64)
    for i, j, win in _conv_taps(x, kh, kw, stride, padding, ho, wo):
        y += np.einsum("nchw,oc->nohw", win, w[:, :, i, j])
    return y


def conv2d_backward_input(gy, w, x_shape, stride=1, padding=0):
    """gx = scatter of gy through the same index map (GRAD_INPUT mode, src/api/ops/conv.cpp:1119-1150)."""
    gy = np.asarray(gy, np.float64)
    w = np.asarray(w, np.float64)
    n, c, h, wd = x_shape
    o, _, kh, kw = w.shape
    _, _, ho, wo = gy.shape
    gxp = np.zeros((n, c, h + 2 * padding, wd + 2 * padding), np.float64)
    for i in range(kh):
        for j in range(kw):
            gxp[:, :, i:i + (ho - 1) * stride + 1:stride, j:j + (wo - 1) * stride + 1:stride] += np.einsum("nohw,oc->nchw", gy, w[:, :, i, j])
    return gxp[:, :, padding:padding + h, padding:padding + wd]


def conv2d_backward_weight(gy, x, w_shape, stride=1, padding=0):
    """gw[o,c,i,j] = sum_{n,p,q} gy[n,o,p,q] * x[n,c,p*s-pad+i,q*s-pad+j] (GRAD_WEIGHT mode,
    src/api/ops/conv.cpp:1034-1060 sums the same products in split-K partials)."""
    gy = np.asarray(gy, np.float64)
    x = np.asarray(x, np.float64)
    o, c, kh, kw = w_shape
    _, _, ho, wo = gy.shape
    gw = np.zeros(tuple(w_shape), np.float64)
    for i, j, win in _conv_taps(x, kh, kw, stride, padding, ho, wo):
        gw[:, :, i, j] = np.einsum("nohw,nchw->oc", gy, win)
    return gw


# ----------------------------------------------------------------------------- attention
def attention_forward(q, k, v, causal=True, scale=None):
    """softmax(q k^T * scale + mask) v with grouped-query heads (kvh = h // (Hq/Hk)), float64.
    Semantics of src/api/ops/attention.cpp:395-480 and attention_coop.slang:117-222: the causal mask hides
    key > row (top-left aligned for L != S: src/api/ops/attention.cpp:107-112, attention_coop.slang:53-56, which
    is also ATen's is_causal rule); a row without a visible key (only possible for S = 0) gives out = 0, lse = +inf.
    q: [B, Hq, L, D], k/v: [B, Hk, S, D]. Returns (out, lse, p)."""
    q, k, v = (np.asarray(t, np.float64) for t in (q, k, v))
    B, Hq, L, D = q.shape
    Hk, S = k.shape[1], k.shape[2]
    g = Hq // Hk
    scale = D ** -0.5 if scale is None else scale
    kk, vv = np.repeat(k, g, axis=1), np.repeat(v, g, axis=1)
    s = np.einsum("bhld,bhsd->bhls", q, kk) * scale
    if causal:
        vis = np.arange(S)[None, :] <= np.arange(L)[:, None]
        s = np.where(vis[None, None], s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    dead = ~np.isfinite(m)
    with np.errstate(invalid="ignore"):
        e = np.where(dead, 0.0, np.exp(s - np.where(dead, 0.0, m)))
    den = e.sum(axis=-1, keepdims=True)
    p = np.where(dead, 0.0, e / np.where(den == 0, 1.0, den))
    lse = np.where(dead[..., 0], np.inf, (m + np.log(np.where(den == 0, 1.0, den)))[..., 0])
    return np.einsum("bhls,bhsd->bhld", p, vv), lse, p


def attention_backward(dout, q, k, v, causal=True, scale=None):
    """Gradients of attention_forward: delta = sum(dO*O), dS = P*(dP - delta)*scale, K/V gradients summed
    over the query heads of each group (src/api/ops/attention.cpp:641-665)."""
    dout, q, k, v = (np.asarray(t, np.float64) for t in (dout, q, k, v))
    B, Hq, L, D = q.shape
    Hk, S = k.shape[1], k.shape[2]
    g = Hq // Hk
    scale = D ** -0.5 if scale is None else scale
    out, _, p = attention_forward(q, k, v, causal, scale)
    kk, vv = np.repeat(k, g, axis=1), np.repeat(v, g, axis=1)
    dp = np.einsum("bhld,bhsd->bhls", dout, vv)
    delta = (dout * out).sum(axis=-1, keepdims=True)
    ds = p * (dp - delta) * scale
    dq = np.einsum("bhls,bhsd->bhld", ds, kk)
    dk = np.einsum("bhls,bhld->bhsd", ds, q).reshape(B, Hk, g, S, D).sum(axis=2)
    dv = np.einsum("bhls,bhld->bhsd", p, dout).reshape(B, Hk, g, S, D).sum(axis=2)
    return dq, dk, dv


# ----------------------------------------------------------------------------- layer / group norm
def layernorm_forward(x, weight=None, bias=None, norm_dims=1, eps=1e-5):
    """(x - mean) * rstd * w + b over the last `norm_dims` axes, biased variance, mean first then the centred squares
    (rowForward, src/shaders/ops/norm.slang:193-226; host src/api/ops/norm.cpp:264-290). Returns (y, mean, rstd)."""
    x = np.asarray(x, np.float64)
    axes = tuple(range(x.ndim - norm_dims, x.ndim))
    mean = x.mean(axis=axes, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=axes, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    y = (x - mean) * rstd
    if weight is not None:
        y = y * np.asarray(weight, np.float64)
    if bias is not None:
        y = y + np.asarray(bias, np.float64)
    return y, mean.reshape(x.shape[:x.ndim - norm_dims]), rstd.reshape(x.shape[:x.ndim - norm_dims])


def layernorm_backward(grad_y, x, weight, mean, rstd, norm_dims=1):
    """rowBackwardInput / rowBackwardParams (src/shaders/ops/norm.slang:228-317): grad_x = rstd * (g - mean(g) - xhat *
    mean(g * xhat)) with g = grad_y * w; grad_w = sum grad_y * xhat and grad_b = sum grad_y over the rows."""
    gy, x = np.asarray(grad_y, np.float64), np.asarray(x, np.float64)
    axes = tuple(range(x.ndim - norm_dims, x.ndim))
    lead = tuple(range(x.ndim - norm_dims))
    shape = x.shape[:x.ndim - norm_dims] + (1,) * norm_dims
    xhat = (x - np.asarray(mean, np.float64).reshape(shape)) * np.asarray(rstd, np.float64).reshape(shape)
    g = gy * (np.asarray(weight, np.float64) if weight is not None else 1.0)
    gx = np.asarray(rstd, np.float64).reshape(shape) * (g - g.mean(axis=axes, keepdims=True) - xhat * (g * xhat).mean(axis=axes, keepdims=True))
    return gx, (gy * xhat).sum(axis=lead), gy.sum(axis=lead)


def groupnorm_forward(x, groups, weight=None, bias=None, eps=1e-5):
    """native_group_norm: statistics over (C / G, H, W) of every (sample, group), affine per channel
    (src/api/ops/norm.cpp:264-325 in its row mode). Returns (y, mean [n, G], rstd [n, G])."""
    x = np.asarray(x, np.float64)
    n, c = x.shape[:2]
    xg = x.reshape(n, groups, -1)
    mean = xg.mean(axis=2)
    var = ((xg - mean[..., None]) ** 2).mean(axis=2)
    rstd = 1.0 / np.sqrt(var + eps)
    y = ((xg - mean[..., None]) * rstd[..., None]).reshape(x.shape)
    bshape = (1, c) + (1,) * (x.ndim - 2)
    if weight is not None:
        y = y * np.asarray(weight, np.float64).reshape(bshape)
    if bias is not None:
        y = y + np.asarray(bias, np.float64).reshape(bshape)
    return y, mean, rstd


def groupnorm_backward(grad_y, x, weight, mean, rstd, groups):
    gy, x = np.asarray(grad_y, np.float64), np.asarray(x, np.float64)
    n, c = x.shape[:2]
    bshape = (1, c) + (1,) * (x.ndim - 2)
    xhat = ((x.reshape(n, groups, -1) - np.asarray(mean, np.float64)[..., None]) * np.asarray(rstd, np.float64)[..., None]).reshape(x.shape)
    g = gy * (np.asarray(weight, np.float64).reshape(bshape) if weight is not None else 1.0)
    gg, xg = g.reshape(n, groups, -1), xhat.reshape(n, groups, -1)
    gx = np.asarray(rstd, np.float64)[..., None] * (gg - gg.mean(axis=2, keepdims=True) - xg * (gg * xg).mean(axis=2, keepdims=True))
    red = (0,) + tuple(range(2, x.ndim))
    return gx.reshape(x.shape), (gy * xhat).sum(axis=red), gy.sum(axis=red)


# ----------------------------------------------------------------------------- cross-entropy (fused form)
def cross_entropy_forward(logits, target, weight=None, reduction="mean", ignore_index=-100):
    """nll_loss(log_softmax(logits)) as one function (src/api/decompositions.cpp:506-571 followed by
    src/api/ops/nllloss.cpp:79-174; ignored / out-of-range targets contribute nothing, nllloss.slang:20-39).
    Returns (loss, total_weight, lse)."""
    x = np.asarray(logits, np.float64)
    m = x.max(axis=1, keepdims=True)
    lse = (m + np.log(np.exp(x - m).sum(axis=1, keepdims=True)))[:, 0]
    loss, total = nll_loss_forward(x - lse[:, None], target, weight, reduction, ignore_index)
    return loss, total, lse


def cross_entropy_backward(grad_out, logits, lse, target, weight=None, reduction="mean", ignore_index=-100, total_weight=None):
    """(softmax - onehot) * w[t] * g (/ total_weight): log_softmax_backward of nll_loss_backward in one expression."""
    x = np.asarray(logits, np.float64)
    n, c = x.shape
    sm = np.exp(x - np.asarray(lse, np.float64)[:, None])
    g = nll_loss_backward(grad_out, target, c, weight, reduction, ignore_index, total_weight)      # -w*g/total at the target
    return g - sm * g.sum(axis=1, keepdims=True)


# ----------------------------------------------------------------------------- scans
def scan(op, x, axis):
    """Inclusive scan (src/shaders/ops/scan.slang: SumScanOp, ProdScanOp, LogAddExpScanOp)."""
    x = np.asarray(x)
    if op == "cumsum":
        return np.cumsum(x, axis=axis)
    if op == "cumprod":
        return np.cumprod(x, axis=axis)
    if op == "logcumsumexp":
        return np.logaddexp.accumulate(np.asarray(x, np.float64), axis=axis)
    raise ValueError(op)


# ----------------------------------------------------------------------------- embedding
def embedding_forward(table, idx):
    """Row gather (src/api/ops/indexing.cpp:299-314); bit-exact copy."""
    return np.asarray(table)[np.asarray(idx, np.int64)]


def embedding_backward(grad, idx, num_rows, padding_idx=-1):
    """Per table row, the fp32 sum of its gradient rows in increasing position
    (src/shaders/ops/embedding_backward.slang:36-56). Sequential float32 accumulation, so the
    result is reproducible bit for bit."""
    grad = np.asarray(grad, np.float32)
    idx = np.asarray(idx, np.int64).reshape(-1)
    grad = grad.reshape(idx.shape[0], -1)
    out = np.zeros((num_rows, grad.shape[1]), np.float32)
    for i, r in enumerate(idx):
        if r != padding_idx and 0 <= r < num_rows:
            out[r] += grad[i]
    return out


# ----------------------------------------------------------------------------- optimizers
def adam_step(p, g, m, v, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-2, decoupled=True,
              maximize=False):
    """One Adam/AdamW step in float32, in the order of adam_step (src/api/ops/optim.cpp:46-86).
    Returns float32 (p, m, v) before the final rounding to the storage dtype."""
    f = np.float32
    p, g, m, v = (np.asarray(t, f) for t in (p, g, m, v))
    if maximize:
        g = -g
    if weight_decay != 0.0:
        if decoupled:
            p = p * f(1.0 - lr * weight_decay)
        else:
            g = g + f(weight_decay) * p
    m = m + f(1.0 - beta1) * (g - m)
    v = v * f(beta2) + (g * f(1.0 - beta2)) * g
    bc1 = 1.0 - beta1 ** step
    bc2_sqrt = math.sqrt(1.0 - beta2 ** step)
    denom = np.sqrt(v) / f(bc2_sqrt) + f(eps)
    p = p - (m * f(lr / bc1)) / denom
    return p.astype(f), m.astype(f), v.astype(f)


def sgd_step(p, g, buf, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, maximize=False,
             first_step=False):
    """src/api/ops/optim.cpp:195-205. Returns float32 (p, buf)."""
    f = np.float32
    p, g = np.asarray(p, f), np.asarray(g, f)
    if maximize:
        g = -g
    if weight_decay != 0.0:
        g = g + f(weight_decay) * p
    if momentum != 0.0:
        buf = g if first_step else np.asarray(buf, f) * f(momentum) + g * f(1.0 - dampening)
        g = g + f(momentum) * buf if nesterov else buf
    p = p - g * f(lr)
    return p.astype(f), (None if buf is None else np.asarray(buf, f))


def gelu_tanh(x):
    """gelu(approximate='tanh') — src/shaders/core/dtype.slang:738."""
    x = np.asarray(x, dtype=np.float64)
    return 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def gelu_tanh_backward(grad, x):
    """src/shaders/core/dtype.slang:745-751."""
    grad, x = np.asarray(grad, dtype=np.float64), np.asarray(x, dtype=np.float64)
    x2 = x * x
    t = np.tanh(0.7978845608028654 * (x + 0.044715 * x2 * x))
    dinner = 0.7978845608028654 * (1.0 + 3.0 * 0.044715 * x2)
    return grad * (0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * dinner)


# ----------------------------------------------------------------------------- elementwise
_UNARY = {
    "neg": lambda x: -x, "exp": np.exp, "log": np.log, "sqrt": np.sqrt, "rsqrt": lambda x: 1.0 / np.sqrt(x),
    "sigmoid": lambda x: 1.0 / (1.0 + np.exp(-x)), "relu": lambda x: np.where(np.isnan(x), x, np.maximum(x, 0.0)),
    "gelu": gelu, "tanh": np.tanh, "abs": np.abs, "silu": lambda x: x / (1.0 + np.exp(-x)),
    "reciprocal": lambda x: 1.0 / x, "square": lambda x: x * x, "sin": np.sin, "cos": np.cos, "gelu_tanh": gelu_tanh,
}


def unary(op, x):
    """float64 value of the unary maps of src/api/ops/unary.cpp:14-64 that the configs use."""
    with np.errstate(all="ignore"):
        return _UNARY[op](np.asarray(x, np.float64))


def binary(op, a, b, alpha=1.0):
    """float64 value of the binary maps (src/api/ops/binary.cpp:20-43) that the configs use."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    with np.errstate(all="ignore"):
        if op == "add":
            return a + alpha * b
        if op == "add_relu":        # relu(add(a, b, alpha)), src/api/ops/binary.cpp:655-657
            v = a + alpha * b
            return np.where(np.isnan(v), v, np.maximum(v, 0.0))
        if op == "sub":
            return a - alpha * b
        if op == "mul":
            return a * b
        if op == "div":
            return a / b
        if op == "maximum":
            return np.where(np.isnan(a) | np.isnan(b), np.nan, np.maximum(a, b))
        if op == "minimum":
            return np.where(np.isnan(a) | np.isnan(b), np.nan, np.minimum(a, b))
        if op == "pow":
            return np.power(a, b)
        if op == "gelu_backward":
            return gelu_backward(a, b)
        if op == "gelu_tanh_backward":
            return gelu_tanh_backward(a, b)
        if op == "threshold_backward":
            return np.where(b <= alpha, 0.0, a)
        if op == "silu_backward":
            s = 1.0 / (1.0 + np.exp(-b))
            return a * s * (1.0 + b * (1.0 - s))
        if op == "sigmoid_backward":
            return a * (1.0 - b) * b
        if op == "tanh_backward":
            return a * (1.0 - b * b)
    raise ValueError(op)


# ----------------------------------------------------------------------------- config 2: MLP step
def mlp_step(x, labels, weights, biases):
    """Forward + backward of the MLP of examples/mlp.py:5-23 (Linear, GELU, ..., Linear, mean
    cross-entropy) in float64 on the given parameter values. Returns
    (loss, logits, [grad_w...], [grad_b...])."""
    h = np.asarray(x, np.float64)
    acts, pre = [h], []
    nl = len(weights)
    for i, (w, b) in enumerate(zip(weights, biases)):
        z = h @ np.asarray(w, np.float64).T + np.asarray(b, np.float64)
        pre.append(z)
        h = gelu(z) if i < nl - 1 else z
        acts.append(h)
    logits = h
    lp = log_softmax(logits)
    loss, total = nll_loss_forward(lp, labels)
    g = nll_loss_backward(1.0, labels, logits.shape[1], total_weight=total)
    g = log_softmax_backward(g, lp)
    gws, gbs = [None] * nl, [None] * nl
    for i in reversed(range(nl)):
        gws[i] = g.T @ acts[i]
        gbs[i] = g.sum(axis=0)
        if i > 0:
            g = g @ np.asarray(weights[i], np.float64)
            g = gelu_backward(g, pre[i - 1])
    return loss, logits, gws, gbs

"""Calls into the tvk C-ABI with ``torch.cuda`` tensors as the device buffers.

torch is used here for device memory and streams only: every function passes raw pointers,
sizes and strides to ``libtvk.so`` and launches on torch's current CUDA stream. Used by the GPU
tests and by ``bench.py``; the ``vulkan`` device of the ATen extension goes through the same
entry points from C++.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi

_DT = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16, torch.int64: capi.I64,
       torch.int32: capi.I32, torch.uint8: capi.U8, torch.bool: capi.U8, torch.float64: capi.F64}

UNARY = {"neg": capi.U_NEG, "exp": capi.U_EXP, "log": capi.U_LOG, "sqrt": capi.U_SQRT, "rsqrt": capi.U_RSQRT,
         "sigmoid": capi.U_SIGMOID, "relu": capi.U_RELU, "gelu": capi.U_GELU, "tanh": capi.U_TANH, "abs": capi.U_ABS,
         "silu": capi.U_SILU, "reciprocal": capi.U_RECIPROCAL, "square": capi.U_SQUARE, "sin": capi.U_SIN,
         "cos": capi.U_COS, "gelu_tanh": capi.U_GELU_TANH}
BINARY = {"add": capi.B_ADD, "sub": capi.B_SUB, "mul": capi.B_MUL, "div": capi.B_DIV, "maximum": capi.B_MAXIMUM,
          "minimum": capi.B_MINIMUM, "pow": capi.B_POW, "gelu_backward": capi.B_GELU_BACKWARD,
          "threshold_backward": capi.B_THRESHOLD_BACKWARD, "silu_backward": capi.B_SILU_BACKWARD,
          "sigmoid_backward": capi.B_SIGMOID_BACKWARD, "tanh_backward": capi.B_TANH_BACKWARD,
          "gelu_tanh_backward": capi.B_GELU_TANH_BACKWARD, "add_relu": capi.B_ADD_RELU}
COMPARE = {"eq": capi.C_EQ, "ne": capi.C_NE, "lt": capi.C_LT, "le": capi.C_LE, "gt": capi.C_GT, "ge": capi.C_GE}
TERNARY = {"addcmul": capi.T_ADDCMUL, "addcdiv": capi.T_ADDCDIV, "lerp": capi.T_LERP, "where": capi.T_WHERE}
REDUCE = {"sum": capi.R_SUM, "mean": capi.R_MEAN, "amax": capi.R_AMAX, "amin": capi.R_AMIN}
ACT = {None: capi.ACT_NONE, "none": capi.ACT_NONE, "relu": capi.ACT_RELU, "gelu": capi.ACT_GELU}


def dt(t: torch.Tensor) -> int:
    return _DT[t.dtype]


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ws(nbytes: int, device) -> torch.Tensor | None:
    return torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None


def check_device_status(device: int = 0) -> None:
    capi.call("tvk_check_device_status", device)


# ------------------------------------------------------------------------------- contraction
AUX = {None: capi.AUX_NONE, "gelu_backward": capi.AUX_GELU_BACKWARD, "relu_backward": capi.AUX_RELU_BACKWARD}


def gemm_desc(a, b, out, bias=None, alpha=1.0, beta=1.0, act=None, force_path=0, out2=None, aux=None, aux_op=None) -> capi.GemmDesc:
    """a: [B?, m, k], b: [B?, k, n] (any strides), out: [B?, m, n] with contiguous rows.
    out2 (same shape and strides as out): out then receives the value before the activation and out2 the activated one.
    aux + aux_op ("gelu_backward" / "relu_backward"): out = (alpha * a @ b + beta * bias) * act'(aux), aux of out's shape."""
    a3 = a if a.dim() == 3 else a.unsqueeze(0)
    b3 = b if b.dim() == 3 else b.unsqueeze(0)
    o3 = out if out.dim() == 3 else out.unsqueeze(0)
    batch = max(a3.shape[0], b3.shape[0])
    m, k = a3.shape[1], a3.shape[2]
    n = b3.shape[2]
    assert b3.shape[1] == k and tuple(o3.shape) == (batch, m, n) and (n <= 1 or o3.stride(2) == 1)
    d = capi.GemmDesc()
    d.dtype, d.activation = dt(a), ACT[act]
    d.batch, d.m, d.n, d.k = batch, m, n, k
    d.a, d.a_rs, d.a_cs, d.a_bs = a3.data_ptr(), a3.stride(1), a3.stride(2), (a3.stride(0) if a3.shape[0] > 1 else 0)
    d.b, d.b_rs, d.b_cs, d.b_bs = b3.data_ptr(), b3.stride(1), b3.stride(2), (b3.stride(0) if b3.shape[0] > 1 else 0)
    d.c, d.c_rs, d.c_bs = o3.data_ptr(), (o3.stride(1) if m > 1 else n), o3.stride(0) if batch > 1 else 0
    if bias is not None:
        bb = bias.expand(batch, m, n) if bias.dim() == 3 else bias.expand(m, n).unsqueeze(0).expand(batch, m, n)
        d.bias, d.bias_rs, d.bias_cs, d.bias_bs = bias.data_ptr(), bb.stride(1), bb.stride(2), bb.stride(0)
    d.alpha, d.beta, d.force_path = alpha, beta, force_path
    if out2 is not None:
        assert out2.shape == out.shape and out2.stride() == out.stride() and out2.dtype == out.dtype
        d.c2 = out2.data_ptr()
    if aux_op is not None:
        x3 = aux if aux.dim() == 3 else aux.unsqueeze(0)
        assert tuple(x3.shape) == (batch, m, n) and (n <= 1 or x3.stride(2) == 1) and aux.dtype == out.dtype
        d.aux, d.aux_rs, d.aux_bs, d.aux_op = x3.data_ptr(), (x3.stride(1) if m > 1 else n), (x3.stride(0) if batch > 1 else 0), AUX[aux_op]
    return d


def gemm_splits(d: capi.GemmDesc) -> int:
    """K slices the tensor-core path cuts this product into (1 = one launch; more = slices + a finishing pass in which
    the fused forms are free)."""
    n = C.c_int(0)
    capi.call("tvk_gemm_splits", C.byref(d), C.byref(n))
    return n.value


def gemm(a, b, bias=None, alpha=1.0, beta=1.0, act=None, out=None, force_path=0, out2=None, aux=None, aux_op=None):
    batch = max(a.shape[0] if a.dim() == 3 else 1, b.shape[0] if b.dim() == 3 else 1)
    m, n = a.shape[-2], b.shape[-1]
    if out is None:
        shape = (batch, m, n) if (a.dim() == 3 or b.dim() == 3) else (m, n)
        out = torch.empty(shape, dtype=a.dtype, device=a.device)
    d = gemm_desc(a, b, out, bias, alpha, beta, act, force_path, out2, aux, aux_op)
    nbytes = C.c_uint64(0)
    capi.call("tvk_gemm_workspace_size", C.byref(d), C.byref(nbytes))
    ws = _ws(nbytes.value, a.device)
    capi.call("tvk_gemm", C.byref(d), ptr(ws), nbytes.value, stream())
    return out


def scaled_mm(a, b, scale_a, scale_b, out_dtype=torch.bfloat16, bias=None, scale_result=None, out=None):
    """out = cast((a * scale_a) @ (b * scale_b) + bias) for float8 a [m, k] and b [k, n] (any strides; k-contiguous operands are
    read in place by the float8 tensor-core kernel). scale_a: fp32 scalar or [m, 1]; scale_b: fp32 scalar or [1, n]."""
    kinds = {torch.float8_e4m3fn: capi.F8_E4M3, torch.float8_e5m2: capi.F8_E5M2}
    outs = {torch.float32: capi.SCALED_OUT_F32, torch.float16: capi.SCALED_OUT_F16, torch.bfloat16: capi.SCALED_OUT_BF16,
            torch.float8_e4m3fn: capi.SCALED_OUT_E4M3, torch.float8_e5m2: capi.SCALED_OUT_E5M2}
    m, k = a.shape
    n = b.shape[1]
    assert b.shape[0] == k and scale_a.dtype == torch.float32 and scale_b.dtype == torch.float32
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    d = capi.ScaledMmDesc()
    d.a_kind, d.b_kind, d.out_kind = kinds[a.dtype], kinds[b.dtype], outs[out.dtype]
    d.m, d.n, d.k = m, n, k
    d.a, d.a_rs, d.a_cs = a.data_ptr(), a.stride(0), a.stride(1)
    d.b, d.b_rs, d.b_cs = b.data_ptr(), b.stride(0), b.stride(1)
    d.out = out.data_ptr()
    d.scale_a, d.sa_stride = scale_a.data_ptr(), (1 if scale_a.numel() > 1 else 0)
    d.scale_b, d.sb_stride = scale_b.data_ptr(), (1 if scale_b.numel() > 1 else 0)
    if bias is not None:
        d.bias, d.bias_dtype = bias.data_ptr(), dt(bias)
    if scale_result is not None:
        d.scale_result = scale_result.data_ptr()
    nbytes = C.c_uint64(0)
    capi.call("tvk_scaled_mm_workspace_size", C.byref(d), C.byref(nbytes))
    ws = _ws(nbytes.value, a.device)
    capi.call("tvk_scaled_mm", C.byref(d), ptr(ws), nbytes.value, stream())
    return out


def gemm_path(a, b, out, **kw) -> int:
    d = gemm_desc(a, b, out, **kw)
    p = C.c_int(0)
    capi.call("tvk_gemm_path", C.byref(d), C.byref(p))
    return p.value


# ------------------------------------------------------------------------------- elementwise
def unary(op, x, out=None):
    out = torch.empty_like(x) if out is None else out
    capi.call("tvk_unary", UNARY[op], dt(x), ptr(out), ptr(x), x.numel(), stream())
    return out


def binary(op, a, b, alpha=1.0, out=None):
    out = torch.empty_like(a) if out is None else out
    if isinstance(b, torch.Tensor):
        capi.call("tvk_binary", BINARY[op], dt(a), ptr(out), ptr(a), ptr(b), 0.0, alpha, a.numel(), stream())
    else:
        capi.call("tvk_binary", BINARY[op], dt(a), ptr(out), ptr(a), None, float(b), alpha, a.numel(), stream())
    return out


def compare(op, a, b):
    out = torch.empty(a.shape, dtype=torch.bool, device=a.device)
    if isinstance(b, torch.Tensor):
        capi.call("tvk_compare", COMPARE[op], dt(a), ptr(out), ptr(a), ptr(b), 0.0, a.numel(), stream())
    else:
        capi.call("tvk_compare", COMPARE[op], dt(a), ptr(out), ptr(a), None, float(b), a.numel(), stream())
    return out


def ternary(op, a, b, c=None, value=1.0, out=None):
    out = torch.empty_like(a) if out is None else out
    capi.call("tvk_ternary", TERNARY[op], dt(a), ptr(out), ptr(a), ptr(b), ptr(c), value, a.numel(), stream())
    return out


def make_iter(shape, *stride_lists) -> capi.Iter:
    it = capi.Iter()
    it.ndim, it.noperands = len(shape), len(stride_lists)
    for d, s in enumerate(shape):
        it.sizes[d] = s
    for o, st in enumerate(stride_lists):
        for d, s in enumerate(st):
            it.strides[o][d] = s
    return it


def _bstrides(t, shape):
    return t.expand(shape).stride()


def binary_strided(op, a, b, alpha=1.0):
    shape = torch.broadcast_shapes(a.shape, b.shape)
    out = torch.empty(shape, dtype=a.dtype, device=a.device)
    it = make_iter(shape, out.stride(), _bstrides(a, shape), _bstrides(b, shape))
    capi.call("tvk_binary_strided", BINARY[op], dt(a), ptr(out), ptr(a), ptr(b), alpha, C.byref(it), stream())
    return out


def unary_strided(op, x):
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    it = make_iter(x.shape, out.stride(), x.stride())
    capi.call("tvk_unary_strided", UNARY[op], dt(x), ptr(out), ptr(x), C.byref(it), stream())
    return out


def compare_strided(op, a, b):
    shape = torch.broadcast_shapes(a.shape, b.shape)
    out = torch.empty(shape, dtype=torch.bool, device=a.device)
    it = make_iter(shape, out.stride(), _bstrides(a, shape), _bstrides(b, shape))
    capi.call("tvk_compare_strided", COMPARE[op], dt(a), ptr(out), ptr(a), ptr(b), C.byref(it), stream())
    return out


def ternary_strided(op, a, b, c, value=1.0):
    shape = torch.broadcast_shapes(a.shape, b.shape, c.shape)
    out = torch.empty(shape, dtype=a.dtype, device=a.device)
    it = make_iter(shape, out.stride(), _bstrides(a, shape), _bstrides(b, shape), _bstrides(c, shape))
    capi.call("tvk_ternary_strided", TERNARY[op], dt(a), ptr(out), ptr(a), ptr(b), ptr(c), value, C.byref(it), stream())
    return out


def fill(t, value):
    capi.call("tvk_fill", dt(t), ptr(t), float(value), t.numel(), stream())
    return t


def cast(x, dtype):
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    capi.call("tvk_cast", _DT[dtype], ptr(out), dt(x), ptr(x), x.numel(), stream())
    return out


def copy_strided(src, dtype=None):
    """Contiguous copy (optionally cast) of an arbitrarily strided tensor."""
    dtype = dtype or src.dtype
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    it = make_iter(src.shape, out.stride(), src.stride())
    capi.call("tvk_copy_strided", _DT[dtype], ptr(out), dt(src), ptr(src), C.byref(it), stream())
    return out


# ------------------------------------------------------------------------------- reductions
def _split(shape, dim):
    outer = 1
    for s in shape[:dim]:
        outer *= s
    inner = 1
    for s in shape[dim + 1:]:
        inner *= s
    return outer, shape[dim], inner


def reduce(op, x, dim=None, out_dtype=None):
    """x contiguous. dim None reduces everything."""
    assert x.is_contiguous()
    out_dtype = out_dtype or x.dtype
    if dim is None:
        outer, red, inner, oshape = 1, x.numel(), 1, ()
    else:
        dim %= x.dim()
        outer, red, inner = _split(x.shape, dim)
        oshape = x.shape[:dim] + x.shape[dim + 1:]
    out = torch.empty(oshape, dtype=out_dtype, device=x.device)
    nbytes = C.c_uint64(0)
    capi.call("tvk_reduce_workspace_size", outer, red, inner, C.byref(nbytes))
    ws = _ws(nbytes.value, x.device)
    capi.call("tvk_reduce", REDUCE[op], dt(x), _DT[out_dtype], ptr(out), ptr(x), outer, red, inner, ptr(ws), nbytes.value, stream())
    return out


def argreduce(x, dim=None, is_max=True):
    assert x.is_contiguous()
    if dim is None:
        outer, red, inner, oshape = 1, x.numel(), 1, ()
    else:
        dim %= x.dim()
        outer, red, inner = _split(x.shape, dim)
        oshape = x.shape[:dim] + x.shape[dim + 1:]
    out = torch.empty(oshape, dtype=torch.int64, device=x.device)
    nbytes = C.c_uint64(0)
    capi.call("tvk_reduce_workspace_size", outer, red, inner, C.byref(nbytes))
    ws = _ws(nbytes.value, x.device)
    capi.call("tvk_argreduce", int(is_max), dt(x), ptr(out), ptr(x), outer, red, inner, ptr(ws), nbytes.value, stream())
    return out


def topk(x, k, descending=True):
    assert x.is_contiguous()
    n = x.shape[-1]
    lines = x.numel() // n if n else 0
    values = torch.empty(x.shape[:-1] + (k,), dtype=x.dtype, device=x.device)
    indices = torch.empty(x.shape[:-1] + (k,), dtype=torch.int64, device=x.device)
    nbytes = C.c_uint64(0)
    capi.call("tvk_sort_workspace_size", dt(x), lines, n, C.byref(nbytes))
    ws = _ws(nbytes.value, x.device)
    capi.call("tvk_topk", dt(x), ptr(values), ptr(indices), ptr(x), lines, n, k, int(descending), ptr(ws), nbytes.value, stream())
    return values, indices


# ------------------------------------------------------------------------------- row-wise
def softmax(x, log=False, out_dtype=None):
    assert x.is_contiguous()
    out_dtype = out_dtype or x.dtype
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    cols = x.shape[-1]
    capi.call("tvk_softmax_forward", int(log), dt(x), _DT[out_dtype], ptr(out), ptr(x), x.numel() // max(cols, 1), cols, stream())
    return out


def softmax_backward(grad, y, log=False):
    out = torch.empty_like(y)
    cols = y.shape[-1]
    capi.call("tvk_softmax_backward", int(log), dt(y), ptr(out), ptr(grad), ptr(y), y.numel() // max(cols, 1), cols, stream())
    return out


_RED = {"none": 0, "mean": 1, "sum": 2}


def nll_loss_forward(logp, target, weight=None, reduction="mean", ignore_index=-100):
    n, c = logp.shape
    out = torch.empty((n,) if reduction == "none" else (), dtype=logp.dtype, device=logp.device)
    total = torch.empty((), dtype=logp.dtype, device=logp.device)
    capi.call("tvk_nll_loss_forward", dt(logp), ptr(out), ptr(total), ptr(logp), ptr(target), ptr(weight), n, c, _RED[reduction],
              ignore_index, stream())
    return out, total


def nll_loss_backward(grad_out, target, c, weight=None, reduction="mean", ignore_index=-100, total_weight=None):
    n = target.shape[0]
    gin = torch.empty((n, c), dtype=grad_out.dtype, device=grad_out.device)
    capi.call("tvk_nll_loss_backward", dt(grad_out), ptr(gin), ptr(grad_out), ptr(target), ptr(weight), ptr(total_weight), n, c,
              _RED[reduction], ignore_index, stream())
    return gin


def rmsnorm_forward(x, weight=None, eps=None):
    eps = torch.finfo(torch.float32).eps if eps is None else eps
    cols = x.shape[-1]
    rows = x.numel() // cols
    y = torch.empty_like(x)
    rstd = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    capi.call("tvk_rmsnorm_forward", dt(x), ptr(y), ptr(rstd), ptr(x), ptr(weight), rows, cols, float(eps), stream())
    return y, rstd


def rmsnorm_backward(grad_y, x, weight, rstd, need_weight_grad=True):
    cols = x.shape[-1]
    rows = x.numel() // cols
    gx = torch.empty_like(x)
    gw = torch.empty(cols, dtype=x.dtype, device=x.device) if need_weight_grad else None
    nbytes = C.c_uint64(0)
    capi.call("tvk_rmsnorm_backward_workspace_size", rows, cols, C.byref(nbytes))
    ws = _ws(nbytes.value, x.device)
    capi.call("tvk_rmsnorm_backward", dt(x), ptr(gx), ptr(gw), ptr(grad_y), ptr(x), ptr(weight), ptr(rstd), rows, cols, ptr(ws),
              nbytes.value, stream())
    return gx, gw


def layernorm_forward(x, weight=None, bias=None, norm_dims=1, eps=1e-5):
    cols = 1
    for d in x.shape[x.dim() - norm_dims:]:
        cols *= d
    rows = x.numel() // max(cols, 1)
    y = torch.empty_like(x)
    mean = torch.empty(x.shape[:x.dim() - norm_dims], dtype=torch.float32, device=x.device)
    rstd = torch.empty_like(mean)
    capi.call("tvk_layernorm_forward", dt(x), ptr(y), ptr(mean), ptr(rstd), ptr(x), ptr(weight), ptr(bias), rows, cols, float(eps), stream())
    return y, mean, rstd


def layernorm_backward(grad_y, x, weight, mean, rstd, norm_dims=1, need_params=True):
    cols = 1
    for d in x.shape[x.dim() - norm_dims:]:
        cols *= d
    rows = x.numel() // max(cols, 1)
    gx = torch.empty_like(x)
    gw = torch.empty(x.shape[x.dim() - norm_dims:], dtype=x.dtype, device=x.device) if need_params else None
    gb = torch.empty_like(gw) if need_params else None
    nbytes = C.c_uint64(0)
    capi.call("tvk_layernorm_backward_workspace_size", rows, cols, C.byref(nbytes))
    ws = _ws(nbytes.value, x.device)
    capi.call("tvk_layernorm_backward", dt(x), ptr(gx), ptr(gw), ptr(gb), ptr(grad_y), ptr(x), ptr(weight), ptr(mean), ptr(rstd), rows, cols,
              ptr(ws), nbytes.value, stream())
    return gx, gw, gb


def groupnorm_forward(x, groups, weight=None, bias=None, eps=1e-5):
    n, c = x.shape[0], x.shape[1]
    hw = x.numel() // max(n * c, 1)
    y = torch.empty_like(x)
    mean = torch.empty((n, groups), dtype=torch.float32, device=x.device)
    rstd = torch.empty_like(mean)
    capi.call("tvk_groupnorm_forward", dt(x), ptr(y), ptr(mean), ptr(rstd), ptr(x), ptr(weight), ptr(bias), n, c, hw, groups, float(eps), stream())
    return y, mean, rstd


def groupnorm_backward(grad_y, x, weight, mean, rstd, groups):
    n, c = x.shape[0], x.shape[1]
    hw = x.numel() // max(n * c, 1)
    gx = torch.empty_like(x)
    gw = torch.empty(c, dtype=x.dtype, device=x.device)
    gb = torch.empty_like(gw)
    capi.call("tvk_groupnorm_backward", dt(x), ptr(gx), ptr(gw), ptr(gb), ptr(grad_y), ptr(x), ptr(weight), ptr(mean), ptr(rstd), n, c, hw, groups,
              stream())
    return gx, gw, gb


def cross_entropy_forward(logits, target, weight=None, reduction="mean", ignore_index=-100):
    n, c = logits.shape
    loss = torch.empty((n,) if reduction == "none" else (), dtype=logits.dtype, device=logits.device)
    total = torch.empty((), dtype=logits.dtype, device=logits.device)
    lse = torch.empty(n, dtype=torch.float32, device=logits.device)
    nbytes = C.c_uint64(0)
    capi.call("tvk_cross_entropy_workspace_size", n, C.byref(nbytes))
    ws = _ws(max(nbytes.value, 8), logits.device)
    capi.call("tvk_cross_entropy_forward", dt(logits), ptr(loss), ptr(total), ptr(lse), ptr(logits), ptr(target), ptr(weight), n, c, _RED[reduction],
              ignore_index, ptr(ws), ws.numel(), stream())
    return loss, total, lse


def cross_entropy_backward(grad_out, logits, lse, target, weight=None, reduction="mean", ignore_index=-100, total_weight=None):
    n, c = logits.shape
    g = torch.empty_like(logits)
    capi.call("tvk_cross_entropy_backward", dt(logits), ptr(g), ptr(grad_out), ptr(logits), ptr(lse), ptr(target), ptr(weight), ptr(total_weight), n, c,
              _RED[reduction], ignore_index, stream())
    return g


SCAN = {"cumsum": capi.SCAN_SUM, "cumprod": capi.SCAN_PROD, "logcumsumexp": capi.SCAN_LOGADDEXP}


def scan(op, x, dim):
    assert x.is_contiguous()
    dim %= x.dim()
    outer, n, inner = _split(x.shape, dim)
    out = torch.empty_like(x)
    capi.call("tvk_scan", SCAN[op], dt(x), ptr(out), ptr(x), outer, n, inner, stream())
    return out


def batchnorm_forward(x, weight, bias, running_mean, running_var, momentum=0.1, eps=1e-5):
    n, c = x.shape[0], x.shape[1]
    hw = x.numel() // max(n * c, 1)
    y = torch.empty_like(x)
    mean = torch.empty(c, dtype=torch.float32, device=x.device)
    invstd = torch.empty(c, dtype=torch.float32, device=x.device)
    nbytes = C.c_uint64(0)
    capi.call("tvk_batchnorm_workspace_size", n, c, hw, C.byref(nbytes))
    ws = _ws(nbytes.value, x.device)
    sdt = dt(running_mean) if running_mean is not None else capi.F32
    if _is_cl(x):       # channels-last storage: [n*hw, c] rows
        capi.call("tvk_batchnorm_cl_workspace_size", n * hw, c, C.byref(nbytes))
        ws = _ws(nbytes.value, x.device)
        capi.call("tvk_batchnorm_forward_cl", dt(x), ptr(y), ptr(mean), ptr(invstd), ptr(x), ptr(weight), ptr(bias), sdt, ptr(running_mean),
                  ptr(running_var), n * hw, c, momentum, eps, ptr(ws), nbytes.value, stream())
        return y, mean, invstd
    capi.call("tvk_batchnorm_forward", dt(x), ptr(y), ptr(mean), ptr(invstd), ptr(x), ptr(weight), ptr(bias), sdt, ptr(running_mean),
              ptr(running_var), n, c, hw, momentum, eps, ptr(ws), nbytes.value, stream())
    return y, mean, invstd


def batchnorm_backward(grad_y, x, weight, mean, invstd):
    n, c = x.shape[0], x.shape[1]
    hw = x.numel() // max(n * c, 1)
    gx = torch.empty_like(x)
    gw = torch.empty(c, dtype=x.dtype, device=x.device)
    gb = torch.empty(c, dtype=x.dtype, device=x.device)
    nbytes = C.c_uint64(0)
    capi.call("tvk_batchnorm_workspace_size", n, c, hw, C.byref(nbytes))
    ws = _ws(nbytes.value, x.device)
    if _is_cl(x):
        assert _is_cl(grad_y)
        capi.call("tvk_batchnorm_cl_workspace_size", n * hw, c, C.byref(nbytes))
        ws = _ws(nbytes.value, x.device)
        capi.call("tvk_batchnorm_backward_cl", dt(x), ptr(gx), ptr(gw), ptr(gb), ptr(grad_y), ptr(x), ptr(weight), ptr(mean), ptr(invstd),
                  n * hw, c, ptr(ws), nbytes.value, stream())
        return gx, gw, gb
    capi.call("tvk_batchnorm_backward", dt(x), ptr(gx), ptr(gw), ptr(gb), ptr(grad_y), ptr(x), ptr(weight), ptr(mean), ptr(invstd), n,
              c, hw, ptr(ws), nbytes.value, stream())
    return gx, gw, gb


def embedding_forward(table, idx):
    out = torch.empty(idx.shape + (table.shape[1],), dtype=table.dtype, device=table.device)
    capi.call("tvk_embedding_forward", dt(table), ptr(out), ptr(table), ptr(idx), idx.numel(), table.shape[0], table.shape[1], stream())
    return out


def embedding_backward(grad, idx, num_rows, padding_idx=-1):
    dim = grad.shape[-1]
    out = torch.empty((num_rows, dim), dtype=grad.dtype, device=grad.device)
    capi.call("tvk_embedding_backward", dt(grad), ptr(out), ptr(grad), ptr(idx), idx.numel(), num_rows, dim, padding_idx, stream())
    return out


# ------------------------------------------------------------------------------- attention
def attention_forward(q, k, v, causal=True, scale=None):
    """q: [B, Hq, L, D], k/v: [B, Hk, S, D], contiguous. Returns (out, lse)."""
    B, Hq, L, D = q.shape
    Hk, S = k.shape[1], k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    out = torch.empty_like(q)
    lse = torch.empty((B, Hq, L), dtype=torch.float32, device=q.device)
    nbytes = C.c_uint64(0)
    capi.call("tvk_attention_workspace_size", dt(q), B, Hq, Hk, L, S, D, 0, C.byref(nbytes))
    ws = _ws(nbytes.value, q.device)
    capi.call("tvk_attention_forward", dt(q), ptr(out), ptr(lse), ptr(q), ptr(k), ptr(v), B, Hq, Hk, L, S, D, scale, int(causal), ptr(ws),
              nbytes.value, stream())
    return out, lse


def attention_backward(dout, q, k, v, out, lse, causal=True, scale=None):
    B, Hq, L, D = q.shape
    Hk, S = k.shape[1], k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    nbytes = C.c_uint64(0)
    capi.call("tvk_attention_workspace_size", dt(q), B, Hq, Hk, L, S, D, 1, C.byref(nbytes))
    ws = _ws(nbytes.value, q.device)
    capi.call("tvk_attention_backward", dt(q), ptr(dq), ptr(dk), ptr(dv), ptr(dout), ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), B, Hq, Hk, L,
              S, D, scale, int(causal), ptr(ws), nbytes.value, stream())
    return dq, dk, dv


# ------------------------------------------------------------------------------- conv2d
def _is_cl(t) -> bool:
    """True for a 4-D tensor stored channels-last (and not also plain-contiguous, e.g. 1x1 spatial)."""
    return t.dim() == 4 and not t.is_contiguous() and t.is_contiguous(memory_format=torch.channels_last)


def conv2d_desc(x_shape, w_shape, dtype, stride=1, padding=0, dilation=1, groups=1, layout=0):
    pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)  # noqa: E731
    (sh, sw), (ph, pw), (dh, dw) = pair(stride), pair(padding), pair(dilation)
    n, cin, h, w = x_shape
    cout, _, kh, kw = w_shape
    return capi.Conv2dDesc(_DT[dtype], n, cin, h, w, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups, layout)


def _conv_out_hw(d):
    return (d.h + 2 * d.pad_h - d.kh) // d.stride_h + 1, (d.w + 2 * d.pad_w - d.kw) // d.stride_w + 1


def _conv_ws(d, mode, device):
    nbytes = C.c_uint64(0)
    capi.call("tvk_conv2d_workspace_size", C.byref(d), mode, C.byref(nbytes))
    return _ws(nbytes.value, device), nbytes.value


def _empty4(shape, like, channels_last):
    return torch.empty(tuple(shape), dtype=like.dtype, device=like.device, memory_format=torch.channels_last if channels_last else torch.contiguous_format)


def conv2d_forward(x, w, stride=1, padding=0, dilation=1, groups=1):
    """x: [n, cin, h, w], w: [cout, cin, kh, kw], fp16/bf16, each plain-contiguous or channels-last. The result is
    channels-last when x is."""
    xcl, wcl = _is_cl(x), _is_cl(w)
    layout = (capi.CONV_X_CHANNELS_LAST | capi.CONV_Y_CHANNELS_LAST if xcl else 0) | (capi.CONV_W_CHANNELS_LAST if wcl else 0)
    d = conv2d_desc(x.shape, w.shape, x.dtype, stride, padding, dilation, groups, layout)
    ws, nb = _conv_ws(d, 0, x.device)
    ho, wo = _conv_out_hw(d)
    y = _empty4((d.n, d.cout, ho, wo), x, xcl)
    capi.call("tvk_conv2d_forward", C.byref(d), ptr(y), ptr(x), ptr(w), ptr(ws), nb, stream())
    return y


def conv2d_backward_input(dy, w, x_shape, stride=1, padding=0, dilation=1, groups=1):
    ycl, wcl = _is_cl(dy), _is_cl(w)
    layout = (capi.CONV_X_CHANNELS_LAST | capi.CONV_Y_CHANNELS_LAST if ycl else 0) | (capi.CONV_W_CHANNELS_LAST if wcl else 0)
    d = conv2d_desc(x_shape, w.shape, dy.dtype, stride, padding, dilation, groups, layout)
    ws, nb = _conv_ws(d, 1, dy.device)
    dx = _empty4(x_shape, dy, ycl)
    capi.call("tvk_conv2d_backward_input", C.byref(d), ptr(dx), ptr(dy), ptr(w), ptr(ws), nb, stream())
    return dx


def conv2d_backward_weight(dy, x, w_shape, stride=1, padding=0, dilation=1, groups=1, channels_last_weight=False):
    layout = (capi.CONV_X_CHANNELS_LAST if _is_cl(x) else 0) | (capi.CONV_Y_CHANNELS_LAST if _is_cl(dy) else 0) | \
             (capi.CONV_W_CHANNELS_LAST if channels_last_weight else 0)
    d = conv2d_desc(x.shape, w_shape, dy.dtype, stride, padding, dilation, groups, layout)
    ws, nb = _conv_ws(d, 2, dy.device)
    dw = _empty4(w_shape, dy, channels_last_weight)
    capi.call("tvk_conv2d_backward_weight", C.byref(d), ptr(dw), ptr(dy), ptr(x), ptr(ws), nb, stream())
    return dw


def conv2d_backward(dy, x, w, stride=1, padding=0, dilation=1, groups=1, need_dx=True, need_dw=True):
    """Both gradients in one call (an NCHW dy is brought into the kernels' layout once). dx follows x's memory format, dw
    follows w's. Returns (dx, dw); a gradient that was not requested is None."""
    xcl, ycl, wcl = _is_cl(x), _is_cl(dy), _is_cl(w)
    layout = (capi.CONV_X_CHANNELS_LAST if xcl else 0) | (capi.CONV_Y_CHANNELS_LAST if ycl else 0) | (capi.CONV_W_CHANNELS_LAST if wcl else 0)
    d = conv2d_desc(x.shape, w.shape, dy.dtype, stride, padding, dilation, groups, layout)
    ws, nb = _conv_ws(d, 3, dy.device)
    dx = _empty4(x.shape, dy, xcl) if need_dx else None
    dw = _empty4(w.shape, dy, wcl) if need_dw else None
    capi.call("tvk_conv2d_backward", C.byref(d), ptr(dx) if need_dx else None, ptr(dw) if need_dw else None, ptr(dy), ptr(x), ptr(w), ptr(ws), nb, stream())
    return dx, dw


# ------------------------------------------------------------------------------- optimizers
def adam_step(p, g, m, v, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-2, decoupled=True, maximize=False):
    capi.call("tvk_adam_step", dt(p), ptr(p), ptr(g), ptr(m), ptr(v), p.numel(), lr, beta1, beta2, eps, weight_decay, step,
              int(decoupled), int(maximize), stream())


def sgd_step(p, g, buf, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, maximize=False, first_step=False):
    capi.call("tvk_sgd_step", dt(p), ptr(p), ptr(g), ptr(buf), p.numel(), lr, momentum, dampening, weight_decay, int(nesterov),
              int(maximize), int(first_step), stream())

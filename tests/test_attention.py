"""Attention: the numpy oracle against ATen CPU's scaled_dot_product_attention (CPU test), and the
CUDA path against the oracle through the C-ABI (GPU tests). Bar: relative Frobenius error <= 1e-2 for
fp16/bf16 results against the float64 oracle on the same rounded inputs."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from conftest import rel_fro


def _inputs(B, Hq, Hk, L, S, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, L, D, generator=g).to(dtype)
    k = torch.randn(B, Hk, S, D, generator=g).to(dtype)
    v = torch.randn(B, Hk, S, D, generator=g).to(dtype)
    do = torch.randn(B, Hq, L, D, generator=g).to(dtype)
    return q, k, v, do


def f64(t):
    return t.detach().float().cpu().double().numpy()


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("Hq,Hk,L,S", [(4, 2, 16, 16), (8, 2, 12, 20), (2, 2, 20, 12), (2, 2, 7, 7)])
def test_oracle_matches_aten_sdpa(causal, Hq, Hk, L, S):
    q, k, v, do = _inputs(2, Hq, Hk, L, S, 8, torch.float64, 0)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    ref = F.scaled_dot_product_attention(q, k, v, is_causal=causal, enable_gqa=True)
    gq, gk, gv = torch.autograd.grad(ref, (q, k, v), do)
    out, lse, _ = oracle.attention_forward(q.detach().numpy(), k.detach().numpy(), v.detach().numpy(), causal)
    np.testing.assert_allclose(out, ref.detach().numpy(), rtol=1e-10, atol=1e-12)
    dq, dk, dv = oracle.attention_backward(do.numpy(), q.detach().numpy(), k.detach().numpy(), v.detach().numpy(), causal)
    np.testing.assert_allclose(dq, gq.numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(dk, gk.numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(dv, gv.numpy(), rtol=1e-9, atol=1e-11)


def test_oracle_causal_mask_is_top_left_aligned():
    # the reference hides key > row (src/api/ops/attention.cpp:107-112): with L != S query row 0 still sees exactly key 0
    for L, S in ((6, 4), (4, 6)):
        q, k, v, _ = _inputs(1, 2, 1, L, S, 8, torch.float64, 1)
        out, lse, p = oracle.attention_forward(q.numpy(), k.numpy(), v.numpy(), True)
        assert np.all(np.isfinite(lse))
        assert np.all(p[:, :, 0, 1:] == 0) and np.allclose(p[:, :, 0, 0], 1.0)
        vis = np.tril(np.ones((L, S), bool))
        assert np.all(p[0, 0][~vis] == 0) and np.all(p[0, 0][vis] > 0)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,Hq,Hk,L,S,D,causal", [(2, 8, 2, 256, 256, 64, True), (1, 4, 4, 128, 128, 64, False), (3, 6, 2, 40, 72, 32, True),
                                                  (2, 2, 1, 72, 40, 64, True), (1, 8, 2, 264, 264, 128, True),
                                                  # head size 64, <= 256 keys, 128-row groups: the fused forward kernel
                                                  (1, 2, 1, 256, 128, 64, True), (2, 4, 2, 64, 200, 64, False), (1, 4, 1, 32, 8, 64, True),
                                                  (2, 4, 2, 12, 24, 64, True), (2, 4, 2, 24, 16, 64, True), (1, 2, 2, 12, 24, 32, True), (1, 2, 2, 40, 24, 32, True),
                                                  # head size 64, keys a multiple of 128: the fused backward kernel (1 to 4 key blocks, tiles that
                                                  # straddle heads, L < S and L > S under a causal mask)
                                                  (1, 4, 2, 64, 384, 64, False), (2, 4, 2, 64, 384, 64, True), (1, 2, 2, 512, 512, 64, True),
                                                  (1, 2, 1, 384, 256, 64, True)])
def test_gpu_attention_forward_backward(cuda, dtype, B, Hq, Hk, L, S, D, causal):
    from torchvulkan_b200 import cuda_ops as ops

    q, k, v, do = _inputs(B, Hq, Hk, L, S, D, dtype, 2)
    out, lse = ops.attention_forward(q.to(cuda), k.to(cuda), v.to(cuda), causal)
    ro, rl, _ = oracle.attention_forward(f64(q), f64(k), f64(v), causal)
    assert not torch.isnan(out).any()
    assert rel_fro(f64(out), ro) <= 1e-2
    got_l = f64(lse)
    assert np.array_equal(np.isinf(got_l), np.isinf(rl))                     # rows that attend to nothing
    fin = np.isfinite(rl)
    assert np.max(np.abs(got_l[fin] - rl[fin])) <= 2e-2
    assert np.all(f64(out)[~fin] == 0)
    dq, dk, dv = ops.attention_backward(do.to(cuda), q.to(cuda), k.to(cuda), v.to(cuda), out, lse, causal)
    rq, rk, rv = oracle.attention_backward(f64(do), f64(q), f64(k), f64(v), causal)
    assert rel_fro(f64(dq), rq) <= 1e-2 and rel_fro(f64(dk), rk) <= 1e-2 and rel_fro(f64(dv), rv) <= 1e-2
    ops.check_device_status()


@pytest.mark.gpu
def test_gpu_config3_attention_shape(cuda):
    """BASELINE config 3's attention: B=32, 8 query / 2 KV heads, L=S=256, D=64, causal, fp16."""
    from torchvulkan_b200 import cuda_ops as ops

    q, k, v, do = _inputs(32, 8, 2, 256, 256, 64, torch.float16, 3)
    out, lse = ops.attention_forward(q.to(cuda), k.to(cuda), v.to(cuda), True)
    dq, dk, dv = ops.attention_backward(do.to(cuda), q.to(cuda), k.to(cuda), v.to(cuda), out, lse, True)
    sl = slice(0, 32, 11)                                                     # a sample of the batch keeps the float64 oracle quick
    ro, _, _ = oracle.attention_forward(f64(q[sl]), f64(k[sl]), f64(v[sl]), True)
    rq, rk, rv = oracle.attention_backward(f64(do[sl]), f64(q[sl]), f64(k[sl]), f64(v[sl]), True)
    assert rel_fro(f64(out[sl]), ro) <= 1e-2
    assert rel_fro(f64(dq[sl]), rq) <= 1e-2 and rel_fro(f64(dk[sl]), rk) <= 1e-2 and rel_fro(f64(dv[sl]), rv) <= 1e-2
    ops.check_device_status()

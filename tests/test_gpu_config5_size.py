"""BASELINE config 5 (ii) at its own size: fp32 add / exp / sum / argmax over 2^30 elements through the C-ABI.

A 2^30-element fp32 tensor is 4 GiB: byte offsets pass 2^31 half way through it, so an offset kept in a signed 32-bit
integer anywhere in a kernel (or a packet count in a 32-bit loop variable) shows up here and nowhere else. The
reference allows exactly this size on its device (every operand must have numel < 2^31 and a 32-bit element offset,
src/api/ops/helpers.h:169-186). Inputs are generated on the CPU in chunks from a fixed seed and copied up chunk by
chunk; the CPU side keeps what the checks need (an fp64 running sum, the running first maximum, and a few 1 Mi-element
windows), so host memory stays bounded.

Bars: add bit-exact (one IEEE fp32 addition per element), exp within 1e-4 relative (held to 4 ulp), sum within 1e-4
relative of the fp64 CPU sum, argmax / argmin bit-exact with the first-maximum / first-NaN rule of
src/shaders/ops/arg_reduce.slang:49-65.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

N = 1 << 30
CHUNK = 1 << 26
WIN = 1 << 20
# windows kept on the CPU: the first, one that straddles element 2^29 (byte offset 2^31), one above it, and the last
WINDOWS = [0, (1 << 29) - WIN // 2, (1 << 29) + 5 * WIN + 12345, 3 * (1 << 28) + 777, N - WIN]


def ops():
    from torchvulkan_b200 import cuda_ops
    return cuda_ops


def _upload(cuda, seed):
    """N(0,1) fp32 tensor of 2^30 elements on the device + (fp64 sum, first argmax, first argmin, CPU windows)."""
    g = torch.Generator().manual_seed(seed)
    dev = torch.empty(N, dtype=torch.float32, device=cuda)
    total = 0.0
    best_max, best_max_i, best_min, best_min_i = -np.inf, -1, np.inf, -1
    wins = {}
    for c in range(N // CHUNK):
        x = torch.randn(CHUNK, generator=g)
        base = c * CHUNK
        dev[base:base + CHUNK].copy_(x)
        total += float(x.double().sum())
        m, i = x.max(0)
        if float(m) > best_max:                       # strict: an equal value later does not replace the first maximum
            best_max, best_max_i = float(m), base + int((x == m).nonzero()[0])
        m, i = x.min(0)
        if float(m) < best_min:
            best_min, best_min_i = float(m), base + int((x == m).nonzero()[0])
        for w in WINDOWS:
            lo, hi = max(w, base), min(w + WIN, base + CHUNK)
            if lo < hi:
                wins.setdefault(w, []).append(x[lo - base:hi - base].clone())
    wins = {w: torch.cat(parts) for w, parts in wins.items()}
    assert all(v.numel() == WIN for v in wins.values())
    torch.cuda.synchronize()
    return dev, total, best_max_i, best_min_i, wins


@pytest.fixture(scope="module")
def big(cuda):
    free, _ = torch.cuda.mem_get_info()
    if free < 16 << 30:
        pytest.skip("needs 16 GB of free device memory")
    a = _upload(cuda, 5)
    yield a
    del a
    torch.cuda.empty_cache()


def test_sum_2p30_against_fp64(big, cuda):
    a, total, *_ = big
    out = ops().reduce("sum", a)
    got = float(out)
    # 1e-4 relative to the fp64 sum; the sum of 2^30 N(0,1) values has magnitude ~sqrt(N) = 32768, so the scale is floored
    # there (a sum that happens to land near zero must not turn the relative bar into an absolute one of nothing)
    assert abs(got - total) <= 1e-4 * max(abs(total), np.sqrt(N)), (got, total)
    mean = float(ops().reduce("mean", a))
    assert abs(mean - total / N) <= 1e-4 * max(abs(total), np.sqrt(N)) / N
    ops().check_device_status(0)


def test_argmax_argmin_2p30_natural(big, cuda):
    a, _, imax, imin, _ = big
    assert int(ops().argreduce(a, None, True)) == imax
    assert int(ops().argreduce(a, None, False)) == imin
    assert float(ops().reduce("amax", a)) == float(a[imax]) and float(ops().reduce("amin", a)) == float(a[imin])


def test_argmax_2p30_planted_above_the_32bit_byte_offset(big, cuda):
    a, *_ = big
    saved = {}

    def plant(i, v):
        saved.setdefault(i, float(a[i]))
        a[i] = v

    try:
        hi = (1 << 29) + 123457                      # byte offset 2^31 + ...
        plant(hi, 100.0)
        assert int(ops().argreduce(a, None, True)) == hi
        plant(N - 1, 100.0)                          # a tie in the very last element: the first maximum wins
        assert int(ops().argreduce(a, None, True)) == hi
        plant(N - 1, 200.0); plant(N - 3, 200.0)     # a tie pair inside the last 16-byte packet
        assert int(ops().argreduce(a, None, True)) == N - 3
        plant(3 * (1 << 28) + 1, -300.0); plant(N - 2, -300.0)
        assert int(ops().argreduce(a, None, False)) == 3 * (1 << 28) + 1
        plant(N - 2, float("nan"))                   # NaN counts as the extreme of both; the first NaN wins
        assert int(ops().argreduce(a, None, True)) == N - 2 and int(ops().argreduce(a, None, False)) == N - 2
        plant((1 << 29) + 5, float("nan"))
        assert int(ops().argreduce(a, None, True)) == (1 << 29) + 5
        plant(17, float("nan"))
        assert int(ops().argreduce(a, None, True)) == 17
    finally:
        for i, v in saved.items():
            a[i] = v
    ops().check_device_status(0)


def test_exp_2p30_windows(big, cuda):
    a, _, _, _, wins = big
    z = ops().unary("exp", a)
    for w, x in wins.items():
        got = z[w:w + WIN].cpu().double().numpy()
        ref = np.exp(x.double().numpy())
        rel = np.abs(got - ref) / ref
        assert rel.max() <= 1e-4, (w, rel.max())
        ulp = np.abs(got - ref) / np.spacing(ref.astype(np.float32)).astype(np.float64)
        assert ulp.max() <= 4.0, (w, ulp.max())
    del z
    ops().check_device_status(0)


def test_add_2p30_windows_bit_exact(big, cuda):
    a, _, _, _, wins = big
    # the second operand: the same data rotated by a quarter of the tensor (no second 4 GiB generation on the host)
    q = N // 4
    b = torch.empty_like(a)
    b[:N - q].copy_(a[q:]); b[N - q:].copy_(a[:q])
    z = ops().binary("add", a, b)
    for w, x in wins.items():
        j = (w + q) % N
        if j + WIN <= N:
            other = a[j:j + WIN].cpu()
        else:
            other = torch.cat([a[j:].cpu(), a[:WIN - (N - j)].cpu()])
        assert torch.equal(a[w:w + WIN].cpu(), x)                 # the upload itself
        assert torch.equal(z[w:w + WIN].cpu(), x + other), w
    # linearity as a whole-tensor property: sum(a + b) = 2 * sum(a), both through the reduction kernel in fp64 partials
    s_a, s_z = float(ops().reduce("sum", a)), float(ops().reduce("sum", z))
    assert abs(s_z - 2 * s_a) <= 1e-4 * max(abs(2 * s_a), np.sqrt(N))
    del z, b
    ops().check_device_status(0)

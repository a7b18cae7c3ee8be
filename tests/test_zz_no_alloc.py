"""tvk_reduce_noalloc: the reduction entry point for hosts that must not allocate.

A caller that lives inside a memory pool owning the whole device, or whose application forbids
driver allocations once it is running, cannot hand tvk_reduce a freshly allocated workspace. The
no-alloc variant keeps the per-CTA partials in a fixed array inside the library, so only inputs
and outputs are passed. This test calls it through the C-ABI twice in a row (the second call
finds the first call's partials still in the array) and compares with tvk_reduce on the same
inputs; it also checks that an oversized shape is refused. The file sorts behind the operator and
device tests on purpose so that a run stopping at the first failure has already gone through them."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def test_reduce_noalloc_matches_reduce_on_two_consecutive_calls(cuda):
    from torchvulkan_b200 import capi, cuda_ops

    lib = capi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(123)
    cases = [((1 << 22) + 7, 1, (1 << 22) + 7, 1),      # one long line: many CTAs, partials in the scratch
             (5 * 70000, 5, 70000, 1),                   # a few long lines
             (4096 * 64, 1, 4096, 64)]                   # strided lines split over the reduce axis
    for dtype in (torch.float32, torch.float16):
        for numel, outer, red, inner in cases:
            x1 = torch.randn(numel, generator=g).to(dtype).to(cuda)
            x2 = (torch.randn(numel, generator=g) * 3 + 1).to(dtype).to(cuda)   # different data for the second call
            need = C.c_uint64(0)
            capi.call("tvk_reduce_workspace_size", outer, red, inner, C.byref(need))
            assert 0 < need.value <= (128 << 10), "the case should need scratch that fits the built-in array"
            for op in (capi.R_SUM, capi.R_AMAX):
                for x in (x1, x2):                                               # two calls in a row
                    out = torch.full((outer * inner,), float("nan"), dtype=torch.float32, device=cuda)
                    capi.call("tvk_reduce_noalloc", op, cuda_ops.dt(x), capi.F32, out.data_ptr(), x.data_ptr(), outer, red, inner, stream)
                    ws = torch.empty(need.value, dtype=torch.uint8, device=cuda)
                    ref = torch.empty_like(out)
                    capi.call("tvk_reduce", op, cuda_ops.dt(x), capi.F32, ref.data_ptr(), x.data_ptr(), outer, red, inner, ws.data_ptr(),
                              need.value, stream)
                    # same kernels, same launch geometry, same summation order: identical bits
                    assert torch.equal(out, ref), (dtype, op, outer, red, inner)
                    # and against the CPU oracle (float64 on the same rounded inputs), so that the pair cannot be wrong
                    # together: these shapes all go through the partials in the built-in array
                    xin = x.float().cpu().double().numpy().reshape(outer, red, inner)
                    want = oracle.reduce("sum" if op == capi.R_SUM else "amax", xin, 1).reshape(-1)
                    got = out.cpu().double().numpy()
                    if op == capi.R_AMAX:
                        assert np.array_equal(got, want), (dtype, outer, red, inner)
                    else:   # fp32 accumulation: 1e-5 of the size of the sum (floored at the spread of a zero-mean sum)
                        assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 3 * np.sqrt(red))), (dtype, outer, red, inner)
    # a short reduction needs no partials at all and still works
    x = torch.randn(8, 100, generator=g).to(cuda)
    out = torch.empty(8, device=cuda)
    capi.call("tvk_reduce_noalloc", capi.R_SUM, capi.F32, capi.F32, out.data_ptr(), x.data_ptr(), 8, 100, 1, stream)
    assert torch.allclose(out.cpu(), x.cpu().sum(1), rtol=1e-5, atol=1e-5)
    cuda_ops.check_device_status()


def test_reduce_noalloc_rejects_shapes_beyond_the_builtin_scratch(cuda):
    from torchvulkan_b200 import capi

    lib = capi.lib()
    # 4000 columns reduced over 4096 rows: three splits of the reduce axis, 12000 partials (188 KiB)
    outer, red, inner = 1, 4096, 4000
    need = C.c_uint64(0)
    capi.call("tvk_reduce_workspace_size", outer, red, inner, C.byref(need))
    assert need.value > (128 << 10)
    rc = lib.tvk_reduce_noalloc(capi.R_SUM, capi.F32, capi.F32, 1, 1, outer, red, inner, None)   # pointers are never touched
    assert rc == capi.ERR_INVALID
    msg = lib.tvk_last_error().decode()
    assert "built-in scratch" in msg and "tvk_reduce" in msg

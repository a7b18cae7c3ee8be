"""CPU-only checks of the C-ABI library: it loads, exports every declared symbol, validates
arguments, and its caching allocator follows the reference's ladder (cache hit -> device malloc
-> release cache and retry -> OutOfMemory, src/vulkan/allocator.cpp:171-201). The allocator tests
run in a child process with a fake raw allocator so no GPU (and no CUDA call) is involved."""
import ctypes as C
import re
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    from torchvulkan_b200 import capi

    hdr = (ROOT / "include" / "tvk.h").read_text()
    declared = set(re.findall(r"TVK_API\s+[\w\s\*]+?\b(tvk_\w+)\s*\(", hdr))
    assert declared, "no declarations found"
    assert declared == set(capi.SIGNATURES), declared ^ set(capi.SIGNATURES)
    lib = C.CDLL(str(capi.library_path()))
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/tvk.h but not exported"
    assert b"sm_100a" in capi.lib().tvk_version()


def test_header_is_plain_c():
    """The boundary is a C ABI: the header must compile as C (no torch or C++ types in it)."""
    src = '#include "tvk.h"\nint main(void) { tvk_gemm_desc d; (void)d; return (int)sizeof(tvk_iter) == 0; }\n'
    p = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-I", str(ROOT / "include"), "-x", "c", "-"],
                       input=src, text=True, capture_output=True)
    assert p.returncode == 0, p.stderr


def test_size_classes():
    from torchvulkan_b200 import capi

    r = capi.lib().tvk_round_size
    assert r(1) == 256 and r(256) == 256 and r(257) == 320
    assert r(1024) == 1024 and r(1025) == 1280 and r(5 << 20) == 5 << 20
    for s in (300, 1000, 4097, 123456, (1 << 30) + 1):
        q = r(s)
        assert s <= q <= s * 1.25 + 1  # at most a quarter-octave of slack (src/vulkan/cache.cpp:78-87)


def test_argument_validation_without_a_gpu():
    from torchvulkan_b200 import capi

    lib = capi.lib()
    d = capi.GemmDesc()
    d.dtype, d.batch, d.m, d.n, d.k = capi.I64, 1, 4, 4, 4
    n = C.c_uint64()
    assert lib.tvk_gemm_workspace_size(C.byref(d), C.byref(n)) == capi.ERR_INVALID
    assert b"matmul" in lib.tvk_last_error()
    d.dtype, d.m = capi.F16, -1
    assert lib.tvk_gemm(C.byref(d), None, 0, None) == capi.ERR_INVALID
    assert lib.tvk_unary(999, capi.F32, 1, 1, 16, None) == capi.ERR_INVALID
    assert lib.tvk_topk(capi.F32, 1, 1, 1, 1, 4, 9, 1, None, 0, None) == capi.ERR_INVALID   # k > n
    assert lib.tvk_reduce(capi.R_AMAX, capi.F32, capi.F32, 1, 1, 2, 0, 1, None, 0, None) == capi.ERR_INVALID
    # empty problems succeed without touching the device
    assert lib.tvk_unary(capi.U_EXP, capi.F32, None, None, 0, None) == capi.OK
    d = capi.GemmDesc()
    d.dtype, d.batch, d.m, d.n, d.k = capi.F16, 1, 0, 8, 8
    assert lib.tvk_gemm(C.byref(d), None, 0, None) == capi.OK


def test_validation_of_pooling_random_and_logical_calls_without_a_gpu():
    """The argument checks of the pooling, random-fill, dropout and logical entry points run before any launch."""
    from torchvulkan_b200 import capi

    lib = capi.lib()
    ok = capi.Pool2dDesc(capi.F16, 6, 8, 8, 4, 4, 2, 2, 2, 2, 0, 0, 1, 1, 1, 0)
    assert C.sizeof(capi.Pool2dDesc) == 8 + 13 * 8 + 8 + 8            # the struct the header declares (with its padding)
    assert lib.tvk_max_pool2d_forward(C.byref(ok), None, None, None, None) == capi.ERR_INVALID and b"null pointer" in lib.tvk_last_error()
    for field, value, what in (("kh", 0, b"bad kernel"), ("stride_w", 0, b"bad kernel"), ("pad_h", 2, b"half of the kernel"), ("ho", 0, b"bad extent")):
        d = capi.Pool2dDesc(capi.F16, 6, 8, 8, 4, 4, 2, 2, 2, 2, 0, 0, 1, 1, 1, 0)
        setattr(d, field, value)
        assert lib.tvk_max_pool2d_forward(C.byref(d), 1, 1, 1, None) == capi.ERR_INVALID and what in lib.tvk_last_error(), field
    d = capi.Pool2dDesc(capi.F16, 6, 8, 8, 4, 4, 2, 2, 2, 2, 0, 0, 2, 1, 1, 0)
    assert lib.tvk_avg_pool2d_forward(C.byref(d), 1, 1, None) == capi.ERR_INVALID and b"no dilation" in lib.tvk_last_error()
    empty = capi.Pool2dDesc(capi.F16, 0, 8, 8, 4, 4, 2, 2, 2, 2, 0, 0, 1, 1, 1, 0)
    assert lib.tvk_max_pool2d_backward(C.byref(empty), None, None, None, None) == capi.OK      # no planes: nothing to do
    assert lib.tvk_random_fill(7, capi.F32, 1, 16, 0.0, 1.0, 0, 0, None, None) == capi.ERR_INVALID and b"distribution" in lib.tvk_last_error()
    assert lib.tvk_random_fill(0, capi.F32, 1, 16, 2.0, 1.0, 0, 0, None, None) == capi.ERR_INVALID      # from > to
    assert lib.tvk_random_fill(2, capi.F32, 1, 16, 1.5, 0.0, 0, 0, None, None) == capi.ERR_INVALID      # p > 1
    assert lib.tvk_random_fill(1, capi.F32, None, 0, 0.0, 1.0, 0, 0, None, None) == capi.OK
    assert lib.tvk_dropout(capi.F16, 1, 1, 1, 16, 1.5, 0, 0, None, None) == capi.ERR_INVALID and b"keep probability" in lib.tvk_last_error()
    assert lib.tvk_logical(9, 1, 1, 1, 16, None) == capi.ERR_INVALID
    assert lib.tvk_logical(capi.L_AND, 1, 1, None, 16, None) == capi.ERR_INVALID                        # and needs two operands
    assert lib.tvk_logical(capi.L_NOT, None, None, None, 0, None) == capi.OK


CHILD = textwrap.dedent(
    """
    import ctypes as C, sys
    sys.path.insert(0, {root!r})
    from torchvulkan_b200 import capi
    lib = capi.lib()
    live, budget, fail_next = {{}}, [1 << 20], [0]
    calls = {{"alloc": 0, "free": 0}}
    @capi.RAW_ALLOC_FN
    def raw_alloc(pp, n):
        calls["alloc"] += 1
        if fail_next[0] > 0:
            fail_next[0] -= 1
            return 1
        if sum(live.values()) + n > budget[0]:
            return 1
        buf = C.create_string_buffer(16)            # a unique fake address
        addr = C.addressof(buf)
        live[addr] = n; keep.append(buf)
        pp[0] = addr
        return 0
    @capi.RAW_FREE_FN
    def raw_free(p):
        calls["free"] += 1
        del live[p]
        return 0
    keep = []
    assert lib.tvk_debug_set_raw_allocator(raw_alloc, raw_free, 2) == 0
    n = C.c_int(); assert lib.tvk_device_count(C.byref(n)) == 0 and n.value == 2
    st = capi.MemStats()
    def stats(dev=0):
        assert lib.tvk_mem_get_stats(dev, C.byref(st)) == 0
        return st
    p = C.c_void_p(); q = C.c_void_p()
    # malloc -> free -> malloc of the same class is a cache hit
    assert lib.tvk_malloc(0, 1000, C.byref(p)) == 0 and calls["alloc"] == 1
    assert stats().allocated_bytes == 1024 and stats().reserved_bytes == 1024
    first = p.value
    assert lib.tvk_free(0, p) == 0
    assert stats().allocated_bytes == 0 and stats().cached_bytes == 1024 and stats().reserved_bytes == 1024
    assert lib.tvk_malloc(0, 1001, C.byref(p)) == 0 and p.value == first and calls["alloc"] == 1
    assert stats().num_cache_hits == 1 and stats().peak_allocated_bytes == 1024
    # zero bytes -> null, freeing null is fine, freeing a foreign pointer is an error
    assert lib.tvk_malloc(0, 0, C.byref(q)) == 0 and q.value is None
    assert lib.tvk_free(0, None) == 0
    assert lib.tvk_free(0, C.c_void_p(12345)) == capi.ERR_INVALID
    # per-device accounting
    assert lib.tvk_malloc(1, 4096, C.byref(q)) == 0 and stats(1).allocated_bytes == 4096 and stats(0).allocated_bytes == 1024
    assert lib.tvk_free(1, q) == 0
    # release-and-retry: the cache holds 768 KiB, the next request only fits once it is released
    assert lib.tvk_free(0, p) == 0
    assert lib.tvk_malloc(0, 768 << 10, C.byref(p)) == 0 and lib.tvk_free(0, p) == 0
    frees_before = calls["free"]
    assert lib.tvk_malloc(0, 512 << 10, C.byref(p)) == 0
    assert calls["free"] > frees_before and stats().num_oom_retries == 1 and stats().cached_bytes == 0
    # a request that can never fit: OOM status + message, counters unchanged
    before = stats().allocated_bytes
    assert lib.tvk_malloc(0, 8 << 20, C.byref(q)) == capi.ERR_OOM and q.value is None
    assert b"out of memory" in lib.tvk_last_error() and stats().allocated_bytes == before
    # a transient failure of the raw allocator is survived by the retry
    fail_next[0] = 1
    assert lib.tvk_malloc(0, 100, C.byref(q)) == 0 and lib.tvk_free(0, q) == 0
    # peak / reset / empty_cache
    assert stats().peak_allocated_bytes >= 768 << 10
    assert lib.tvk_mem_reset_peak(0) == 0 and stats().peak_allocated_bytes == stats().allocated_bytes
    assert lib.tvk_free(0, p) == 0 and lib.tvk_empty_cache(0) == 0 and stats().reserved_bytes == 0
    assert stats().total_allocated_bytes - stats().total_freed_bytes == 0
    # A graph's private pool: blocks handed out during a capture are parked with the graph when freed, reused inside the
    # capture only, invisible to other allocations and to empty_cache until the graph is destroyed.
    g = C.c_void_p(); a = C.c_void_p(); b = C.c_void_p(); c = C.c_void_p()
    assert lib.tvk_malloc(0, 2000, C.byref(a)) == 0 and lib.tvk_free(0, a) == 0          # one 2 KiB block in the shared cache
    shared = a.value
    assert lib.tvk_graph_begin_capture(0) == 0
    assert lib.tvk_graph_begin_capture(0) == capi.ERR_INVALID                            # one capture per device
    assert lib.tvk_malloc(0, 2000, C.byref(a)) == 0 and a.value == shared                 # a cached block may join the pool
    assert lib.tvk_malloc(0, 3000, C.byref(b)) == 0
    inside = b.value
    assert lib.tvk_free(0, b) == 0                                                       # freed during the capture: parked
    assert lib.tvk_malloc(0, 3000, C.byref(c)) == 0 and c.value == inside                 # ... and reused by the same capture
    assert lib.tvk_free(0, c) == 0
    frees = calls["free"]
    assert lib.tvk_empty_cache(0) == 0 and calls["free"] == frees                        # no-op while capturing
    fail_next[0] = 1
    assert lib.tvk_malloc(0, 5000, C.byref(c)) == capi.ERR_OOM and b"during a graph capture" in lib.tvk_last_error()   # no ladder
    assert lib.tvk_graph_end_capture(0, C.byref(g)) == 0 and g.value
    reserved = stats().reserved_bytes
    assert lib.tvk_malloc(0, 3000, C.byref(c)) == 0 and c.value != inside                 # between replays: not the parked block
    assert lib.tvk_free(0, c) == 0
    assert lib.tvk_free(0, a) == 0                                                       # a pool block freed after the capture: parked too
    assert lib.tvk_malloc(0, 2000, C.byref(c)) == 0 and c.value != shared
    assert lib.tvk_free(0, c) == 0
    frees = calls["free"]
    assert lib.tvk_empty_cache(0) == 0 and calls["free"] > frees                         # frees the shared cache only
    assert stats().reserved_bytes == 2048 + 3072                                         # the two parked blocks stay reserved
    assert lib.tvk_graph_launch(1, g) == capi.ERR_INVALID and lib.tvk_graph_launch(0, g) == 0
    assert lib.tvk_graph_destroy(g) == 0
    assert stats().cached_bytes == 2048 + 3072                                           # back in the shared cache
    assert lib.tvk_malloc(0, 3000, C.byref(c)) == 0 and c.value == inside and lib.tvk_free(0, c) == 0
    assert lib.tvk_empty_cache(0) == 0 and stats().reserved_bytes == 0
    assert lib.tvk_graph_end_capture(0, C.byref(g)) == capi.ERR_INVALID                  # nothing to end
    # RNG bookkeeping: reserve hands out consecutive offsets (src/vulkan/generator.cpp:165-167)
    s = C.c_uint64(); o = C.c_uint64()
    assert lib.tvk_rng_set_seed(0, 42) == 0
    assert lib.tvk_rng_reserve(0, 4, C.byref(s), C.byref(o)) == 0 and (s.value, o.value) == (42, 0)
    assert lib.tvk_rng_reserve(0, 1, C.byref(s), C.byref(o)) == 0 and o.value == 4
    assert lib.tvk_rng_get_state(0, C.byref(s), C.byref(o)) == 0 and o.value == 5
    assert lib.tvk_rng_set_state(0, 7, 100) == 0 and lib.tvk_rng_get_state(0, C.byref(s), C.byref(o)) == 0 and (s.value, o.value) == (7, 100)
    # current device is per thread and validated
    assert lib.tvk_set_device(1) == 0
    d = C.c_int(); assert lib.tvk_get_device(C.byref(d)) == 0 and d.value == 1
    assert lib.tvk_set_device(5) == capi.ERR_INVALID
    import threading
    seen = []
    def other():
        e = C.c_int(); lib.tvk_get_device(C.byref(e)); seen.append(e.value)
    t = threading.Thread(target=other); t.start(); t.join()
    assert seen == [0]
    # fork guard: a child of an initialised parent is refused (src/vulkan/vulkan_context.cpp:119-133)
    import os
    pid = os.fork()
    if pid == 0:
        ok = lib.tvk_is_in_bad_fork() == 1 and lib.tvk_malloc(0, 16, C.byref(q)) == capi.ERR_BAD_FORK
        os._exit(0 if ok else 1)
    _, status = os.waitpid(pid, 0)
    assert os.WEXITSTATUS(status) == 0
    print("ALLOCATOR-OK")
    """
)


def test_caching_allocator_ladder_with_fake_device():
    p = subprocess.run([sys.executable, "-c", CHILD.format(root=str(ROOT))], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "ALLOCATOR-OK" in p.stdout, p.stdout + p.stderr


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from torchvulkan_b200 import capi

    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "_LIB_PATH", tmp_path / "libtvk.so")
    with pytest.raises(ImportError, match="no fallback"):
        capi.lib()


RESIZE_CHILD = textwrap.dedent(
    """
    import ctypes as C, sys
    sys.path.insert(0, {root!r})
    from torchvulkan_b200 import capi
    lib = capi.lib()
    keep = []
    @capi.RAW_ALLOC_FN
    def raw_alloc(pp, n):
        buf = C.create_string_buffer(max(int(n), 16))     # real host bytes stand in for device memory
        keep.append(buf)
        pp[0] = C.addressof(buf)
        return 0
    @capi.RAW_FREE_FN
    def raw_free(p):
        return 0
    assert lib.tvk_debug_set_raw_allocator(raw_alloc, raw_free, 2) == 0
    import torch, torchvulkan
    assert torchvulkan.device_count() == 2
    st = capi.MemStats()
    def allocated(dev):
        assert lib.tvk_mem_get_stats(dev, C.byref(st)) == 0
        return st.allocated_bytes
    t = torch.empty(16, dtype=torch.uint8, device="vulkan:1")
    assert torchvulkan.current_device() == 0 and t.device.index == 1
    a0, a1 = allocated(0), allocated(1)
    t.resize_(100000)                                     # grows the storage while vulkan:0 is the current device
    assert t.numel() == 100000 and t.device.index == 1 and t.untyped_storage().device.index == 1
    assert allocated(0) == a0, "the new block was taken from the current device instead of the storage's"
    assert allocated(1) >= a1 + 100000 - 256
    assert torchvulkan.current_device() == 0
    # an event recorded on one device and waited on from the other goes through tvk_event_wait
    ev = C.c_void_p(64)                                   # no CUDA here: any non-null handle
    assert lib.tvk_event_wait(1, ev) == 0
    assert lib.tvk_event_wait(5, ev) != 0 and lib.tvk_event_wait(1, None) == capi.ERR_INVALID
    print("RESIZE-OK")
    """
)


def test_resize_allocates_on_the_storage_device_with_two_fake_devices():
    """resize_ of a vulkan:1 tensor while vulkan:0 is current must take the new block from device 1 (the hook
    resizePrivateUse1Bytes, src/api/hook.cpp:53-83 in the reference)."""
    out = subprocess.run([sys.executable, "-c", RESIZE_CHILD.format(root=str(ROOT))], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "RESIZE-OK" in out.stdout, out.stdout[-2000:] + out.stderr[-4000:]

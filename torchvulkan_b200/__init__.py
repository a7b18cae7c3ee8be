"""torchvulkan_b200: the torchvulkan Python API over a B200-native runtime.

Importing this package (or its alias ``torchvulkan``) registers PyTorch's PrivateUse1 backend
under the name ``vulkan`` and exposes the same module-level functions as the reference's
``torchvulkan/__init__.py`` (is_available, device_count, synchronize, memory_*, RNG helpers,
``Tensor.vulkan()`` ...), so scripts written against the reference run unchanged. Underneath,
tensors live in CUDA device memory managed by ``lib/libtvk.so`` and every operator on the hot
path is a hand-written sm_100a kernel reached through the C-ABI in ``include/tvk.h``.

The native pieces are required: if ``_C`` or ``libtvk.so`` has not been built
(``python -m torchvulkan_b200.build --aten``) the import of the device API fails; there is no
Python or CPU fallback. The ctypes binding (``torchvulkan_b200.capi``) and the torch.cuda-buffer
helpers (``torchvulkan_b200.cuda_ops``) can be imported on their own without ``_C``.
"""
from __future__ import annotations

import sys as _sys
from collections import namedtuple as _namedtuple

__version__ = "0.1.0"

_C = None
_backend_error = None


def _load_backend():
    """Imports the ATen extension and registers the device module (once)."""
    global _C, _backend_error
    if _C is not None:
        return _C
    import ctypes
    import torch
    from . import capi

    # libtvk.so must be resident before _C (which links against it) is loaded.
    ctypes.CDLL(str(capi.library_path()), mode=ctypes.RTLD_GLOBAL)
    import importlib

    _C = importlib.import_module(__name__ + "._C")
    torch.utils.rename_privateuse1_backend("vulkan")
    torch._register_device_module("vulkan", _sys.modules[__name__])
    try:  # only newer PyTorch versions have this hook
        from torch._functorch._aot_autograd.utils import register_graphsafe_rng_device_type
        register_graphsafe_rng_device_type("vulkan")
    except ImportError:
        pass
    # torch.Tensor already carries `vulkan`/`is_vulkan` for PyTorch's own mobile Vulkan backend:
    # point them at this device, and let torch generate the Module/Storage methods.
    def _to_vulkan(self, device=None, non_blocking=False, **kwargs):
        if isinstance(device, (str, torch.device)) and torch.device(device).type != "vulkan":
            raise RuntimeError("Invalid device, must be vulkan device")
        return self.to(torch.device("vulkan", _index(device)), non_blocking=non_blocking, **kwargs)

    torch.Tensor.vulkan = _to_vulkan
    torch.Tensor.is_vulkan = property(lambda self: self.device.type == "vulkan")
    torch.utils.generate_methods_for_privateuse1_backend(for_tensor=False)
    # The tensor formatter gathers its statistics (min / max of the finite values) on the tensor's device in float64;
    # this device computes in fp32, fp16 and bf16, so printing uses float32 there, as the reference does for devices
    # without fp64 (torchvulkan/__init__.py:208-215).
    import torch._tensor_str as _ts

    _totype = _ts.tensor_totype

    def _vulkan_tensor_totype(t):
        if t.device.type == "vulkan":
            return t.to(dtype=torch.float)
        return _totype(t)

    _ts.tensor_totype = _vulkan_tensor_totype
    _install_pickling(torch)
    return _C


def _install_pickling(torch):
    """Tensors cross process boundaries through the CPU (as the reference's reducer does)."""
    from multiprocessing.reduction import ForkingPickler
    from torch.multiprocessing import reductions

    stock = reductions.reduce_tensor
    if getattr(stock, "_tvk", False):
        return

    def reduce_tensor(t):
        if t.device.type != "vulkan" or (t.requires_grad and not t.is_leaf):
            return stock(t)
        return _rebuild, (t.detach().cpu(), t.device.index, t.requires_grad, isinstance(t, torch.nn.Parameter))

    reduce_tensor._tvk = True
    reductions.reduce_tensor = reduce_tensor
    for cls in (*torch._tensor_classes, torch.Tensor, torch.nn.Parameter):
        ForkingPickler.register(cls, reduce_tensor)


def _rebuild(cpu, index, requires_grad, is_parameter):
    import torch

    t = cpu.to(torch.device("vulkan", index))
    return torch.nn.Parameter(t, requires_grad=requires_grad) if is_parameter else t.requires_grad_(requires_grad)


def _index(dev) -> int:
    import torch

    if isinstance(dev, int):
        return dev
    idx = None if dev is None else torch.device(dev).index
    return current_device() if idx is None else idx


# ----------------------------------------------------------------------------- device API
def is_available() -> bool:
    return _load_backend().is_available()


def device_count() -> int:
    return _load_backend().device_count()


def current_device() -> int:
    return _load_backend().current_device()


def set_device(device) -> None:
    import torch

    i = _index(device)
    if i >= 0:
        torch.accelerator.set_device_index(i)


def is_initialized() -> bool:
    return _load_backend()._is_initialized()


def _lazy_init() -> None:
    _load_backend()._lazy_init()


def device(dev):
    import torch

    idx = dev if isinstance(dev, int) or dev is None else torch.device(dev).index
    return torch.accelerator.device_index(idx)


def synchronize(device=None) -> None:
    _load_backend().synchronize(_index(device))


class Graph:
    """One captured step of device work, replayed with a single call.

    The reference batches a step's operators into one submission itself (deferred op list + hazard DAG); on this
    runtime the device's in-order stream is captured into a CUDA graph. Usage::

        for _ in range(3): train_step()          # warm-up: kernels, workspaces and the allocator's cache settle
        g = torchvulkan.Graph()
        with g.capture():
            train_step()                          # recorded, not run
        for _ in range(n): g.replay()             # every replay is one more train_step()

    The captured step must not wait for the device (no .item(), .cpu(), print of a device tensor) and must not copy
    from host memory: keep its inputs on the device and overwrite them in place between replays (``x.copy_(batch)``
    before the replay). Optimizers must keep their step count on the device (``fused=True``). Tensors created during
    the capture that are still referenced afterwards (the loss, the gradients) are rewritten by every replay.

    Memory: every block the allocator hands out during the capture belongs to the graph. Temporaries that are freed
    are parked with the graph (and reused only inside the same capture), not returned to the shared cache, so work done
    between replays (``x.copy_(batch)`` with a cast, another model, ``empty_cache()``) can never be given, or free,
    memory a replay writes into. ``reset()`` (or deleting the Graph) releases the pool. Tensors that existed before
    the capture (parameters, inputs) must be kept alive by the caller.
    """

    def __init__(self, device=None):
        self._dev = _index(device)
        self._handle = None

    def capture(self):
        import contextlib

        from . import capi

        @contextlib.contextmanager
        def _ctx():
            import ctypes

            _load_backend()
            if self._handle is not None:
                raise RuntimeError("torchvulkan [ERROR]: this Graph already holds a captured step")
            capi.call("tvk_graph_begin_capture", self._dev)
            handle = ctypes.c_void_p()
            try:
                yield self
            except BaseException:
                try:
                    capi.call("tvk_graph_end_capture", self._dev, ctypes.byref(handle))
                    capi.call("tvk_graph_destroy", handle)
                except Exception:
                    pass
                raise
            capi.call("tvk_graph_end_capture", self._dev, ctypes.byref(handle))
            self._handle = handle

        return _ctx()

    def replay(self) -> None:
        from . import capi

        if self._handle is None:
            raise RuntimeError("torchvulkan [ERROR]: Graph.replay() before a successful capture")
        capi.call("tvk_graph_launch", self._dev, self._handle)

    def reset(self) -> None:
        from . import capi

        if self._handle is not None:
            capi.call("tvk_graph_destroy", self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.reset()
        except Exception:
            pass


def current_stream(device=None):
    import torch

    return torch.accelerator.current_stream(torch.device("vulkan", _index(device)))


def default_stream(device=None):
    import torch

    return torch.Stream(stream_id=0, device_index=_index(device), device_type=torch.accelerator.current_stream().device_type)


def set_stream(stream) -> None:
    import torch

    torch.accelerator.set_stream(stream)


def empty_cache() -> None:
    _load_backend().empty_cache()


def memory_allocated(device=None) -> int:
    return _load_backend()._memory_allocated(_index(device))


def max_memory_allocated(device=None) -> int:
    return _load_backend()._max_memory_allocated(_index(device))


def memory_reserved(device=None) -> int:
    return _load_backend()._memory_reserved(_index(device))


def mem_get_info(device=None) -> tuple:
    return _load_backend()._mem_get_info(_index(device))


def reset_peak_memory_stats(device=None) -> None:
    _load_backend()._reset_peak_memory_stats(_index(device))


def memory_stats(device=None) -> dict:
    i = _index(device)
    c = _load_backend()
    cur, peak = c._memory_allocated(i), c._max_memory_allocated(i)
    return {"active_bytes.all.current": cur, "active_bytes.all.peak": peak, "allocated_bytes.all.current": cur,
            "allocated_bytes.all.peak": peak, "reserved_bytes.all.current": c._memory_reserved(i)}


DeviceProperties = _namedtuple("DeviceProperties", ["name", "total_memory", "vendor_id", "device_id", "api_version", "driver_version",
                                                    "subgroup_size", "has_fp64", "has_int64", "has_fp16", "has_bf16", "has_int16",
                                                    "has_int8"])


def get_device_properties(device=None) -> DeviceProperties:
    return DeviceProperties(**_load_backend()._device_properties(_index(device)))


def get_device_name(device=None) -> str:
    return get_device_properties(device).name


# ----------------------------------------------------------------------------- RNG
def _default_generator(dev=None):
    return _load_backend()._default_generator(_index(dev))


_get_generator = _default_generator


def __getattr__(name):
    if name == "default_generators":
        return tuple(_default_generator(i) for i in range(device_count()))
    if name == "_initialized":
        return is_initialized()
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def _u64(seed) -> int:
    seed = int(seed)
    return seed + (1 << 64) if seed < 0 else seed


def manual_seed(seed) -> None:
    _load_backend()._manual_seed(current_device(), _u64(seed))


def manual_seed_all(seed) -> None:
    _load_backend()._manual_seed_all(_u64(seed))


def seed() -> None:
    _default_generator().seed()


def seed_all() -> None:
    s = _default_generator(0).seed()
    for i in range(1, device_count()):
        _default_generator(i).manual_seed(s)


def initial_seed() -> int:
    return _default_generator().initial_seed()


def get_rng_state(device="vulkan"):
    return _default_generator(device).get_state()


def set_rng_state(new_state, device="vulkan") -> None:
    import torch

    _default_generator(device).set_state(new_state.clone(memory_format=torch.contiguous_format))


def get_rng_state_all() -> list:
    return [get_rng_state(i) for i in range(device_count())]


def set_rng_state_all(new_states) -> None:
    for i, s in enumerate(new_states):
        set_rng_state(s, i)


def get_amp_supported_dtype() -> list:
    return _load_backend()._amp_supported_dtypes(current_device())


def is_bf16_supported() -> bool:
    import torch

    return torch.bfloat16 in get_amp_supported_dtype()


def _is_in_bad_fork() -> bool:
    return _load_backend()._is_in_bad_fork()


def enable() -> None:
    """Registers the ``vulkan`` device with PyTorch. ``import torchvulkan`` calls this."""
    _load_backend()

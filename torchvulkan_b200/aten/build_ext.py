"""Builds the ATen PrivateUse1 extension (`torchvulkan_b200/_C*.so`) in-tree with g++.

The extension holds no device code: it registers the `vulkan` device's allocator, guard, hooks
and operator kernels with PyTorch and calls `lib/libtvk.so` (the C-ABI) for everything else.
Objects are rebuilt only when their source or a header changed.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
PKG = HERE.parent
OBJ = PKG / "build" / "aten"


def target() -> Path:
    return PKG / ("_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(verbose: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(parents=True, exist_ok=True)
    sources = sorted(HERE.glob("*.cpp"))
    headers = list(HERE.glob("*.h")) + list((PKG.parent / "include").glob("*.h"))
    newest_header = max(h.stat().st_mtime for h in headers)
    includes = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    cuda_home = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    includes.append(f"-I{cuda_home}/include")      # nvtx3 (header-only) for TORCHVULKAN_PROFILE ranges
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function", "-Wno-unknown-pragmas",
             f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H"]

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, newest_header):
            return obj
        cmd = ["g++", *flags, *includes, "-c", str(src), "-o", str(obj)]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"g++ failed for {src.name}:\n{p.stderr[-6000:]}")
        if verbose and p.stderr:
            print(p.stderr)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources))
    out = target()
    if not out.exists() or any(o.stat().st_mtime > out.stat().st_mtime for o in objs):
        torch_lib = Path(torch.__file__).resolve().parent / "lib"
        cmd = ["g++", "-shared", "-o", str(out), *map(str, objs), f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python",
               f"-L{PKG / 'lib'}", "-ltvk", "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{torch_lib}"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"link of {out.name} failed:\n{p.stderr[-4000:]}")
    return out


if __name__ == "__main__":
    print(build(verbose=True))

"""In-tree build of the two native pieces of the package.

1. ``libwush_int4_b200.so`` -- every ``csrc/*.cu`` compiled by nvcc for sm_100a only
   (``-gencode arch=compute_100a,code=sm_100a``); exports the C ABI of
   ``include/wush_int4.h`` and depends on nothing but the CUDA runtime.
2. ``_C.<abi>.so`` -- the torch-facing pybind11 module (``csrc/bindings.cpp``) compiled by
   g++ against torch's headers and linked to (1) with an ``$ORIGIN`` rpath.

Both land next to this file so that they travel with the source tree.  nvcc cross-compiles
without a GPU.  ``python -m wush_int4_kernel_b200.build`` builds both.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libwush_int4_b200.so")
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
BINDING = os.path.join(PKG, "_C" + EXT_SUFFIX)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--threads", "4",
]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def build_library(force: bool = False, verbose: bool = False) -> str:
    """One object per ``.cu`` (kept under ``csrc/build/``, rebuilt only when its source or a shared
    header changed), then one link.  No translation unit refers to another's device symbols, so
    no relocatable device code is needed."""
    from concurrent.futures import ThreadPoolExecutor

    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(PKG, "..", "include", "wush_int4.h")]
    if not force and _newer(LIB, sources + headers):
        return LIB
    objdir = os.path.join(CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    nvcc = nvcc_path()
    flags = [f for f in NVCC_FLAGS if f not in ("--threads", "4")]
    jobs = []
    objects = []
    for src in sources:
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if force or not _newer(obj, [src] + headers):
            cmd = [nvcc, *flags, "-c", src, "-o", obj]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        list(pool.map(_run, jobs))
    _run([nvcc, *flags, "-shared", "-o", LIB, *objects])
    return LIB


def build_binding(force: bool = False) -> str:
    src = os.path.join(CSRC, "bindings.cpp")
    if not force and _newer(BINDING, [src, LIB, os.path.join(PKG, "..", "include", "wush_int4.h")]):
        return BINDING
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cmd = [
        cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wno-attributes",
        f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
        *inc, src, "-o", BINDING,
        f"-L{PKG}", "-lwush_int4_b200", f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
        "-ltorch", "-ltorch_python", "-Wl,-rpath,$ORIGIN",
    ]
    _run(cmd)
    return BINDING


def build_all(force: bool = False) -> None:
    build_library(force)
    build_binding(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print(LIB)
    print(BINDING)

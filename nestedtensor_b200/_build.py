"""In-tree build of the native libraries (sm_100a only).

  lib/libntb200.so        the C-ABI kernel library (no torch dependency)   <- csrc/*.cu
  lib/ntb200_dispatch.so  the torch operator layer that calls it           <- csrc/dispatch.cpp

Both are rebuilt only when a source is newer than the library.  Run as
``python -m nestedtensor_b200._build`` or through ``__graft_entry__.build()``.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT_DIR = os.path.dirname(PKG_DIR)
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
INCLUDE_DIR = os.path.join(ROOT_DIR, "include")
CABI_LIB = os.path.join(LIB_DIR, "libntb200.so")
DISPATCH_LIB = os.path.join(LIB_DIR, "ntb200_dispatch.so")

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _stale(target: str, sources) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print("[ntb200 build]", " ".join(cmd), flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + proc.stdout)
    if verbose and proc.stdout.strip():
        print(proc.stdout)


def build_cabi(force: bool = False, verbose: bool = False) -> str:
    """Compile every csrc/*.cu into lib/libntb200.so (one object per file, then link)."""
    os.makedirs(LIB_DIR, exist_ok=True)
    cus = sorted(glob.glob(os.path.join(CSRC_DIR, "*.cu")))
    deps = cus + glob.glob(os.path.join(CSRC_DIR, "*.cuh")) + glob.glob(os.path.join(INCLUDE_DIR, "*.h"))
    if not force and not _stale(CABI_LIB, deps):
        return CABI_LIB
    objdir = os.path.join(PKG_DIR, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    headers = [d for d in deps if not d.endswith(".cu")]
    for cu in cus:
        obj = os.path.join(objdir, os.path.basename(cu)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [cu] + headers):
            _run([_nvcc(), "-O3", "-std=c++17", *NVCC_ARCH, "-lineinfo", "-Xcompiler", "-fPIC",
                  "-Xptxas", "-v" if verbose else "-warn-spills",
                  "-I", INCLUDE_DIR, "-I", CSRC_DIR, "-c", cu, "-o", obj], verbose)
    _run([_nvcc(), "-shared", *NVCC_ARCH, "-o", CABI_LIB, *objs], verbose)
    return CABI_LIB


def build_dispatch(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/dispatch.cpp (TORCH_LIBRARY operator layer) against the installed torch."""
    src = os.path.join(CSRC_DIR, "dispatch.cpp")
    if not os.path.exists(src):
        return ""
    build_cabi(force=False, verbose=verbose)
    deps = [src] + glob.glob(os.path.join(INCLUDE_DIR, "*.h"))
    if not force and not _stale(DISPATCH_LIB, deps):
        return DISPATCH_LIB
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], INCLUDE_DIR, "/usr/local/cuda/include"]:
        inc += ["-I", p]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DNDEBUG",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi, "-DTORCH_EXTENSION_NAME=ntb200_dispatch",
           *inc, src, "-o", DISPATCH_LIB,
           "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           "-L", LIB_DIR, "-lntb200",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    _run(cmd, verbose)
    return DISPATCH_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cabi(force=force, verbose=verbose)
    build_dispatch(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)

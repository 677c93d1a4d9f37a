"""Builds oracle/_ref/libntref_cuda.so: the REFERENCE's own CUDA padding kernels and attention helper kernels
(masked softmax, bias add + pad, transpose + remove padding), compiled for sm_100a from the reference's source files
where they lie (never copied), behind the C names of oracle/ref_cuda_shim.cu.

    python oracle/build_ref.py [path of the reference checkout]

Test infrastructure only.  The output directory is git-ignored; the built library travels with the tree to a GPU
machine, where the reference checkout itself is absent.  Needs nvcc and the c10 headers of the installed torch
(`c10/util/Half.h`); does not run the reference's build system.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT_LIB = os.path.join(OUT_DIR, "libntref_cuda.so")


def build(reference="/root/reference", verbose=False):
    src = os.path.join(reference, "nestedtensor", "csrc", "cuda", "padding.cu")
    src_attn = os.path.join(reference, "nestedtensor", "csrc", "cuda", "attention.cu")
    if not (os.path.exists(src) and os.path.exists(src_attn)):
        return None
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    import torch
    from torch.utils import cpp_extension as ce
    inc = []
    for p in [reference] + ce.include_paths():
        inc += ["-I", p]
    shim = os.path.join(HERE, "ref_cuda_shim.cu")
    if os.path.exists(OUT_LIB) and os.path.getmtime(OUT_LIB) >= max(os.path.getmtime(src), os.path.getmtime(src_attn), os.path.getmtime(shim)):
        return OUT_LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-shared",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI), *inc, src, src_attn, shim, "-o", OUT_LIB]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or proc.returncode != 0:
        print(" ".join(cmd))
        print(proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError("the reference's padding.cu / attention.cu did not compile for sm_100a")
    return OUT_LIB


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), verbose=True))

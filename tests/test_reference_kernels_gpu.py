"""The reference's own CUDA padding kernels (nestedtensor/csrc/cuda/padding.cu, compiled unmodified for sm_100a by
oracle/build_ref.py into oracle/_ref/) against this library and against the CPU oracle, bit for bit, on the shapes
where the reference's 32-bit indexing holds: configurations 1, 3 and a configuration-4-shaped batch, fp32 and fp16.
Skipped where the reference library has not been built (it is built where the reference checkout is present and
travels with the tree)."""
import ctypes
import os

import pytest
import torch

from nestedtensor_b200 import workloads
from oracle import ntref
from _helpers import assert_bit_equal, cabi_pad, cabi_unpad, sizes_of, stream_ptr

pytestmark = pytest.mark.gpu

REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libntref_cuda.so")


@pytest.fixture(scope="module")
def ref_lib():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libntref_cuda.so has not been built (python oracle/build_ref.py)")
    lib = ctypes.CDLL(REF_LIB)
    lib.ntref_add_padding.restype = ctypes.c_int
    lib.ntref_add_padding.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                      ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.ntref_remove_padding.restype = ctypes.c_int
    lib.ntref_remove_padding.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return lib


def _collapse(tensors):
    """What the reference does before its kernel: a regular last dimension of 3-D nested tensors is folded into the
    one before it (nestedtensor/csrc/masking.cpp:573-575)."""
    if tensors[0].dim() == 2 and all(t.size(1) == tensors[0].size(1) for t in tensors):
        return [t.reshape(-1) for t in tensors]
    return tensors


def ref_pad(lib, tensors, padding, device):
    flat = _collapse(tensors)
    sizes = sizes_of(flat)
    B, dim = sizes.shape
    numel = sizes.prod(1)
    offsets = torch.zeros(B, dtype=torch.int64)
    offsets[1:] = numel.cumsum(0)[:-1]
    mx = sizes.max(0).values.tolist()
    assert B * int(torch.tensor(mx).prod()) < 2 ** 31, "beyond the reference's int indexing"
    buf = torch.cat([t.reshape(-1) for t in flat]).to(device)
    d_off = offsets.to(torch.int32).to(device)
    d_sizes = sizes.to(torch.int32).contiguous().to(device)
    out = torch.empty([B] + mx, dtype=buf.dtype, device=device)
    out_sizes = (ctypes.c_int64 * (dim + 1))(*([B] + mx))
    rc = lib.ntref_add_padding(buf.data_ptr(), out.data_ptr(), float(padding), d_off.data_ptr(), d_sizes.data_ptr(), dim, out_sizes, B,
                               0 if buf.dtype == torch.float32 else 1, stream_ptr())
    assert rc == 0, rc
    torch.cuda.synchronize()
    full = sizes_of(tensors).max(0).values.tolist()
    return out.reshape([B] + full)


def _cases():
    g = torch.Generator().manual_seed(404)
    c1 = workloads.config1().tensors()
    c3 = [t for t in workloads.config3(batch=6).tensors()]
    L4 = workloads.lengths_c4(workloads._gen(4), 16).tolist()
    c4 = [torch.randn(l, 768, generator=g) for l in L4]
    odd = [torch.randn(int(a), int(b), generator=g) for a, b in torch.randint(1, 40, (9, 2), generator=g)]
    return {"config1": c1, "config3 (6 images)": c3, "config4-shaped": c4, "ragged 2-D": odd}


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=str)
@pytest.mark.parametrize("name", ["config1", "config3 (6 images)", "config4-shaped", "ragged 2-D"])
def test_pad_matches_the_reference_kernels(native_libs, cuda_device, ref_lib, name, dtype):
    tensors = [t.to(dtype) for t in _cases()[name]]
    for padding in (0.0, -1.0):
        want = ref_pad(ref_lib, tensors, padding, cuda_device)
        assert_bit_equal(want, ntref.to_padded_tensor(tensors, padding), "reference kernel vs CPU oracle")
        assert_bit_equal(cabi_pad(tensors, padding, cuda_device), want.cpu(), "this library vs reference kernel")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=str)
@pytest.mark.parametrize("name", ["config3 (6 images)", "ragged 2-D"])
def test_unpad_matches_the_reference_kernels(native_libs, cuda_device, ref_lib, name, dtype):
    """remove_padding with two and three ragged dimensions (the one-dimensional case of the reference reads sizes it was
    not given and is never run)."""
    tensors = [t.to(dtype) for t in _cases()[name]]
    sizes = sizes_of(tensors)
    B, dim = sizes.shape
    padded = ntref.to_padded_tensor(tensors, 0).to(cuda_device)
    offsets = torch.zeros(B, dtype=torch.int64)
    offsets[1:] = sizes.prod(1).cumsum(0)[:-1]
    d_off = offsets.to(torch.int32).to(cuda_device)
    d_target = sizes.to(torch.int32).contiguous().to(cuda_device)
    d_padded_sizes = torch.tensor(list(padded.shape), dtype=torch.int32, device=cuda_device)
    out = torch.empty(int(sizes.prod(1).sum()), dtype=dtype, device=cuda_device)
    rc = ref_lib.ntref_remove_padding(padded.data_ptr(), out.data_ptr(), d_off.data_ptr(), d_padded_sizes.data_ptr(), d_target.data_ptr(),
                                      dim, B, 0 if dtype == torch.float32 else 1, stream_ptr())
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert_bit_equal(out, torch.cat([t.reshape(-1) for t in tensors]), "reference kernel vs the constituents")
    assert_bit_equal(cabi_unpad(padded, sizes), out.cpu(), "this library vs reference kernel")

"""The reference's own CUDA padding kernels (nestedtensor/csrc/cuda/padding.cu, compiled unmodified for sm_100a by
oracle/build_ref.py into oracle/_ref/) against this library and against the CPU oracle, bit for bit, on the shapes
where the reference's 32-bit indexing holds: configurations 1, 3 and a configuration-4-shaped batch, fp32 and fp16;
and its attention helper kernels (nestedtensor/csrc/cuda/attention.cu: masked softmax, bias add + pad, transpose +
remove padding) against this library's reference-shaped helpers at BERT-base head shapes.
Skipped where the reference library has not been built (it is built where the reference checkout is present and
travels with the tree)."""
import ctypes
import os

import pytest
import torch

from nestedtensor_b200 import workloads
from oracle import ntref
from nestedtensor_b200 import _cabi
from nestedtensor_b200.nested import build_meta
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


# ------------------------------------------------------------------------------------ attention helpers
def _attn_lib(lib):
    if not hasattr(lib, "ntref_softmax"):
        pytest.skip("oracle/_ref/libntref_cuda.so predates the attention helpers (python oracle/build_ref.py)")
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.ntref_softmax.restype = I
    lib.ntref_softmax.argtypes = [P, P, I, I, I, F, I, P]
    lib.ntref_add_qkv_bias_padding.restype = I
    lib.ntref_add_qkv_bias_padding.argtypes = [P] * 9 + [I] * 5 + [P, P, P]
    lib.ntref_transpose_rm_padding.restype = I
    lib.ntref_transpose_rm_padding.argtypes = [P, P, I, I, I, I, I, P, P, P]
    return lib


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.float16, 1e-3)], ids=str)
@pytest.mark.parametrize("B,H,L", [(4, 12, 128), (4, 12, 77), (11, 12, 301), (32, 12, 512), (3, 4, 20), (2, 12, 1024)])
def test_masked_softmax_matches_the_reference_kernel(native_libs, cuda_device, ref_lib, dtype, tol, B, H, L):
    """Every branch of the reference's launcher (odd length with few / many rows, even length, <= 32, many heads x
    batch) against `ntb200_softmax_masked` on the same scores and lengths: the same arithmetic (scale, -10000 on masked
    keys, row sum + 1e-6), so the results agree to the rounding of two exponential implementations."""
    ref = _attn_lib(ref_lib)
    lib = _cabi.load()
    g = torch.Generator().manual_seed(B * 1000 + L)
    lengths = torch.randint(1, L + 1, (B,), generator=g)
    lengths[0] = L
    scores = (torch.randn(B, H, L, L, generator=g) * 3).to(dtype).to(cuda_device)
    valid = torch.arange(L)[None, :] < lengths[:, None]
    mask = (valid[:, :, None] & valid[:, None, :]).to(dtype).to(cuda_device).contiguous()
    theirs = scores.clone()
    assert ref.ntref_softmax(theirs.data_ptr(), mask.data_ptr(), B, H, L, 0.125, 0 if dtype == torch.float32 else 1, stream_ptr()) == 0
    ours = scores.clone()
    meta = build_meta(lengths[:, None].clone(), cuda_device)
    _cabi.check("ntb200_softmax_masked", lib.ntb200_softmax_masked(ours.data_ptr(), meta.data_ptr(), 1, B, H, L, L, 0.125,
                                                                   0 if dtype == torch.float32 else 1, stream_ptr()))
    torch.cuda.synchronize()
    assert bool(torch.isfinite(theirs.float()).all())
    for b, l in enumerate(lengths.tolist()):  # rows of valid queries (the others are never read by the path)
        diff = (ours[b, :, :l].float() - theirs[b, :, :l].float()).abs().max().item()
        assert diff <= tol, (b, l, diff)


def test_bias_pad_and_transpose_match_the_reference_kernels(native_libs, cuda_device, ref_lib):
    """fp32 (all the reference instantiates), 12 heads x 64: q/k/v + bias scattered into padded head-major buffers, and
    the way back, bit for bit."""
    ref = _attn_lib(ref_lib)
    lib = _cabi.load()
    H, d = 12, 64
    E = H * d
    lengths = [40, 1, 33, 17, 64]
    B, T, L = len(lengths), sum(lengths), max(lengths)
    g = torch.Generator().manual_seed(77)
    qkv = torch.randn(T, 3 * E, generator=g).to(cuda_device)
    bias = torch.randn(3 * E, generator=g).to(cuda_device)
    meta = build_meta(torch.tensor([[l, E] for l in lengths]), cuda_device)
    batch_idx = torch.cat([torch.full((l,), b, dtype=torch.int32) for b, l in enumerate(lengths)]).to(cuda_device)
    word_idx = torch.cat([torch.arange(l, dtype=torch.int32) for l in lengths]).to(cuda_device)
    ours = [torch.full((B, H, L, d), 7.0, device=cuda_device) for _ in range(3)]
    theirs = [torch.full((B, H, L, d), 7.0, device=cuda_device) for _ in range(3)]
    _cabi.check("ntb200_add_qkv_bias_pad", lib.ntb200_add_qkv_bias_pad(qkv.data_ptr(), bias.data_ptr(), ours[0].data_ptr(), ours[1].data_ptr(),
                                                                       ours[2].data_ptr(), meta.data_ptr(), B, T, H, d, L, 0, stream_ptr()))
    q, k, v = (qkv[:, i * E:(i + 1) * E].contiguous() for i in range(3))
    bq, bk, bv = (bias[i * E:(i + 1) * E].contiguous() for i in range(3))
    assert ref.ntref_add_qkv_bias_padding(q.data_ptr(), bq.data_ptr(), k.data_ptr(), bk.data_ptr(), v.data_ptr(), bv.data_ptr(),
                                          theirs[0].data_ptr(), theirs[1].data_ptr(), theirs[2].data_ptr(), T, B, L, H, d,
                                          batch_idx.data_ptr(), word_idx.data_ptr(), stream_ptr()) == 0
    torch.cuda.synchronize()
    for i in range(3):
        assert_bit_equal(ours[i], theirs[i], "q/k/v buffer %d" % i)
    back_ours = torch.empty(T, E, device=cuda_device)
    back_theirs = torch.empty(T, E, device=cuda_device)
    _cabi.check("ntb200_transpose_rm_padding", lib.ntb200_transpose_rm_padding(ours[0].data_ptr(), back_ours.data_ptr(), meta.data_ptr(), B, T,
                                                                               H, d, L, 0, stream_ptr()))
    assert ref.ntref_transpose_rm_padding(theirs[0].data_ptr(), back_theirs.data_ptr(), T, B, L, H, d, batch_idx.data_ptr(),
                                          word_idx.data_ptr(), stream_ptr()) == 0
    torch.cuda.synchronize()
    assert_bit_equal(back_ours, back_theirs, "transpose_rm_padding")
    assert_bit_equal(back_ours, (qkv[:, :E] + bias[:E]).contiguous(), "transpose_rm_padding against q + bias")


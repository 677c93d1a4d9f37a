"""Construction of the packed buffer on the GPU (pointer-array gather) and the packed embedding lookup:
bit-exact against concatenation / the oracle."""
import ctypes

import pytest
import torch

import nestedtensor_b200 as nt
from nestedtensor_b200 import _cabi
from nestedtensor_b200.nested import build_meta
from oracle import ntref
from _helpers import assert_bit_equal, random_list, sizes_of, stream_ptr

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.uint8, torch.bool, torch.int16]


def _cabi_pack(srcs, device):
    lib = _cabi.load()
    numel = [t.numel() for t in srcs]
    offs = torch.zeros(len(srcs) + 1, dtype=torch.int64)
    offs[1:] = torch.tensor(numel, dtype=torch.int64).cumsum(0)
    ptrs = torch.tensor([t.data_ptr() for t in srcs], dtype=torch.int64).to(device)
    d_offs = offs.to(device)
    total = int(offs[-1])
    out = torch.empty(total, dtype=srcs[0].dtype, device=device)
    rc = lib.ntb200_pack_pointers(ptrs.data_ptr(), d_offs.data_ptr(), len(srcs), out.data_ptr(), total, srcs[0].element_size(),
                                  stream_ptr())
    _cabi.check("ntb200_pack_pointers", rc)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
def test_cabi_pack_pointers_misaligned_sources_and_empty_entries(native_libs, cuda_device, dtype):
    """Sources are views into one arena starting at every element phase (so most are not 16-byte aligned), with
    empty constituents in between and sizes from 1 element to several tiles."""
    g = torch.Generator().manual_seed(7)
    if dtype == torch.bool:
        arena = torch.randint(0, 2, (600000,), generator=g).to(torch.bool).to(cuda_device)
    elif dtype.is_floating_point:
        arena = torch.randn(600000, generator=g).to(dtype).to(cuda_device)
    else:
        arena = torch.randint(0, 100, (600000,), generator=g).to(dtype).to(cuda_device)
    lens = [1, 0, 3, 17, 0, 0, 4096, 5, 33000, 2, 70001, 0, 9, 131072, 1]
    srcs, pos = [], 0
    for k, n in enumerate(lens):
        pos += k % 5  # shift the phase
        srcs.append(arena[pos:pos + n])
        pos += n
    got = _cabi_pack(srcs, cuda_device)
    assert_bit_equal(got, torch.cat([s.cpu() for s in srcs]), "pack_pointers")


@pytest.mark.parametrize("tdim", [1, 2, 3])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64], ids=str)
def test_nested_tensor_from_cuda_list(native_libs, cuda_device, dtype, tdim):
    g = torch.Generator().manual_seed(tdim)
    tensors = random_list(g, 9, tdim, 1, 33, dtype)
    on_gpu = [t.to(cuda_device) for t in tensors]
    x = nt.nested_tensor(on_gpu, device=cuda_device, dtype=dtype)
    assert_bit_equal(x._buffer, torch.cat([t.reshape(-1) for t in tensors]), "nested_tensor(cuda list)")
    assert torch.equal(x._sizes, sizes_of(tensors))
    assert torch.equal(x._record()[2].cpu(), build_meta(sizes_of(tensors), "cpu"))
    # non-contiguous constituents are compacted first
    y = nt.nested_tensor([t.t() if t.dim() == 2 else t for t in on_gpu], device=cuda_device, dtype=dtype)
    want = torch.cat([(t.t() if t.dim() == 2 else t).reshape(-1) for t in tensors])
    assert_bit_equal(y._buffer, want, "nested_tensor(non-contiguous cuda list)")
    # and the operators accept the result
    assert_bit_equal(x.to_padded_tensor(0), ntref.to_padded_tensor(tensors, 0), "pad after pack")


def test_nested_tensor_from_host_list_uses_pinned_staging(native_libs, cuda_device):
    g = torch.Generator().manual_seed(3)
    tensors = [torch.randn(int(l), 48, generator=g) for l in torch.randint(1, 70, (40,), generator=g)]
    x = nt.nested_tensor(tensors, device=cuda_device, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert_bit_equal(x._buffer, torch.cat([t.reshape(-1) for t in tensors]).to(torch.bfloat16), "nested_tensor(host list)")


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32], ids=str)
@pytest.mark.parametrize("dtype,E", [(torch.bfloat16, 1024), (torch.float32, 64), (torch.float32, 7), (torch.float16, 20)], ids=str)
def test_embedding_matches_oracle(native_libs, cuda_device, dtype, E, idx_dtype):
    g = torch.Generator().manual_seed(E)
    V = 1000
    weight = torch.randn(V, E, generator=g).to(dtype)
    idx = [torch.randint(0, V, (int(l),), generator=g).to(idx_dtype) for l in torch.randint(1, 90, (21,), generator=g)]
    x = nt.nested_tensor(idx, device=cuda_device, dtype=idx_dtype)
    w = weight.to(cuda_device)
    got = torch.nn.functional.embedding(x, w)
    assert isinstance(got, nt.NestedTensor)
    assert [tuple(r) for r in got._sizes.tolist()] == [(len(i), E) for i in idx]
    want = ntref.embedding(idx, weight)
    for a, b in zip(got.unbind(), want):
        assert_bit_equal(a, b, "embedding")
    assert _cabi.load().ntb200_device_error_flags() == 0
    # the module form
    emb = torch.nn.Embedding(V, E).to(cuda_device).to(dtype)
    with torch.no_grad():
        emb.weight.copy_(w)
    got2 = emb(x)
    assert_bit_equal(got2._buffer, got._buffer.cpu(), "nn.Embedding")


def test_embedding_out_of_range_index_is_reported_not_trapped(native_libs, cuda_device):
    lib = _cabi.load()
    lib.ntb200_device_error_flags()
    V, E = 10, 8
    w = torch.arange(V * E, dtype=torch.float32, device=cuda_device).reshape(V, E)
    idx = torch.tensor([0, 9, 10, -1, 3], dtype=torch.int64, device=cuda_device)
    out = torch.full((5, E), 7.0, device=cuda_device)
    _cabi.check("ntb200_embedding", lib.ntb200_embedding(w.data_ptr(), idx.data_ptr(), 8, out.data_ptr(), 5, V, E, 4, stream_ptr()))
    flags = lib.ntb200_device_error_flags()
    assert flags == 1 << 16
    assert torch.equal(out[0], w[0]) and torch.equal(out[1], w[9]) and torch.equal(out[4], w[3])
    assert bool((out[2] == 0).all()) and bool((out[3] == 0).all())
    assert lib.ntb200_device_error_flags() == 0


def test_full_size_construction_embedding_and_transposes(native_libs, cuda_device):
    """Size-independent properties at the benchmark sizes: packing 4096 separately allocated (L_i, 1024) bf16
    tensors reproduces their concatenation, the packed embedding equals an index-select, and the ragged transposes
    are inverse to each other."""
    from nestedtensor_b200 import workloads
    L = workloads.lengths_c2(workloads._gen(2), 4096)
    g = torch.Generator(device=cuda_device).manual_seed(1)
    parts = [torch.randn(int(l), 1024, device=cuda_device, generator=g).to(torch.bfloat16) for l in L[:4096]]
    x = nt.nested_tensor(parts, device=cuda_device, dtype=torch.bfloat16)
    for i in (0, 1, 77, 2048, 4095):
        start = int(L[:i].sum()) * 1024
        assert torch.equal(x._buffer[start:start + parts[i].numel()].view(torch.int16), parts[i].reshape(-1).view(torch.int16))
    assert x._buffer.numel() == int(L.sum()) * 1024
    checksum = sum(int(p.view(torch.int16).to(torch.int64).sum()) for p in parts[::64])
    got = 0
    for i in range(0, 4096, 64):
        start = int(L[:i].sum()) * 1024
        got += int(x._buffer[start:start + parts[i].numel()].view(torch.int16).to(torch.int64).sum())
    assert got == checksum
    del parts, x
    torch.cuda.empty_cache()

    c5 = workloads.config5()
    T = int(c5.sizes[:, 0].sum())
    table = torch.randn(30522, 1024, device=cuda_device, generator=g).to(torch.bfloat16)
    idx = torch.randint(0, 30522, (T,), device=cuda_device, generator=g)
    ids = nt.NestedTensor(idx, c5.sizes[:, :1].contiguous())
    emb = torch.nn.functional.embedding(ids, table)
    assert torch.equal(emb._buffer.view(T, 1024).view(torch.int16), table.index_select(0, idx).view(torch.int16))
    assert _cabi.load().ntb200_device_error_flags() == 0

    hw = torch.randint(100, 169, (32, 2), generator=torch.Generator().manual_seed(2))
    isz = torch.cat([torch.full((32, 1), 256), hw], 1).contiguous()
    n = int((isz[:, 0] * isz[:, 1] * isz[:, 2]).sum())
    img = nt.NestedTensor(torch.randn(n, device=cuda_device, generator=g).to(torch.float16), isz)
    nhwc = nt.nn.transpose_nchw_nhwc(img)
    back = nt.nn.transpose_nhwc_nchw(nhwc)
    assert torch.equal(back._buffer.view(torch.int16), img._buffer.view(torch.int16))
    first = img.unbind()[0]
    assert torch.equal(nhwc.unbind()[0], first.permute(1, 2, 0))

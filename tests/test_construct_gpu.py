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


def test_operator_layer_random_sweep(native_libs, cuda_device):
    """150 random batches through the operator layer against the oracle, bit for bit: construction from separately
    allocated device tensors (pointer-table gather), to_tensor_mask with every mask_dim (or the same error as the
    oracle), to_padded_tensor, and both constructors that take a padded tensor back (by padding value, by mask)."""
    for seed in range(150):
        g = torch.Generator().manual_seed(91000 + seed)
        r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
        dtype = [torch.uint8, torch.bfloat16, torch.float16, torch.float32, torch.float64, torch.int64][r(0, 5)]
        tdim = r(1, 3)
        B = [1, 2, r(3, 12), r(13, 80), r(100, 600)][r(0, 4)]
        wide = [r(1, 9), r(1, 70), r(60, 700), r(600, 2400)][r(0, 3)]
        reg = r(1, 9) if tdim >= 2 and r(0, 2) == 0 else None
        outer = [1, 3, 12][r(0, 2)] if B < 100 else r(1, 2)
        tensors = []
        for _ in range(B):
            n_outer = max(0, tdim - 1 - (1 if reg is not None else 0))
            shape = [r(1, outer) for _ in range(n_outer)] + [r(max(1, wide - 7), wide)] + ([reg] if reg is not None else [])
            if tdim == 1:
                shape = [r(max(1, wide - 7), wide)]
            x = torch.randn(shape, generator=g)
            if dtype.is_floating_point:  # no element equals a padding value used below
                tensors.append((x.abs() + 0.01).to(dtype) * torch.where(x < 0, -1, 1).to(dtype))
            else:
                tensors.append(((x * 40).abs() + 1).to(dtype))
        tag = "seed %d %s tdim %d B %d first %s" % (seed, dtype, tdim, B, [tuple(t.shape) for t in tensors[:3]])
        a = nt.nested_tensor([t.to(cuda_device) for t in tensors], device=cuda_device, dtype=dtype)
        assert_bit_equal(a._buffer, torch.cat([t.reshape(-1) for t in tensors]), "construction " + tag)
        for mask_dim in [None] + list(range(1, tdim + 2)):
            try:
                want = ntref.to_tensor_mask(tensors, mask_dim)
            except RuntimeError:
                with pytest.raises(RuntimeError):
                    a.to_tensor_mask(mask_dim=mask_dim)
                continue
            data, mask = a.to_tensor_mask(mask_dim=mask_dim)
            assert mask.dtype == want[1].dtype, (tag, mask_dim)
            assert_bit_equal(data, want[0], "to_tensor_mask data, mask_dim %s, %s" % (mask_dim, tag))
            assert_bit_equal(mask, want[1], "to_tensor_mask mask, mask_dim %s, %s" % (mask_dim, tag))
        padding = -7 if dtype != torch.uint8 else 0
        dense = a.to_padded_tensor(padding=padding)
        assert_bit_equal(dense, ntref.to_padded_tensor(tensors, padding), "to_padded_tensor " + tag)
        back = nt.nested_tensor_from_padded_tensor(dense, padding=padding)
        assert [tuple(t.shape) for t in back.unbind()] == [tuple(t.shape) for t in tensors], tag
        assert_bit_equal(back._buffer, a._buffer.cpu(), "nested_tensor_from_padded_tensor " + tag)
        data, mask = a.to_tensor_mask()
        back = nt.nested_tensor_from_tensor_mask(data, mask)
        assert_bit_equal(back._buffer, a._buffer.cpu(), "nested_tensor_from_tensor_mask " + tag)
    assert _cabi.load().ntb200_device_error_flags() == 0

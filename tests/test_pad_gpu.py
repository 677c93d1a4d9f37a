"""Parity of the CUDA ragged<->dense / mask kernels with the CPU oracle: bit-exact, through the raw
C ABI (ctypes on device pointers) and through the Python operator surface."""
import math

import pytest
import torch

import nestedtensor_b200 as nt
from nestedtensor_b200 import workloads
from oracle import ntref
from nestedtensor_b200 import _cabi
from _helpers import (assert_bit_equal, bits_of, cabi_mask, cabi_pad, cabi_unpad, random_list, sizes_of, stream_ptr)

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.uint8, torch.bool, torch.int16]


def _oracle_pad(tensors, padding):
    if tensors[0].dtype == torch.bool:
        return ntref.to_padded_tensor([t.to(torch.uint8) for t in tensors], padding).to(torch.bool)
    return ntref.to_padded_tensor(tensors, padding)


@pytest.mark.parametrize("dtype", DTYPES, ids=str)
@pytest.mark.parametrize("tdim", [1, 2, 3])
def test_cabi_pad_unpad_small(native_libs, cuda_device, dtype, tdim):
    """5 random tensors with extents 3..30 per dim (test/test_nested_tensor_class.py:754-792), every
    element width, odd extents so that rows start at every 16-byte phase."""
    g = torch.Generator().manual_seed(1010 + tdim)
    tensors = random_list(g, 5, tdim, 3, 30, dtype)
    padding = 1
    want = _oracle_pad(tensors, padding)
    got = cabi_pad(tensors, padding, cuda_device)
    assert_bit_equal(got, want, "pad")
    buf = cabi_unpad(got, sizes_of(tensors))
    assert_bit_equal(buf, torch.cat([t.reshape(-1) for t in tensors]), "unpad")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.uint8], ids=str)
@pytest.mark.parametrize("tdim,regular_last", [(2, 8), (2, 7), (3, 5), (3, 16), (2, 1)])
def test_cabi_pad_regular_last(native_libs, cuda_device, dtype, tdim, regular_last):
    """(L_i, D) style constituents: trailing regular dims are folded into `inner`."""
    g = torch.Generator().manual_seed(7 + tdim + regular_last)
    tensors = random_list(g, 9, tdim, 1, 19, dtype, regular_last=regular_last)
    for padding in (0, -1):
        if dtype == torch.uint8 and padding < 0:
            continue
        want = _oracle_pad(tensors, padding)
        got = cabi_pad(tensors, padding, cuda_device)
        assert_bit_equal(got, want, "pad")
        assert_bit_equal(cabi_unpad(got, sizes_of(tensors)), torch.cat([t.reshape(-1) for t in tensors]), "unpad")


def test_exhaustive_tiny(native_libs, cuda_device):
    """Every combination of lengths 1..5 for 3 sequences and row widths 1..5 (fp32 and bf16):
    covers every alignment residue and vectors that span rows and entries."""
    for dtype in (torch.float32, torch.bfloat16):
        for D in range(1, 6):
            for l0 in range(1, 6):
                for l1 in range(1, 6):
                    for l2 in (1, 3, 5):
                        tensors = [torch.arange(l * D, dtype=torch.float32).reshape(l, D).add(100 * i).to(dtype)
                                   for i, l in enumerate((l0, l1, l2))]
                        want = ntref.to_padded_tensor(tensors, -1)
                        got = cabi_pad(tensors, -1, cuda_device)
                        assert_bit_equal(got, want, "pad D=%d L=%s" % (D, (l0, l1, l2)))
                        back = cabi_unpad(got, sizes_of(tensors))
                        assert_bit_equal(back, torch.cat([t.reshape(-1) for t in tensors]), "unpad")


def test_negative_zero_and_nan_bits(native_libs, cuda_device):
    a = torch.tensor([[-0.0, float("nan")], [1.0, -0.0]])
    b = torch.tensor([[float("inf"), -0.0]])
    got = cabi_pad([a, b], -0.0, cuda_device)
    want = ntref.to_padded_tensor([a, b], -0.0)
    assert_bit_equal(got, want, "special values")


def test_empty_constituents(native_libs, cuda_device):
    tensors = [torch.randn(0, 4), torch.randn(3, 4), torch.randn(0, 4), torch.randn(2, 4), torch.randn(0, 4)]
    got = cabi_pad(tensors, 7, cuda_device)
    want = torch.full((5, 3, 4), 7.0)
    want[1] = tensors[1]
    want[3, :2] = tensors[3]
    assert_bit_equal(got, want, "pad with empty entries")
    back = cabi_unpad(got, sizes_of(tensors))
    assert_bit_equal(back, torch.cat([t.reshape(-1) for t in tensors]), "unpad with empty entries")


@pytest.mark.parametrize("mask_nd", [1, 2, 3])
def test_cabi_mask(native_libs, cuda_device, mask_nd):
    g = torch.Generator().manual_seed(5)
    tensors = random_list(g, 7, 3, 1, 21, torch.float32)
    got = cabi_mask(sizes_of(tensors), mask_nd, cuda_device)
    want = ntref.to_mask(tensors, mask_nd + 1) if mask_nd < 3 else ntref.to_tensor_mask(tensors, 4)[1]
    assert_bit_equal(got, want.to(torch.uint8), "mask")


def test_config1_roundtrip(native_libs, cuda_device):
    """Configuration 1: 64 fp32 (L_i, 256): pad(0) -> mask -> from padded, bit-exact."""
    w = workloads.config1()
    tensors = w.tensors()
    a = nt.nested_tensor(tensors, device=cuda_device, dtype=torch.float32)
    padded = a.to_padded_tensor(padding=0)
    assert_bit_equal(padded, ntref.to_padded_tensor(tensors, 0), "to_padded_tensor")
    data, mask = a.to_tensor_mask(mask_dim=2)
    odata, omask = ntref.to_tensor_mask(tensors, mask_dim=2)
    assert_bit_equal(data, odata, "to_tensor_mask data")
    assert mask.dtype == torch.bool and omask.dtype == torch.bool
    assert_bit_equal(mask, omask, "to_tensor_mask mask")
    back = nt.nested_tensor_from_padded_tensor(padded, padding=0)
    assert back.nested_size() == a.nested_size()
    assert_bit_equal(back._buffer, a._buffer, "nested_tensor_from_padded_tensor")
    back2 = nt.from_padded_tensor(padded, a)
    assert_bit_equal(back2._buffer, a._buffer, "from_padded_tensor")
    # default padding of the API is -1
    assert_bit_equal(a.to_padded_tensor(), ntref.to_padded_tensor(tensors, -1), "padding=-1")

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.uint8, torch.float64], ids=str)
@pytest.mark.parametrize("tdim", [2, 3])
def test_unpad_many_entries_per_tile(native_libs, cuda_device, dtype, tdim):
    """2 and 3 ragged dims with large and tiny constituents interleaved: tiles that start in the middle of a
    large constituent, tiles that span dozens of tiny ones (more than the kernel's per-tile table of
    per-constituent divisors holds), and extents of 1."""
    g = torch.Generator().manual_seed(4242 + tdim)
    big = random_list(g, 4, tdim, 40, 90 if tdim == 2 else 60, dtype)
    tiny = random_list(g, 60, tdim, 1, 5, dtype)
    tensors = tiny[:25] + big[:2] + tiny[25:40] + big[2:] + tiny[40:]
    want = _oracle_pad(tensors, 0)
    got = cabi_pad(tensors, 0, cuda_device)
    assert_bit_equal(got, want, "pad")
    assert_bit_equal(cabi_unpad(got, sizes_of(tensors)), torch.cat([t.reshape(-1) for t in tensors]), "unpad")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.uint8, torch.float64], ids=str)
@pytest.mark.parametrize("tdim,regular_last", [(2, None), (3, None), (3, 3), (2, 5)])
def test_long_rows(native_libs, cuda_device, dtype, tdim, regular_last):
    """2 and 3 ragged dims whose innermost padded rows are a few KB long (images): the warp-per-row kernels.  Odd widths (every source row starts at another phase of a 16-byte vector), widths below
    one vector, an empty constituent, one of a single element, a regular folded trailing dim; pad, data + mask in one
    pass, unpad, and the size scan of the padded result."""
    g = torch.Generator().manual_seed(977 + tdim)
    es = torch.empty(0, dtype=dtype).element_size()
    hi = 3300 // es + 37  # rows of 3.3 KB and more: beyond every threshold of the row kernels
    tensors = random_list(g, 9, tdim, 3, 11, dtype, regular_last)
    for i, t in enumerate(tensors):  # widen the innermost ragged dim
        shape = list(t.shape)
        j = tdim - 1 if regular_last is None else tdim - 2
        shape[j] = [hi, 1, hi - 1, 3, hi // 2 + 1, 17, hi - 16, 2, hi - 5][i]
        x = torch.randn(shape, generator=g)
        tensors[i] = ((x * 40).abs() + 1).to(dtype) if dtype == torch.uint8 else x.to(dtype)
    empty = list(tensors[0].shape)
    empty[0] = 0
    tensors.insert(4, torch.zeros(empty, dtype=dtype))
    pad_value = 0 if dtype == torch.uint8 else 777.0  # a value the data cannot hold
    full = tensors[:4] + tensors[5:]  # the operators (as the reference's) reject empty constituents; the C ABI takes them
    a = nt.nested_tensor(full, device=cuda_device, dtype=dtype)
    want = ntref.to_padded_tensor(full, pad_value)
    padded = a.to_padded_tensor(padding=pad_value)
    assert_bit_equal(padded, want, "to_padded_tensor")
    want_e = torch.cat([want[:4], torch.full_like(want[:1], pad_value), want[4:]])
    padded_e = cabi_pad(tensors, pad_value, cuda_device)
    assert_bit_equal(padded_e, want_e, "ntb200_pad_nd")
    data, mask = a.to_tensor_mask()
    odata, omask = ntref.to_tensor_mask(full)
    assert_bit_equal(data, odata, "to_tensor_mask data")
    assert_bit_equal(mask, omask, "to_tensor_mask mask")
    flat = torch.cat([t.reshape(-1) for t in tensors])
    assert_bit_equal(cabi_unpad(padded_e, sizes_of(tensors)), flat, "ntb200_unpad_nd")
    assert_bit_equal(nt.from_padded_tensor(padded, a)._buffer, flat, "from_padded_tensor")
    # an unaligned view of the dense tensor as the source of the unpad (rows start at every phase)
    shifted = torch.empty(padded_e.numel() + 1, dtype=dtype, device=cuda_device)[1:].view(padded_e.shape)
    shifted.copy_(padded_e)
    assert_bit_equal(cabi_unpad(shifted, sizes_of(tensors)), flat, "ntb200_unpad_nd, unaligned source")
    back = nt.nested_tensor_from_padded_tensor(padded_e, padding=pad_value)
    oback = ntref.from_padded_by_value_fast(want_e, pad_value)
    for got_t, want_t in zip(back.unbind(), oback):
        assert got_t.numel() == want_t.numel() and (want_t.numel() == 0 or tuple(got_t.shape) == tuple(want_t.shape))
    assert_bit_equal(back._buffer, torch.cat([t.reshape(-1) for t in oback]), "nested_tensor_from_padded_tensor")


@pytest.mark.parametrize("seed", range(24))
def test_row_and_vector_walks_random_shapes(native_libs, cuda_device, seed):
    """Random batches around the switch between the vector walk and the warp-per-row kernels (innermost padded rows of
    2 to 3 KB): 2 and 3 ragged dims, four element sizes, optional regular trailing dim, extents of zero in any position,
    one to six constituents; pad, unpad and the size scan through the C ABI against plain torch on the CPU."""
    g = torch.Generator().manual_seed(9000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    dtype = [torch.uint8, torch.bfloat16, torch.float32, torch.float64][r(0, 3)]
    es = torch.empty(0, dtype=dtype).element_size()
    tdim, B = r(2, 3), r(1, 6)
    regular_last = r(2, 6) if r(0, 2) == 0 else None
    width_hi = max(2, (r(1200, 4200) // es) // (regular_last or 1))  # the switch lies between 2 and 3 KB
    tensors = []
    for _ in range(B):
        shape = [r(0, 5) if r(0, 5) == 0 else r(1, 6) for _ in range(tdim - 1)] + [r(0, width_hi) if r(0, 4) == 0 else r(max(1, width_hi - 40), width_hi)]
        if regular_last is not None:
            shape[-1], shape[-2] = regular_last, shape[-1]
        x = torch.randn(shape, generator=g)
        tensors.append(((x * 40).abs() + 1).to(dtype) if dtype == torch.uint8 else x.to(dtype))
    sizes = sizes_of(tensors)
    mx = sizes.max(0).values.tolist()
    pad_value = 0 if dtype == torch.uint8 else 777.0
    want = torch.full([B] + mx, pad_value, dtype=dtype)
    for b, t in enumerate(tensors):
        want[(b,) + tuple(slice(0, n) for n in t.shape)] = t
    if min(mx) == 0:
        return  # nothing to pad: the entry points return at once (covered by the edge-case tests)
    got = cabi_pad(tensors, pad_value, cuda_device)
    assert_bit_equal(got, want, "ntb200_pad_nd %s %s" % (dtype, sizes.tolist()))
    flat = torch.cat([t.reshape(-1) for t in tensors])
    if flat.numel():
        assert_bit_equal(cabi_unpad(got, sizes), flat, "ntb200_unpad_nd %s %s" % (dtype, sizes.tolist()))
    # size scan of the padded tensor: extents of each entry's bounding box of non-padding elements, and their count
    lib = _cabi.load()
    nd = len(mx)
    out = torch.empty(B * (nd + 1), dtype=torch.int64, device=cuda_device)
    kind = 0 if dtype == torch.uint8 else (2 if dtype == torch.bfloat16 else 1)
    rc = lib.ntb200_sizes_from_padded(got.data_ptr(), out.data_ptr(), out.data_ptr() + 8 * B * nd, nd, B, _cabi.host_i64(mx), es, kind,
                                      bits_of(pad_value, dtype), stream_ptr())
    _cabi.check("ntb200_sizes_from_padded", rc)
    torch.cuda.synchronize()
    got_sizes, got_counts = out[:B * nd].view(B, nd).cpu(), out[B * nd:].cpu()
    for b, t in enumerate(tensors):
        assert int(got_counts[b]) == t.numel(), (b, sizes.tolist())
        assert got_sizes[b].tolist() == (list(t.shape) if t.numel() else [0] * nd), (b, sizes.tolist())


def test_copy_kernels_wide_random_sweep(native_libs, cuda_device):
    """300 random batches over everything the dispatch of the copy kernels looks at: six dtypes, 1 to 4 tensor dims
    (at most three ragged after folding), 1 to 400 constituents, innermost rows from a few bytes to 9 KB, extents of
    zero, regular trailing dims, padding values 777, NaN, +0 and -0; pad, unpad and the size scan through the C ABI
    against plain torch on the CPU, bit for bit."""
    lib = _cabi.load()
    for seed in range(300):
        g = torch.Generator().manual_seed(777000 + seed)
        r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
        dtype = [torch.uint8, torch.bfloat16, torch.float16, torch.float32, torch.float64, torch.int32][r(0, 5)]
        es = torch.empty(0, dtype=dtype).element_size()
        tdim = r(1, 4)
        B = [1, 2, 3, r(4, 12), r(13, 60), r(100, 400)][r(0, 5)]
        regular_last = r(1, 9) if (tdim >= 2 and (r(0, 2) == 0 or tdim == 4)) else None
        width_bytes = [r(1, 64), r(64, 1024), r(1024, 4200), r(4200, 9000)][r(0, 3)]
        width_hi = max(1, (width_bytes // es) // (regular_last or 1))
        outer_hi = [1, 2, 6, 20][r(0, 3)] if B < 100 else r(1, 3)
        n_outer = max(0, tdim - 1 - (1 if regular_last is not None else 0))
        while B * outer_hi ** n_outer * width_hi * (regular_last or 1) * es > 64e6 and outer_hi > 1:
            outer_hi -= 1
        tensors = []
        for _ in range(B):
            shape = [(0 if r(0, 9) == 0 else r(1, outer_hi)) for _ in range(n_outer)]
            w = r(0, width_hi) if r(0, 3) == 0 else r(max(1, width_hi - 9), width_hi)
            if r(0, 12) == 0:
                w = 0
            shape = [w] if tdim == 1 else shape + [w] + ([regular_last] if regular_last is not None else [])
            x = torch.randn(shape, generator=g)
            tensors.append(((x * 40).abs() + 1).to(dtype) if dtype in (torch.uint8, torch.int32) else x.to(dtype))
        sizes = sizes_of(tensors)
        mx = sizes.max(0).values.tolist()
        if min(mx) == 0:
            continue
        pad_value = 0 if dtype in (torch.uint8, torch.int32) else [777.0, float("nan"), -0.0, 0.0][r(0, 3)]
        want = torch.full([B] + mx, pad_value, dtype=dtype)
        for b, t in enumerate(tensors):
            want[(b,) + tuple(slice(0, n) for n in t.shape)] = t
        tag = "seed %d %s B=%d max %s padding %s" % (seed, dtype, B, mx, pad_value)
        got = cabi_pad(tensors, pad_value, cuda_device)
        assert_bit_equal(got, want, "ntb200_pad_nd " + tag)
        flat = torch.cat([t.reshape(-1) for t in tensors])
        if flat.numel():
            assert_bit_equal(cabi_unpad(got, sizes), flat, "ntb200_unpad_nd " + tag)
        nd = len(mx)
        if nd > 3:
            continue  # the scan takes at most three dims
        out = torch.empty(B * (nd + 1), dtype=torch.int64, device=cuda_device)
        kind = 0 if dtype in (torch.uint8, torch.int32) else (2 if dtype == torch.bfloat16 else 1)
        rc = lib.ntb200_sizes_from_padded(got.data_ptr(), out.data_ptr(), out.data_ptr() + 8 * B * nd, nd, B, _cabi.host_i64(mx), es, kind,
                                          bits_of(pad_value, dtype), stream_ptr())
        _cabi.check("ntb200_sizes_from_padded", rc)
        torch.cuda.synchronize()
        got_sizes, got_counts = out[:B * nd].view(B, nd).cpu(), out[B * nd:].cpu()
        for b, t in enumerate(tensors):
            if pad_value != pad_value:  # NaN differs from everything: every element of the padded box counts
                assert int(got_counts[b]) == math.prod(mx) and got_sizes[b].tolist() == mx, (tag, b)
                continue
            n_valid = int((t != pad_value).sum()) if t.numel() else 0  # (a value equal to the padding is not counted)
            assert int(got_counts[b]) == n_valid, (tag, b)
            if n_valid == t.numel():
                assert got_sizes[b].tolist() == (list(t.shape) if n_valid else [0] * nd), (tag, b)
    assert lib.ntb200_device_error_flags() == 0


def test_config3_images(native_libs, cuda_device):
    """Configuration 3: 32 fp32 images (3, H_i, W_i): 4-D pad, the un-collapsible 4-D mask, and the
    DETR (B, maxH, maxW) mask = channel 0 of it."""
    w = workloads.config3()
    tensors = w.tensors()
    a = nt.nested_tensor(tensors, device=cuda_device, dtype=torch.float32)
    padded = a.to_padded_tensor(padding=0)
    want = ntref.to_padded_tensor(tensors, 0)
    assert_bit_equal(padded, want, "to_padded_tensor 4-D")
    data, mask = a.to_tensor_mask()
    odata, omask = ntref.to_tensor_mask(tensors)
    assert mask.dtype == omask.dtype == torch.uint8 and mask.dim() == 4
    assert_bit_equal(mask, omask, "4-D mask")
    assert_bit_equal(data, odata, "4-D data")
    with pytest.raises(RuntimeError, match="Mask dimension is too small"):
        a.to_tensor_mask(mask_dim=3)
    back = nt.from_padded_tensor(padded, a)
    assert_bit_equal(back._buffer, a._buffer, "unpad 4-D")
    m3 = nt.to_mask(a, 3)  # leading dims (B, C, maxH)
    assert_bit_equal(m3, ntref.to_mask(tensors, 3), "to_mask(3)")


def test_config2_properties_full_size(native_libs, cuda_device):
    """Configuration 2 at full size (4096 bf16 sequences, 8.6 GB dense): the oracle cannot run it in
    seconds, so check size-independent properties: unpad(pad(x)) == x bit-exactly, the padding region
    holds only the padding value (count and checksum), and a sampled set of rows equals the source."""
    free, _ = torch.cuda.mem_get_info()
    if free < 14 * (1 << 30):
        pytest.skip("needs 14 GB of free device memory")
    w = workloads.config2(with_values=False)
    L = w.sizes[:, 0]
    T = int(L.sum())
    g = torch.Generator(device="cuda").manual_seed(2)
    buf = torch.randn(T * 1024, generator=g, device=cuda_device, dtype=torch.float32).to(torch.bfloat16)
    a = nt.NestedTensor(buf, w.sizes)
    pad_value = 3.0
    padded = a.to_padded_tensor(padding=pad_value)
    assert tuple(padded.shape) == (4096, int(L.max()), 1024)
    back = nt.from_padded_tensor(padded, a)
    assert torch.equal(back._buffer.view(torch.int16), buf.view(torch.int16))
    # padding region: number of elements equal to the padding value >= padded - valid, and the sum of the
    # integer views is the valid checksum plus pad_bits * (number of padding elements)
    n_pad = padded.numel() - buf.numel()
    pad_bits = int(torch.tensor(pad_value, dtype=torch.bfloat16).view(torch.int16))
    chk_valid = int(buf.view(torch.int16).to(torch.int64).sum())
    chk = 0
    for b0 in range(0, 4096, 256):
        chk += int(padded[b0:b0 + 256].view(torch.int16).to(torch.int64).sum())
    assert chk == chk_valid + pad_bits * n_pad
    offs = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(L, 0)])
    for b in (0, 1, 17, 2048, 4095):
        l = int(L[b])
        src = buf[int(offs[b]) * 1024:(int(offs[b]) + l) * 1024].reshape(l, 1024)
        assert torch.equal(padded[b, :l].view(torch.int16), src.view(torch.int16))
        assert bool((padded[b, l:] == pad_value).all())
    del padded, back
    # mask
    m = nt.to_mask(a, 2)
    assert int(m.sum()) == T and bool((m.sum(1).cpu() == L).all())


def test_big_index_path(native_libs, cuda_device):
    """One padded entry above 2^30 elements takes the 64-bit division path of the kernels."""
    free, _ = torch.cuda.mem_get_info()
    if free < 6 * (1 << 30):
        pytest.skip("needs 6 GB of free device memory")
    big = (1 << 30) + 4096 + 3
    x = torch.arange(big, device=cuda_device, dtype=torch.int32).to(torch.uint8)
    y = x[:1000].clone()
    a = nt.NestedTensor(torch.cat([x, y]), torch.tensor([[big], [1000]], dtype=torch.int64))
    padded = a.to_padded_tensor(padding=9)
    assert torch.equal(padded[0], x)
    assert torch.equal(padded[1, :1000], y) and bool((padded[1, 1000:] == 9).all())
    back = nt.from_padded_tensor(padded, a)
    assert torch.equal(back._buffer, a._buffer)

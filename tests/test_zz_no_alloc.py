"""The allocation-free offsets entry point (ntb200_offsets_from_sizes_static) against the regular one.

Some hosts of this library may not allocate device memory once they are running - a server that
reserved one fixed arena at start-up, or a binding from a language runtime that has no device allocator
to offer - so they cannot supply the workspace ntb200_offsets_from_sizes asks for.  The static variant
keeps that scratch inside the library.  This test calls it through the C ABI twice in a row (the second
call reuses the scratch the first one left dirty) and requires bit-identical offsets to the regular
entry point.
"""
import ctypes

import pytest
import torch

from nestedtensor_b200 import _cabi

pytestmark = pytest.mark.gpu


def _regular(lib, d_sizes, B, nd, inner):
    offsets = torch.full((B + 1,), -1, dtype=torch.int64, device=d_sizes.device)
    nbytes = lib.ntb200_offsets_workspace_bytes(B)
    ws = torch.empty(max(nbytes // 8, 1), dtype=torch.int64, device=d_sizes.device)
    rc = lib.ntb200_offsets_from_sizes(d_sizes.data_ptr(), nd, nd, inner, B, offsets.data_ptr(),
                                       ws.data_ptr() if nbytes else None, nbytes,
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _cabi.check("ntb200_offsets_from_sizes", rc)
    return offsets


def _static(lib, d_sizes, B, nd, inner):
    offsets = torch.full((B + 1,), -1, dtype=torch.int64, device=d_sizes.device)
    rc = lib.ntb200_offsets_from_sizes_static(d_sizes.data_ptr(), nd, nd, inner, B, offsets.data_ptr(),
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _cabi.check("ntb200_offsets_from_sizes_static", rc)
    return offsets


def test_static_offsets_match_regular_twice_in_a_row(native_libs, cuda_device):
    lib = _cabi.load()
    assert lib.ntb200_offsets_static_max_batch() == 4096 * 1024
    # two different multi-block problems back to back, then a single-block one
    for seed, B, nd, inner in ((1, 70000, 2, 3), (2, 5000, 1, 1024), (3, 300, 3, 1)):
        g = torch.Generator().manual_seed(seed)
        sizes = torch.randint(0, 12, (B, nd), generator=g)
        d_sizes = sizes.to(cuda_device)
        want = _regular(lib, d_sizes, B, nd, inner)
        got = _static(lib, d_sizes, B, nd, inner)
        torch.cuda.synchronize()
        host = torch.cat([torch.zeros(1, dtype=torch.int64), (sizes.prod(1) * inner).cumsum(0)])
        assert torch.equal(got, want), "static and regular entry points disagree (B=%d)" % B
        assert torch.equal(got.cpu(), host)


def test_static_offsets_rejects_oversized_batch(native_libs, cuda_device):
    lib = _cabi.load()
    too_big = lib.ntb200_offsets_static_max_batch() + 1
    dummy = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    rc = lib.ntb200_offsets_from_sizes_static(dummy.data_ptr(), 1, 1, 1, too_big, dummy.data_ptr(), None)
    assert rc == -8
    assert b"built-in scratch" in lib.ntb200_status_string(rc)

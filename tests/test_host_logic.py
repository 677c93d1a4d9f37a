"""CPU-only checks: the C-ABI library loads and exports what include/ntb200.h declares, the
host-side data model and argument errors behave like the reference's, and there is no CPU fallback."""
import os
import re

import pytest
import torch

import nestedtensor_b200 as nt
from nestedtensor_b200 import _cabi, sharding, workloads

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "ntb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ntb200_[a-z0-9_]+)\s*\(", text)))


def test_cabi_exports_every_declared_symbol(native_libs):
    lib = _cabi.load()
    names = _declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), name
        assert name in _cabi.SIGNATURES, "ctypes prototype missing for " + name
    assert lib.ntb200_version() >= 1000
    assert lib.ntb200_status_string(0) == b"ok"
    assert lib.ntb200_status_string(-3) == b"misaligned pointer"


def test_cabi_rejects_bad_arguments_without_launching(native_libs):
    """Validation happens on the host: these calls touch no device."""
    lib = _cabi.load()
    mx = _cabi.host_i64([4])
    assert lib.ntb200_pad_nd(None, None, None, None, 1, 0, 1, 1, mx, 4, 0, None) == -1   # nd out of range
    assert lib.ntb200_pad_nd(None, None, None, None, 1, 1, 1, 1, mx, 3, 0, None) == -2   # element size
    assert lib.ntb200_pad_nd(None, None, None, None, 1, 1, 0, 1, mx, 4, 0, None) == -1   # inner < 1
    assert lib.ntb200_pad_nd(None, None, None, None, 1, 1, 1, 1, mx, 4, 0, None) == -1   # null pointers
    assert lib.ntb200_pad_nd(None, 8, 16, 16, 1, 1, 1, 1, mx, 4, 0, None) == -3          # misaligned output
    assert lib.ntb200_pad_nd(None, None, None, None, 1, 1, 1, 0, mx, 4, 0, None) == 0    # empty batch: no-op
    assert lib.ntb200_unpad_nd(None, None, None, None, 1, 4, 1, 1, mx, 1, 4, None) == -1
    assert lib.ntb200_offsets_workspace_bytes(10) == 0
    assert lib.ntb200_offsets_workspace_bytes(5000) == 8 * 5


def test_cabi_rejects_bad_arguments_of_the_surrounding_operators(native_libs):
    """The entry points around the core path validate on the host too (no device is touched here)."""
    lib = _cabi.load()
    assert lib.ntb200_layer_norm(None, None, None, 1e-5, None, -1, 8, 0, None) == -1            # negative rows
    assert lib.ntb200_layer_norm(16, 16, None, 1e-5, 16, 1, 8, 0, None) == -1                   # gamma without beta
    assert lib.ntb200_layer_norm(16, None, None, 1e-5, 16, 1, 8, 7, None) == -2                 # dtype
    assert lib.ntb200_layer_norm(None, None, None, 1e-5, None, 0, 8, 0, None) == 0              # no rows: no-op
    assert lib.ntb200_add_bias_gelu(None, None, None, 3, 8, 0, None) == -1                      # null pointers
    assert lib.ntb200_gemm_bias_act(16, 16, None, None, 16, 4, 4, 4, 0, 3, 0, None) == -1       # activation code
    assert lib.ntb200_gemm_bias_act(16, 16, None, None, 16, 4, 4, 4, 9, 0, 0, None) == -2       # dtype
    assert lib.ntb200_pack_pointers(16, 16, 2, 8, 10, 4, None) == -3                            # misaligned output
    assert lib.ntb200_pack_pointers(16, 16, 2, 16, 10, 3, None) == -2                           # element size
    assert lib.ntb200_pack_pointers(None, None, 0, None, 0, 4, None) == 0                       # empty batch
    assert lib.ntb200_embedding(16, 16, 2, 16, 4, 10, 8, 4, None) == -1                         # index width
    assert lib.ntb200_embedding(16, 16, 8, 16, 4, 0, 8, 4, None) == -1                          # empty vocabulary
    assert lib.ntb200_transpose_ragged(16, 16, 16, 2, 8, 1, 10, 4, None) == -1                  # in place
    assert lib.ntb200_transpose_ragged(16, 32, 16, 2, 8, 1, 10, 3, None) == -2                  # element size
    assert lib.ntb200_varlen_cross_attention(16, 4, 16, 64, 16, 64, 16, 16, 16, 1, 4, 1, 64, 4, 1.0, 2, 0, None) == -1  # ldq < E
    assert lib.ntb200_varlen_cross_attention(16, 64, 16, 64, 16, 64, 16, 16, 16, 1, 4, 1, 64, 4, 1.0, 2, 5, None) == -1  # path
    assert lib.ntb200_varlen_cross_attention(16, 64, 16, 64, 16, 64, 16, 16, 16, 0, 0, 1, 64, 0, 1.0, 2, 0, None) == 0  # empty


def test_no_cpu_fallback(native_libs):
    a = nt.nested_tensor([torch.randn(3, 4), torch.randn(5, 4)])
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        a.to_padded_tensor(0)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        a.to_tensor_mask()
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        torch.ops.nestedtensor.to_mask(a, 2)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        nt.nested_tensor_from_padded_tensor(torch.zeros(2, 3))


def test_metadata_surface():
    ts = [torch.randn(3, 4), torch.randn(5, 4), torch.randn(1, 4)]
    a = nt.nested_tensor(ts)
    assert a.size() == (3, None, 4) and a.dim() == 3 and a.nested_dim() == 1 and len(a) == 3
    assert a.nested_size() == (torch.Size([3, 4]), torch.Size([5, 4]), torch.Size([1, 4]))
    assert a.nested_size(1) == (3, 5, 1)
    assert a.nested_stride() == ((4, 1), (4, 1), (4, 1))
    assert a.numel() == 36 and a.dtype == torch.float32 and a.device.type == "cpu"
    assert a.is_contiguous() and not a.requires_grad
    for x, y in zip(a.unbind(), ts):
        assert torch.equal(x, y)
    assert a.unbind()[0].data_ptr() != ts[0].data_ptr()      # pack always copies
    b = nt.nested_tensor([ts[0]])
    assert b.unbind()[0].data_ptr() != ts[0].data_ptr()
    assert nt.as_nested_tensor(a) is a
    e = nt.nested_tensor([])
    assert len(e) == 0 and e.dim() == 1 and e.size() == (0,)
    h = nt.nested_tensor(ts, dtype=torch.float16)
    assert h.dtype == torch.float16


def test_constructor_errors():
    with pytest.raises(RuntimeError, match="does not support autograd"):
        nt.nested_tensor([torch.randn(2)], requires_grad=True)
    with pytest.raises(RuntimeError, match="constiuent of dimension 2 doesn't match another constiuent of dimension 1"):
        nt.nested_tensor([torch.randn(2), torch.randn(2, 2)])
    with pytest.raises(RuntimeError, match="scalar type"):
        nt.nested_tensor([torch.randn(2), torch.zeros(2, dtype=torch.int64)])
    with pytest.raises(RuntimeError, match="Currently only supporting a sequence of Tensors."):
        nt.nested_tensor([1, 2])
    with pytest.raises(RuntimeError, match="Currently do not support NestedTensor entries."):
        nt.nested_tensor([nt.nested_tensor([torch.randn(2)])])


def test_from_mask_argument_errors():
    from golden import reference_cases as rc
    for _, tensor, mask, nested_dim, msg in rc.FROM_TENSOR_MASK_ERRORS:
        with pytest.raises(RuntimeError, match=msg):
            nt.nested_tensor_from_tensor_mask(tensor, mask, nested_dim)
    with pytest.raises(RuntimeError):
        nt.nested_tensor_from_tensor_mask(None, None)
    with pytest.raises(RuntimeError, match="can't be bigger than data tensor dimension"):
        nt.nested_tensor_from_tensor_mask(torch.zeros(2), torch.ones(2, dtype=torch.bool), nested_dim=2)


def test_unsupported_function_is_loud():
    a = nt.nested_tensor([torch.randn(3), torch.randn(2)])
    with pytest.raises(NotImplementedError):
        torch.nn.functional.relu(a)


def test_token_balanced_partition():
    L = workloads.lengths_c5(workloads._gen(5)).tolist()
    for world in (1, 2, 4, 8):
        parts = sharding.token_balanced_partition(L, world)
        assert parts[0][0] == 0 and parts[-1][1] == len(L)
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        assert sharding.imbalance(L, parts) < 1.02
    parts = sharding.token_balanced_partition([5, 5], 4)
    assert parts[0][0] == 0 and parts[-1][1] == 2 and all(a <= b for a, b in parts)
    assert sharding.token_balanced_partition([], 2) == [(0, 0), (0, 0)]


def test_workloads_are_deterministic():
    a, b = workloads.config1(), workloads.config1()
    assert torch.equal(a.sizes, b.sizes) and torch.equal(a.buffer, b.buffer)
    c2 = workloads.config2(with_values=False)
    L = c2.sizes[:, 0]
    assert c2.batch == 4096 and int(L.min()) >= 1 and int(L.max()) <= 1024
    c5 = workloads.config5()
    assert c5.batch == 1024 and c5.weights["in_proj_weight"].shape == (3072, 1024) and c5.dtype == torch.bfloat16
    s = c5.slice(10, 20)
    assert s.batch == 10 and s.buffer.numel() == int(c5.sizes[10:20].prod(1).sum())


def test_host_pipeline_range_plan():
    """Ranges are contiguous, non-empty, cover the batch in order and never outnumber the sequences."""
    from nestedtensor_b200.host_pipeline import plan_ranges
    w = [5, 1, 1, 1, 8, 2, 2, 40, 1, 1]
    for n in (1, 2, 3, 8, 50):
        parts = plan_ranges(w, n)
        assert parts[0][0] == 0 and parts[-1][1] == len(w)
        assert all(b > a for a, b in parts)
        assert all(parts[i][1] == parts[i + 1][0] for i in range(len(parts) - 1))
        assert len(parts) <= min(n, len(w))
    assert plan_ranges([3], 8) == [(0, 1)]


def test_host_pipeline_rejects_pageable_memory_before_touching_the_gpu():
    import nestedtensor_b200 as nt
    sizes = torch.tensor([[2, 4], [3, 4]], dtype=torch.int64)
    with pytest.raises(ValueError, match="pinned"):
        nt.to_padded_tensor_host(torch.zeros(20), sizes, 0)
    with pytest.raises(ValueError, match="pinned"):
        nt.from_padded_tensor_host(torch.zeros(2, 3, 4), sizes)


def test_merge_tensor_mask_operator_matches_the_oracle(native_libs):
    """torch.ops.nestedtensor.merge_tensor_mask (nestedtensor/csrc/masking.cpp:12-43) is a plain-tensor operator: the
    reference's own cases (test/test_nested_tensor_masking.py: all-true, all-false, mixed and ragged masks, with and
    without a target mask_dim) against the CPU restatement."""
    from oracle import ntref
    op = torch.ops.nestedtensor.merge_tensor_mask
    t = torch.arange(24.0).reshape(2, 3, 4)
    ragged = torch.tensor([[[1, 1, 0, 0], [1, 1, 0, 0], [0, 0, 0, 0]], [[1, 1, 1, 1], [1, 1, 1, 1], [1, 1, 1, 1]]], dtype=torch.uint8)
    rows = torch.tensor([[[1, 1, 1, 1], [1, 1, 1, 1], [0, 0, 0, 0]], [[1, 1, 1, 1], [0, 0, 0, 0], [0, 0, 0, 0]]], dtype=torch.uint8)
    for mask in (torch.ones(2, 3, 4, dtype=torch.uint8), torch.zeros(2, 3, 4, dtype=torch.uint8), ragged, rows):
        for md in (None, 1, 2, 3):
            try:
                want = ntref.merge_tensor_mask(t, mask, md)
            except RuntimeError as e:
                with pytest.raises(RuntimeError, match="Mask dimension is too small"):
                    op(t, mask, md)
                assert "too small" in str(e)
                continue
            got = op(t, mask, md)
            assert torch.equal(got[0], want[0])
            assert got[1].dtype == want[1].dtype and torch.equal(got[1], want[1]), (md, got[1], want[1])
    assert nt.merge_tensor_mask(t, rows)[1].shape == (2, 3)


def test_device_error_flags_wrapper_needs_a_device(native_libs):
    assert callable(nt.device_error_flags)

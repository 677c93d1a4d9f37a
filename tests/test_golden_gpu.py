"""The reference's known-answer cases (tests/golden/reference_cases.py) replayed on the CUDA path
through the Python surface, with the reference's own comparison rule (cast, then max-abs 1e-5)."""
import pytest
import torch

import nestedtensor_b200 as nt
from golden import reference_cases as rc

pytestmark = pytest.mark.gpu


def _eq(a, b):
    b = b.to(a)
    return a.shape == b.shape and torch.allclose(a.double(), b.double(), atol=1e-5, rtol=0)


def _to_cuda_nt(tensors):
    dtype = tensors[0].dtype if len(tensors) else torch.float32
    return nt.nested_tensor(tensors, device="cuda", dtype=dtype)


@pytest.mark.parametrize("case", rc.TO_TENSOR_MASK, ids=lambda c: c[0])
def test_to_tensor_mask_golden(native_libs, cuda_device, case):
    _, tensors, mask_dim, exp_t, exp_m = case
    t, m = _to_cuda_nt(tensors).to_tensor_mask(mask_dim=mask_dim)
    assert _eq(exp_t, t.cpu())
    assert _eq(exp_m, m.cpu())


@pytest.mark.parametrize("case", rc.TO_TENSOR_MASK_ERRORS, ids=lambda c: c[0])
def test_to_tensor_mask_errors(native_libs, cuda_device, case):
    _, tensors, mask_dim, msg = case
    with pytest.raises(RuntimeError, match=msg):
        _to_cuda_nt(tensors).to_tensor_mask(mask_dim=mask_dim)


@pytest.mark.parametrize("case", rc.FROM_TENSOR_MASK, ids=lambda c: c[0])
def test_from_tensor_mask_golden(native_libs, cuda_device, case):
    _, tensor, mask, nested_dim, expected = case
    got = nt.nested_tensor_from_tensor_mask(tensor.cuda(), mask.cuda(), nested_dim)
    assert len(got) == len(expected)
    for g, e in zip(got.unbind(), expected):
        assert _eq(e, g.cpu())


@pytest.mark.parametrize("case", rc.FROM_TENSOR_MASK_ERRORS, ids=lambda c: c[0])
def test_from_tensor_mask_errors(native_libs, cuda_device, case):
    _, tensor, mask, nested_dim, msg = case
    with pytest.raises(RuntimeError, match=msg):
        nt.nested_tensor_from_tensor_mask(tensor.cuda(), mask.cuda(), nested_dim)


def test_roundtrip_golden(native_libs, cuda_device):
    """test/test_nested_tensor_masking.py:454-477"""
    data1, mask1 = rc.ROUNDTRIP_DATA.cuda(), rc.ROUNDTRIP_MASK.cuda()
    nt2 = nt.nested_tensor_from_tensor_mask(data1, mask1)
    assert nt2.nested_size() == (torch.Size([1, 2]), torch.Size([3, 4]))
    data2, mask2 = nt2.to_tensor_mask()
    assert _eq(data1.cpu(), data2.cpu())
    assert _eq(mask1.cpu(), mask2.cpu())
    data3 = nt2.to_padded_tensor(padding=rc.ROUNDTRIP_PADDING)
    assert _eq((data1 + ~mask1 * rc.ROUNDTRIP_PADDING).cpu(), data3.cpu())
    nt3 = nt.nested_tensor_from_padded_tensor(data3, padding=rc.ROUNDTRIP_PADDING)
    assert nt3.nested_size() == nt2.nested_size()
    assert torch.equal(nt3._buffer, nt2._buffer)


def test_hole_in_mask_is_rejected(native_libs, cuda_device):
    t = torch.arange(12.0).reshape(1, 3, 4).cuda()
    m = torch.ones(1, 3, 4, dtype=torch.bool).cuda()
    m[0, 1, 1] = False
    with pytest.raises(RuntimeError, match="not a padding mask"):
        nt.nested_tensor_from_tensor_mask(t, m)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32], ids=str)
def test_to_tensor_mask_cuda(native_libs, cuda_device, dtype):
    """test/test_nested_tensor_class.py:794-807 and :809-816"""
    import random
    from oracle import ntref
    random.seed(110)
    tensors = [torch.arange(t * 3).reshape(t, 3).float().to(dtype) for t in [random.randint(2, 4) for _ in range(3)]]
    a = nt.nested_tensor(tensors, device="cuda", dtype=dtype)
    data, mask = a.to_tensor_mask(mask_dim=2)
    data1, mask1 = ntref.to_tensor_mask(tensors, mask_dim=2)
    assert _eq(data1, data.cpu()) and _eq(mask1, mask.cpu())
    assert _eq(mask.cpu(), torch.ops.nestedtensor.to_mask(a, 2).cpu())

"""Ragged NCHW <-> NHWC transposes (bit-exact against per-image permutes) and the convolution / pooling callers
of the padding path against the per-image oracle."""
import pytest
import torch

import nestedtensor_b200 as nt
from nestedtensor_b200 import _cabi
from oracle import ntref
from _helpers import assert_bit_equal

pytestmark = pytest.mark.gpu


def _images(g, n, C, lo, hi, dtype):
    out = []
    for _ in range(n):
        h, w = (int(v) for v in torch.randint(lo, hi + 1, (2,), generator=g))
        if dtype.is_floating_point:
            out.append(torch.randn(C, h, w, generator=g).to(dtype))
        else:
            out.append(torch.randint(0, 100, (C, h, w), generator=g).to(dtype))
    return out


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.int64, torch.uint8], ids=str)
@pytest.mark.parametrize("C,lo,hi", [(1, 1, 9), (3, 1, 70), (64, 5, 40), (100, 1, 33), (256, 60, 70), (8, 1, 50), (72, 3, 30)])
def test_transposes_bit_exact_and_round_trip(native_libs, cuda_device, dtype, C, lo, hi):
    g = torch.Generator().manual_seed(C + hi)
    imgs = _images(g, 7, C, lo, hi, dtype)
    x = nt.nested_tensor(imgs, device=cuda_device, dtype=dtype)
    y = torch.ops.nestedtensor.transpose_nchw_nhwc(x)
    assert [tuple(s) for s in y._sizes.tolist()] == [(t.size(1), t.size(2), C) for t in imgs]
    for a, b in zip(y.unbind(), ntref.transpose_nchw_nhwc(imgs)):
        assert_bit_equal(a, b, "transpose_nchw_nhwc")
    z = torch.ops.nestedtensor.transpose_nhwc_nchw(y)
    assert torch.equal(z._sizes, x._sizes)
    assert_bit_equal(z._buffer, x._buffer.cpu(), "transpose round trip")


def test_transposes_random_sweep(native_libs, cuda_device):
    """150 random batches (five element types, 1 to 320 channels, 1 to 9 images of 1 to 80 pixels a side): both
    transposes bit for bit against torch.permute, and the round trip."""
    for seed in range(150):
        g = torch.Generator().manual_seed(41000 + seed)
        r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
        dtype = [torch.float16, torch.bfloat16, torch.float32, torch.uint8, torch.int64][r(0, 4)]
        C = [1, 3, r(2, 40), 8 * r(1, 40), 64, 256][r(0, 5)]
        lo = r(1, 20)
        imgs = _images(g, r(1, 9), C, lo, lo + r(0, 60), dtype)
        x = nt.nested_tensor(imgs, device=cuda_device, dtype=dtype)
        y = torch.ops.nestedtensor.transpose_nchw_nhwc(x)
        for a, b in zip(y.unbind(), imgs):
            assert_bit_equal(a, b.permute(1, 2, 0).contiguous(), "transpose_nchw_nhwc seed %d %s C %d" % (seed, dtype, C))
        z = torch.ops.nestedtensor.transpose_nhwc_nchw(y)
        assert_bit_equal(z._buffer, x._buffer.cpu(), "transpose round trip seed %d %s C %d" % (seed, dtype, C))


def test_transpose_errors(native_libs, cuda_device):
    x = nt.nested_tensor([torch.randn(3, 4), torch.randn(2, 4)], device=cuda_device)
    with pytest.raises(RuntimeError, match="transpose_nchw_nhwc needs 4d input."):
        torch.ops.nestedtensor.transpose_nchw_nhwc(x)
    y = nt.nested_tensor([torch.randn(3, 4, 5), torch.randn(2, 4, 5)], device=cuda_device)
    with pytest.raises(RuntimeError, match="Expected first dimension to be regular."):
        torch.ops.nestedtensor.transpose_nchw_nhwc(y)
    z = nt.nested_tensor([torch.randn(4, 5, 3), torch.randn(4, 5, 2)], device=cuda_device)
    with pytest.raises(RuntimeError, match="Expected last dimension to be regular."):
        torch.ops.nestedtensor.transpose_nhwc_nchw(z)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.float16, 2e-2), (torch.bfloat16, 3e-2)], ids=str)
def test_pointwise_conv2d_is_one_packed_gemm(native_libs, cuda_device, dtype, tol):
    """1x1 convolution, no bias (nestedtensor/csrc/conv2d.cpp:33-73): transpose, one GEMM over all pixels of all
    images, transpose back."""
    g = torch.Generator().manual_seed(2)
    imgs = _images(g, 6, 64, 3, 40, dtype)
    w = (torch.randn(128, 64, 1, 1, generator=g) * 0.1).to(dtype)
    x = nt.nested_tensor(imgs, device=cuda_device, dtype=dtype)
    got = torch.nn.functional.conv2d(x, w.to(cuda_device))
    want = ntref.conv2d(imgs, w)
    assert [tuple(s) for s in got._sizes.tolist()] == [tuple(t.shape) for t in want]
    err = max((a.float().cpu() - b).abs().max().item() for a, b in zip(got.unbind(), want))
    assert err <= tol, err
    assert _cabi.load().ntb200_device_error_flags() == 0


@pytest.mark.parametrize("k,stride,padding,dilation,bias", [(3, 2, 1, 1, True), (7, 2, 3, 1, False), (3, 1, 0, 2, True), (1, 2, 0, 1, True)])
def test_conv2d_through_the_padding_path(native_libs, cuda_device, k, stride, padding, dilation, bias):
    """pad -> dense convolution -> unpad with the per-image output sizes (nestedtensor/csrc/conv2d.cpp:75-90)."""
    g = torch.Generator().manual_seed(k)
    imgs = _images(g, 5, 8, 20, 45, torch.float32)
    w = torch.randn(12, 8, k, k, generator=g) * 0.1
    b = torch.randn(12, generator=g) if bias else None
    x = nt.nested_tensor(imgs, device=cuda_device)
    prev = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        got = torch.nn.functional.conv2d(x, w.to(cuda_device), None if b is None else b.to(cuda_device), stride, padding, dilation)
    finally:
        torch.backends.cudnn.allow_tf32 = prev
    want = ntref.conv2d(imgs, w, b, stride, padding, dilation)
    assert [tuple(s) for s in got._sizes.tolist()] == [tuple(t.shape) for t in want]
    err = max((a.cpu() - b_).abs().max().item() for a, b_ in zip(got.unbind(), want))
    assert err <= 1e-4, err


@pytest.mark.parametrize("k,stride,padding", [(3, 2, 1), (2, 2, 0), (3, 1, 1)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32], ids=str)
def test_max_pool2d_matches_per_image_pooling(native_libs, cuda_device, dtype, k, stride, padding):
    """All-negative images: padding the batch with 0 (as the reference does, pooling.cpp:41) would leak zeros into
    the border windows; padding with -inf reproduces per-image pooling bit for bit."""
    g = torch.Generator().manual_seed(k + stride)
    imgs = [-(t.abs() + 0.5) for t in _images(g, 6, 5, 9, 31, dtype)]
    x = nt.nested_tensor(imgs, device=cuda_device, dtype=dtype)
    got = torch.nn.functional.max_pool2d(x, k, stride, padding)
    want = ntref.max_pool2d([t.float() for t in imgs], k, stride, padding)
    assert [tuple(s) for s in got._sizes.tolist()] == [tuple(t.shape) for t in want]
    for a, b in zip(got.unbind(), want):
        assert_bit_equal(a, b.to(dtype), "max_pool2d")


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32], ids=str)
def test_channels_last_nested_tensor(native_libs, cuda_device, dtype):
    """nested_tensor(..., channels_last=True) (nestedtensor/csrc/creation.cpp:197,217-220): logical (C, H_i, W_i)
    constituents stored pixel-major; unbind() gives channels_last-strided views with the same values, the operators see
    the logical layout, contiguous() converts both ways, and a 1x1 convolution stays channels_last without a transpose."""
    g = torch.Generator().manual_seed(21)
    C = 24
    imgs = [torch.randn(C, int(torch.randint(3, 40, (1,), generator=g)), int(torch.randint(3, 40, (1,), generator=g)), generator=g).to(dtype)
            for _ in range(6)]
    a = nt.nested_tensor(imgs, device=cuda_device, dtype=dtype, channels_last=True)
    assert a.is_contiguous(memory_format=torch.channels_last) and not a.is_contiguous()
    assert a.nested_size() == tuple(torch.Size(t.shape) for t in imgs)
    for view, t in zip(a.unbind(), imgs):
        assert view.stride() == (1, t.size(2) * C, C)
        assert torch.equal(view.cpu(), t)
    assert a.nested_stride()[0] == (1, imgs[0].size(2) * C, C)
    # stored bytes are those of the NHWC transpose
    want_buf = torch.cat([t.permute(1, 2, 0).reshape(-1) for t in imgs])
    assert torch.equal(a._buffer.cpu(), want_buf)
    # operators work on the logical layout
    assert_equal = lambda x, y: torch.equal(x.cpu().view(torch.int16 if dtype == torch.float16 else torch.int32),
                                            y.view(torch.int16 if dtype == torch.float16 else torch.int32))
    assert_equal(a.to_padded_tensor(padding=0), ntref.to_padded_tensor(imgs, 0))
    b = a.contiguous()
    assert b.is_contiguous() and torch.equal(b._buffer.cpu(), torch.cat([t.reshape(-1) for t in imgs]))
    assert b.contiguous(memory_format=torch.channels_last)._buffer.equal(a._buffer)
    assert a.contiguous(memory_format=torch.channels_last) is a
    # pointwise convolution keeps the storage format
    w = (torch.randn(16, C, 1, 1, generator=g) * 0.2).to(dtype).to(cuda_device)
    y = torch.nn.functional.conv2d(a, w)
    assert y.is_contiguous(memory_format=torch.channels_last)
    for got, t in zip(y.unbind(), imgs):
        want = torch.nn.functional.conv2d(t.float().unsqueeze(0), w.float().cpu())[0]
        assert (got.float().cpu() - want).abs().max().item() <= (2e-2 if dtype == torch.float16 else 1e-4)
    with pytest.raises(RuntimeError, match="4d input"):
        nt.nested_tensor([torch.randn(3, 4)], device=cuda_device, channels_last=True)

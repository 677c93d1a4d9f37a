"""Empty and degenerate inputs through the operators around the core path: they must return the same (empty or
trivial) results as the oracle, launch nothing harmful and leave the device flags clear."""
import pytest
import torch

import nestedtensor_b200 as nt
from nestedtensor_b200 import _cabi
from oracle import ntref
from _helpers import assert_bit_equal

pytestmark = pytest.mark.gpu


def test_layer_norm_with_empty_constituents(native_libs, cuda_device):
    ts = [torch.randn(0, 16), torch.randn(3, 16), torch.randn(0, 16), torch.randn(1, 16)]
    x = nt.nested_tensor(ts, device=cuda_device)
    m = torch.nn.LayerNorm(16).to(cuda_device)
    got = m(x)
    want = ntref.layer_norm(ts, (16,), m.weight.detach().cpu(), m.bias.detach().cpu(), m.eps)
    assert [tuple(t.shape) for t in got.unbind()] == [tuple(t.shape) for t in want]
    for a, b in zip(got.unbind(), want):
        assert (a.cpu() - b).abs().max().item() <= 4e-5 if b.numel() else True
    all_empty = nt.nested_tensor([torch.randn(0, 16), torch.randn(0, 16)], device=cuda_device)
    assert m(all_empty)._buffer.numel() == 0


def test_embedding_with_empty_sequences(native_libs, cuda_device):
    w = torch.randn(11, 8)
    idx = [torch.tensor([], dtype=torch.int64), torch.tensor([3, 10, 0]), torch.tensor([], dtype=torch.int64)]
    x = nt.nested_tensor(idx, device=cuda_device, dtype=torch.int64)
    got = torch.nn.functional.embedding(x, w.to(cuda_device))
    for a, b in zip(got.unbind(), ntref.embedding(idx, w)):
        assert tuple(a.shape) == tuple(b.shape)
        assert_bit_equal(a, b, "embedding")
    assert _cabi.load().ntb200_device_error_flags() == 0


def test_construction_from_device_list_with_empty_tensors(native_libs, cuda_device):
    ts = [torch.randn(0, 5), torch.randn(2, 5), torch.randn(0, 5)]
    x = nt.nested_tensor([t.to(cuda_device) for t in ts], device=cuda_device)
    assert_bit_equal(x._buffer, torch.cat([t.reshape(-1) for t in ts]), "pack with empty tensors")
    assert x.nested_size() == nt.nested_tensor(ts).nested_size()
    only_empty = nt.nested_tensor([torch.randn(0, 5).to(cuda_device)], device=cuda_device)
    assert only_empty._buffer.numel() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=str)
def test_self_attention_with_length_one_and_long_sequences(native_libs, cuda_device, dtype):
    """A batch mixing single-token sequences with one far longer than a key block."""
    E, H = 128, 2
    g = torch.Generator().manual_seed(1)
    xs = [torch.randn(l, E, generator=g).to(dtype) for l in (1, 1, 700, 1, 129, 1)]
    torch.manual_seed(2)
    mha = torch.nn.MultiheadAttention(E, H).eval().to(dtype).to(cuda_device)
    x = nt.nested_tensor(xs, device=cuda_device, dtype=dtype)
    with torch.no_grad():
        got, _ = mha(x, x, x, need_weights=False)
    want = ntref.min_mha(H, E // H, xs, xs, xs, mha.in_proj_weight.cpu(), mha.in_proj_bias.cpu(), float(E // H) ** -0.5,
                         mha.out_proj.weight.cpu(), mha.out_proj.bias.cpu())
    err = max((a.float().cpu() - b).abs().max().item() for a, b in zip(got.unbind(), want))
    assert err <= (1e-5 if dtype == torch.float32 else 2e-2), err
    assert _cabi.load().ntb200_device_error_flags() == 0


def test_cross_attention_with_empty_memory_sequence(native_libs, cuda_device):
    """A query sequence whose memory is empty receives the output projection of zeros (its bias)."""
    E, H = 64, 1
    g = torch.Generator().manual_seed(4)
    qs = [torch.randn(3, E, generator=g), torch.randn(2, E, generator=g)]
    ks = [torch.randn(0, E), torch.randn(5, E, generator=g)]
    torch.manual_seed(3)
    mha = torch.nn.MultiheadAttention(E, H).eval().to(cuda_device)
    q = nt.nested_tensor(qs, device=cuda_device)
    k = nt.nested_tensor(ks, device=cuda_device)
    with torch.no_grad():
        got, _ = mha(q, k, k, need_weights=False)
    outs = got.unbind()
    bias = mha.out_proj.bias.detach()
    assert (outs[0] - bias).abs().max().item() <= 1e-6
    want = ntref.min_mha(H, E, qs[1:], ks[1:], ks[1:], mha.in_proj_weight.cpu(), mha.in_proj_bias.cpu(), float(E) ** -0.5,
                         mha.out_proj.weight.cpu(), mha.out_proj.bias.cpu())
    assert (outs[1].cpu() - want[0]).abs().max().item() <= 1e-5


def test_host_entry_points_with_a_single_sequence(native_libs, cuda_device):
    h = torch.randn(7 * 4).pin_memory()
    sizes = torch.tensor([[7, 4]], dtype=torch.int64)
    got = nt.to_padded_tensor_host(h, sizes, 0, device=cuda_device)
    torch.cuda.synchronize()
    assert_bit_equal(got, h.view(1, 7, 4), "to_padded_tensor_host, one sequence")


def test_conv2d_rejects_images_smaller_than_the_kernel(native_libs, cuda_device):
    x = nt.nested_tensor([torch.randn(3, 2, 9), torch.randn(3, 8, 8)], device=cuda_device)
    w = torch.randn(4, 3, 5, 5, device=cuda_device)
    with pytest.raises(RuntimeError):
        torch.nn.functional.conv2d(x, w)


def test_remaining_operator_names_of_the_reference_surface(native_libs, cuda_device):
    """get_max_size, pad_nt and min_mha under torch.ops.nestedtensor (nestedtensor/csrc/masking.cpp:652-675,
    nestedtensor/csrc/mha.cpp:71-74), called with the wrapper like the reference's own tests do."""
    g = torch.Generator().manual_seed(8)
    ts = [torch.randn(3, 5, generator=g), torch.randn(6, 2, generator=g), torch.randn(1, 7, generator=g)]
    x = nt.nested_tensor(ts, device=cuda_device)
    assert torch.ops.nestedtensor.get_max_size(x) == [6, 7]
    data, mask = torch.ops.nestedtensor.pad_nt(x, [8, 9])
    assert mask.dtype == torch.uint8 and tuple(data.shape) == (3, 8, 9) and tuple(mask.shape) == (3, 8, 9)
    want = torch.stack([torch.nn.functional.pad(t, (0, 9 - t.size(1), 0, 8 - t.size(0))) for t in ts])
    wmask = torch.stack([torch.nn.functional.pad(torch.ones_like(t, dtype=torch.uint8), (0, 9 - t.size(1), 0, 8 - t.size(0)))
                         for t in ts])
    assert_bit_equal(data, want, "pad_nt data")
    assert torch.equal(mask.cpu(), wmask)
    with pytest.raises(RuntimeError, match="smaller than the largest constituent"):
        torch.ops.nestedtensor.pad_nt(x, [5, 9])
    with pytest.raises(RuntimeError, match="Empty tensors are not yet supported."):
        torch.ops.nestedtensor.pad_nt(nt.nested_tensor([torch.randn(0, 3), torch.randn(2, 3)], device=cuda_device), [4, 4])

    E, H = 32, 2
    xs = [torch.randn(l, E, generator=g) for l in (4, 9)]
    ks = [torch.randn(l, E, generator=g) for l in (7, 2)]
    torch.manual_seed(5)
    mha = torch.nn.MultiheadAttention(E, H).eval().to(cuda_device)
    q, k = nt.nested_tensor(xs, device=cuda_device), nt.nested_tensor(ks, device=cuda_device)
    args = (mha.in_proj_weight, mha.in_proj_bias, float(E // H) ** -0.5, mha.out_proj.weight, mha.out_proj.bias)
    cpu = [a.detach().cpu() if torch.is_tensor(a) else a for a in args]
    for key in (q, k):
        got = torch.ops.nestedtensor.min_mha(H, E // H, 0.0, False, q, key, key, *args)
        kk = xs if key is q else ks
        want = ntref.min_mha(H, E // H, xs, kk, kk, *cpu)
        assert max((a.cpu() - b).abs().max().item() for a, b in zip(got.unbind(), want)) <= 1e-5

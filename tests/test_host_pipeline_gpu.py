"""The host-buffer entry points (pinned host in, pinned host out, ranges pipelined on three streams) must
return exactly what the oracle returns for the whole batch, whatever the number of ranges."""
import pytest
import torch

import nestedtensor_b200 as nt
from nestedtensor_b200 import workloads
from oracle import ntref
from _helpers import assert_bit_equal, random_list, sizes_of

pytestmark = pytest.mark.gpu


def _pinned(t):
    return t.contiguous().pin_memory()


@pytest.mark.parametrize("ranges", [1, 3, 8, 64])
@pytest.mark.parametrize("tdim,dtype", [(1, torch.float32), (2, torch.bfloat16), (3, torch.int16)], ids=str)
def test_to_padded_tensor_host_matches_oracle(native_libs, cuda_device, ranges, tdim, dtype):
    g = torch.Generator().manual_seed(77 + tdim)
    tensors = random_list(g, 23, tdim, 1, 40, dtype)
    sizes = sizes_of(tensors)
    h = _pinned(torch.cat([t.reshape(-1) for t in tensors]))
    got = nt.to_padded_tensor_host(h, sizes, 3, device=cuda_device, ranges=ranges)
    torch.cuda.synchronize()
    assert got.is_pinned()
    assert_bit_equal(got, ntref.to_padded_tensor(tensors, 3), "to_padded_tensor_host")
    # and back
    back = nt.from_padded_tensor_host(got, sizes, device=cuda_device, ranges=ranges)
    torch.cuda.synchronize()
    assert_bit_equal(back, h, "from_padded_tensor_host")


def test_host_pad_regular_trailing_dim_and_out_argument(native_libs, cuda_device):
    """(L_i, 64) rows: the regular trailing dim is folded; a caller-provided pinned output is filled in place
    and a range whose own maximum is below the batch maximum is still padded to the batch maximum."""
    g = torch.Generator().manual_seed(5)
    lengths = [1, 90, 2, 3, 2, 1, 77, 5, 4, 1, 1, 2]
    tensors = [torch.randn(l, 64, generator=g).to(torch.float16) for l in lengths]
    sizes = sizes_of(tensors)
    h = _pinned(torch.cat([t.reshape(-1) for t in tensors]))
    out = torch.full((len(lengths), 90, 64), 9.0, dtype=torch.float16).pin_memory()
    got = nt.to_padded_tensor_host(h, sizes, -1, out=out, device=cuda_device, ranges=5)
    torch.cuda.synchronize()
    assert got.data_ptr() == out.data_ptr()
    assert_bit_equal(out, ntref.to_padded_tensor(tensors, -1), "to_padded_tensor_host(out=)")


def test_host_argument_errors(native_libs, cuda_device):
    sizes = torch.tensor([[2, 4], [3, 4]], dtype=torch.int64)
    pageable = torch.zeros(20)
    with pytest.raises(ValueError, match="pinned"):
        nt.to_padded_tensor_host(pageable, sizes, 0, device=cuda_device)
    with pytest.raises(ValueError, match="sum\\(numel\\)"):
        nt.to_padded_tensor_host(torch.zeros(19).pin_memory(), sizes, 0, device=cuda_device)
    with pytest.raises(ValueError, match="shape"):
        nt.to_padded_tensor_host(torch.zeros(20).pin_memory(), sizes, 0, out=torch.zeros(2, 3, 5).pin_memory(),
                                 device=cuda_device)
    with pytest.raises(TypeError):
        nt.to_padded_tensor_host(torch.zeros(20).pin_memory(), sizes.to(torch.int32), 0, device=cuda_device)
    with pytest.raises(RuntimeError, match="smaller than the largest constituent"):
        buf = torch.zeros(20, device=cuda_device)
        from nestedtensor_b200.nested import build_meta
        torch.ops.nestedtensor.to_padded_tensor_out(buf, sizes, build_meta(sizes, cuda_device), 0.0,
                                                    torch.zeros(2, 2, 4, device=cuda_device))


@pytest.mark.parametrize("ranges", [1, 4, 8])
def test_multi_head_attention_host_matches_device_operator(native_libs, cuda_device, ranges):
    """Sequences are independent, so the pipelined host entry point must reproduce the one-call device
    operator bit for bit, and agree with the fp32 oracle within the bf16 bar."""
    E, H = 128, 2
    g = torch.Generator().manual_seed(31)
    lengths = [int(v) for v in torch.randint(1, 200, (37,), generator=g)]
    w = workloads._mha_weights(g, E, torch.bfloat16)
    wd = {k: v.to(cuda_device) for k, v in w.items()}
    xs = [torch.randn(l, E, generator=g).to(torch.bfloat16) for l in lengths]
    sizes = sizes_of(xs)
    h = _pinned(torch.cat(xs))
    got = nt.multi_head_attention_host(h, sizes, H, wd["in_proj_weight"], wd["in_proj_bias"], wd["out_proj_weight"],
                                       wd["out_proj_bias"], ranges=ranges)
    torch.cuda.synchronize()
    x = nt.nested_tensor(xs, device=cuda_device, dtype=torch.bfloat16)
    buf, sz, meta = x._record()
    ref = torch.ops.nestedtensor.bt_min_mha(H, E // H, 0.0, False, buf, sz, meta, wd["in_proj_weight"], wd["in_proj_bias"],
                                            float(E // H) ** -0.5, wd["out_proj_weight"], wd["out_proj_bias"])
    assert_bit_equal(got.reshape(-1), ref.reshape(-1).cpu(), "multi_head_attention_host vs bt_min_mha")
    xf = [t.float() for t in xs]
    want = ntref.min_mha(H, E // H, xf, xf, xf, w["in_proj_weight"].float(), w["in_proj_bias"].float(),
                         float(E // H) ** -0.5, w["out_proj_weight"].float(), w["out_proj_bias"].float())
    err = (got.float() - torch.cat(want)).abs().max().item()
    assert err <= 2e-2, err  # bf16 bar for MHA against the fp32 oracle

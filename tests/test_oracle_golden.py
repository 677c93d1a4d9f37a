"""Pins the CPU oracle (oracle/ntref.py) to the reference's own known-answer tests, and its MHA
to stock torch multi-head attention the way the reference's tests do."""
import random

import pytest
import torch
import torch.nn.functional as F

from oracle import ntref
from golden import reference_cases as rc


def _eq(a, b):
    """The reference's assertEqual casts b to a's dtype/device first (test/utils_test_case.py:224-283)."""
    b = b.to(a)
    return a.shape == b.shape and torch.allclose(a.double(), b.double(), atol=1e-5, rtol=0)


@pytest.mark.parametrize("case", rc.TO_TENSOR_MASK, ids=lambda c: c[0])
def test_to_tensor_mask_golden(case):
    _, tensors, mask_dim, exp_t, exp_m = case
    t, m = ntref.to_tensor_mask(tensors, mask_dim)
    assert _eq(exp_t, t)
    assert _eq(exp_m, m)


@pytest.mark.parametrize("case", rc.TO_TENSOR_MASK_ERRORS, ids=lambda c: c[0])
def test_to_tensor_mask_errors(case):
    _, tensors, mask_dim, msg = case
    with pytest.raises(RuntimeError, match=msg):
        ntref.to_tensor_mask(tensors, mask_dim)


@pytest.mark.parametrize("case", rc.FROM_TENSOR_MASK, ids=lambda c: c[0])
def test_from_tensor_mask_golden(case):
    _, tensor, mask, nested_dim, expected = case
    got = ntref.nested_tensor_from_tensor_mask(tensor, mask, nested_dim)
    assert len(got) == len(expected)
    for g, e in zip(got, expected):
        assert _eq(e, g)


@pytest.mark.parametrize("case", rc.FROM_TENSOR_MASK_ERRORS, ids=lambda c: c[0])
def test_from_tensor_mask_errors(case):
    _, tensor, mask, nested_dim, msg = case
    with pytest.raises(RuntimeError, match=msg):
        ntref.nested_tensor_from_tensor_mask(tensor, mask, nested_dim)


def test_none_arguments():
    with pytest.raises(RuntimeError):
        ntref.nested_tensor_from_tensor_mask(None, None)
    with pytest.raises(RuntimeError):
        ntref.nested_tensor_from_tensor_mask(torch.tensor([]), None)


def test_roundtrip_golden():
    """test/test_nested_tensor_masking.py:454-477"""
    nt2 = ntref.nested_tensor_from_tensor_mask(rc.ROUNDTRIP_DATA, rc.ROUNDTRIP_MASK)
    assert [tuple(t.shape) for t in nt2] == [(1, 2), (3, 4)]
    data2, mask2 = ntref.to_tensor_mask(nt2)
    assert _eq(rc.ROUNDTRIP_DATA, data2)
    assert _eq(rc.ROUNDTRIP_MASK, mask2)
    data3 = ntref.to_padded_tensor(nt2, rc.ROUNDTRIP_PADDING)
    assert _eq(rc.ROUNDTRIP_DATA + ~rc.ROUNDTRIP_MASK * rc.ROUNDTRIP_PADDING, data3)
    # and through the value-driven constructor
    nt3 = ntref.nested_tensor_from_padded_tensor(data3, padding=rc.ROUNDTRIP_PADDING)
    for a, b in zip(nt2, nt3):
        assert torch.equal(a, b)
    nt4 = ntref.from_padded_by_value_fast(data3, rc.ROUNDTRIP_PADDING)
    for a, b in zip(nt2, nt4):
        assert torch.equal(a, b)


@pytest.mark.parametrize("tdim", [1, 2, 3])
def test_padded_equals_masked_fill(tdim):
    """The identity the reference checks in test/test_nested_tensor_class.py:754-792:
    to_padded_tensor(padding=1) == to_tensor_mask() data with the invalid part filled with 1."""
    random.seed(1010)
    tensors = [torch.randn(*[random.randint(3, 30) for _ in range(tdim)]) for _ in range(5)]
    data0 = ntref.to_padded_tensor(tensors, 1)
    data1, mask1 = ntref.to_tensor_mask(tensors)
    data1 = data1.masked_fill(mask1.logical_not(), 1)
    assert torch.equal(data0, data1)
    back = ntref.from_padded_tensor(data0, [list(t.shape) for t in tensors])
    for a, b in zip(tensors, back):
        assert torch.equal(a, b)


def test_to_mask_equals_tensor_mask():
    """test/test_nested_tensor_class.py:809-816"""
    random.seed(110)
    tensors = [torch.arange(t * 3).reshape(t, 3).float() for t in [random.randint(2, 4) for _ in range(3)]]
    _, mask0 = ntref.to_tensor_mask(tensors, mask_dim=2)
    mask1 = ntref.to_mask(tensors, 2)
    assert _eq(mask0, mask1)


def test_to_mask_leading_dims():
    tensors = [torch.randn(3, 4, 5), torch.randn(3, 2, 7)]
    m = ntref.to_mask(tensors, 3)
    assert tuple(m.shape) == (2, 3, 4)
    assert m[0].all() and m[1, :, :2].all() and not m[1, :, 2:].any()


def _dense_mha(tensors, E, H, w):
    """Stock torch attention on the zero-padded batch with key_padding_mask, as
    test/test_nested_tensor_functional.py:1103-1140 does."""
    data, mask = ntref.to_tensor_mask(tensors, mask_dim=2)
    x = data.transpose(0, 1)
    out, _ = F.multi_head_attention_forward(
        x, x, x, E, H, w["in_proj_weight"], w["in_proj_bias"], None, None, False, 0.0, w["out_proj_weight"],
        w["out_proj_bias"], training=False, key_padding_mask=~mask.to(torch.bool), need_weights=False)
    return out.transpose(0, 1), mask.to(torch.bool)


@pytest.mark.parametrize("H,B,Lmax,d", [(2, 1, 2, 1), (1, 3, 5, 4), (2, 3, 5, 2), (8, 8, 50, 16), (16, 16, 50, 16),
                                         (4, 8, 50, 64)])
def test_min_mha_matches_stock_attention(H, B, Lmax, d):
    """Shapes from test/test_nested_tensor_functional.py:1149-1161 (batch reduced for CPU time);
    tolerance 5e-4 as at :1135."""
    g = torch.Generator().manual_seed(1010 + H + B)
    E = H * d
    tensors = [torch.randn(int(torch.randint(1, Lmax + 1, (1,), generator=g)), E, generator=g) for _ in range(B)]
    w = {"in_proj_weight": torch.randn(3 * E, E, generator=g) * E ** -0.5,
         "in_proj_bias": torch.randn(3 * E, generator=g) * 0.1,
         "out_proj_weight": torch.randn(E, E, generator=g) * E ** -0.5,
         "out_proj_bias": torch.randn(E, generator=g) * 0.1}
    got = ntref.min_mha(H, d, tensors, tensors, tensors, w["in_proj_weight"], w["in_proj_bias"], float(d) ** -0.5,
                        w["out_proj_weight"], w["out_proj_bias"])
    ref, mask = _dense_mha(tensors, E, H, w)
    got_padded = ntref.to_padded_tensor(got, 0) if len({t.shape[0] for t in got}) > 1 or len(got) > 1 else got[0][None]
    ref = ref * mask.unsqueeze(-1)
    assert torch.allclose(got_padded, ref, atol=5e-4, rtol=1e-8)


def test_masked_softmax_matches_exact():
    g = torch.Generator().manual_seed(3)
    s = torch.randn(2, 3, 6, 6, generator=g)
    lens = [4, 6]
    m = torch.zeros(2, 6)
    for i, l in enumerate(lens):
        m[i, :l] = 1
    mask = m.unsqueeze(1) * m.unsqueeze(2)
    p = ntref.masked_softmax(s, mask, 0.5)
    for b, l in enumerate(lens):
        exact = torch.softmax(s[b, :, :l, :l] * 0.5, -1)
        assert torch.allclose(p[b, :, :l, :l], exact, atol=2e-6)


# ------------------------------------------------------------------ layer norm / encoder layer
@pytest.mark.parametrize("size", [1024, 512, 256, 128, 2, 4, 32])
def test_oracle_layer_norm_matches_module_per_constituent(size):
    """test/test_nested_tensor_functional.py:895-957: LayerNorm of the nested tensor equals the module applied
    to each constituent."""
    g = torch.Generator().manual_seed(size)
    ts = [torch.randn(2, size, generator=g), torch.randn(3, size, generator=g)]
    m = torch.nn.LayerNorm(size)
    with torch.no_grad():
        m.weight.copy_(torch.randn(size, generator=g))
        m.bias.copy_(torch.randn(size, generator=g))
        want = [m(t) for t in ts]
    got = ntref.layer_norm(ts, (size,), m.weight.detach(), m.bias.detach(), m.eps)
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=1e-6, rtol=1e-6)


def test_oracle_layer_norm_errors():
    ts = [torch.randn(3, 4), torch.randn(2, 4)]
    with pytest.raises(RuntimeError, match="Currently only singleton tuples"):
        ntref.layer_norm(ts, (2, 4), None, None)
    with pytest.raises(RuntimeError, match=r"Normalized shape \[3\] does not match the size of the last dimension \(4\)"):
        ntref.layer_norm(ts, (3,), None, None)
    with pytest.raises(RuntimeError, match="Either both weight and bias"):
        ntref.layer_norm(ts, (4,), torch.ones(4), None)
    with pytest.raises(RuntimeError, match="Cannot normalize across irregular dimension 2"):
        ntref.layer_norm([torch.randn(3, 4), torch.randn(2, 5)], (4,), None, None)


@pytest.mark.parametrize("norm_first", [False, True])
@pytest.mark.parametrize("act", ["gelu_tanh", "relu"])
def test_oracle_encoder_layer_matches_stock_module(act, norm_first):
    """The oracle's encoder layer is pinned to torch.nn.TransformerEncoderLayer evaluated per sequence (with
    gradients enabled the stock module takes its plain Python path; its fused inference path replaces the
    tanh GELU by the erf form)."""
    torch.manual_seed(5)
    activation = torch.nn.GELU(approximate="tanh") if act == "gelu_tanh" else torch.nn.functional.relu
    layer = torch.nn.TransformerEncoderLayer(64, 4, dim_feedforward=128, dropout=0.0, activation=activation, batch_first=True,
                                             norm_first=norm_first).eval()
    p = {"in_proj_weight": layer.self_attn.in_proj_weight, "in_proj_bias": layer.self_attn.in_proj_bias,
         "out_proj_weight": layer.self_attn.out_proj.weight, "out_proj_bias": layer.self_attn.out_proj.bias,
         "linear1_weight": layer.linear1.weight, "linear1_bias": layer.linear1.bias, "linear2_weight": layer.linear2.weight,
         "linear2_bias": layer.linear2.bias, "norm1_weight": layer.norm1.weight, "norm1_bias": layer.norm1.bias,
         "norm2_weight": layer.norm2.weight, "norm2_bias": layer.norm2.bias}
    p = {k: v.detach() for k, v in p.items()}
    xs = [torch.randn(l, 64) for l in (5, 17, 1)]
    got = ntref.encoder_layer(xs, 4, p, act, norm_first)
    want = [layer(x.unsqueeze(0)).squeeze(0).detach() for x in xs]
    for a, b in zip(got, want):
        assert (a - b).abs().max().item() <= 2e-6


def test_oracle_attention_weights_pinned_to_stock_module():
    """ntref.mha_weights against torch.nn.MultiheadAttention(need_weights=True) run on one sequence at a time
    (self- and cross-attention, averaged over heads and per head)."""
    E, H = 96, 3
    g = torch.Generator().manual_seed(1)
    qs = [torch.randn(l, E, generator=g) for l in (7, 1, 30)]
    ks = [torch.randn(l, E, generator=g) for l in (9, 4, 50)]
    torch.manual_seed(3)
    mha = torch.nn.MultiheadAttention(E, H).eval()
    with torch.no_grad():
        mha.in_proj_bias.normal_(0, 0.05)
    for keys in (qs, ks):
        for average in (True, False):
            want = ntref.mha_weights(H, E // H, qs, keys, mha.in_proj_weight, mha.in_proj_bias, float(E // H) ** -0.5, average)
            with torch.no_grad():
                for xq, xk, b in zip(qs, keys, want):
                    _, ws = mha(xq.unsqueeze(1), xk.unsqueeze(1), xk.unsqueeze(1), need_weights=True, average_attn_weights=average)
                    assert torch.allclose(ws[0], b, atol=2e-6)

"""Parity of the packed row operators (LayerNorm, bias + residual + LayerNorm, bias + GELU), of the fused
projection epilogues and of the encoder layer built from them with the fp32 oracle
(oracle.ntref.layer_norm = nestedtensor/csrc/functions.cpp:65-110, gelu_tanh =
nestedtensor/csrc/cuda/cuda_kernels.cu:29-36, encoder_layer pinned to torch.nn.TransformerEncoderLayer).
Tolerances (max-abs on O(1) outputs): fp32 1e-5 for the row operators and 1e-4 for a whole layer,
fp16 / bf16 2e-2 (3e-2 for a whole bf16 layer, whose intermediates are rounded four times; relative to
1 + |y| at BERT-large width, where outputs reach |y| ~ 5)."""
import pytest
import torch

import nestedtensor_b200 as nt
from nestedtensor_b200 import _cabi, workloads
from oracle import ntref
from _helpers import random_list, sizes_of, stream_ptr

pytestmark = pytest.mark.gpu

CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
TOL = {torch.float32: 1e-5, torch.float16: 2e-2, torch.bfloat16: 2e-2}


def _ptr(t):
    return t.data_ptr() if t is not None else None


def _layer_norm(x, res, bias, gamma, beta, eps, inplace=False):
    lib = _cabi.load()
    out = x if inplace else torch.empty_like(x)
    if res is None and bias is None:
        rc = lib.ntb200_layer_norm(x.data_ptr(), _ptr(gamma), _ptr(beta), eps, out.data_ptr(), x.size(0), x.size(1),
                                   CODE[x.dtype], stream_ptr())
    else:
        rc = lib.ntb200_add_bias_residual_layer_norm(x.data_ptr(), _ptr(res), _ptr(bias), _ptr(gamma), _ptr(beta), eps,
                                                     out.data_ptr(), x.size(0), x.size(1), CODE[x.dtype], stream_ptr())
    _cabi.check("ntb200_layer_norm", rc)
    torch.cuda.synchronize()
    return out


# the reference's test sizes (test/test_nested_tensor_functional.py:953) plus rows handled by a whole block
# (cols * element size > 4 KB), rows that are not a multiple of 16 bytes and a row longer than 32 KB
@pytest.mark.parametrize("cols", [1024, 512, 256, 128, 2, 4, 32, 8, 40, 3000, 4096, 8192, 1023, 20000, 64, 96, 768, 1280, 1536, 2560, 3072,
                                  6144, 10240, 12288])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=str)
def test_cabi_layer_norm(native_libs, cuda_device, dtype, cols):
    g = torch.Generator().manual_seed(cols)
    rows = 37 if cols <= 4096 else 5
    x = (torch.randn(rows, cols, generator=g) * 2 + 0.5).to(dtype)
    gamma = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
    beta = (0.1 * torch.randn(cols, generator=g)).to(dtype)
    want = torch.nn.functional.layer_norm(x.float(), (cols,), gamma.float(), beta.float(), 1e-5)
    got = _layer_norm(x.to(cuda_device), None, None, gamma.to(cuda_device), beta.to(cuda_device), 1e-5)
    assert (got.float().cpu() - want).abs().max().item() <= TOL[dtype] * (4 if dtype == torch.float32 else 1)
    # no affine
    got = _layer_norm(x.to(cuda_device), None, None, None, None, 1e-5)
    want = torch.nn.functional.layer_norm(x.float(), (cols,), None, None, 1e-5)
    assert (got.float().cpu() - want).abs().max().item() <= TOL[dtype] * (4 if dtype == torch.float32 else 1)


@pytest.mark.parametrize("cols", [1024, 768, 64, 6, 4104, 96, 1280, 1536, 3072, 6144])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=str)
def test_cabi_add_bias_residual_layer_norm(native_libs, cuda_device, dtype, cols):
    g = torch.Generator().manual_seed(cols + 1)
    rows = 53
    x = torch.randn(rows, cols, generator=g).to(dtype)
    res = torch.randn(rows, cols, generator=g).to(dtype)
    bias = (0.2 * torch.randn(cols, generator=g)).to(dtype)
    gamma = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
    beta = (0.1 * torch.randn(cols, generator=g)).to(dtype)
    d = lambda t: t.to(cuda_device)
    want = torch.nn.functional.layer_norm(x.float() + res.float() + bias.float(), (cols,), gamma.float(), beta.float(), 1e-6)
    got = _layer_norm(d(x), d(res), d(bias), d(gamma), d(beta), 1e-6)
    assert (got.float().cpu() - want).abs().max().item() <= TOL[dtype] * (4 if dtype == torch.float32 else 1)
    # in place, residual only
    xin = d(x).clone()
    got = _layer_norm(xin, d(res), None, d(gamma), d(beta), 1e-6, inplace=True)
    want = torch.nn.functional.layer_norm(x.float() + res.float(), (cols,), gamma.float(), beta.float(), 1e-6)
    assert got.data_ptr() == xin.data_ptr()
    assert (got.float().cpu() - want).abs().max().item() <= TOL[dtype] * (4 if dtype == torch.float32 else 1)


@pytest.mark.parametrize("cols", [1024, 512, 256, 64, 200])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=str)
@pytest.mark.parametrize("fused", [False, True])
def test_cabi_layer_norm_many_rows(native_libs, cuda_device, dtype, cols, fused):
    """Thousands of rows (more than one wave of CTAs), plain and with residual + bias, out of place and in place."""
    g = torch.Generator().manual_seed(cols + int(fused))
    rows = 9001
    x = (torch.randn(rows, cols, generator=g) + 0.3).to(dtype)
    res = torch.randn(rows, cols, generator=g).to(dtype) if fused else None
    bias = (0.2 * torch.randn(cols, generator=g)).to(dtype) if fused else None
    gamma = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
    beta = (0.1 * torch.randn(cols, generator=g)).to(dtype)
    d = lambda t: None if t is None else t.to(cuda_device)
    ref_in = x.float() + (res.float() if fused else 0) + (bias.float() if fused else 0)
    want = torch.nn.functional.layer_norm(ref_in, (cols,), gamma.float(), beta.float(), 1e-5)
    tol = TOL[dtype] * (4 if dtype == torch.float32 else 1)
    got = _layer_norm(d(x), d(res), d(bias), d(gamma), d(beta), 1e-5)
    assert (got.float().cpu() - want).abs().max().item() <= tol
    xin = d(x).clone()
    got = _layer_norm(xin, d(res), d(bias), d(gamma), d(beta), 1e-5, inplace=True)
    assert (got.float().cpu() - want).abs().max().item() <= tol


@pytest.mark.parametrize("cols", [4096, 24, 7])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=str)
def test_cabi_add_bias_gelu(native_libs, cuda_device, dtype, cols):
    g = torch.Generator().manual_seed(cols + 2)
    x = (2 * torch.randn(29, cols, generator=g)).to(dtype)
    bias = torch.randn(cols, generator=g).to(dtype)
    lib = _cabi.load()
    xd, bd = x.to(cuda_device), bias.to(cuda_device)
    out = torch.empty_like(xd)
    _cabi.check("ntb200_add_bias_gelu", lib.ntb200_add_bias_gelu(xd.data_ptr(), bd.data_ptr(), out.data_ptr(), 29, cols,
                                                                 CODE[dtype], stream_ptr()))
    torch.cuda.synchronize()
    want = ntref.gelu_tanh(x.float() + bias.float())
    assert (out.float().cpu() - want).abs().max().item() <= (1e-5 if dtype == torch.float32 else 4e-2)
    rel = ((out.float().cpu() - want).abs() / (want.abs() + 1)).max().item()
    assert rel <= (1e-5 if dtype == torch.float32 else 1e-2)


def _gemm_act(A, W, bias, res, act, path):
    lib = _cabi.load()
    M, K = A.shape
    N = W.shape[0]
    C = torch.empty(M, N, dtype=A.dtype, device=A.device)
    rc = lib.ntb200_gemm_bias_act(A.data_ptr(), W.data_ptr(), _ptr(bias), _ptr(res), C.data_ptr(), M, N, K, CODE[A.dtype], act,
                                  path, stream_ptr())
    _cabi.check("ntb200_gemm_bias_act", rc)
    torch.cuda.synchronize()
    assert lib.ntb200_device_error_flags() == 0
    return C


def _act_ref(v, act):
    return [lambda t: t, ntref.gelu_tanh, torch.relu][act](v)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
@pytest.mark.parametrize("M,N,K", [(300, 512, 256), (1000, 4096, 1024), (129, 264, 72), (4099, 1024, 4096)])
@pytest.mark.parametrize("act", [0, 1, 2])
def test_gemm_fused_epilogue_tensor_core(native_libs, cuda_device, dtype, M, N, K, act):
    g = torch.Generator().manual_seed(M + N + K + act)
    A = torch.randn(M, K, generator=g).to(dtype).to(cuda_device)
    W = (torch.randn(N, K, generator=g) * K ** -0.5).to(dtype).to(cuda_device)
    b = (torch.randn(N, generator=g) * 0.1).to(dtype).to(cuda_device)
    res = torch.randn(M, N, generator=g).to(dtype).to(cuda_device)
    base = _act_ref(A.float() @ W.float().t() + b.float(), act)
    for path in (3, 2, 1, 0):
        got = _gemm_act(A, W, b, res, act, path)
        assert (got.float() - (base + res.float())).abs().max().item() <= 3e-2, path
        got = _gemm_act(A, W, b, None, act, path)
        assert (got.float() - base).abs().max().item() <= 2e-2, path


@pytest.mark.parametrize("act", [0, 1, 2])
def test_gemm_fused_epilogue_fp32(native_libs, cuda_device, act):
    g = torch.Generator().manual_seed(act)
    M, N, K = 130, 66, 100
    A = torch.randn(M, K, generator=g).to(cuda_device)
    W = (torch.randn(N, K, generator=g) * K ** -0.5).to(cuda_device)
    b = torch.randn(N, generator=g).to(cuda_device)
    res = torch.randn(M, N, generator=g).to(cuda_device)
    want = _act_ref((A.double() @ W.double().t() + b.double()).float(), act) + res
    assert (_gemm_act(A, W, b, res, act, 0) - want).abs().max().item() <= 1e-5
    lib = _cabi.load()
    assert lib.ntb200_gemm_bias_act(A.data_ptr(), W.data_ptr(), None, None, A.data_ptr(), M, N, K, 0, 3, 0, None) == -1  # bad act


def test_row_operators_and_gemm_random_sweep(native_libs, cuda_device):
    """120 random shapes: LayerNorm (1 to 9000 columns, 1 to 6000 rows, with / without affine, plain and with bias and
    residual fused) and the projection with every epilogue (bias, activation, residual) on every kernel that takes the
    shape (default, SIMT, single-CTA and CTA-pair tcgen05, per-thread residual), against fp32 torch."""
    lib = _cabi.load()
    for seed in range(120):
        g = torch.Generator().manual_seed(31000 + seed)
        r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
        dtype = [torch.float32, torch.float16, torch.bfloat16][r(0, 2)]
        tol = {torch.float32: 8e-5, torch.float16: 1.6e-2, torch.bfloat16: 0.12}[dtype]  # outputs reach |y| ~ 8
        cols = [r(1, 64), r(1, 64) * 8, r(64, 1100), r(16, 1600) * 8, r(1100, 9000), 128 * r(1, 96)][r(0, 5)]
        rows = [1, r(2, 40), r(41, 700), r(1000, 6000)][r(0, 3)]
        if rows * cols > 8e6:
            rows = max(1, int(8e6 // cols))
        x = (torch.randn(rows, cols, generator=g) * 2 + 0.5).to(dtype).to(cuda_device)
        affine = r(0, 3) != 0
        gamma = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype).to(cuda_device) if affine else None
        beta = (0.1 * torch.randn(cols, generator=g)).to(dtype).to(cuda_device) if affine else None
        fused = r(0, 1)
        res = torch.randn(rows, cols, generator=g).to(dtype).to(cuda_device) if fused and r(0, 3) != 0 else None
        bias = (0.3 * torch.randn(cols, generator=g)).to(dtype).to(cuda_device) if fused and (res is None or r(0, 1)) else None
        got = _layer_norm(x, res, bias, gamma, beta, 1e-5)
        pre = x.float() + (res.float() if res is not None else 0) + (bias.float() if bias is not None else 0)
        want = torch.nn.functional.layer_norm(pre, (cols,), gamma.float() if affine else None, beta.float() if affine else None, 1e-5)
        tag = "seed %d %s rows %d cols %d residual %s bias %s affine %s" % (seed, dtype, rows, cols, res is not None, bias is not None, affine)
        assert float((got.float() - want).abs().max()) <= tol, "layer norm " + tag
        if dtype == torch.float32 and r(0, 3) != 0:
            continue
        M = [r(1, 130), r(130, 1200), r(1200, 9000)][r(0, 2)]
        N = [8 * r(1, 40), 64 * r(1, 48), r(1, 300), 256 * r(1, 12)][r(0, 3)]
        K = [8 * r(1, 40), 64 * r(1, 48), r(1, 300), 1024, 2048, 4096][r(0, 5)]
        if dtype == torch.float32:
            M, N, K = min(M, 1500), min(N, 600), min(K, 600)
        act = r(0, 2)
        A = torch.randn(M, K, generator=g).to(dtype).to(cuda_device)
        W = (torch.randn(N, K, generator=g) * K ** -0.5).to(dtype).to(cuda_device)
        b = (torch.randn(N, generator=g) * 0.1).to(dtype).to(cuda_device) if r(0, 4) else None
        rs = torch.randn(M, N, generator=g).to(dtype).to(cuda_device) if r(0, 1) else None
        base = _act_ref(A.float() @ W.float().t() + (b.float() if b is not None else 0), act) + (rs.float() if rs is not None else 0)
        for path in (0, 1, 2, 3, 4):
            C = torch.full((M, N), float("nan"), dtype=dtype, device=cuda_device)
            rc = lib.ntb200_gemm_bias_act(A.data_ptr(), W.data_ptr(), _ptr(b), _ptr(rs), C.data_ptr(), M, N, K, CODE[dtype], act, path,
                                          stream_ptr())
            torch.cuda.synchronize()
            if rc == -7 and path >= 2:
                continue  # NTB200_UNSUPPORTED_SHAPE: that kernel does not take the shape
            _cabi.check("ntb200_gemm_bias_act", rc)
            err = float((C.float() - base).abs().max())
            assert err <= (1e-4 if dtype == torch.float32 else 4e-2), "gemm seed %d %s M %d N %d K %d act %d path %d: %g" % (seed, dtype, M, N, K, act, path, err)
    assert lib.ntb200_device_error_flags() == 0


@pytest.mark.parametrize("size", [1024, 512, 256, 128, 2, 4, 32])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32], ids=str)
def test_layer_norm_module_on_nested_tensor(native_libs, cuda_device, dtype, size):
    """test/test_nested_tensor_functional.py:895-957: torch.nn.LayerNorm applied to the nested tensor equals
    the module applied to each constituent."""
    g = torch.Generator().manual_seed(size)
    t0 = torch.randn(2, size, generator=g)
    t1 = torch.randn(2, size, generator=g)
    ts = [t0, t1, t0, t1]
    x = nt.nested_tensor(ts, device=cuda_device, dtype=dtype)
    m = torch.nn.LayerNorm(size).to(cuda_device).to(dtype)
    with torch.no_grad():
        m.weight.copy_(1 + 0.1 * torch.randn(size, generator=g))
        m.bias.copy_(0.1 * torch.randn(size, generator=g))
    got = m(x)
    assert isinstance(got, nt.NestedTensor) and got.nested_size() == x.nested_size()
    want = ntref.layer_norm([t.to(dtype) for t in ts], (size,), m.weight.detach().cpu(), m.bias.detach().cpu(), m.eps)
    for a, b in zip(got.unbind(), want):
        assert (a.float().cpu() - b).abs().max().item() <= (4e-5 if dtype == torch.float32 else 2e-2)


def test_layer_norm_errors(native_libs, cuda_device):
    x = nt.nested_tensor([torch.randn(3, 4), torch.randn(2, 4)], device=cuda_device)
    with pytest.raises(RuntimeError, match="Currently only singleton tuples of integers supported for layer_norm."):
        torch.nn.functional.layer_norm(x, (2, 4))
    with pytest.raises(RuntimeError, match=r"Normalized shape \[3\] does not match the size of the last dimension \(4\) of input."):
        torch.nn.functional.layer_norm(x, (3,))
    with pytest.raises(RuntimeError, match="Either both weight and bias are used or not."):
        torch.nn.functional.layer_norm(x, (4,), torch.ones(4, device=cuda_device), None)
    y = nt.nested_tensor([torch.randn(3, 4), torch.randn(2, 5)], device=cuda_device)
    with pytest.raises(RuntimeError, match="Cannot normalize across irregular dimension 2"):
        torch.nn.functional.layer_norm(y, (4,))


def _params(layer):
    p = {"in_proj_weight": layer.self_attn.in_proj_weight, "in_proj_bias": layer.self_attn.in_proj_bias,
         "out_proj_weight": layer.self_attn.out_proj.weight, "out_proj_bias": layer.self_attn.out_proj.bias,
         "linear1_weight": layer.linear1.weight, "linear1_bias": layer.linear1.bias, "linear2_weight": layer.linear2.weight,
         "linear2_bias": layer.linear2.bias, "norm1_weight": layer.norm1.weight, "norm1_bias": layer.norm1.bias,
         "norm2_weight": layer.norm2.weight, "norm2_bias": layer.norm2.bias}
    return {k: v.detach().float().cpu() for k, v in p.items()}


@pytest.mark.parametrize("norm_first", [False, True])
@pytest.mark.parametrize("dtype,E,H,F,act,tol", [(torch.float32, 64, 4, 128, "relu", 1e-4), (torch.float32, 48, 3, 96, "gelu_tanh", 1e-4),
                                                 (torch.bfloat16, 128, 2, 512, "gelu_tanh", 3e-2), (torch.float16, 256, 4, 1024, "relu", 2e-2)])
def test_transformer_encoder_layer(native_libs, cuda_device, dtype, E, H, F, act, tol, norm_first):
    torch.manual_seed(E + F)
    activation = torch.nn.GELU(approximate="tanh") if act == "gelu_tanh" else torch.nn.functional.relu
    layer = torch.nn.TransformerEncoderLayer(E, H, dim_feedforward=F, dropout=0.1, activation=activation, norm_first=norm_first)
    layer = layer.eval().to(dtype)
    g = torch.Generator().manual_seed(3)
    xs = [torch.randn(int(l), E, generator=g).to(dtype) for l in torch.randint(1, 160, (19,), generator=g)]
    want = ntref.encoder_layer(xs, H, _params(layer), act, norm_first, layer.norm1.eps)
    x = nt.nested_tensor(xs, device=cuda_device, dtype=dtype)
    got = nt.nn.transformer_encoder_layer(layer.to(cuda_device), x)
    assert got.nested_size() == x.nested_size()
    err = max((a.float().cpu() - b).abs().max().item() for a, b in zip(got.unbind(), want))
    assert err <= tol, err
    assert _cabi.load().ntb200_device_error_flags() == 0


def test_encoder_layer_bert_large_sampled(native_libs, cuda_device):
    """Configuration 5 through a BERT-large layer (E=1024, 16 heads, FFN 4096, bf16): full batch on the GPU,
    oracle on every 64th sequence (sequences are independent)."""
    wl = workloads.config5()
    E, H, F = 1024, 16, 4096
    torch.manual_seed(11)
    layer = torch.nn.TransformerEncoderLayer(E, H, dim_feedforward=F, dropout=0.0, activation=torch.nn.GELU(approximate="tanh"))
    layer = layer.eval().to(torch.bfloat16)
    x = nt.NestedTensor(wl.buffer.to(cuda_device), wl.sizes)
    got = nt.nn.transformer_encoder_layer(layer.to(cuda_device), x)
    torch.cuda.synchronize()
    assert _cabi.load().ntb200_device_error_flags() == 0
    outs = got.unbind()
    ins = nt.NestedTensor(wl.buffer, wl.sizes).unbind()
    idx = list(range(0, len(ins), 64))
    want = ntref.encoder_layer([ins[i] for i in idx], H, _params(layer), "gelu_tanh", False, layer.norm1.eps)
    # LayerNorm outputs reach |y| ~ 5 at this width, where one bf16 rounding is already 0.02: the bar is on the
    # error relative to 1 + |y| (2e-2, the bf16 bar), with a loose absolute cap
    rel = max(((outs[i].float().cpu() - w).abs() / (1 + w.abs())).max().item() for i, w in zip(idx, want))
    err = max((outs[i].float().cpu() - w).abs().max().item() for i, w in zip(idx, want))
    assert rel <= 2e-2 and err <= 8e-2, (rel, err)
    assert not torch.isnan(got._buffer.float()).any()


def test_transformer_encoder_stack_from_token_ids(native_libs, cuda_device):
    """Embedding lookup on packed token ids, three encoder layers and a final LayerNorm, never padded; against the
    per-sequence fp32 oracle."""
    torch.manual_seed(21)
    V, E, H, F = 97, 64, 4, 128
    emb = torch.nn.Embedding(V, E)
    layer = torch.nn.TransformerEncoderLayer(E, H, dim_feedforward=F, dropout=0.0, activation=torch.nn.functional.relu)
    enc = torch.nn.TransformerEncoder(layer, num_layers=3, norm=torch.nn.LayerNorm(E), enable_nested_tensor=False).eval()
    g = torch.Generator().manual_seed(4)
    ids = [torch.randint(0, V, (int(l),), generator=g) for l in torch.randint(1, 90, (11,), generator=g)]
    want = ntref.embedding(ids, emb.weight.detach())
    for lyr in enc.layers:
        want = ntref.encoder_layer(want, H, _params(lyr), "relu", False, lyr.norm1.eps)
    want = ntref.layer_norm(want, (E,), enc.norm.weight.detach(), enc.norm.bias.detach(), enc.norm.eps)
    x = nt.nested_tensor(ids, device=cuda_device, dtype=torch.int64)
    got = nt.nn.transformer_encoder(enc.to(cuda_device), emb.to(cuda_device)(x))
    err = max((a.cpu() - b).abs().max().item() for a, b in zip(got.unbind(), want))
    assert err <= 3e-4, err

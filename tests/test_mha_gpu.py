"""Parity of the CUDA projection / varlen attention kernels and of the MHA operator with the fp32
oracle (oracle.ntref.min_mha = nestedtensor/csrc/mha.cpp:18-69).  Tolerances: max-abs 2e-2 for
fp16/bf16 and 1e-5 for fp32, against the oracle evaluated in fp32 on the same (cast) inputs."""
import ctypes

import pytest
import torch

import nestedtensor_b200 as nt
from nestedtensor_b200 import _cabi, workloads
from nestedtensor_b200.nested import build_meta
from oracle import ntref
from _helpers import stream_ptr

pytestmark = pytest.mark.gpu

CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
TOL = {torch.float32: 1e-5, torch.float16: 2e-2, torch.bfloat16: 2e-2}


def _gemm(A, W, bias, force_simt=0):
    lib = _cabi.load()
    M, K = A.shape
    N = W.shape[0]
    C = torch.empty(M, N, dtype=A.dtype, device=A.device)
    rc = lib.ntb200_gemm_bias(A.data_ptr(), W.data_ptr(), bias.data_ptr() if bias is not None else None, C.data_ptr(),
                              M, N, K, CODE[A.dtype], force_simt, stream_ptr())
    _cabi.check("ntb200_gemm_bias", rc)
    torch.cuda.synchronize()
    assert lib.ntb200_device_error_flags() == 0
    return C


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 512, 256), (1000, 3072, 1024), (129, 264, 72), (5, 8, 64),
                                   (4099, 1024, 1024), (20000, 768, 768)])
def test_gemm_bias_tensor_core(native_libs, cuda_device, dtype, M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    A = torch.randn(M, K, generator=g).to(dtype).to(cuda_device)
    W = (torch.randn(N, K, generator=g) * K ** -0.5).to(dtype).to(cuda_device)
    b = (torch.randn(N, generator=g) * 0.1).to(dtype).to(cuda_device)
    want = A.float() @ W.float().t() + b.float()
    for path, name in ((3, "CTA-pair tcgen05"), (2, "single-CTA tcgen05"), (1, "SIMT"), (0, "default")):
        got = _gemm(A, W, b, force_simt=path)
        err = (got.float() - want).abs().max().item()
        assert err <= 2e-2, "%s path max-abs %g" % (name, err)
    got3 = _gemm(A, W, None)
    assert (got3.float() - (want - b.float())).abs().max().item() <= 2e-2


@pytest.mark.parametrize("M,N,K", [(7, 5, 3), (130, 66, 100), (1000, 768, 256)])
def test_gemm_bias_fp32(native_libs, cuda_device, M, N, K):
    g = torch.Generator().manual_seed(M)
    A = torch.randn(M, K, generator=g).to(cuda_device)
    W = (torch.randn(N, K, generator=g) * K ** -0.5).to(cuda_device)
    b = torch.randn(N, generator=g).to(cuda_device)
    want = (A.double() @ W.double().t() + b.double()).float()
    got = _gemm(A, W, b)
    assert (got - want).abs().max().item() <= 1e-5


def _attention(qkv, lengths, H, d, path=0):
    """path 0 = best available, 1 = SIMT, 2 = mma.sync flash kernel, 3 = tcgen05 kernel"""
    lib = _cabi.load()
    E = H * d
    T = qkv.shape[0]
    sizes = torch.tensor([[l, E] for l in lengths], dtype=torch.int64)
    meta = build_meta(sizes, qkv.device)
    out = torch.full((T, E), float("nan"), dtype=qkv.dtype, device=qkv.device)
    nbytes = lib.ntb200_varlen_attention_workspace_bytes(len(lengths), T, H, d, CODE[qkv.dtype])
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=qkv.device)
    rc = lib.ntb200_varlen_attention(qkv.data_ptr(), out.data_ptr(), meta.data_ptr(), len(lengths), T, H, d, max(lengths),
                                     float(d) ** -0.5, CODE[qkv.dtype], path, ws.data_ptr() if nbytes else None, nbytes,
                                     stream_ptr())
    _cabi.check("ntb200_varlen_attention", rc)
    torch.cuda.synchronize()
    assert lib.ntb200_device_error_flags() == 0
    return out


def _attention_oracle(qkv, lengths, H, d):
    E = H * d
    x = qkv.float().cpu()
    out, off = [], 0
    for l in lengths:
        blk = x[off:off + l]
        q = blk[:, :E].reshape(l, H, d).transpose(0, 1) * float(d) ** -0.5
        k = blk[:, E:2 * E].reshape(l, H, d).transpose(0, 1)
        v = blk[:, 2 * E:].reshape(l, H, d).transpose(0, 1)
        w = torch.softmax(q @ k.transpose(1, 2), -1)
        out.append((w @ v).transpose(0, 1).reshape(l, E))
        off += l
    return torch.cat(out)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
def test_varlen_attention_d64(native_libs, cuda_device, dtype):
    lengths = [1, 63, 64, 65, 128, 200, 512, 7, 129, 16]
    H, d = 4, 64
    g = torch.Generator().manual_seed(4)
    qkv = torch.randn(sum(lengths), 3 * H * d, generator=g).to(dtype).to(cuda_device)
    want = _attention_oracle(qkv, lengths, H, d)
    for path, name in ((3, "tcgen05"), (2, "mma.sync"), (1, "SIMT"), (0, "default")):
        got = _attention(qkv, lengths, H, d, path=path)
        err = (got.float().cpu() - want).abs().max().item()
        assert err <= 2e-2, "%s attention max-abs %g" % (name, err)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
@pytest.mark.parametrize("H,d", [(8, 32), (3, 128), (1, 32)])
def test_varlen_attention_flash_other_head_dims(native_libs, cuda_device, dtype, H, d):
    """The mma.sync flash kernel at head_dim 32 and 128 (the default for these sizes), against the SIMT kernel's
    oracle."""
    lengths = [1, 63, 64, 65, 130, 200, 7, 16]
    g = torch.Generator().manual_seed(H * d)
    qkv = torch.randn(sum(lengths), 3 * H * d, generator=g).to(dtype).to(cuda_device)
    want = _attention_oracle(qkv, lengths, H, d)
    for path, name in ((2, "mma.sync"), (1, "SIMT"), (0, "default")):
        got = _attention(qkv, lengths, H, d, path=path)
        err = (got.float().cpu() - want).abs().max().item()
        assert err <= 2e-2, "%s attention max-abs %g" % (name, err)


@pytest.mark.parametrize("lengths", [[1], [128], [129], [256, 1, 255], [300, 512, 700, 1024, 33], [16] * 40 + [1000]],
                         ids=lambda l: "L" + "_".join(map(str, l[:5])))
def test_varlen_attention_tcgen05_lengths(native_libs, cuda_device, lengths):
    """Block boundaries (128 keys / 128 queries), multi-block online softmax and the work-list order."""
    H, d = 2, 64
    g = torch.Generator().manual_seed(sum(lengths))
    qkv = (torch.randn(sum(lengths), 3 * H * d, generator=g) * 1.5).to(torch.bfloat16).to(cuda_device)
    want = _attention_oracle(qkv, lengths, H, d)
    got = _attention(qkv, lengths, H, d, path=3)
    err = (got.float().cpu() - want).abs().max().item()
    assert err <= 2e-2, "tcgen05 attention max-abs %g" % err


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
@pytest.mark.parametrize("H,d", [(4, 64), (8, 32), (3, 128), (1, 64)])
@pytest.mark.parametrize("max_len", [16, 32, 9, 17])
def test_varlen_attention_short_sequences(native_libs, cuda_device, dtype, H, d, max_len):
    """Batches whose longest sequence has at most 32 tokens run on the warp-per-(sequence, head) kernel (path 4; the
    default picks it from max_len): every length from 1 to max_len, against the oracle and the SIMT kernel."""
    g = torch.Generator().manual_seed(100 * max_len + d)
    lengths = list(range(1, max_len + 1)) + [max_len, 1, 7, max_len, 2]
    lengths = [lengths[i] for i in torch.randperm(len(lengths), generator=g).tolist()]
    qkv = (torch.randn(sum(lengths), 3 * H * d, generator=g) * 1.5).to(dtype).to(cuda_device)
    want = _attention_oracle(qkv, lengths, H, d)
    got = {}
    for path, name in ((4, "warp per (sequence, head)"), (0, "default"), (1, "SIMT")):
        got[path] = _attention(qkv, lengths, H, d, path=path)
        err = (got[path].float().cpu() - want).abs().max().item()
        assert err <= 2e-2, "%s attention max-abs %g" % (name, err)
    assert torch.equal(got[0].view(torch.int16), got[4].view(torch.int16)), "the default did not take the short-sequence kernel"


def test_varlen_attention_short_sequences_large_batch(native_libs, cuda_device):
    """30 000 sequences of 1..8 tokens, 16 heads x 64: more (sequence, head) pairs than one grid dimension of the
    other kernels holds; compared on the GPU with the SIMT kernel."""
    H, d = 16, 64
    g = torch.Generator().manual_seed(8)
    lengths = torch.randint(1, 9, (30000,), generator=g).tolist()
    qkv = torch.randn(sum(lengths), 3 * H * d, generator=g).to(torch.bfloat16).to(cuda_device)
    got = _attention(qkv, lengths, H, d, path=0)
    ref = _attention(qkv, lengths, H, d, path=1)
    assert bool(torch.isfinite(got.float()).all())
    assert (got.float() - ref.float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
def test_varlen_attention_mostly_short_sequences(native_libs, cuda_device, dtype):
    """Mostly short sequences with a few longer ones: the default splits the batch between the warp-per-(sequence,
    head) kernel (at most 32 tokens) and the tcgen05 work list (the rest); every row must be written exactly once
    and agree with the SIMT kernel and, for a sample, with the oracle."""
    H, d = 4, 64
    g = torch.Generator().manual_seed(77)
    lengths = torch.randint(1, 33, (1500,), generator=g).tolist()
    for pos, l in ((3, 100), (700, 300), (701, 64), (1200, 33), (1499, 40), (0, 32)):
        lengths[pos] = l
    qkv = (torch.randn(sum(lengths), 3 * H * d, generator=g) * 1.5).to(dtype).to(cuda_device)
    got = _attention(qkv, lengths, H, d, path=0)
    ref = _attention(qkv, lengths, H, d, path=1)
    assert bool(torch.isfinite(got.float()).all()), "rows left unwritten"
    # two 16-bit roundings of one value may lie an ulp apart (0.031 for values of 4..8): the 2e-2 bar is the one against
    # the fp32 oracle, checked below on the first 300 sequences (among them the long ones at 3 and 0)
    assert (got.float() - ref.float()).abs().max().item() <= 4e-2
    only_tc = _attention(qkv, lengths, H, d, path=3)
    assert (got.float() - only_tc.float()).abs().max().item() <= 4e-2
    head = sum(lengths[:300])
    want = _attention_oracle(qkv[:head], lengths[:300], H, d)
    assert (got[:head].float().cpu() - want).abs().max().item() <= 2e-2
    tail = sum(lengths[:-300])
    want = _attention_oracle(qkv[tail:], lengths[-300:], H, d)
    assert (got[tail:].float().cpu() - want).abs().max().item() <= 2e-2


def test_varlen_attention_default_path_random_sweep(native_libs, cuda_device):
    """100 random batches (1 to 3000 sequences of 1 to 600 tokens, head sizes 32 / 64 / 128, 1 to 20 heads, fp16 / bf16,
    with and without a workspace) through the default path, whatever kernels it picks, against the SIMT kernel's
    fp32 arithmetic on the GPU: every row written, within the 16-bit bar relative to the largest output."""
    lib = _cabi.load()
    for seed in range(100):
        g = torch.Generator().manual_seed(55000 + seed)
        r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
        dtype, code = [(torch.bfloat16, 2), (torch.float16, 1)][r(0, 1)]
        d = [64, 64, 64, 32, 128][r(0, 4)]
        H = [1, 2, 3, 8, 16, 20][r(0, 5)]
        B = [1, 2, 5, r(6, 40), r(41, 300), r(500, 3000)][r(0, 5)]
        hi = [4, 16, 32, 33, 64, 130, 300, 600][r(0, 7)]
        if B > 300:
            hi = min(hi, 64)
        L = torch.randint(1, hi + 1, (B,), generator=g).tolist()
        if r(0, 3) == 0:
            L[r(0, B - 1)] = hi
        E, T = H * d, sum(L)
        qkv = (torch.randn(T, 3 * E, generator=g) * [0.5, 1.0, 2.0][r(0, 2)]).to(dtype).to(cuda_device)
        meta = build_meta(torch.tensor([[l, E] for l in L]), cuda_device)
        nb = lib.ntb200_varlen_attention_workspace_bytes(B, T, H, d, code)
        use_ws = nb > 0 and r(0, 4) != 0
        ws = torch.empty(max(nb, 16), dtype=torch.uint8, device=cuda_device)
        outs = {}
        for path in (0, 1):
            out = torch.full((T, E), float("nan"), dtype=dtype, device=cuda_device)
            _cabi.check("ntb200_varlen_attention",
                        lib.ntb200_varlen_attention(qkv.data_ptr(), out.data_ptr(), meta.data_ptr(), B, T, H, d, max(L), d ** -0.5, code,
                                                    path, ws.data_ptr() if use_ws else None, nb if use_ws else 0, stream_ptr()))
            torch.cuda.synchronize()
            outs[path] = out.float()
        tag = "seed %d %s d=%d H=%d B=%d longest %d workspace %s" % (seed, dtype, d, H, B, max(L), use_ws)
        assert bool(torch.isfinite(outs[0]).all()), "rows left unwritten: " + tag
        bar = 2e-2 * max(1.0, float(outs[1].abs().max()))
        assert float((outs[0] - outs[1]).abs().max()) <= bar, tag
    assert lib.ntb200_device_error_flags() == 0


UNSUPPORTED_SHAPE = -7  # NTB200_UNSUPPORTED_SHAPE


def test_varlen_attention_short_sequence_kernel_limits(native_libs, cuda_device):
    """Path 4 refuses a batch whose longest sequence exceeds 32 tokens, fp32 data and other head sizes; a non-finite
    value stays inside its sequence."""
    lib = _cabi.load()
    H, d = 2, 64
    E = H * d

    def call(qkv, lengths, max_len, code, path, head_dim=d, heads=H):
        meta = build_meta(torch.tensor([[l, heads * head_dim] for l in lengths], dtype=torch.int64), cuda_device)
        out = torch.full((sum(lengths), heads * head_dim), float("nan"), dtype=qkv.dtype, device=cuda_device)
        rc = lib.ntb200_varlen_attention(qkv.data_ptr(), out.data_ptr(), meta.data_ptr(), len(lengths), sum(lengths), heads, head_dim,
                                         max_len, head_dim ** -0.5, code, path, None, 0, stream_ptr())
        torch.cuda.synchronize()
        return rc, out

    lengths = [5, 33, 2]
    qkv = torch.randn(sum(lengths), 3 * E).to(torch.bfloat16).to(cuda_device)
    assert call(qkv, lengths, 33, 2, 4)[0] == UNSUPPORTED_SHAPE
    assert call(qkv.float(), [5, 7, 2], 7, 0, 4)[0] == UNSUPPORTED_SHAPE
    q40 = torch.randn(14, 3 * 2 * 40).to(torch.bfloat16).to(cuda_device)
    assert call(q40, [5, 7, 2], 7, 2, 4, head_dim=40)[0] == UNSUPPORTED_SHAPE
    for bad in (float("nan"), float("inf")):
        lengths = [7, 16, 3, 32, 1, 20]
        x = torch.randn(sum(lengths), 3 * E)
        x[7:23] = bad  # every token of sequence 1
        rc, out = call(x.to(torch.bfloat16).to(cuda_device), lengths, 32, 2, 4)
        assert rc == 0
        off = 0
        for b, l in enumerate(lengths):
            if b != 1:
                assert bool(torch.isfinite(out[off:off + l].float()).all()), "sequence %d picked up a non-finite value" % b
            off += l


@pytest.mark.parametrize("H", [1, 3, 7, 40, 300])
def test_varlen_attention_tcgen05_head_counts(native_libs, cuda_device, H):
    """The persistent kernel steps through the flattened (item, head) list by its grid size: head counts that do not
    divide it, exceed it, or equal 1."""
    d = 64
    lengths = [5, 130, 64, 1, 257] if H < 100 else [5, 70]
    g = torch.Generator().manual_seed(H)
    qkv = torch.randn(sum(lengths), 3 * H * d, generator=g).to(torch.bfloat16).to(cuda_device)
    want = _attention_oracle(qkv, lengths, H, d)
    got = _attention(qkv, lengths, H, d, path=3)
    assert (got.float().cpu() - want).abs().max().item() <= 2e-2


@pytest.mark.parametrize("H,d", [(2, 1), (1, 4), (2, 2), (8, 16), (4, 256), (3, 40), (16, 64)])
def test_varlen_attention_fp32(native_libs, cuda_device, H, d):
    lengths = [5, 1, 33, 50, 2, 64, 100]
    g = torch.Generator().manual_seed(H * 100 + d)
    qkv = torch.randn(sum(lengths), 3 * H * d, generator=g).to(cuda_device)
    want = _attention_oracle(qkv, lengths, H, d)
    got = _attention(qkv, lengths, H, d)
    assert (got.cpu() - want).abs().max().item() <= 1e-5


def _run_mha(tensors, H, w, dtype, device):
    a = nt.nested_tensor(tensors, device=device, dtype=dtype)
    E = tensors[0].shape[1]
    d = E // H
    wd = {k: v.to(dtype).to(device) for k, v in w.items()}
    out = torch.ops.nestedtensor.bt_min_mha(H, d, 0.5, False, a, a, a, wd["in_proj_weight"], wd["in_proj_bias"],
                                            float(d) ** -0.5, wd["out_proj_weight"], wd["out_proj_bias"])
    torch.cuda.synchronize()
    assert _cabi.load().ntb200_device_error_flags() == 0
    cast = [t.to(dtype) for t in tensors]
    wc = {k: v.to(dtype) for k, v in w.items()}
    want = ntref.min_mha(H, d, cast, cast, cast, wc["in_proj_weight"], wc["in_proj_bias"], float(d) ** -0.5,
                         wc["out_proj_weight"], wc["out_proj_bias"])
    return out, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=str)
@pytest.mark.parametrize("H,B,Lmax,d", [(2, 1, 2, 1), (1, 3, 5, 4), (2, 3, 5, 2), (2, 1, 2, 2), (8, 8, 50, 16),
                                         (16, 64, 50, 16), (16, 128, 50, 16), (4, 64, 50, 256), (16, 64, 50, 64)])
def test_bt_min_mha_reference_shapes(native_libs, cuda_device, dtype, H, B, Lmax, d):
    """Shape list of test/test_nested_tensor_functional.py:1149-1161 (largest batches reduced to keep the CPU
    oracle in seconds)."""
    g = torch.Generator().manual_seed(1010 + H + B + d)
    E = H * d
    tensors = [torch.randn(int(torch.randint(1, Lmax + 1, (1,), generator=g)), E, generator=g) for _ in range(B)]
    w = {"in_proj_weight": torch.randn(3 * E, E, generator=g) * E ** -0.5,
         "in_proj_bias": torch.randn(3 * E, generator=g) * 0.02,
         "out_proj_weight": torch.randn(E, E, generator=g) * E ** -0.5,
         "out_proj_bias": torch.randn(E, generator=g) * 0.02}
    out, want = _run_mha(tensors, H, w, dtype, cuda_device)
    assert out.nested_size() == tuple(torch.Size(t.shape) for t in tensors)
    for o, r in zip(out.unbind(), want):
        err = (o.float().cpu() - r).abs().max().item()
        assert err <= TOL[dtype], "max-abs %g" % err


def test_config4_bert_base_fp16(native_libs, cuda_device):
    """Configuration 4: batch 128, L ~ U[32,512], E=768, 12 heads x 64, fp16, non-zero biases."""
    w = workloads.config4()
    tensors = w.tensors()
    out, want = _run_mha([t.float() for t in tensors], 12, {k: v.float() for k, v in w.weights.items()}, torch.float16,
                         cuda_device)
    worst = max((o.float().cpu() - r).abs().max().item() for o, r in zip(out.unbind(), want))
    assert worst <= 2e-2, "max-abs %g" % worst


def test_config5_bert_large_bf16_sampled(native_libs, cuda_device):
    """Configuration 5 at full size on the GPU (batch 1024, bf16, E=1024, 16 x 64); the fp32 oracle is
    evaluated on every 16th sequence only (sequences are independent)."""
    w = workloads.config5()
    a = nt.NestedTensor(w.buffer.to(cuda_device), w.sizes)
    wd = {k: v.to(cuda_device) for k, v in w.weights.items()}
    mha = nt.nn.MultiheadAttention(1024, 16).to(torch.bfloat16).to(cuda_device)
    with torch.no_grad():
        mha.in_proj_weight.copy_(wd["in_proj_weight"])
        mha.in_proj_bias.copy_(wd["in_proj_bias"])
        mha.out_proj.weight.copy_(wd["out_proj_weight"])
        mha.out_proj.bias.copy_(wd["out_proj_bias"])
        out, none = mha(a, a, a, need_weights=False)
    assert none is None
    torch.cuda.synchronize()
    assert _cabi.load().ntb200_device_error_flags() == 0
    tensors = w.tensors()
    idx = list(range(0, w.batch, 16))
    sample = [tensors[i] for i in idx]
    want = ntref.min_mha(16, 64, sample, sample, sample, w.weights["in_proj_weight"], w.weights["in_proj_bias"],
                         64 ** -0.5, w.weights["out_proj_weight"], w.weights["out_proj_bias"])
    outs = out.unbind()
    worst = max((outs[i].float().cpu() - r).abs().max().item() for i, r in zip(idx, want))
    assert worst <= 2e-2, "max-abs %g" % worst


def test_stock_module_matches_dense_attention(native_libs, cuda_device):
    """test/test_nested_tensor_functional.py:1103-1140: stock torch.nn.MultiheadAttention on NestedTensor inputs
    equals the dense module with key_padding_mask on the zero-padded batch (atol 5e-4, fp32)."""
    torch.manual_seed(1010)
    E, H = 128, 8
    g = torch.Generator().manual_seed(5)
    tensors = [torch.randn(int(torch.randint(1, 51, (1,), generator=g)), E, generator=g) for _ in range(8)]
    a = nt.nested_tensor(tensors, device=cuda_device, dtype=torch.float32)
    mha = torch.nn.MultiheadAttention(E, H).to(cuda_device).eval()
    with torch.no_grad():
        mha.in_proj_bias.normal_(0, 0.02)
        mha.out_proj.bias.normal_(0, 0.02)
        got, _ = mha(a, a, a, need_weights=False)
        data, mask = a.to_tensor_mask(mask_dim=2)
        x = data.transpose(0, 1)
        dense, _ = mha(x, x, x, key_padding_mask=~mask, need_weights=False)
    dense = dense.transpose(0, 1) * mask.unsqueeze(-1)
    assert torch.allclose(got.to_padded_tensor(padding=0), dense, atol=5e-4, rtol=1e-8)


@pytest.mark.parametrize("dtype,E,H", [(torch.float32, 8, 2), (torch.float32, 96, 3), (torch.bfloat16, 128, 2), (torch.float16, 256, 4),
                                       (torch.float16, 256, 8), (torch.bfloat16, 256, 2)], ids=str)
@pytest.mark.parametrize("separate_value", [False, True])
def test_cross_attention_matches_oracle(native_libs, cuda_device, dtype, E, H, separate_value):
    """query != key (a DETR-style decoder: a fixed number of object queries per image over a ragged memory,
    test/test_nested_tensor_functional.py:960-1032), with key == value and with a separate value tensor,
    against min_mha (nestedtensor/csrc/mha.cpp:18-69) in fp32."""
    g = torch.Generator().manual_seed(E + int(separate_value))
    lk = [int(v) for v in torch.randint(1, 150, (9,), generator=g)]
    lq = [10, 10, 10, 10, 1, 70, 10, 129, 10]
    qs = [torch.randn(l, E, generator=g).to(dtype) for l in lq]
    ks = [torch.randn(l, E, generator=g).to(dtype) for l in lk]
    vs = [torch.randn(l, E, generator=g).to(dtype) for l in lk] if separate_value else ks
    torch.manual_seed(1)
    mha = torch.nn.MultiheadAttention(E, H).eval().to(dtype).to(cuda_device)
    q = nt.nested_tensor(qs, device=cuda_device, dtype=dtype)
    k = nt.nested_tensor(ks, device=cuda_device, dtype=dtype)
    v = nt.nested_tensor(vs, device=cuda_device, dtype=dtype) if separate_value else k
    with torch.no_grad():
        got, _ = mha(q, k, v, need_weights=False)
    assert got.nested_size() == q.nested_size()
    want = ntref.min_mha(H, E // H, qs, ks, vs, mha.in_proj_weight.cpu(), mha.in_proj_bias.cpu(), float(E // H) ** -0.5,
                         mha.out_proj.weight.cpu(), mha.out_proj.bias.cpu())
    err = max((a.float().cpu() - b).abs().max().item() for a, b in zip(got.unbind(), want))
    assert err <= TOL[dtype], err


@pytest.mark.parametrize("dtype,E,H", [(torch.float32, 96, 3), (torch.bfloat16, 128, 2), (torch.float16, 256, 8)], ids=str)
@pytest.mark.parametrize("cross", [False, True])
@pytest.mark.parametrize("average", [True, False])
def test_need_weights_returns_the_attention_probabilities(native_libs, cuda_device, dtype, E, H, cross, average):
    """need_weights=True: one (L_q, L_k) matrix per sequence (averaged over the heads) or (H, L_q, L_k), against the
    oracle; the oracle itself is pinned to stock torch.nn.MultiheadAttention(need_weights=True) run per sequence."""
    g = torch.Generator().manual_seed(E + 2 * int(cross))
    lq = [7, 1, 130, 33, 64]
    lk = [int(v) for v in torch.randint(1, 200, (5,), generator=g)] if cross else lq
    qs = [torch.randn(l, E, generator=g).to(dtype) for l in lq]
    ks = [torch.randn(l, E, generator=g).to(dtype) for l in lk] if cross else qs
    torch.manual_seed(2)
    mha = torch.nn.MultiheadAttention(E, H).eval().to(dtype).to(cuda_device)
    with torch.no_grad():
        mha.in_proj_bias.normal_(0, 0.05)
    q = nt.nested_tensor(qs, device=cuda_device, dtype=dtype)
    k = nt.nested_tensor(ks, device=cuda_device, dtype=dtype) if cross else q
    with torch.no_grad():
        out, w = mha(q, k, k, need_weights=True, average_attn_weights=average)
    assert out.nested_size() == q.nested_size()
    want = ntref.mha_weights(H, E // H, qs, ks, mha.in_proj_weight.cpu(), mha.in_proj_bias.cpu(), float(E // H) ** -0.5, average)
    got = w.unbind()
    assert len(got) == len(want)
    for a, b in zip(got, want):
        assert tuple(a.shape) == tuple(b.shape)
        assert (a.float().cpu() - b).abs().max().item() <= (1e-5 if dtype == torch.float32 else 4e-3)
        assert abs(float(a.float().sum(-1).mean()) - 1.0) <= (1e-4 if dtype == torch.float32 else 1e-2)
    if dtype == torch.float32:  # pin the oracle to the stock module, one sequence at a time
        cpu = torch.nn.MultiheadAttention(E, H).eval()
        cpu.load_state_dict({n: p.cpu() for n, p in mha.state_dict().items()})
        with torch.no_grad():
            for xq, xk, b in zip(qs, ks, want):
                _, ws = cpu(xq.unsqueeze(1), xk.unsqueeze(1), xk.unsqueeze(1), need_weights=True, average_attn_weights=average)
                assert torch.allclose(ws[0], b, atol=2e-6)


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, 2), (torch.float16, 1)], ids=["bf16", "f16"])
@pytest.mark.parametrize("packed_kv", [True, False])
def test_cabi_cross_attention_tcgen05_against_simt(native_libs, cuda_device, dtype, code, packed_kv):
    """The tcgen05 kernel with separate query / key / value tensor maps (path 3) against the SIMT kernel (path 1):
    query tiles of more than 128 rows, key sequences of one to several blocks, a sequence without keys (zeros), one
    without queries, and k / v either as the halves of one [Tk, 2E] matrix or as two matrices."""
    lib = _cabi.load()
    H, d = 4, 64
    E = H * d
    g = torch.Generator().manual_seed(77 + int(packed_kv))
    lq = [5, 300, 0, 129, 64, 100, 1]
    lk = [700, 33, 50, 0, 128, 129, 1]
    B, Tq, Tk = len(lq), sum(lq), sum(lk)
    q = torch.randn(Tq, E, generator=g).to(dtype).to(cuda_device)
    if packed_kv:
        kv = torch.randn(Tk, 2 * E, generator=g).to(dtype).to(cuda_device)
        kp, vp, ld = kv.data_ptr(), kv.data_ptr() + E * 2, 2 * E
    else:
        k = torch.randn(Tk, E, generator=g).to(dtype).to(cuda_device)
        v = torch.randn(Tk, E, generator=g).to(dtype).to(cuda_device)
        kp, vp, ld = k.data_ptr(), v.data_ptr(), E
    mq = build_meta(torch.tensor([[l, E] for l in lq]), cuda_device)
    mk = build_meta(torch.tensor([[l, E] for l in lk]), cuda_device)
    nb = lib.ntb200_varlen_cross_attention_workspace_bytes(B, Tq, H, d, code)
    assert nb > 0
    ws = torch.empty(nb, dtype=torch.uint8, device=cuda_device)
    outs = []
    for path in (3, 1):
        o = torch.full((Tq, E), 7.0, dtype=dtype, device=cuda_device)
        rc = lib.ntb200_varlen_cross_attention_ws(q.data_ptr(), E, kp, ld, vp, ld, o.data_ptr(), mq.data_ptr(), mk.data_ptr(), B, Tq, Tk,
                                                  H, d, max(lq), d ** -0.5, code, path, ws.data_ptr(), nb, stream_ptr())
        _cabi.check("ntb200_varlen_cross_attention_ws", rc)
        outs.append(o)
    torch.cuda.synchronize()
    assert lib.ntb200_device_error_flags() == 0
    assert (outs[0].float() - outs[1].float()).abs().max().item() <= 2e-2
    off = sum(lq[:3])
    assert int(outs[0][off:off + lq[3]].count_nonzero()) == 0  # the sequence without keys
    # too small a workspace is refused, nothing is launched
    assert lib.ntb200_varlen_cross_attention_ws(q.data_ptr(), E, kp, ld, vp, ld, outs[0].data_ptr(), mq.data_ptr(), mk.data_ptr(), B, Tq, Tk,
                                                H, d, max(lq), d ** -0.5, code, 3, ws.data_ptr(), 16, stream_ptr()) == -6


def test_cabi_cross_attention_random_sweep(native_libs, cuda_device):
    """100 random cross-attention batches (1 to 400 sequences, up to 300 queries over up to 900 keys, sequences without
    keys or without queries, head sizes 32 / 64 / 128, k / v packed in one matrix or apart): every kernel that takes the
    shape (default, mma.sync, tcgen05) against the SIMT kernel; rows of a sequence without keys are zeros."""
    lib = _cabi.load()
    for seed in range(100):
        g = torch.Generator().manual_seed(66000 + seed)
        r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
        dtype, code = [(torch.bfloat16, 2), (torch.float16, 1)][r(0, 1)]
        d, H = [64, 64, 32, 128][r(0, 3)], [1, 2, 4, 8, 11][r(0, 4)]
        E = H * d
        B = [1, 2, r(3, 10), r(11, 60), r(100, 400)][r(0, 4)]
        hq, hk = [3, 40, 130, 300][r(0, 3)], [3, 40, 130, 300, 900][r(0, 4)]
        if B >= 100:
            hq, hk = min(hq, 130), min(hk, 130)
        lq = [0 if r(0, 14) == 0 else r(1, hq) for _ in range(B)]
        lk = [0 if r(0, 14) == 0 else r(1, hk) for _ in range(B)]
        lq[0], lk[0] = max(lq[0], 1), max(lk[0], 1)
        Tq, Tk = sum(lq), sum(lk)
        q = torch.randn(Tq, E, generator=g).to(dtype).to(cuda_device)
        if r(0, 1):
            kv = torch.randn(Tk, 2 * E, generator=g).to(dtype).to(cuda_device)
            kp, vp, ld = kv.data_ptr(), kv.data_ptr() + E * 2, 2 * E
        else:
            k = torch.randn(Tk, E, generator=g).to(dtype).to(cuda_device)
            v = torch.randn(Tk, E, generator=g).to(dtype).to(cuda_device)
            kp, vp, ld = k.data_ptr(), v.data_ptr(), E
        mq = build_meta(torch.tensor([[l, E] for l in lq]), cuda_device)
        mk = build_meta(torch.tensor([[l, E] for l in lk]), cuda_device)
        nb = lib.ntb200_varlen_cross_attention_workspace_bytes(B, Tq, H, d, code)
        ws = torch.empty(max(nb, 16), dtype=torch.uint8, device=cuda_device)
        outs = {}
        for path in (1, 0, 2, 3):
            o = torch.full((Tq, E), float("nan"), dtype=dtype, device=cuda_device)
            rc = lib.ntb200_varlen_cross_attention_ws(q.data_ptr(), E, kp, ld, vp, ld, o.data_ptr(), mq.data_ptr(), mk.data_ptr(), B, Tq,
                                                      Tk, H, d, max(lq), d ** -0.5, code, path, ws.data_ptr() if nb else None, nb,
                                                      stream_ptr())
            torch.cuda.synchronize()
            if rc == UNSUPPORTED_SHAPE and path >= 2:
                continue
            _cabi.check("ntb200_varlen_cross_attention_ws", rc)
            outs[path] = o.float()
        tag = "seed %d %s d %d H %d B %d" % (seed, dtype, d, H, B)
        for path, o in outs.items():
            assert bool(torch.isfinite(o).all()), "rows left unwritten, path %d, %s" % (path, tag)
            assert float((o - outs[1]).abs().max()) <= 2e-2 * max(1.0, float(outs[1].abs().max())), "path %d, %s" % (path, tag)
        off = 0
        for b in range(B):
            if lk[b] == 0 and lq[b] > 0:
                assert int(outs[0][off:off + lq[b]].count_nonzero()) == 0, tag
            off += lq[b]
    assert lib.ntb200_device_error_flags() == 0


def test_cabi_cross_attention_paths_and_empty_key_sequence(native_libs, cuda_device):
    """SIMT and mma.sync kernels agree with plain torch; a query whose key sequence is empty gets zeros."""
    lib = _cabi.load()
    H, d = 2, 64
    E = H * d
    g = torch.Generator().manual_seed(9)
    lq, lk = [5, 70, 3], [33, 0, 129]
    q = torch.randn(sum(lq), E, generator=g).to(torch.bfloat16).to(cuda_device)
    kv = torch.randn(sum(lk), 2 * E, generator=g).to(torch.bfloat16).to(cuda_device)
    mq = build_meta(torch.tensor([[l, E] for l in lq]), cuda_device)
    mk = build_meta(torch.tensor([[l, E] for l in lk]), cuda_device)
    want, oq, ok = [], 0, 0
    for a, b in zip(lq, lk):
        qq = q[oq:oq + a].float().reshape(a, H, d).transpose(0, 1) * d ** -0.5
        kk = kv[ok:ok + b, :E].float().reshape(b, H, d).transpose(0, 1)
        vv = kv[ok:ok + b, E:].float().reshape(b, H, d).transpose(0, 1)
        o = torch.softmax(qq @ kk.transpose(1, 2), -1) @ vv if b > 0 else torch.zeros(H, a, d, device=cuda_device)
        want.append(o.transpose(0, 1).reshape(a, E))
        oq += a
        ok += b
    want = torch.cat(want)
    for path in (1, 2, 0):
        out = torch.full((sum(lq), E), float("nan"), dtype=torch.bfloat16, device=cuda_device)
        rc = lib.ntb200_varlen_cross_attention(q.data_ptr(), E, kv.data_ptr(), 2 * E, kv.data_ptr() + 2 * E, 2 * E, out.data_ptr(),
                                               mq.data_ptr(), mk.data_ptr(), 3, sum(lq), H, d, max(lq), d ** -0.5, 2, path,
                                               stream_ptr())
        _cabi.check("ntb200_varlen_cross_attention", rc)
        torch.cuda.synchronize()
        assert (out.float() - want).abs().max().item() <= 2e-2, path


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=str)
def test_reference_shaped_helpers(native_libs, cuda_device, dtype):
    """add_qkv_bias_pad / transpose_rm_padding / softmax_masked against plain torch."""
    lib = _cabi.load()
    H, d = 3, 8
    E = H * d
    lengths = [4, 1, 6, 3]
    B, T, maxL = len(lengths), sum(lengths), max(lengths)
    g = torch.Generator().manual_seed(9)
    qkv = torch.randn(T, 3 * E, generator=g).to(dtype).to(cuda_device)
    bias = torch.randn(3 * E, generator=g).to(dtype).to(cuda_device)
    meta = build_meta(torch.tensor([[l, E] for l in lengths], dtype=torch.int64), cuda_device)
    bufs = [torch.zeros(B, H, maxL, d, dtype=dtype, device=cuda_device) for _ in range(3)]
    rc = lib.ntb200_add_qkv_bias_pad(qkv.data_ptr(), bias.data_ptr(), bufs[0].data_ptr(), bufs[1].data_ptr(),
                                     bufs[2].data_ptr(), meta.data_ptr(), B, T, H, d, maxL, CODE[dtype], stream_ptr())
    _cabi.check("ntb200_add_qkv_bias_pad", rc)
    torch.cuda.synchronize()
    biased = (qkv.float() + bias.float()).to(dtype)
    off = 0
    for b, l in enumerate(lengths):
        for which in range(3):
            want = biased[off:off + l, which * E:(which + 1) * E].reshape(l, H, d).transpose(0, 1)
            assert torch.equal(bufs[which][b, :, :l], want)
            assert bool((bufs[which][b, :, l:] == 0).all())
        off += l
    back = torch.empty(T, E, dtype=dtype, device=cuda_device)
    rc = lib.ntb200_transpose_rm_padding(bufs[0].data_ptr(), back.data_ptr(), meta.data_ptr(), B, T, H, d, maxL,
                                         CODE[dtype], stream_ptr())
    _cabi.check("ntb200_transpose_rm_padding", rc)
    torch.cuda.synchronize()
    assert torch.equal(back, biased[:, :E])
    # masked softmax with the reference's arithmetic
    scores = torch.randn(B, H, maxL, maxL, generator=g).to(dtype).to(cuda_device)
    m = torch.zeros(B, maxL)
    for b, l in enumerate(lengths):
        m[b, :l] = 1
    want = ntref.masked_softmax(scores.cpu(), m.unsqueeze(1) * m.unsqueeze(2), 0.35)
    rc = lib.ntb200_softmax_masked(scores.data_ptr(), meta.data_ptr(), E, B, H, maxL, maxL, 0.35, CODE[dtype], stream_ptr())
    _cabi.check("ntb200_softmax_masked", rc)
    torch.cuda.synchronize()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for b, l in enumerate(lengths):
        assert (scores[b, :, :l, :l].float().cpu() - want[b, :, :l, :l]).abs().max().item() <= tol


def test_offsets_scan_and_token_index(native_libs, cuda_device):
    """Device-side offsets (exclusive scan, with and without the block-sum workspace) and token index."""
    for B in (1, 7, 1024, 1025, 5000, 70000):
        g = torch.Generator().manual_seed(B)
        sizes = torch.randint(0, 9, (B, 2), generator=g)
        d_sizes = sizes.to(cuda_device)
        meta = torch.ops.nestedtensor.meta_from_device_sizes(d_sizes)
        want = build_meta(sizes, "cpu")
        assert torch.equal(meta.cpu(), want)
    lengths = torch.tensor([3, 0, 5, 1, 0, 2])
    offs = torch.cat([torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)]).to(cuda_device)
    bi, wi = torch.ops.nestedtensor.token_index(offs, int(lengths.sum()))
    assert bi.cpu().tolist() == [0, 0, 0, 2, 2, 2, 2, 2, 3, 5, 5]
    assert wi.cpu().tolist() == [0, 1, 2, 0, 1, 2, 3, 4, 0, 0, 1]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32, torch.uint8],
                         ids=str)
def test_sizes_from_padded_semantics(native_libs, cuda_device, dtype):
    """`tensor != padding` follows the dtype's comparison: -0.0 counts as padding 0.0, NaN never does."""
    t = torch.zeros(3, 4, 6, dtype=dtype)
    t[0, :2, :3] = 1
    t[1, :4, :6] = 2
    t[2, :1, :1] = 3
    if dtype.is_floating_point:
        t[0, 3, 5] = -0.0            # still padding
    a = nt.nested_tensor_from_padded_tensor(t.to(cuda_device), padding=0)
    assert a.nested_size() == (torch.Size([2, 3]), torch.Size([4, 6]), torch.Size([1, 1]))
    if dtype.is_floating_point:
        t2 = t.clone()
        t2[2, 0, 1] = float("nan")   # NaN != 0 -> valid
        b = nt.nested_tensor_from_padded_tensor(t2.to(cuda_device), padding=0)
        assert b.nested_size()[2] == torch.Size([1, 2])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32, torch.uint8],
                         ids=str)
@pytest.mark.parametrize("odd", [0, 3])
def test_sizes_from_padded_semantics_long_rows(native_libs, cuda_device, dtype, odd):
    """The same comparison rules in the warp-per-row scan (rows of 3.3 KB; three elements less: rows that start at
    every phase of a 16-byte vector): -0.0 is padding 0.0, NaN is never padding, a NaN padding value matches nothing,
    and a box that holds the padding value inside is refused."""
    width = 3328 // torch.empty(0, dtype=dtype).element_size() - odd
    t = torch.zeros(3, 4, width, dtype=dtype)
    t[0, :2, :333] = 1
    t[1, :4, :width] = 2
    t[2, :1, :17] = 3
    if dtype.is_floating_point:
        t[0, 3, width - 1] = -0.0    # still padding
    a = nt.nested_tensor_from_padded_tensor(t.to(cuda_device), padding=0)
    assert a.nested_size() == (torch.Size([2, 333]), torch.Size([4, width]), torch.Size([1, 17]))
    assert_close_bits = torch.equal(a.unbind()[0].cpu(), t[0, :2, :333])
    assert assert_close_bits
    if dtype.is_floating_point:
        t2 = t.clone()
        t2[2, 0, 17] = float("nan")  # NaN != 0 -> valid
        b = nt.nested_tensor_from_padded_tensor(t2.to(cuda_device), padding=0)
        assert b.nested_size()[2] == torch.Size([1, 18])
        c = nt.nested_tensor_from_padded_tensor(t.to(cuda_device), padding=float("nan"))
        assert c.nested_size() == (torch.Size([4, width]),) * 3
    t3 = t.clone()
    t3[1, 2, 100] = 0                # a padding value inside the box
    with pytest.raises(RuntimeError, match="not a padding mask"):
        nt.nested_tensor_from_padded_tensor(t3.to(cuda_device), padding=0)

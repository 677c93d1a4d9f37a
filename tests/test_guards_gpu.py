"""Write-side checks that stand in for a memory checker: every C-ABI output below is a view into a larger
allocation with 256 guard bytes of a known pattern on either side, and the guards must be untouched after
the call.  The boundary passes of the copy kernels, the 32-byte stores of the tcgen05 epilogues and the
ragged last tiles are where an overrun by one vector would not show in a value comparison.

Also here: the data + mask single-pass kernel at every element width, the tcgen05 attention against the
SIMT fp32-math path on every sequence of configuration 5, a non-finite value in a neighbouring sequence,
the reference-shaped helper kernels at BERT-sized shapes, a second device in the same process, and the
NCCL verification gather on two GPUs (the last two are skipped when the machine shows fewer than two).
"""
import ctypes
import math
import os
import subprocess
import sys

import pytest
import torch

import nestedtensor_b200 as nt
from nestedtensor_b200 import _cabi, workloads
from nestedtensor_b200.nested import build_meta
from oracle import ntref
from _helpers import assert_bit_equal, bits_of, fold, random_list, sizes_of, stream_ptr

pytestmark = pytest.mark.gpu

GUARD = 256
PATTERN = 0xA5


class Guarded:
    """A tensor of `shape` / `dtype` placed between two guard regions of one uint8 allocation."""

    def __init__(self, shape, dtype, device, fill=None):
        n = int(math.prod(shape)) if len(shape) else 1
        es = torch.empty(0, dtype=dtype).element_size()
        body = (n * es + 15) // 16 * 16
        self.raw = torch.full((GUARD + body + GUARD,), PATTERN, dtype=torch.uint8, device=device)
        self.nbytes = n * es
        self.t = self.raw[GUARD:GUARD + n * es].view(dtype).view(shape)
        assert self.t.data_ptr() % 16 == 0
        if fill is not None:
            self.t.fill_(fill)

    def check(self, what):
        torch.cuda.synchronize()
        head = self.raw[:GUARD]
        tail = self.raw[GUARD + self.nbytes:]
        assert bool((head == PATTERN).all()), "%s: bytes BEFORE the output were written" % what
        assert bool((tail == PATTERN).all()), "%s: bytes AFTER the output were written (first at +%d)" % (
            what, int((tail != PATTERN).nonzero()[0]))


def _lib():
    return _cabi.load()


# ------------------------------------------------------------------------------------ copies and masks
@pytest.mark.parametrize("dtype", [torch.uint8, torch.bfloat16, torch.float32, torch.float64], ids=str)
@pytest.mark.parametrize("tdim", [1, 2, 3])
def test_guards_pad_unpad_mask(native_libs, cuda_device, dtype, tdim):
    g = torch.Generator().manual_seed(4100 + tdim)
    tensors = random_list(g, 7, tdim, 1, 23, dtype)
    sizes = sizes_of(tensors)
    B = sizes.size(0)
    mx = sizes.max(0).values.tolist()
    buf = torch.cat([t.reshape(-1) for t in tensors]).to(cuda_device)
    meta = build_meta(sizes, cuda_device)
    d_off, d_sz = meta.data_ptr(), meta.data_ptr() + 8 * (B + 1)
    nd, inner = fold(sizes)
    lib = _lib()
    out = Guarded([B] + mx, dtype, cuda_device)
    _cabi.check("pad", lib.ntb200_pad_nd(buf.data_ptr(), out.t.data_ptr(), d_off, d_sz, tdim, nd, inner, B, _cabi.host_i64(mx),
                                         buf.element_size(), bits_of(1, dtype), stream_ptr()))
    out.check("ntb200_pad_nd")
    assert_bit_equal(out.t, ntref.to_padded_tensor(tensors, 1), "pad")
    back = Guarded([buf.numel()], dtype, cuda_device)
    _cabi.check("unpad", lib.ntb200_unpad_nd(out.t.data_ptr(), back.t.data_ptr(), d_off, d_sz, tdim, nd, inner, B,
                                             _cabi.host_i64(mx), buf.numel(), buf.element_size(), stream_ptr()))
    back.check("ntb200_unpad_nd")
    assert_bit_equal(back.t, buf, "unpad")
    for mask_nd in range(1, tdim + 1):
        mask = Guarded([B] + mx[:mask_nd], torch.uint8, cuda_device)
        _cabi.check("mask", lib.ntb200_mask_from_sizes(mask.t.data_ptr(), d_sz, tdim, mask_nd, B, _cabi.host_i64(mx[:mask_nd]), stream_ptr()))
        mask.check("ntb200_mask_from_sizes")


@pytest.mark.parametrize("dtype", [torch.uint8, torch.float16, torch.float32, torch.int64], ids=str)
@pytest.mark.parametrize("tdim,regular_last", [(1, None), (2, None), (3, None), (2, 8), (3, 3), (2, 5)])
def test_pad_with_mask_single_pass(native_libs, cuda_device, dtype, tdim, regular_last):
    """Data + element-wise mask through ntb200_pad_with_mask (the same-shape case runs as one kernel) against the
    oracle's pad_nt, at every element width, with guards around both outputs; then the coarser mask (one byte per
    row), which takes the two-launch route."""
    g = torch.Generator().manual_seed(5200 + tdim + (regular_last or 0))
    tensors = random_list(g, 6, tdim, 1, 21, dtype, regular_last=regular_last)
    sizes = sizes_of(tensors)
    B = sizes.size(0)
    mx = sizes.max(0).values.tolist()
    buf = torch.cat([t.reshape(-1) for t in tensors]).to(cuda_device)
    meta = build_meta(sizes, cuda_device)
    d_off, d_sz = meta.data_ptr(), meta.data_ptr() + 8 * (B + 1)
    nd, inner = fold(sizes)
    lib = _lib()
    want_data, want_mask = ntref.pad_nt(tensors, mx)
    for mask_nd in sorted({tdim, nd}):
        data = Guarded([B] + mx, dtype, cuda_device)
        mask = Guarded([B] + mx[:mask_nd], torch.uint8, cuda_device)
        rc = lib.ntb200_pad_with_mask(buf.data_ptr(), data.t.data_ptr(), mask.t.data_ptr(), d_off, d_sz, tdim, nd, inner, B,
                                      _cabi.host_i64(mx), buf.element_size(), d_sz, tdim, mask_nd, _cabi.host_i64(mx[:mask_nd]),
                                      stream_ptr())
        _cabi.check("ntb200_pad_with_mask", rc)
        data.check("pad_with_mask data")
        mask.check("pad_with_mask mask")
        assert_bit_equal(data.t, want_data, "data")
        wm = want_mask
        while wm.dim() > mask_nd + 1:  # a coarser mask: an entry is valid when its whole trailing slab is
            wm = wm.amax(-1)
        assert_bit_equal(mask.t, wm.to(torch.uint8), "mask over %d dims" % mask_nd)


def test_guards_scan_offsets_token_index(native_libs, cuda_device):
    lib = _lib()
    g = torch.Generator().manual_seed(77)
    tensors = random_list(g, 9, 2, 1, 40, torch.float32)
    sizes = sizes_of(tensors)
    B = sizes.size(0)
    padded = ntref.to_padded_tensor(tensors, 0).to(cuda_device)
    dims = list(padded.shape[1:])
    o_sizes = Guarded([B, 2], torch.int64, cuda_device)
    o_counts = Guarded([B], torch.int64, cuda_device)
    _cabi.check("scan", lib.ntb200_sizes_from_padded(padded.data_ptr(), o_sizes.t.data_ptr(), o_counts.t.data_ptr(), 2, B,
                                                     _cabi.host_i64(dims), 4, 1, 0, stream_ptr()))
    o_sizes.check("sizes_from_padded sizes")
    o_counts.check("sizes_from_padded counts")
    d_sizes = sizes.to(cuda_device)
    offs = Guarded([B + 1], torch.int64, cuda_device)
    nbytes = lib.ntb200_offsets_workspace_bytes(B)
    ws = Guarded([max(nbytes, 8)], torch.uint8, cuda_device)
    _cabi.check("offsets", lib.ntb200_offsets_from_sizes(d_sizes.data_ptr(), 2, 2, 1, B, offs.t.data_ptr(), ws.t.data_ptr(), nbytes, stream_ptr()))
    offs.check("offsets_from_sizes")
    ws.check("offsets workspace")
    want = torch.zeros(B + 1, dtype=torch.int64)
    want[1:] = sizes.prod(1).cumsum(0)
    assert torch.equal(offs.t.cpu(), want)
    L = sizes[:, 0]
    tok = torch.zeros(B + 1, dtype=torch.int64)
    tok[1:] = L.cumsum(0)
    T = int(L.sum())
    bi = Guarded([T], torch.int32, cuda_device)
    wi = Guarded([T], torch.int32, cuda_device)
    d_tok = tok.to(cuda_device)
    _cabi.check("token_index", lib.ntb200_token_index(d_tok.data_ptr(), B, T, bi.t.data_ptr(), wi.t.data_ptr(), stream_ptr()))
    bi.check("token_index batch_idx")
    wi.check("token_index word_idx")


# ------------------------------------------------------------------------------------ GEMM / attention / rows
@pytest.mark.parametrize("M,N,K", [(300, 264, 64), (129, 8, 128), (1000, 3072 + 8, 1024), (5, 1000, 72)])
@pytest.mark.parametrize("force", [0, 2, 3])
def test_guards_gemm(native_libs, cuda_device, M, N, K, force):
    """N not a multiple of 16 (nor of the 256-column tile): the 32-byte stores of the epilogue end inside a tile."""
    lib = _lib()
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_device)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(cuda_device)
    c = Guarded([M, N], torch.bfloat16, cuda_device)
    _cabi.check("gemm", lib.ntb200_gemm_bias(a.data_ptr(), w.data_ptr(), b.data_ptr(), c.t.data_ptr(), M, N, K, 2, force, stream_ptr()))
    c.check("ntb200_gemm_bias force=%d" % force)
    want = a.float() @ w.float().t() + b.float()
    assert float((c.t.float() - want).abs().max()) <= 2e-2 * (1 + float(want.abs().max()))
    assert lib.ntb200_device_error_flags() == 0


@pytest.mark.parametrize("M,N,K", [(300, 264, 64), (1000, 1024 + 8, 1024), (257, 72, 128), (2100, 1024, 256)])
@pytest.mark.parametrize("force", [0, 2, 3])
def test_guards_gemm_residual(native_libs, cuda_device, M, N, K, force):
    """The residual epilogue (CTA pairs: the residual tile staged in shared memory by TMA, several tiles per CTA pair at
    M = 2100 so that boxes are reloaded; single CTA: per-thread row reads): guard bytes around the output, result
    against fp32, error flags clear."""
    lib = _lib()
    g = torch.Generator().manual_seed(M * 7 + N)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_device)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(cuda_device)
    r = Guarded([M, N], torch.bfloat16, cuda_device)
    r.t.copy_((torch.randn(M, N, generator=g) * 3).to(torch.bfloat16))
    c = Guarded([M, N], torch.bfloat16, cuda_device)
    _cabi.check("gemm", lib.ntb200_gemm_bias_act(a.data_ptr(), w.data_ptr(), b.data_ptr(), r.t.data_ptr(), c.t.data_ptr(), M, N, K, 2,
                                                 0, force, stream_ptr()))
    c.check("ntb200_gemm_bias_act + residual, force=%d" % force)
    want = a.float() @ w.float().t() + b.float() + r.t.float()
    assert float((c.t.float() - want).abs().max()) <= 2e-2 * (1 + float(want.abs().max()))
    assert lib.ntb200_device_error_flags() == 0


@pytest.mark.parametrize("path", [1, 2, 3])
def test_guards_attention(native_libs, cuda_device, path):
    lib = _lib()
    H, d = 4, 64
    E = H * d
    lengths = [1, 127, 128, 129, 300, 17, 64, 65]
    T, B = sum(lengths), len(lengths)
    g = torch.Generator().manual_seed(31)
    qkv = torch.randn(T, 3 * E, generator=g).to(torch.bfloat16).to(cuda_device)
    meta = build_meta(torch.tensor([[l, E] for l in lengths]), cuda_device)
    out = Guarded([T, E], torch.bfloat16, cuda_device)
    nb = lib.ntb200_varlen_attention_workspace_bytes(B, T, H, d, 2)
    ws = Guarded([max(nb, 16)], torch.uint8, cuda_device)
    rc = lib.ntb200_varlen_attention(qkv.data_ptr(), out.t.data_ptr(), meta.data_ptr(), B, T, H, d, max(lengths), d ** -0.5, 2, path,
                                     ws.t.data_ptr(), nb, stream_ptr())
    _cabi.check("ntb200_varlen_attention", rc)
    out.check("attention path %d" % path)
    ws.check("attention workspace path %d" % path)
    assert lib.ntb200_device_error_flags() == 0
    assert bool(torch.isfinite(out.t.float()).all())


def test_guards_rows_transpose_pack_embedding(native_libs, cuda_device):
    lib = _lib()
    g = torch.Generator().manual_seed(9)
    rows, cols = 77, 1000
    x = torch.randn(rows, cols, generator=g).to(torch.float16).to(cuda_device)
    gam = torch.randn(cols, generator=g).to(torch.float16).to(cuda_device)
    bet = torch.randn(cols, generator=g).to(torch.float16).to(cuda_device)
    o = Guarded([rows, cols], torch.float16, cuda_device)
    _cabi.check("ln", lib.ntb200_layer_norm(x.data_ptr(), gam.data_ptr(), bet.data_ptr(), 1e-5, o.t.data_ptr(), rows, cols, 1, stream_ptr()))
    o.check("layer_norm")
    o2 = Guarded([rows, cols], torch.float16, cuda_device)
    _cabi.check("gelu", lib.ntb200_add_bias_gelu(x.data_ptr(), bet.data_ptr(), o2.t.data_ptr(), rows, cols, 1, stream_ptr()))
    o2.check("add_bias_gelu")
    # ragged transposes: 5 maps of 24 channels, odd pixel counts
    C = 24
    px = [7, 130, 64, 1, 999]
    offs = torch.zeros(len(px) + 1, dtype=torch.int64)
    offs[1:] = torch.tensor([p * C for p in px]).cumsum(0)
    d_offs = offs.to(cuda_device)
    src = torch.randn(int(offs[-1]), generator=g).to(torch.float16).to(cuda_device)
    for to_nhwc in (1, 0):
        t = Guarded([int(offs[-1])], torch.float16, cuda_device)
        _cabi.check("transpose", lib.ntb200_transpose_ragged(src.data_ptr(), t.t.data_ptr(), d_offs.data_ptr(), len(px), C, to_nhwc,
                                                               max(px), 2, stream_ptr()))
        t.check("transpose_ragged to_nhwc=%d" % to_nhwc)
    # pack: four separate allocations, one of them at an odd element phase
    parts = [torch.randn(n + 1, generator=g).to(torch.float16).to(cuda_device)[1:] for n in (5, 300, 1, 64)]
    ptrs = torch.tensor([p.data_ptr() for p in parts], dtype=torch.int64, device=cuda_device)
    po = torch.zeros(5, dtype=torch.int64)
    po[1:] = torch.tensor([p.numel() for p in parts]).cumsum(0)
    d_po = po.to(cuda_device)
    packed = Guarded([int(po[-1])], torch.float16, cuda_device)
    _cabi.check("pack", lib.ntb200_pack_pointers(ptrs.data_ptr(), d_po.data_ptr(), 4, packed.t.data_ptr(), int(po[-1]), 2, stream_ptr()))
    packed.check("pack_pointers")
    assert_bit_equal(packed.t, torch.cat(parts), "pack")
    # embedding
    table = torch.randn(50, 40, generator=g).to(torch.float16).to(cuda_device)
    idx = torch.randint(0, 50, (33,), generator=g).to(cuda_device)
    emb = Guarded([33, 40], torch.float16, cuda_device)
    _cabi.check("embedding", lib.ntb200_embedding(table.data_ptr(), idx.data_ptr(), 8, emb.t.data_ptr(), 33, 50, 40, 2, stream_ptr()))
    emb.check("embedding")
    assert_bit_equal(emb.t, table[idx], "embedding")


# ------------------------------------------------------------------------------------ attention coverage
def test_config5_tcgen05_against_simt_every_sequence(native_libs, cuda_device):
    """The whole configuration-5 batch (1024 sequences, 16 heads): the tcgen05 kernel against the SIMT kernel (fp32
    arithmetic on the same bf16 inputs) on every sequence, so every item switch and deferred output write of the
    persistent kernel is compared, not a sample."""
    lib = _lib()
    L = workloads.lengths_c5(workloads._gen(5)).tolist()
    H, d = 16, 64
    E = H * d
    T, B = sum(L), len(L)
    g = torch.Generator(device=cuda_device).manual_seed(5)
    qkv = torch.randn(T, 3 * E, generator=g, device=cuda_device).to(torch.bfloat16)
    meta = build_meta(torch.tensor([[l, E] for l in L]), cuda_device)
    outs = []
    nb = lib.ntb200_varlen_attention_workspace_bytes(B, T, H, d, 2)
    ws = torch.empty(max(nb, 16), dtype=torch.uint8, device=cuda_device)
    for path in (3, 1):
        o = torch.empty(T, E, dtype=torch.bfloat16, device=cuda_device)
        _cabi.check("attention", lib.ntb200_varlen_attention(qkv.data_ptr(), o.data_ptr(), meta.data_ptr(), B, T, H, d, max(L), d ** -0.5, 2,
                                                               path, ws.data_ptr(), nb, stream_ptr()))
        outs.append(o)
    torch.cuda.synchronize()
    assert lib.ntb200_device_error_flags() == 0
    err = (outs[0].float() - outs[1].float()).abs()
    worst = int(err.reshape(-1).argmax())
    assert float(err.max()) <= 2e-2, "max-abs %g at token %d" % (float(err.max()), worst // E)


@pytest.mark.parametrize("bad", [float("nan"), float("inf")])
def test_nonfinite_value_stays_in_its_sequence(native_libs, cuda_device, bad):
    """A NaN / Inf in sequence b+1 must not reach the output of sequence b (whose last key tile is read past its end
    into the neighbour's tokens), as with the reference's zero-padded per-sequence tensors."""
    lib = _lib()
    H, d = 2, 64
    E = H * d
    lengths = [70, 33, 129, 250, 5]
    T, B = sum(lengths), len(lengths)
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(T, 3 * E, generator=g).to(torch.bfloat16)
    victim = 2  # every token of this sequence is non-finite in q, k and v
    a = sum(lengths[:victim])
    qkv[a:a + lengths[victim]] = bad
    qkv = qkv.to(cuda_device)
    meta = build_meta(torch.tensor([[l, E] for l in lengths]), cuda_device)
    nb = lib.ntb200_varlen_attention_workspace_bytes(B, T, H, d, 2)
    ws = torch.empty(max(nb, 16), dtype=torch.uint8, device=cuda_device)
    for path in (3, 2, 1):
        out = torch.empty(T, E, dtype=torch.bfloat16, device=cuda_device)
        _cabi.check("attention", lib.ntb200_varlen_attention(qkv.data_ptr(), out.data_ptr(), meta.data_ptr(), B, T, H, d, max(lengths),
                                                               d ** -0.5, 2, path, ws.data_ptr(), nb, stream_ptr()))
        torch.cuda.synchronize()
        off = 0
        for b, l in enumerate(lengths):
            if b != victim:
                assert bool(torch.isfinite(out[off:off + l].float()).all()), "path %d: sequence %d picked up a non-finite value" % (path, b)
            off += l


# ------------------------------------------------------------------------------------ reference-shaped helpers
@pytest.mark.parametrize("dtype,code", [(torch.float16, 1), (torch.bfloat16, 2), (torch.float32, 0)], ids=["f16", "bf16", "f32"])
def test_reference_shaped_helpers_bert_sizes(native_libs, cuda_device, dtype, code):
    """add_QKV_bias_padding, masked softmax (the reference's -10000 / +1e-6 arithmetic) and transpose_rm_padding at
    H=16, d=64 with sequences up to 512 tokens: rows longer than a warp, keys beyond 32, offsets beyond 2^16."""
    lib = _lib()
    H, d = 16, 64
    E = H * d
    lengths = [512, 1, 33, 300, 64, 257]
    B, T, maxL = len(lengths), sum(lengths), max(lengths)
    g = torch.Generator().manual_seed(12)
    qkv = torch.randn(T, 3 * E, generator=g).to(dtype)
    bias = torch.randn(3 * E, generator=g).to(dtype)
    meta = build_meta(torch.tensor([[l, E] for l in lengths]), cuda_device)
    bufs = [Guarded([B, H, maxL, d], dtype, cuda_device, fill=0) for _ in range(3)]
    d_qkv, d_bias = qkv.to(cuda_device), bias.to(cuda_device)
    _cabi.check("add_qkv_bias_pad", lib.ntb200_add_qkv_bias_pad(d_qkv.data_ptr(), d_bias.data_ptr(), bufs[0].t.data_ptr(), bufs[1].t.data_ptr(),
                                                                  bufs[2].t.data_ptr(), meta.data_ptr(), B, T, H, d, maxL, code, stream_ptr()))
    for i, gbuf in enumerate(bufs):
        gbuf.check("add_qkv_bias_pad buffer %d" % i)
    x = (qkv.float() + bias.float()).to(dtype)  # one rounding, as the kernel's fp32 add
    off = 0
    for b, l in enumerate(lengths):
        for i in range(3):
            want = x[off:off + l, i * E:(i + 1) * E].reshape(l, H, d).permute(1, 0, 2)
            got = bufs[i].t[b, :, :l].cpu()
            assert_bit_equal(got, want.contiguous(), "q/k/v %d of sequence %d" % (i, b))
            assert int(bufs[i].t[b, :, l:].count_nonzero()) == 0
        off += l
    # masked softmax on random scores
    scores = torch.randn(B, H, maxL, maxL, generator=g)
    sc = Guarded([B, H, maxL, maxL], dtype, cuda_device)
    sc.t.copy_(scores.to(dtype))
    _cabi.check("softmax_masked", lib.ntb200_softmax_masked(sc.t.data_ptr(), meta.data_ptr(), E, B, H, maxL, maxL, 0.125, code, stream_ptr()))
    sc.check("softmax_masked")
    lens = torch.tensor(lengths)
    valid = torch.arange(maxL)[None, :] < lens[:, None]
    mask = (valid[:, :, None] & valid[:, None, :]).float()
    want = ntref.masked_softmax(scores.to(dtype).float(), mask, 0.125)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    got = sc.t.float().cpu()
    for b, l in enumerate(lengths):  # rows of valid queries over valid keys
        assert float((got[b, :, :l, :l] - want[b, :, :l, :l]).abs().max()) <= tol
    # transpose_rm_padding of the padded q buffer gives the packed q + bias back
    packed = Guarded([T, E], dtype, cuda_device)
    _cabi.check("transpose_rm_padding", lib.ntb200_transpose_rm_padding(bufs[0].t.data_ptr(), packed.t.data_ptr(), meta.data_ptr(), B, T, H, d,
                                                                          maxL, code, stream_ptr()))
    packed.check("transpose_rm_padding")
    assert_bit_equal(packed.t, x[:, :E].contiguous(), "transpose_rm_padding")


# ------------------------------------------------------------------------------------ more than one GPU
_TWO = torch.cuda.is_available() and torch.cuda.device_count() >= 2


@pytest.mark.skipif(not _TWO, reason="needs two GPUs")
def test_second_device_in_one_process(native_libs):
    """The tcgen05 projection and attention on cuda:1 after cuda:0: the per-kernel shared-memory opt-in is a
    per-device setting and must be repeated on every device the process drives."""
    g = torch.Generator().manual_seed(1)
    xs = [torch.randn(l, 128, generator=g).to(torch.bfloat16) for l in (40, 200, 7)]
    torch.manual_seed(0)
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        mha = torch.nn.MultiheadAttention(128, 2).eval().to(torch.bfloat16)
        torch.manual_seed(0)
        with torch.no_grad():
            for p in mha.parameters():
                p.copy_(torch.randn(p.shape, generator=torch.Generator().manual_seed(p.numel())) * 0.05)
        mha = mha.to(dev)
        x = nt.nested_tensor(xs, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            out, _ = mha(x, x, x, need_weights=False)
        torch.cuda.synchronize(dev)
        outs.append(torch.cat([o.reshape(-1) for o in out.unbind()]).float().cpu())
    assert _cabi.load().ntb200_device_error_flags() >= 0
    assert float((outs[0] - outs[1]).abs().max()) == 0.0


_GATHER_CHILD = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["NTB200_ROOT"])
import nestedtensor_b200 as nt
from nestedtensor_b200 import sharding, workloads
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
w = workloads.config1()
parts = sharding.token_balanced_partition(w.sizes[:, 0].tolist(), world)
a, b = parts[rank]
sub = w.slice(a, b)
x = nt.NestedTensor(sub.buffer.cuda(), sub.sizes)
padded = x.to_padded_tensor(padding=0)
back = nt.from_padded_tensor(padded, x)
buf, sizes = sharding.gather_ragged(back._buffer, sub.sizes)
ok = torch.equal(buf.cpu(), w.buffer) and torch.equal(sizes, w.sizes)
dist.barrier()
dist.destroy_process_group()
sys.exit(0 if ok else 3)
"""


@pytest.mark.skipif(not _TWO, reason="needs two GPUs")
def test_gather_ragged_over_nccl(native_libs, tmp_path):
    """Two ranks, one GPU each: every rank pads and unpads its token-balanced shard of configuration 1, the shard
    results are all-gathered with sharding.gather_ragged over NCCL (plain collectives, NVLS off) and every rank must
    hold the whole configuration bit for bit."""
    script = tmp_path / "child.py"
    script.write_text(_GATHER_CHILD)
    env = dict(os.environ, NTB200_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", str(script)]
    proc = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:]

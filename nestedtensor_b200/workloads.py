"""Seeded synthetic workloads with the shapes, sizes and value distributions of the five
benchmark configurations (stand-ins for BERT / DETR style batches; no dataset is involved).

Draw order for configuration k (one ``torch.Generator`` seeded 20240 + k): all lengths first,
then the values of the whole ragged buffer in one draw, then the weights in the order
in_proj_weight, in_proj_bias, out_proj.weight, out_proj.bias.  Values are drawn in fp32 and
cast to the configuration's dtype.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

SEED_BASE = 20240


@dataclass
class Workload:
    name: str
    dtype: torch.dtype
    sizes: torch.Tensor          # CPU int64 [B, tensor_dim]
    buffer: torch.Tensor         # CPU, 1-D, dtype
    weights: Optional[dict] = None   # MHA configs: in_proj_weight, in_proj_bias, out_proj_weight, out_proj_bias
    num_heads: int = 0

    @property
    def batch(self) -> int:
        return int(self.sizes.size(0))

    def tensors(self) -> List[torch.Tensor]:
        out, off = [], 0
        for row in self.sizes.tolist():
            n = math.prod(row)
            out.append(self.buffer[off:off + n].reshape(row))
            off += n
        return out

    def slice(self, start: int, end: int) -> "Workload":
        numel = self.sizes.prod(1)
        a = int(numel[:start].sum())
        b = int(numel[:end].sum())
        return Workload(self.name, self.dtype, self.sizes[start:end].contiguous(), self.buffer[a:b], self.weights,
                        self.num_heads)


def _gen(k: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(SEED_BASE + k)
    return g


def lengths_c1(g, batch=64):
    return torch.randint(1, 129, (batch,), generator=g)


def lengths_c2(g, batch=4096):
    z = torch.randn(batch, generator=g, dtype=torch.float64)
    return torch.clamp(torch.round(torch.exp(math.log(200.0) + 0.6 * z)), 1, 1024).to(torch.int64)


def lengths_c4(g, batch=128):
    return torch.randint(32, 513, (batch,), generator=g)


def lengths_c5(g, batch=1024):
    u = torch.rand(batch, generator=g)
    short = torch.randint(16, 129, (batch,), generator=g)
    long_ = torch.randint(128, 513, (batch,), generator=g)
    return torch.where(u < 0.7, short, long_)


def _values(g, n, dtype, dist="randn", chunk=1 << 26):
    out = torch.empty(n, dtype=dtype)
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        x = torch.randn(b - a, generator=g) if dist == "randn" else torch.rand(b - a, generator=g)
        out[a:b] = x.to(dtype)
    return out


def _mha_weights(g, E, dtype):
    return {
        "in_proj_weight": (torch.randn(3 * E, E, generator=g) * 0.02).to(dtype),
        "in_proj_bias": (torch.randn(3 * E, generator=g) * 0.02).to(dtype),
        "out_proj_weight": (torch.randn(E, E, generator=g) * 0.02).to(dtype),
        "out_proj_bias": (torch.randn(E, generator=g) * 0.02).to(dtype),
    }


def config1(batch=64) -> Workload:
    """64 fp32 tensors (L_i, 256), L_i ~ U[1,128], N(0,1)."""
    g = _gen(1)
    L = lengths_c1(g, batch)
    sizes = torch.stack([L, torch.full_like(L, 256)], 1)
    return Workload("c1_pad_roundtrip_fp32", torch.float32, sizes, _values(g, int(L.sum()) * 256, torch.float32))


def config2(batch=4096, hidden=1024, with_values=True) -> Workload:
    """4096 bf16 sequences (L_i, 1024), L_i = clip(round(lognormal(ln 200, 0.6)), 1, 1024)."""
    g = _gen(2)
    L = lengths_c2(g, batch)
    sizes = torch.stack([L, torch.full_like(L, hidden)], 1)
    n = int(L.sum()) * hidden
    buf = _values(g, n, torch.bfloat16) if with_values else torch.empty(0, dtype=torch.bfloat16)
    return Workload("c2_pad_bf16_4096x1024", torch.bfloat16, sizes, buf)


def config3(batch=32) -> Workload:
    """32 fp32 images (3, H_i, W_i), H_i, W_i ~ U[400,1024], uniform [0,1]."""
    g = _gen(3)
    H = torch.randint(400, 1025, (batch,), generator=g)
    W = torch.randint(400, 1025, (batch,), generator=g)
    sizes = torch.stack([torch.full_like(H, 3), H, W], 1)
    return Workload("c3_detr_images_fp32", torch.float32, sizes,
                    _values(g, int((3 * H * W).sum()), torch.float32, dist="rand"))


def config4(batch=128) -> Workload:
    """BERT-base varlen self-attention, fp16: L_i ~ U[32,512], E=768, 12 heads x 64."""
    g = _gen(4)
    L = lengths_c4(g, batch)
    E = 768
    sizes = torch.stack([L, torch.full_like(L, E)], 1)
    buf = _values(g, int(L.sum()) * E, torch.float16)
    return Workload("c4_bert_base_mha_fp16", torch.float16, sizes, buf, _mha_weights(g, E, torch.float16), 12)


def config5(batch=1024) -> Workload:
    """BERT-large varlen self-attention, bf16: 70% L~U[16,128] / 30% L~U[128,512], E=1024, 16 heads x 64."""
    g = _gen(5)
    L = lengths_c5(g, batch)
    E = 1024
    sizes = torch.stack([L, torch.full_like(L, E)], 1)
    buf = _values(g, int(L.sum()) * E, torch.bfloat16)
    return Workload("c5_bert_large_mha_bf16", torch.bfloat16, sizes, buf, _mha_weights(g, E, torch.bfloat16), 16)


def mha_flops(lengths, E) -> float:
    """8*T*E^2 (QKV + output projections) + 4*E*sum(L_i^2) (QK^T and PV over all heads)."""
    L = torch.as_tensor(lengths, dtype=torch.float64)
    return float(8.0 * L.sum() * E * E + 4.0 * E * (L * L).sum())

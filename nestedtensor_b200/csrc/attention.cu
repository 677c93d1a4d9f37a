// Variable-length self-attention on the packed QKV buffer of a nested tensor, and the standalone
// B200 equivalents of the reference's attention helper kernels.
//
//   qkv   [T, 3E]  token-major, row t = (q | k | v) of token t, heads contiguous inside each third
//   out   [T, E]   token-major: softmax(scale * Q_b K_b^T) V_b for every sequence b and head h
//
// Padded tokens never exist: a CTA works on one (sequence, head, 64-query tile) and walks only that
// sequence's keys, so the "transpose + remove padding" step of the reference
// (transpose_rm_padding, nestedtensor/csrc/cuda/attention.cu:488-530) is the kernel's own store.
// Replaces steps 2-8 of bt_min_mha (nestedtensor/csrc/cuda/mha.cpp:59-105): pad to (B, maxL, 3E),
// padded batched QK^T, host-built mask, masked softmax kernel (attention.cu:182-482), padded PV, unpad.
//
// Paths: head_dim 64 in fp16/bf16 -> tensor-core flash kernel (mma.sync m16n8k16, fp32 online softmax);
// anything else (fp32, other head sizes) -> a warp-per-(token, head) SIMT kernel with fp32 math.

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "attention_internal.cuh"
#include "attention_tiny.cuh"
#include "common.cuh"

namespace ntb200 {
namespace {

template <typename T>
struct Cvt;
template <>
struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// largest b in [0, batch) with offsets[b] <= e
__device__ __forceinline__ int64_t find_entry(const int64_t* __restrict__ offsets, int64_t batch, int64_t e) {
  int64_t lo = 0, hi = batch - 1;
  while (lo < hi) {
    const int64_t mid = (lo + hi + 1) >> 1;
    if (offsets[mid] <= e) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// ------------------------------------------------------------------ generic SIMT attention
constexpr int kSimtWarps = 8;
constexpr int kMaxHeadDim = 256;

template <typename T>
__global__ void __launch_bounds__(kSimtWarps * 32)
attn_simt_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk, const T* __restrict__ v, int64_t ldv,
                 T* __restrict__ out, const int64_t* __restrict__ offsets_q, const int64_t* __restrict__ offsets_k,
                 int64_t batch, int64_t total_tokens, int H, int d, float scale) {
  // q / k / v: first element of head 0 of token 0, row strides ldq / ldk / ldv (self-attention on a packed
  // [T, 3E] buffer: the three thirds of one row, all strides 3E, offsets_k == offsets_q); offsets in elements
  // of the [tokens, E] matrices of the query and of the key / value nested tensors
  __shared__ float s_q[kSimtWarps][kMaxHeadDim];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t wg = (int64_t)blockIdx.x * kSimtWarps + warp;
  if (wg >= total_tokens * H) return;
  const int64_t t = wg / H;
  const int h = (int)(wg % H);
  const int64_t E = (int64_t)H * d;
  const int64_t b = find_entry(offsets_q, batch, t * E);
  const int64_t tok0 = offsets_k[b] / E;
  const int L = (int)((offsets_k[b + 1] - offsets_k[b]) / E);
  const T* qrow = q + t * ldq + (int64_t)h * d;
  for (int i = lane; i < d; i += 32) s_q[warp][i] = Cvt<T>::to_f(qrow[i]) * scale;
  __syncwarp();
  const T* kbase = k + tok0 * ldk + (int64_t)h * d;
  const T* vbase = v + tok0 * ldv + (int64_t)h * d;
  constexpr int DPL = kMaxHeadDim / 32;
  float acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;
  for (int c0 = 0; c0 < L; c0 += 32) {
    const int j = c0 + lane;
    float s = -INFINITY;
    if (j < L) {
      const T* krow = kbase + (int64_t)j * ldk;
      float dot = 0.0f;
      for (int i = 0; i < d; ++i) dot = fmaf(s_q[warp][i], Cvt<T>::to_f(krow[i]), dot);
      s = dot;
    }
    float cm = s;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
    const float m_new = fmaxf(m, cm);
    const float corr = __expf(m - m_new);  // 0 on the first chunk (m = -inf)
    const float p = (j < L) ? __expf(s - m_new) : 0.0f;
    float ps = p;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l = l * corr + ps;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] *= corr;
    const int nj = (L - c0) < 32 ? (L - c0) : 32;
    for (int jj = 0; jj < nj; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const T* vrow = vbase + (int64_t)(c0 + jj) * ldv;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int dim = lane + 32 * i;
        if (dim < d) acc[i] = fmaf(pj, Cvt<T>::to_f(vrow[dim]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = L > 0 ? 1.0f / l : 0.0f;  // a query whose key sequence is empty gets zeros
  T* orow = out + t * E + (int64_t)h * d;
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int dim = lane + 32 * i;
    if (dim < d) orow[dim] = Cvt<T>::from_f(acc[i] * inv);
  }
}

// ------------------------------------------------------- tensor-core flash kernel, head_dim 32 / 64 / 128
constexpr int kBQ = 64, kBKV = 64, kFaThreads = 128;

// copy rows [row0, row0+64) (clamped to last_row) x D columns of one head from global into a swizzled tile
template <typename T, int D>
__device__ __forceinline__ void load_tile_async(uint32_t smem_tile, const T* __restrict__ gbase, int64_t ld, int row0,
                                                int last_row) {
  constexpr int kChunks = D / 8;  // 16-byte chunks per row
#pragma unroll
  for (int i = 0; i < (64 * kChunks) / kFaThreads; ++i) {
    const int idx = threadIdx.x + i * kFaThreads;
    const int r = idx / kChunks, c = idx % kChunks;
    int gr = row0 + r;
    gr = gr > last_row ? last_row : gr;
    cp_async_16(smem_tile + tile_off<D>(r, c), gbase + (int64_t)gr * ld + c * 8);
  }
}

template <typename T, int kD>
__global__ void __launch_bounds__(kFaThreads)
attn_fa_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk, const T* __restrict__ v,
                   int64_t ldv, T* __restrict__ out, const int64_t* __restrict__ offsets_q, const int64_t* __restrict__ offsets_k,
                   int H, float scale_log2e) {  // arguments as in attn_simt_kernel
  extern __shared__ __align__(128) uint8_t fa_smem[];  // Q tile, two K tiles, two V tiles of 64 x kD each
  constexpr uint32_t kTileBytes = kBKV * kD * 2;
  uint8_t* s_q = fa_smem;
  uint8_t* s_k = fa_smem + kTileBytes;
  uint8_t* s_v = fa_smem + 3 * kTileBytes;

  const int b = blockIdx.z, h = blockIdx.y;
  const int64_t E = (int64_t)H * kD;
  const int64_t off_b = offsets_q[b];
  const int Lq = (int)((offsets_q[b + 1] - off_b) / E);
  const int q0 = blockIdx.x * kBQ;
  if (q0 >= Lq) return;
  const int64_t tok0 = off_b / E;  // first query token (also the first output row)
  const int64_t tokk0 = offsets_k[b] / E;
  const int L = (int)((offsets_k[b + 1] - offsets_k[b]) / E);  // keys
  const T* qbase = q + tok0 * ldq + (int64_t)h * kD;
  const T* kbase = k + tokk0 * ldk + (int64_t)h * kD;
  const T* vbase = v + tokk0 * ldv + (int64_t)h * kD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t sq = (uint32_t)__cvta_generic_to_shared(s_q);
  const uint32_t sk = (uint32_t)__cvta_generic_to_shared(s_k);
  const uint32_t sv = (uint32_t)__cvta_generic_to_shared(s_v);

  const int n_kv = (L + kBKV - 1) / kBKV;
  if (L <= 0) {  // no keys: the output rows of this tile are zeros
    for (int i = threadIdx.x; i < kBQ * (kD / 2); i += kFaThreads) {
      const int r = q0 + i / (kD / 2);
      if (r < Lq) reinterpret_cast<uint32_t*>(out + (tok0 + r) * E + (int64_t)h * kD)[i % (kD / 2)] = 0u;
    }
    return;
  }
  load_tile_async<T, kD>(sq, qbase, ldq, q0, Lq - 1);
  load_tile_async<T, kD>(sk, kbase, ldk, 0, L - 1);
  load_tile_async<T, kD>(sv, vbase, ldv, 0, L - 1);
  cp_async_commit();

  constexpr int KS = kD / 16, NO = kD / 8;
  uint32_t qf[KS][4];  // Q fragments: k-steps of 16 head dims
  float o[NO][4];      // O accumulator: n-tiles of 8 head dims
#pragma unroll
  for (int i = 0; i < NO; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;  // rows g and g+8 of this warp's 16

  for (int it = 0; it < n_kv; ++it) {
    const int buf = it & 1;
    if (it + 1 < n_kv) {
      load_tile_async<T, kD>(sk + (buf ^ 1) * kTileBytes, kbase, ldk, (it + 1) * kBKV, L - 1);
      load_tile_async<T, kD>(sv + (buf ^ 1) * kTileBytes, vbase, ldv, (it + 1) * kBKV, L - 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int ks = 0; ks < KS; ++ks)
        ldmatrix_x4(qf[ks], sq + tile_off<kD>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
    }
    // S = Q K^T for this warp's 16 rows x 64 keys
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
    const uint32_t kt = sk + buf * kTileBytes, vt = sv + buf * kTileBytes;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {  // pairs of key n-tiles
        uint32_t kf[4];
        ldmatrix_x4(kf, kt + tile_off<kD>(np * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
        MmaOp<T>::mma(s[np * 2], qf[ks], kf[0], kf[1]);
        MmaOp<T>::mma(s[np * 2 + 1], qf[ks], kf[2], kf[3]);
      }
    }
    // mask keys beyond the sequence (only the last tile can have any)
    const int kv0 = it * kBKV;
    if (kv0 + kBKV > L) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int key = kv0 + nt * 8 + 2 * (lane & 3);
        if (key >= L) s[nt][0] = s[nt][2] = -INFINITY;
        if (key + 1 >= L) s[nt][1] = s[nt][3] = -INFINITY;
      }
    }
    // online softmax in the exp2 domain
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0 * scale_log2e), mn1 = fmaxf(m1, mx1 * scale_log2e);
    const float c0 = exp2f(m0 - mn0), c1 = exp2f(m1 - mn1);
    float rs0 = 0.0f, rs1 = 0.0f;
    uint32_t pf[4][4];  // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float p0 = exp2f(fmaf(s[nt][0], scale_log2e, -mn0));
      const float p1 = exp2f(fmaf(s[nt][1], scale_log2e, -mn0));
      const float p2 = exp2f(fmaf(s[nt][2], scale_log2e, -mn1));
      const float p3 = exp2f(fmaf(s[nt][3], scale_log2e, -mn1));
      rs0 += p0 + p1;
      rs1 += p2 + p3;
      pf[nt >> 1][(nt & 1) * 2] = MmaOp<T>::pack(p0, p1);
      pf[nt >> 1][(nt & 1) * 2 + 1] = MmaOp<T>::pack(p2, p3);
    }
    l0 = l0 * c0 + rs0;
    l1 = l1 * c1 + rs1;
    m0 = mn0;
    m1 = mn1;
#pragma unroll
    for (int nt = 0; nt < NO; ++nt) {
      o[nt][0] *= c0;
      o[nt][1] *= c0;
      o[nt][2] *= c1;
      o[nt][3] *= c1;
    }
    // O += P V
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int np = 0; np < NO / 2; ++np) {  // pairs of head-dim n-tiles
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vt + tile_off<kD>(ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), np * 2 + (lane >> 4)));
        MmaOp<T>::mma(o[np * 2], pf[ks], vf[0], vf[1]);
        MmaOp<T>::mma(o[np * 2 + 1], pf[ks], vf[2], vf[3]);
      }
    }
    __syncthreads();  // everyone is done with this K/V buffer before it is refilled
  }

  // finish the row sums across the quad, normalise, store token-major
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = 1.0f / l0, i1 = 1.0f / l1;
  const int r0 = q0 + warp * 16 + (lane >> 2), r1 = r0 + 8;
  uint32_t* obase = reinterpret_cast<uint32_t*>(out + (tok0 + r0) * E + (int64_t)h * kD);
  uint32_t* obase1 = reinterpret_cast<uint32_t*>(out + (tok0 + r1) * E + (int64_t)h * kD);
#pragma unroll
  for (int nt = 0; nt < NO; ++nt) {
    const int col2 = nt * 4 + (lane & 3);  // index in 32-bit pairs
    if (r0 < Lq) obase[col2] = MmaOp<T>::pack(o[nt][0] * i0, o[nt][1] * i0);
    if (r1 < Lq) obase1[col2] = MmaOp<T>::pack(o[nt][2] * i1, o[nt][3] * i1);
  }
}

// ---------------------------------------------------- packed QKV + bias -> padded head-major
// q/k/v_buf[b, h, l, :] = qkv[tok, {0,E,2E} + h*d + :] + bias, zero elsewhere is NOT written (the caller
// zero-fills if it needs it, as the reference's caller would).  One warp per (token, head, third).
template <typename T>
__global__ void __launch_bounds__(256) add_qkv_bias_pad_kernel(const T* __restrict__ qkv, const T* __restrict__ bias,
                                                               T* __restrict__ q_buf, T* __restrict__ k_buf,
                                                               T* __restrict__ v_buf, const int64_t* __restrict__ offsets,
                                                               int64_t batch, int64_t total_tokens, int H, int d,
                                                               int64_t max_len) {
  const int64_t E = (int64_t)H * d;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // over T * 3E
  if (idx >= total_tokens * 3 * E) return;
  const int64_t t = idx / (3 * E);
  const int64_t c = idx - t * 3 * E;
  const int which = (int)(c / E);
  const int64_t e = c - which * E;
  const int h = (int)(e / d), i = (int)(e - (int64_t)h * d);
  const int64_t b = find_entry(offsets, batch, t * E);
  const int64_t l = t - offsets[b] / E;
  T* dst = which == 0 ? q_buf : (which == 1 ? k_buf : v_buf);
  const float v = Cvt<T>::to_f(qkv[idx]) + (bias != nullptr ? Cvt<T>::to_f(bias[c]) : 0.0f);
  dst[((b * H + h) * max_len + l) * d + i] = Cvt<T>::from_f(v);
}

// padded head-major [B, H, maxL, d] -> packed token-major [T, H*d]
template <typename T>
__global__ void __launch_bounds__(256) transpose_rm_padding_kernel(const T* __restrict__ src, T* __restrict__ dst,
                                                                   const int64_t* __restrict__ offsets, int64_t batch,
                                                                   int64_t total_tokens, int H, int d, int64_t max_len) {
  const int64_t E = (int64_t)H * d;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // over T * E
  if (idx >= total_tokens * E) return;
  const int64_t t = idx / E;
  const int64_t e = idx - t * E;
  const int h = (int)(e / d), i = (int)(e - (int64_t)h * d);
  const int64_t b = find_entry(offsets, batch, t * E);
  const int64_t l = t - offsets[b] / E;
  dst[idx] = src[((b * H + h) * max_len + l) * d + i];
}

// ---------------------------------------------------- masked softmax on padded scores
// In place over the last dim of scores [B, H, Lq, Lk]; the valid region of batch b is lens[b] x lens[b].
// Same arithmetic as the reference (attention.cu:182-225): masked logits get -10000 added, the row sum
// gets 1e-6.  One warp per row.
template <typename T>
__global__ void __launch_bounds__(256) softmax_masked_kernel(T* __restrict__ scores, const int64_t* __restrict__ offsets,
                                                             int64_t row_elems, int64_t rows_total, int H, int Lq, int Lk,
                                                             float scale) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows_total) return;
  const int64_t b = row / ((int64_t)H * Lq);
  const int qi = (int)(row % Lq);
  const int len = (int)((offsets[b + 1] - offsets[b]) / row_elems);
  T* p = scores + row * Lk;
  const bool qvalid = qi < len;
  float mx = -1e20f;
  for (int j = lane; j < Lk; j += 32) {
    const float mask = (qvalid && j < len) ? 1.0f : 0.0f;
    const float v = Cvt<T>::to_f(p[j]) * scale + (1.0f - mask) * -10000.0f;
    mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.0f;
  for (int j = lane; j < Lk; j += 32) {
    const float mask = (qvalid && j < len) ? 1.0f : 0.0f;
    const float v = Cvt<T>::to_f(p[j]) * scale + (1.0f - mask) * -10000.0f;
    sum += __expf(v - mx);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.0f / (sum + 1e-6f);
  for (int j = lane; j < Lk; j += 32) {
    const float mask = (qvalid && j < len) ? 1.0f : 0.0f;
    const float v = Cvt<T>::to_f(p[j]) * scale + (1.0f - mask) * -10000.0f;
    p[j] = Cvt<T>::from_f(__expf(v - mx) * inv);
  }
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ------------------------------------------------------------------ attention weights (need_weights=True)
// softmax(scale * q_b,h k_b,h^T) itself, for callers that ask for it: one block per query token walks the heads;
// the scores of a row live in shared memory (fp32), the row is written once.  average != 0: mean over heads into a
// (Lq_b x Lk_b) matrix per sequence; average == 0: (H x Lq_b x Lk_b) per sequence.  `weight_offsets[b]` is the element
// offset of sequence b's matrix in `weights`.  Not on the hot path: the attention kernels never materialise this.
constexpr int kWeightsThreads = 128;

template <typename T>
__global__ void __launch_bounds__(kWeightsThreads)
attn_weights_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk, T* __restrict__ weights,
                    const int64_t* __restrict__ offsets_q, const int64_t* __restrict__ offsets_k,
                    const int64_t* __restrict__ weight_offsets, int64_t batch, int H, int d, float scale, int average) {
  extern __shared__ float w_smem[];  // [d] query, [Lk] scores of the current head, [Lk] running mean (average mode)
  __shared__ float s_red[kWeightsThreads / 32];
  __shared__ float s_bcast;
  const int64_t t = blockIdx.x;
  const int64_t E = (int64_t)H * d;
  const int64_t b = find_entry(offsets_q, batch, t * E);
  const int64_t iq = t - offsets_q[b] / E;
  const int Lq = (int)((offsets_q[b + 1] - offsets_q[b]) / E);
  const int64_t tokk0 = offsets_k[b] / E;
  const int Lk = (int)((offsets_k[b + 1] - offsets_k[b]) / E);
  if (Lk <= 0) return;
  float* s_qv = w_smem;
  float* s_sc = w_smem + d;
  float* s_acc = s_sc + Lk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto block_reduce = [&](float v, bool is_max) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, other) : v + other;
    }
    __syncthreads();  // s_red / s_bcast of the previous reduction have been read
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float r = s_red[0];
      for (int w = 1; w < kWeightsThreads / 32; ++w) r = is_max ? fmaxf(r, s_red[w]) : r + s_red[w];
      s_bcast = r;
    }
    __syncthreads();
    return s_bcast;
  };
  if (average)
    for (int j = threadIdx.x; j < Lk; j += kWeightsThreads) s_acc[j] = 0.0f;
  for (int h = 0; h < H; ++h) {
    __syncthreads();
    const T* qrow = q + t * ldq + (int64_t)h * d;
    for (int i = threadIdx.x; i < d; i += kWeightsThreads) s_qv[i] = Cvt<T>::to_f(qrow[i]) * scale;
    __syncthreads();
    float mx = -INFINITY;
    for (int j = threadIdx.x; j < Lk; j += kWeightsThreads) {
      const T* krow = k + (tokk0 + j) * ldk + (int64_t)h * d;
      float dot = 0.0f;
      for (int i = 0; i < d; ++i) dot = fmaf(s_qv[i], Cvt<T>::to_f(krow[i]), dot);
      s_sc[j] = dot;
      mx = fmaxf(mx, dot);
    }
    mx = block_reduce(mx, true);
    float sum = 0.0f;
    for (int j = threadIdx.x; j < Lk; j += kWeightsThreads) {
      const float e = __expf(s_sc[j] - mx);
      s_sc[j] = e;
      sum += e;
    }
    sum = block_reduce(sum, false);
    const float inv = 1.0f / sum;
    if (average) {
      for (int j = threadIdx.x; j < Lk; j += kWeightsThreads) s_acc[j] += s_sc[j] * inv;
    } else {
      T* wrow = weights + weight_offsets[b] + ((int64_t)h * Lq + iq) * Lk;
      for (int j = threadIdx.x; j < Lk; j += kWeightsThreads) wrow[j] = Cvt<T>::from_f(s_sc[j] * inv);
    }
  }
  if (average) {
    const float invh = 1.0f / (float)H;
    T* wrow = weights + weight_offsets[b] + iq * Lk;
    for (int j = threadIdx.x; j < Lk; j += kWeightsThreads) wrow[j] = Cvt<T>::from_f(s_acc[j] * invh);
  }
}

// Separate query / key / value sources (self-attention passes the thirds of one packed row)
struct QkvSrc {
  const void *q, *k, *v;
  int64_t ldq, ldk, ldv;
  const int64_t *offsets_q, *offsets_k;
};

template <typename T>
int launch_attn_simt(const QkvSrc& s, void* out, int64_t batch, int64_t q_tokens, int H, int d, float scale, cudaStream_t st) {
  const int64_t blocks = ceil_div(q_tokens * H, kSimtWarps);
  if (blocks > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  attn_simt_kernel<T><<<(unsigned)blocks, kSimtWarps * 32, 0, st>>>(static_cast<const T*>(s.q), s.ldq, static_cast<const T*>(s.k),
                                                                    s.ldk, static_cast<const T*>(s.v), s.ldv, static_cast<T*>(out),
                                                                    s.offsets_q, s.offsets_k, batch, q_tokens, H, d, scale);
  return status_from_cuda(cudaGetLastError());
}

template <typename T, int D>
int launch_attn_fa(const QkvSrc& s, void* out, int64_t batch, int H, int64_t max_len_q, float scale, cudaStream_t st) {
  constexpr int kSmem = 5 * kBKV * D * 2;  // 20 / 40 / 80 KB
  if (kSmem > 48 * 1024) {
    static std::atomic<int> configured[kMaxDevices];
    if (!once_per_device(configured, [] {
          return cudaFuncSetAttribute(attn_fa_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) == cudaSuccess;
        }))
      return NTB200_LAUNCH_FAILED;
  }
  dim3 grid((unsigned)ceil_div(max_len_q, kBQ), (unsigned)H, (unsigned)batch);
  attn_fa_kernel<T, D><<<grid, kFaThreads, kSmem, st>>>(static_cast<const T*>(s.q), s.ldq, static_cast<const T*>(s.k), s.ldk,
                                                        static_cast<const T*>(s.v), s.ldv, static_cast<T*>(out), s.offsets_q,
                                                        s.offsets_k, H, scale * 1.4426950408889634f);
  return status_from_cuda(cudaGetLastError());
}

template <typename T>
int launch_attn_fa_any(const QkvSrc& s, void* out, int64_t batch, int H, int d, int64_t max_len_q, float scale, cudaStream_t st) {
  if (d == 32) return launch_attn_fa<T, 32>(s, out, batch, H, max_len_q, scale, st);
  if (d == 64) return launch_attn_fa<T, 64>(s, out, batch, H, max_len_q, scale, st);
  return launch_attn_fa<T, 128>(s, out, batch, H, max_len_q, scale, st);
}

template <typename T, int D, int R>
int launch_attn_tiny_dr(const QkvSrc& s, void* out, int64_t batch, int H, float scale, cudaStream_t st) {
  constexpr int kPerWarp = 3 * R * D * 2;  // 3 ... 24 KB
  constexpr int kWarps = 48 * 1024 / kPerWarp > 8 ? 8 : 48 * 1024 / kPerWarp;
  const int64_t blocks = ceil_div(batch * H, kWarps);
  if (blocks > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  attn_tiny_kernel<T, D, R, kWarps><<<(unsigned)blocks, kWarps * 32, kWarps * kPerWarp, st>>>(
      static_cast<const T*>(s.q), s.ldq, static_cast<const T*>(s.k), s.ldk, static_cast<const T*>(s.v), s.ldv, static_cast<T*>(out),
      s.offsets_q, s.offsets_k, batch, H, scale * 1.4426950408889634f);
  return status_from_cuda(cudaGetLastError());
}

template <typename T>
int launch_attn_tiny(const QkvSrc& s, void* out, int64_t batch, int H, int d, int64_t max_len, float scale, cudaStream_t st) {
  const bool r16 = max_len <= 16;
  if (d == 32) return r16 ? launch_attn_tiny_dr<T, 32, 16>(s, out, batch, H, scale, st) : launch_attn_tiny_dr<T, 32, 32>(s, out, batch, H, scale, st);
  if (d == 64) return r16 ? launch_attn_tiny_dr<T, 64, 16>(s, out, batch, H, scale, st) : launch_attn_tiny_dr<T, 64, 32>(s, out, batch, H, scale, st);
  return r16 ? launch_attn_tiny_dr<T, 128, 16>(s, out, batch, H, scale, st) : launch_attn_tiny_dr<T, 128, 32>(s, out, batch, H, scale, st);
}

// The non-tcgen05 kernels behind both entry points: mma.sync flash kernel for head_dim 32 / 64 / 128 in fp16 / bf16 with
// 16-byte aligned rows, SIMT otherwise.  path: 0 best of the two, 1 SIMT, 2 flash (error if unsupported).
int launch_attn_generic(const QkvSrc& s, void* out, int64_t batch, int64_t q_tokens, int H, int d, int64_t max_len_q,
                        float scaling, int dtype, int path, cudaStream_t st) {
  const size_t es = dtype == NTB200_F32 ? 4 : 2;
  auto rows16 = [&](const void* p, int64_t ld) { return aligned16(p) && (ld * (int64_t)es) % 16 == 0; };
  const bool fa = path != 1 && dtype != NTB200_F32 && (d == 32 || d == 64 || d == 128) && rows16(s.q, s.ldq) && rows16(s.k, s.ldk) && rows16(s.v, s.ldv) &&
                  aligned16(out) && batch <= 65535 && H <= 65535 && max_len_q > 0;
  if (path == 2 && !fa) return NTB200_UNSUPPORTED_SHAPE;
  if (fa) {
    if (dtype == NTB200_F16) return launch_attn_fa_any<__half>(s, out, batch, H, d, max_len_q, scaling, st);
    return launch_attn_fa_any<__nv_bfloat16>(s, out, batch, H, d, max_len_q, scaling, st);
  }
  switch (dtype) {
    case NTB200_F32: return launch_attn_simt<float>(s, out, batch, q_tokens, H, d, scaling, st);
    case NTB200_F16: return launch_attn_simt<__half>(s, out, batch, q_tokens, H, d, scaling, st);
    case NTB200_BF16: return launch_attn_simt<__nv_bfloat16>(s, out, batch, q_tokens, H, d, scaling, st);
  }
  return NTB200_UNSUPPORTED_DTYPE;
}

}  // namespace
}  // namespace ntb200

using namespace ntb200;

extern "C" {

size_t ntb200_varlen_attention_workspace_bytes(int64_t batch, int64_t total_tokens, int num_heads, int head_dim, int dtype) {
  if (batch <= 0 || total_tokens <= 0) return 0;
  if (!attn_tcgen05_supported(batch, total_tokens, num_heads, head_dim, dtype)) return 0;
  return attn_tcgen05_workspace_bytes(batch, total_tokens);
}

int ntb200_varlen_attention(const void* qkv, void* out, const int64_t* offsets, int64_t batch, int64_t total_tokens,
                            int num_heads, int head_dim, int64_t max_len, float scaling, int dtype, int path,
                            void* workspace, size_t workspace_bytes, void* stream) {
  const int force_simt = path == 1;
  if (batch < 0 || total_tokens < 0 || num_heads < 1 || head_dim < 1 || max_len < 0) return NTB200_INVALID_ARG;
  if (dtype != NTB200_F32 && dtype != NTB200_F16 && dtype != NTB200_BF16) return NTB200_UNSUPPORTED_DTYPE;
  if (head_dim > kMaxHeadDim) return NTB200_UNSUPPORTED_SHAPE;
  if (batch == 0 || total_tokens == 0) return NTB200_OK;
  if (qkv == nullptr || out == nullptr || offsets == nullptr) return NTB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // path 0: best available (the warp-per-(sequence, head) kernel when no sequence is longer than 32 tokens, else tcgen05
  // when a workspace is given and the shape is supported, else mma.sync, else SIMT); 1: SIMT; 2: mma.sync flash kernel;
  // 3: tcgen05 (error if unsupported); 4: warp-per-(sequence, head) kernel (error if unsupported)
  {
    const int64_t E = (int64_t)num_heads * head_dim;
    const bool tiny_ok = dtype != NTB200_F32 && (head_dim == 32 || head_dim == 64 || head_dim == 128) && aligned16(qkv) &&
                         aligned16(out) && max_len >= 1 && max_len <= kTinyMaxLen;
    if (path == 4 || (path == 0 && tiny_ok)) {
      if (!tiny_ok) return NTB200_UNSUPPORTED_SHAPE;
      const char* base = static_cast<const char*>(qkv);
      const QkvSrc src = {base, base + E * 2, base + 2 * E * 2, 3 * E, 3 * E, 3 * E, offsets, offsets};
      if (dtype == NTB200_F16) return launch_attn_tiny<__half>(src, out, batch, num_heads, head_dim, max_len, scaling, st);
      return launch_attn_tiny<__nv_bfloat16>(src, out, batch, num_heads, head_dim, max_len, scaling, st);
    }
  }
  const bool tc_ok = dtype != NTB200_F32 && (num_heads * (int64_t)head_dim) % 8 == 0 && aligned16(qkv) && aligned16(out) &&
                     attn_tcgen05_supported(batch, total_tokens, num_heads, head_dim, dtype);
  if (path == 3 || (path == 0 && tc_ok && workspace != nullptr)) {
    if (!tc_ok) return NTB200_UNSUPPORTED_SHAPE;
    const size_t need = attn_tcgen05_workspace_bytes(batch, total_tokens);
    if (workspace == nullptr || workspace_bytes < need) return NTB200_WORKSPACE_TOO_SMALL;
    if (!aligned16(workspace)) return NTB200_MISALIGNED;
    // On the default path the sequences of at most 32 tokens are computed by single warps beside the block that builds
    // the work list (same launch), and get no work item: each of them would cost the tensor-memory kernel a whole
    // 128-row item.  Which kernel computes a sequence thus depends on the sequence alone, never on the batch around it,
    // so a batch cut into shards or ranges reproduces the one-call result bit for bit.
    const int skip_short = path == 0 ? (int)kTinyMaxLen : 0;
    return attn_tcgen05_launch(qkv, out, offsets, batch, total_tokens, num_heads, scaling, dtype, workspace, st, skip_short);
  }
  const int64_t E = (int64_t)num_heads * head_dim;
  const size_t es = dtype == NTB200_F32 ? 4 : 2;
  const char* base = static_cast<const char*>(qkv);
  const QkvSrc src = {base, base + E * es, base + 2 * E * es, 3 * E, 3 * E, 3 * E, offsets, offsets};
  return launch_attn_generic(src, out, batch, total_tokens, num_heads, head_dim, max_len, scaling, dtype, force_simt ? 1 : path, st);
}

int ntb200_varlen_cross_attention(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, void* out,
                                  const int64_t* offsets_q, const int64_t* offsets_k, int64_t batch, int64_t q_tokens,
                                  int num_heads, int head_dim, int64_t max_len_q, float scaling, int dtype, int path,
                                  void* stream) {
  if (batch < 0 || q_tokens < 0 || num_heads < 1 || head_dim < 1 || max_len_q < 0 || path < 0 || path > 2) return NTB200_INVALID_ARG;
  if (dtype != NTB200_F32 && dtype != NTB200_F16 && dtype != NTB200_BF16) return NTB200_UNSUPPORTED_DTYPE;
  if (head_dim > kMaxHeadDim) return NTB200_UNSUPPORTED_SHAPE;
  const int64_t E = (int64_t)num_heads * head_dim;
  if (ldq < E || ldk < E || ldv < E) return NTB200_INVALID_ARG;
  if (batch == 0 || q_tokens == 0) return NTB200_OK;
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || offsets_q == nullptr || offsets_k == nullptr)
    return NTB200_INVALID_ARG;
  const QkvSrc src = {q, k, v, ldq, ldk, ldv, offsets_q, offsets_k};
  return launch_attn_generic(src, out, batch, q_tokens, num_heads, head_dim, max_len_q, scaling, dtype, path,
                             static_cast<cudaStream_t>(stream));
}

size_t ntb200_varlen_cross_attention_workspace_bytes(int64_t batch, int64_t q_tokens, int num_heads, int head_dim, int dtype) {
  if (batch <= 0 || q_tokens <= 0) return 0;
  if (!attn_tcgen05_supported(batch, q_tokens, num_heads, head_dim, dtype)) return 0;
  return attn_tcgen05_workspace_bytes(batch, q_tokens);
}

int ntb200_varlen_cross_attention_ws(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, void* out,
                                     const int64_t* offsets_q, const int64_t* offsets_k, int64_t batch, int64_t q_tokens,
                                     int64_t k_tokens, int num_heads, int head_dim, int64_t max_len_q, float scaling, int dtype,
                                     int path, void* workspace, size_t workspace_bytes, void* stream) {
  if (batch < 0 || q_tokens < 0 || k_tokens < 0 || num_heads < 1 || head_dim < 1 || max_len_q < 0 || path < 0 || path > 3)
    return NTB200_INVALID_ARG;
  if (dtype != NTB200_F32 && dtype != NTB200_F16 && dtype != NTB200_BF16) return NTB200_UNSUPPORTED_DTYPE;
  if (head_dim > kMaxHeadDim) return NTB200_UNSUPPORTED_SHAPE;
  const int64_t E = (int64_t)num_heads * head_dim;
  if (ldq < E || ldk < E || ldv < E) return NTB200_INVALID_ARG;
  if (batch == 0 || q_tokens == 0) return NTB200_OK;
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr || offsets_q == nullptr || offsets_k == nullptr)
    return NTB200_INVALID_ARG;
  // path 0: tcgen05 when the shape allows it and a workspace is given, else the mma.sync kernel, else SIMT; 3: tcgen05 or error
  const bool tc_ok = dtype != NTB200_F32 && attn_tcgen05_supported(batch, q_tokens, num_heads, head_dim, dtype) && k_tokens > 0 &&
                     k_tokens < (1ll << 31) - 128 && aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) &&
                     ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0;
  if (path == 3 || (path == 0 && tc_ok && workspace != nullptr)) {
    if (!tc_ok) return NTB200_UNSUPPORTED_SHAPE;
    const size_t need = attn_tcgen05_workspace_bytes(batch, q_tokens);
    if (workspace == nullptr || workspace_bytes < need) return NTB200_WORKSPACE_TOO_SMALL;
    if (!aligned16(workspace)) return NTB200_MISALIGNED;
    return attn_tcgen05_cross_launch(q, ldq, k, ldk, v, ldv, out, offsets_q, offsets_k, batch, q_tokens, k_tokens, num_heads, scaling,
                                     dtype, workspace, static_cast<cudaStream_t>(stream));
  }
  const QkvSrc src = {q, k, v, ldq, ldk, ldv, offsets_q, offsets_k};
  return launch_attn_generic(src, out, batch, q_tokens, num_heads, head_dim, max_len_q, scaling, dtype, path,
                             static_cast<cudaStream_t>(stream));
}

int ntb200_varlen_attention_weights(const void* q, int64_t ldq, const void* k, int64_t ldk, void* weights,
                                    const int64_t* offsets_q, const int64_t* offsets_k, const int64_t* weight_offsets,
                                    int64_t batch, int64_t q_tokens, int num_heads, int head_dim, int64_t max_len_k,
                                    float scaling, int dtype, int average, void* stream) {
  if (batch < 0 || q_tokens < 0 || num_heads < 1 || head_dim < 1 || max_len_k < 0) return NTB200_INVALID_ARG;
  if (dtype != NTB200_F32 && dtype != NTB200_F16 && dtype != NTB200_BF16) return NTB200_UNSUPPORTED_DTYPE;
  if (head_dim > kMaxHeadDim) return NTB200_UNSUPPORTED_SHAPE;
  const int64_t E = (int64_t)num_heads * head_dim;
  if (ldq < E || ldk < E) return NTB200_INVALID_ARG;
  if (batch == 0 || q_tokens == 0 || max_len_k == 0) return NTB200_OK;
  if (q == nullptr || k == nullptr || weights == nullptr || offsets_q == nullptr || offsets_k == nullptr || weight_offsets == nullptr)
    return NTB200_INVALID_ARG;
  if (q_tokens > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  const size_t smem = sizeof(float) * ((size_t)head_dim + 2 * (size_t)max_len_k);
  if (smem > 200 * 1024) return NTB200_UNSUPPORTED_SHAPE;  // key sequences beyond about 25 000 tokens
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define NTB200_LAUNCH_WEIGHTS(T)                                                                                          \
  do {                                                                                                                    \
    if (smem > 48 * 1024) {                                                                                               \
      static std::atomic<int> configured[kMaxDevices];                                                                    \
      if (!once_per_device(configured, [] {                                                                               \
            return cudaFuncSetAttribute(attn_weights_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == \
                   cudaSuccess;                                                                                           \
          }))                                                                                                             \
        return NTB200_LAUNCH_FAILED;                                                                                      \
    }                                                                                                                     \
    attn_weights_kernel<T><<<(unsigned)q_tokens, kWeightsThreads, smem, st>>>(                                            \
        static_cast<const T*>(q), ldq, static_cast<const T*>(k), ldk, static_cast<T*>(weights), offsets_q, offsets_k,     \
        weight_offsets, batch, num_heads, head_dim, scaling, average);                                                    \
  } while (0)
  switch (dtype) {
    case NTB200_F32: NTB200_LAUNCH_WEIGHTS(float); break;
    case NTB200_F16: NTB200_LAUNCH_WEIGHTS(__half); break;
    case NTB200_BF16: NTB200_LAUNCH_WEIGHTS(__nv_bfloat16); break;
  }
#undef NTB200_LAUNCH_WEIGHTS
  return status_from_cuda(cudaGetLastError());
}

#define NTB200_DISPATCH_DTYPE(dtype, CALL)                 \
  switch (dtype) {                                         \
    case NTB200_F32: { using T = float; CALL; } break;     \
    case NTB200_F16: { using T = __half; CALL; } break;    \
    case NTB200_BF16: { using T = __nv_bfloat16; CALL; } break; \
    default: return NTB200_UNSUPPORTED_DTYPE;              \
  }

int ntb200_add_qkv_bias_pad(const void* qkv, const void* bias, void* q_buf, void* k_buf, void* v_buf, const int64_t* offsets,
                            int64_t batch, int64_t total_tokens, int num_heads, int head_dim, int64_t max_len, int dtype,
                            void* stream) {
  if (batch < 0 || total_tokens < 0 || num_heads < 1 || head_dim < 1 || max_len < 0) return NTB200_INVALID_ARG;
  if (batch == 0 || total_tokens == 0) return NTB200_OK;
  if (qkv == nullptr || q_buf == nullptr || k_buf == nullptr || v_buf == nullptr || offsets == nullptr) return NTB200_INVALID_ARG;
  const int64_t n = total_tokens * 3 * num_heads * head_dim;
  const int64_t blocks = ceil_div(n, 256);
  if (blocks > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NTB200_DISPATCH_DTYPE(dtype, (add_qkv_bias_pad_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(
                                   static_cast<const T*>(qkv), static_cast<const T*>(bias), static_cast<T*>(q_buf),
                                   static_cast<T*>(k_buf), static_cast<T*>(v_buf), offsets, batch, total_tokens, num_heads,
                                   head_dim, max_len)));
  return status_from_cuda(cudaGetLastError());
}

int ntb200_transpose_rm_padding(const void* src, void* dst, const int64_t* offsets, int64_t batch, int64_t total_tokens,
                                int num_heads, int head_dim, int64_t max_len, int dtype, void* stream) {
  if (batch < 0 || total_tokens < 0 || num_heads < 1 || head_dim < 1 || max_len < 0) return NTB200_INVALID_ARG;
  if (batch == 0 || total_tokens == 0) return NTB200_OK;
  if (src == nullptr || dst == nullptr || offsets == nullptr) return NTB200_INVALID_ARG;
  const int64_t n = total_tokens * num_heads * head_dim;
  const int64_t blocks = ceil_div(n, 256);
  if (blocks > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NTB200_DISPATCH_DTYPE(dtype, (transpose_rm_padding_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(
                                   static_cast<const T*>(src), static_cast<T*>(dst), offsets, batch, total_tokens, num_heads,
                                   head_dim, max_len)));
  return status_from_cuda(cudaGetLastError());
}

int ntb200_softmax_masked(void* scores, const int64_t* offsets, int64_t row_elems, int64_t batch, int num_heads,
                          int64_t len_q, int64_t len_k, float scaling, int dtype, void* stream) {
  if (batch < 0 || num_heads < 1 || len_q < 0 || len_k < 0 || row_elems < 1) return NTB200_INVALID_ARG;
  if (batch == 0 || len_q == 0 || len_k == 0) return NTB200_OK;
  if (scores == nullptr || offsets == nullptr) return NTB200_INVALID_ARG;
  if (len_q > 0x7fffffffll || len_k > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  const int64_t rows = batch * num_heads * len_q;
  const int64_t blocks = ceil_div(rows, 8);
  if (blocks > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NTB200_DISPATCH_DTYPE(dtype, (softmax_masked_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(
                                   static_cast<T*>(scores), offsets, row_elems, rows, num_heads, (int)len_q, (int)len_k,
                                   scaling)));
  return status_from_cuda(cudaGetLastError());
}

}  // extern "C"

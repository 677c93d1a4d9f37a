// Row operators on the packed token matrix [T = sum(L_i), E] of a nested tensor: the steps of a
// transformer encoder layer that sit between the projections.  All of them stream every element once
// (HBM-bound), never see padding, and keep their arithmetic in fp32 whatever the storage type.
//
//   layer_norm                    out = (x - mean) * rsqrt(var + eps) * gamma + beta          per row
//   add_bias_residual_layer_norm  the same on x + residual + bias (one pass instead of three)
//   add_bias_gelu                 out = gelu_tanh(x + bias)
//
// Replaces fastertransformer::layer_norm (nestedtensor/csrc/cuda/transformer_kernels.cu:260-335) as used by
// cuda::NestedTensor_layer_norm (nestedtensor/csrc/cuda/layernorm.cpp:14-76), add_bias_input_layernorm
// (transformer_kernels.cu:64-156, cuda_kernels.cu:114-159) and add_bias_act / add_bias_gelu
// (cuda_kernels.cu:73-104, transformer_kernels.cu:52-62).

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ntb200 {
namespace {

// 16 bytes of storage <-> fp32 lanes
template <int DT>
struct Vec16;
template <>
struct Vec16<NTB200_F32> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x), f[1] = __uint_as_float(r.y), f[2] = __uint_as_float(r.z), f[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ float load1(const void* p, int64_t i) { return reinterpret_cast<const float*>(p)[i]; }
  static __device__ __forceinline__ void store1(void* p, int64_t i, float v) { reinterpret_cast<float*>(p)[i] = v; }
};
template <>
struct Vec16<NTB200_F16> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
      f[2 * k] = t.x, f[2 * k + 1] = t.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __half2 h = __floats2half2_rn(f[2 * k], f[2 * k + 1]);
      w[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ float load1(const void* p, int64_t i) { return __half2float(reinterpret_cast<const __half*>(p)[i]); }
  static __device__ __forceinline__ void store1(void* p, int64_t i, float v) { reinterpret_cast<__half*>(p)[i] = __float2half_rn(v); }
};
template <>
struct Vec16<NTB200_BF16> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {  // a bf16 is the upper half of an fp32
      f[2 * k] = __uint_as_float(w[k] << 16);
      f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
      w[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ float load1(const void* p, int64_t i) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  }
  static __device__ __forceinline__ void store1(void* p, int64_t i, float v) {
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  }
};

// The same 16 bytes as kElems / 2 packed fp32 pairs (sm_100 adds, subtracts and multiplies two fp32 values
// held in a 64-bit register pair with one instruction: the LayerNorm kernel is otherwise bound by its issue
// slots, not by memory).
template <int DT>
__device__ __forceinline__ void unpack_pairs(const uint4& r, uint64_t* p) {
  float f[Vec16<DT>::kElems];
  Vec16<DT>::unpack(r, f);
#pragma unroll
  for (int k = 0; k < Vec16<DT>::kElems / 2; ++k) p[k] = ptx::f32x2_pack(f[2 * k], f[2 * k + 1]);
}
template <int DT>
__device__ __forceinline__ uint4 pack_pairs(const uint64_t* p) {
  float f[Vec16<DT>::kElems];
#pragma unroll
  for (int k = 0; k < Vec16<DT>::kElems / 2; ++k) ptx::f32x2_unpack(p[k], f[2 * k], f[2 * k + 1]);
  return Vec16<DT>::pack(f);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the GROUP threads that share a row: part of a warp (GROUP == 8, 16: neighbouring lanes), a warp
// (GROUP == 32) or the whole block.
template <int GROUP>
__device__ __forceinline__ float group_sum(float v, float* scratch) {
  if (GROUP < 32) {
#pragma unroll
    for (int o = GROUP / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  }
  v = warp_sum(v);
  if (GROUP == 32) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < GROUP / 32 ? scratch[lane] : 0.0f;
  return warp_sum(t);
}

constexpr int kLnThreads = 256;

// One row per GROUP threads, the row held in registers between the passes (one global read, one global
// write per element).  VPL = 16-byte vectors per thread; vector v of the row belongs to thread v % GROUP.
// Mean and variance are the two-pass forms of the reference kernel (sum, then sum of squared deviations).
// A 16-bit row without the fused additions stays in its packed form (4 registers per vector instead of 8) and is
// widened again in each pass, which is exact: half the registers, twice the rows in flight per SM.
// FULL: the row is exactly VPL * GROUP vectors (no per-vector bound test).
template <int DT, int VPL, int GROUP, bool FUSED, bool FULL>
__global__ void __launch_bounds__(kLnThreads, (!FUSED && FULL && DT != NTB200_F32 && VPL <= 4) ? 6 : 1)
layer_norm_kernel(const void* x, const void* __restrict__ residual, const void* __restrict__ bias,
                  const void* __restrict__ gamma, const void* __restrict__ beta, float eps, void* out, int64_t rows,
                  int cols) {  // out may alias x: a thread has read all it needs of the row before it writes
  constexpr int EPV = Vec16<DT>::kElems;
  constexpr int kRowsPerBlock = kLnThreads / GROUP;
  constexpr bool RAW = !FUSED && DT != NTB200_F32;
  __shared__ float scratch[kLnThreads / 32];
  const int t = threadIdx.x % GROUP;
  const int64_t row = (int64_t)blockIdx.x * kRowsPerBlock + threadIdx.x / GROUP;
  const bool live = row < rows;  // whole groups are live or not; a warp of several short rows may hold both kinds
  if (GROUP == 32 && !live) return;
  const int nv = cols / EPV;
  const uint4* xr = reinterpret_cast<const uint4*>(x) + row * nv;
  const uint4* rr = reinterpret_cast<const uint4*>(residual) + row * nv;
  constexpr int PPV = EPV / 2;  // packed pairs per vector
  uint4 raw[RAW ? VPL : 1];
  uint64_t v[RAW ? 1 : VPL][PPV];
  if (RAW) {  // all loads of the row first
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int vec = t + j * GROUP;
      raw[j] = make_uint4(0u, 0u, 0u, 0u);
      if ((FULL || vec < nv) && live) raw[j] = xr[vec];
    }
  }
  uint64_t sum2 = 0;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int vec = t + j * GROUP;
    if (RAW) {
      uint64_t a[PPV];
      unpack_pairs<DT>(raw[j], a);  // (vectors past the row are zero)
#pragma unroll
      for (int k = 0; k < PPV; ++k) sum2 = ptx::f32x2_add(sum2, a[k]);
    } else if ((FULL || vec < nv) && live) {
      unpack_pairs<DT>(xr[vec], v[j]);
      if (FUSED) {
        uint64_t a[PPV];
        if (residual != nullptr) {
          unpack_pairs<DT>(rr[vec], a);
#pragma unroll
          for (int k = 0; k < PPV; ++k) v[j][k] = ptx::f32x2_add(v[j][k], a[k]);
        }
        if (bias != nullptr) {
          unpack_pairs<DT>(reinterpret_cast<const uint4*>(bias)[vec], a);
#pragma unroll
          for (int k = 0; k < PPV; ++k) v[j][k] = ptx::f32x2_add(v[j][k], a[k]);
        }
      }
#pragma unroll
      for (int k = 0; k < PPV; ++k) sum2 = ptx::f32x2_add(sum2, v[j][k]);
    } else {
#pragma unroll
      for (int k = 0; k < PPV; ++k) v[j][k] = 0;
    }
  }
  // (an empty asm that "rewrites" the packed row: keeps the compiler from carrying the widened copy across the pass)
#define NTB200_LN_LAUNDER()                                                                                     \
  if (RAW) {                                                                                                    \
    _Pragma("unroll") for (int j = 0; j < VPL; ++j)                                                             \
        asm volatile("" : "+r"(raw[j].x), "+r"(raw[j].y), "+r"(raw[j].z), "+r"(raw[j].w));                      \
  }
  NTB200_LN_LAUNDER();
  float s_lo, s_hi;
  ptx::f32x2_unpack(sum2, s_lo, s_hi);
  const float mean = group_sum<GROUP>(s_lo + s_hi, scratch) / (float)cols;
  const uint64_t mean2 = ptx::f32x2_pack(mean, mean);
  uint64_t sq2 = 0;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    if (FULL || t + j * GROUP < nv) {
      if (RAW) {
        uint64_t a[PPV];
        unpack_pairs<DT>(raw[j], a);
#pragma unroll
        for (int k = 0; k < PPV; ++k) {
          const uint64_t d = ptx::f32x2_sub(a[k], mean2);
          sq2 = ptx::f32x2_fma(d, d, sq2);
        }
      } else {
#pragma unroll
        for (int k = 0; k < PPV; ++k) {
          v[j][k] = ptx::f32x2_sub(v[j][k], mean2);  // deviations replace the values
          sq2 = ptx::f32x2_fma(v[j][k], v[j][k], sq2);
        }
      }
    }
  }
  NTB200_LN_LAUNDER();
#undef NTB200_LN_LAUNDER
  ptx::f32x2_unpack(sq2, s_lo, s_hi);
  const float rstd = rsqrtf(group_sum<GROUP>(s_lo + s_hi, scratch) / (float)cols + eps);
  if (!live) return;
  const uint64_t rstd2 = ptx::f32x2_pack(rstd, rstd);
  uint4* orow = reinterpret_cast<uint4*>(out) + row * nv;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int vec = t + j * GROUP;
    if (FULL || vec < nv) {
      uint64_t o[PPV], d[PPV];
      if (RAW) {
        unpack_pairs<DT>(raw[j], d);
#pragma unroll
        for (int k = 0; k < PPV; ++k) d[k] = ptx::f32x2_sub(d[k], mean2);
      } else {
#pragma unroll
        for (int k = 0; k < PPV; ++k) d[k] = v[j][k];
      }
      if (gamma != nullptr) {
        uint64_t g[PPV], b[PPV];
        unpack_pairs<DT>(reinterpret_cast<const uint4*>(gamma)[vec], g);
        unpack_pairs<DT>(reinterpret_cast<const uint4*>(beta)[vec], b);
#pragma unroll
        for (int k = 0; k < PPV; ++k) o[k] = ptx::f32x2_fma(ptx::f32x2_fma(d[k], rstd2, 0ull), g[k], b[k]);
      } else {
#pragma unroll
        for (int k = 0; k < PPV; ++k) o[k] = ptx::f32x2_fma(d[k], rstd2, 0ull);
      }
      orow[vec] = pack_pairs<DT>(o);
    }
  }
}

// Any row length and alignment: one block per row, three passes over global memory.
template <int DT>
__global__ void __launch_bounds__(kLnThreads)
layer_norm_generic_kernel(const void* x, const void* __restrict__ residual, const void* __restrict__ bias,
                          const void* __restrict__ gamma, const void* __restrict__ beta, float eps, void* out, int64_t rows,
                          int cols) {
  __shared__ float scratch[kLnThreads / 32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int64_t base = row * cols;
    auto value = [&](int i) {
      float a = Vec16<DT>::load1(x, base + i);
      if (residual != nullptr) a += Vec16<DT>::load1(residual, base + i);
      if (bias != nullptr) a += Vec16<DT>::load1(bias, i);
      return a;
    };
    float sum = 0.0f;
    for (int i = threadIdx.x; i < cols; i += kLnThreads) sum += value(i);
    const float mean = group_sum<kLnThreads>(sum, scratch) / (float)cols;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < cols; i += kLnThreads) {
      const float d = value(i) - mean;
      sq += d * d;
    }
    const float rstd = rsqrtf(group_sum<kLnThreads>(sq, scratch) / (float)cols + eps);
    for (int i = threadIdx.x; i < cols; i += kLnThreads) {
      float o = (value(i) - mean) * rstd;
      if (gamma != nullptr) o = o * Vec16<DT>::load1(gamma, i) + Vec16<DT>::load1(beta, i);
      Vec16<DT>::store1(out, base + i, o);  // out may alias x: every thread rereads only what it writes itself
    }
  }
}

// tanh form of GELU, the one the reference's fused kernels use (cuda_kernels.cu:29-36)
__device__ __forceinline__ float gelu_tanh(float x) {
  return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

template <int DT>
__global__ void __launch_bounds__(256)
add_bias_gelu_kernel(const void* x, const void* __restrict__ bias, void* out, int64_t n_vec,
                     int vec_per_row) {
  constexpr int EPV = Vec16<DT>::kElems;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * 256) {
    float a[EPV], b[EPV];
    Vec16<DT>::unpack(reinterpret_cast<const uint4*>(x)[i], a);
    if (bias != nullptr) {
      Vec16<DT>::unpack(reinterpret_cast<const uint4*>(bias)[i % vec_per_row], b);
#pragma unroll
      for (int k = 0; k < EPV; ++k) a[k] += b[k];
    }
#pragma unroll
    for (int k = 0; k < EPV; ++k) a[k] = gelu_tanh(a[k]);
    reinterpret_cast<uint4*>(out)[i] = Vec16<DT>::pack(a);
  }
}

template <int DT>
__global__ void __launch_bounds__(256)
add_bias_gelu_scalar_kernel(const void* x, const void* __restrict__ bias, void* out, int64_t n,
                            int cols) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    float a = Vec16<DT>::load1(x, i);
    if (bias != nullptr) a += Vec16<DT>::load1(bias, i % cols);
    Vec16<DT>::store1(out, i, gelu_tanh(a));
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int DT, bool FUSED>
int launch_layer_norm(const void* x, const void* residual, const void* bias, const void* gamma, const void* beta, float eps,
                      void* out, int64_t rows, int64_t cols, cudaStream_t st) {
  constexpr int EPV = Vec16<DT>::kElems;
  const bool vec_ok = cols % EPV == 0 && aligned16(x) && aligned16(out) && (residual == nullptr || aligned16(residual)) &&
                      (bias == nullptr || aligned16(bias)) && (gamma == nullptr || (aligned16(gamma) && aligned16(beta)));
  const int64_t nv = cols / EPV;
#define NTB200_LN_LAUNCH(VPL, GROUP)                                                                              \
  do {                                                                                                            \
    const int64_t rpb = kLnThreads / GROUP;                                                                       \
    const int64_t grid = (rows + rpb - 1) / rpb;                                                                  \
    if (grid > 0x7fffffff) return NTB200_INVALID_ARG;                                                             \
    if (nv == (int64_t)(VPL) * (GROUP))                                                                           \
      layer_norm_kernel<DT, VPL, GROUP, FUSED, true><<<(unsigned)grid, kLnThreads, 0, st>>>(x, residual, bias, gamma, beta, \
                                                                                           eps, out, rows, (int)cols); \
    else                                                                                                          \
      layer_norm_kernel<DT, VPL, GROUP, FUSED, false><<<(unsigned)grid, kLnThreads, 0, st>>>(x, residual, bias, gamma, beta, \
                                                                                            eps, out, rows, (int)cols); \
  } while (0)
  // Vectors per thread = ceil(nv / GROUP): widths such as 768, 1280 or 1536 get an exact fit (3, 5 or 6 vectors per
  // lane, no idle slots, the variant without bound tests) instead of the next power of two.  A packed 16-bit row
  // (no fused additions) stays on one warp up to 512 vectors: 16 loads in flight per lane, no block-wide reduction.
  constexpr bool kPacked = !FUSED && DT != NTB200_F32;
  if (vec_ok && nv <= 8) NTB200_LN_LAUNCH(1, 8);  // short rows: several rows per warp, every lane busy
  else if (vec_ok && nv <= 16) NTB200_LN_LAUNCH(1, 16);
  else if (vec_ok && nv <= 32) NTB200_LN_LAUNCH(1, 32);
  else if (vec_ok && nv <= 64) NTB200_LN_LAUNCH(2, 32);
  else if (vec_ok && nv <= 96) NTB200_LN_LAUNCH(3, 32);
  else if (vec_ok && nv <= 128) NTB200_LN_LAUNCH(4, 32);
  else if (vec_ok && nv <= 160) NTB200_LN_LAUNCH(5, 32);
  else if (vec_ok && nv <= 192) NTB200_LN_LAUNCH(6, 32);
  else if (vec_ok && nv <= 256) NTB200_LN_LAUNCH(8, 32);
  else if (vec_ok && kPacked && nv <= 512) {
    if constexpr (kPacked) {
      if (nv <= 384) NTB200_LN_LAUNCH(12, 32);
      else NTB200_LN_LAUNCH(16, 32);
    }
  } else if (vec_ok && nv <= 512) NTB200_LN_LAUNCH(2, kLnThreads);
  else if (vec_ok && nv <= 768) NTB200_LN_LAUNCH(3, kLnThreads);
  else if (vec_ok && nv <= 1024) NTB200_LN_LAUNCH(4, kLnThreads);
  else if (vec_ok && nv <= 1280) NTB200_LN_LAUNCH(5, kLnThreads);
  else if (vec_ok && nv <= 1536) NTB200_LN_LAUNCH(6, kLnThreads);
  else if (vec_ok && nv <= 2048) NTB200_LN_LAUNCH(8, kLnThreads);
  else {
    const int64_t grid = rows < 148 * 32 ? rows : 148 * 32;
    layer_norm_generic_kernel<DT><<<(unsigned)grid, kLnThreads, 0, st>>>(x, FUSED ? residual : nullptr,
                                                                        FUSED ? bias : nullptr, gamma, beta, eps, out, rows,
                                                                        (int)cols);
  }
#undef NTB200_LN_LAUNCH
  return status_from_cuda(cudaGetLastError());
}

int layer_norm_entry(const void* x, const void* residual, const void* bias, const void* gamma, const void* beta, float eps,
                     void* out, int64_t rows, int64_t cols, int dtype, void* stream) {
  if (rows < 0 || cols < 0 || cols > 0x7fffffff || !(eps >= 0.0f)) return NTB200_INVALID_ARG;
  if ((gamma == nullptr) != (beta == nullptr)) return NTB200_INVALID_ARG;
  if (rows == 0 || cols == 0) return NTB200_OK;
  if (x == nullptr || out == nullptr) return NTB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool fused = residual != nullptr || bias != nullptr;
  switch (dtype) {
    case NTB200_F32:
      return fused ? launch_layer_norm<NTB200_F32, true>(x, residual, bias, gamma, beta, eps, out, rows, cols, st)
                   : launch_layer_norm<NTB200_F32, false>(x, residual, bias, gamma, beta, eps, out, rows, cols, st);
    case NTB200_F16:
      return fused ? launch_layer_norm<NTB200_F16, true>(x, residual, bias, gamma, beta, eps, out, rows, cols, st)
                   : launch_layer_norm<NTB200_F16, false>(x, residual, bias, gamma, beta, eps, out, rows, cols, st);
    case NTB200_BF16:
      return fused ? launch_layer_norm<NTB200_BF16, true>(x, residual, bias, gamma, beta, eps, out, rows, cols, st)
                   : launch_layer_norm<NTB200_BF16, false>(x, residual, bias, gamma, beta, eps, out, rows, cols, st);
    default:
      return NTB200_UNSUPPORTED_DTYPE;
  }
}

template <int DT>
int launch_bias_gelu(const void* x, const void* bias, void* out, int64_t rows, int64_t cols, cudaStream_t st) {
  constexpr int EPV = Vec16<DT>::kElems;
  const int64_t n = rows * cols;
  if (cols % EPV == 0 && aligned16(x) && aligned16(out) && (bias == nullptr || aligned16(bias))) {
    const int64_t n_vec = n / EPV;
    int64_t grid = (n_vec + 255) / 256;
    if (grid > 148 * 64) grid = 148 * 64;
    add_bias_gelu_kernel<DT><<<(unsigned)grid, 256, 0, st>>>(x, bias, out, n_vec, (int)(cols / EPV));
  } else {
    int64_t grid = (n + 255) / 256;
    if (grid > 148 * 64) grid = 148 * 64;
    add_bias_gelu_scalar_kernel<DT><<<(unsigned)grid, 256, 0, st>>>(x, bias, out, n, (int)cols);
  }
  return status_from_cuda(cudaGetLastError());
}

}  // namespace
}  // namespace ntb200

extern "C" {

int ntb200_layer_norm(const void* x, const void* gamma, const void* beta, float eps, void* out, int64_t rows, int64_t cols,
                      int dtype, void* stream) {
  return ntb200::layer_norm_entry(x, nullptr, nullptr, gamma, beta, eps, out, rows, cols, dtype, stream);
}

int ntb200_add_bias_residual_layer_norm(const void* x, const void* residual, const void* bias, const void* gamma,
                                        const void* beta, float eps, void* out, int64_t rows, int64_t cols, int dtype,
                                        void* stream) {
  return ntb200::layer_norm_entry(x, residual, bias, gamma, beta, eps, out, rows, cols, dtype, stream);
}

int ntb200_add_bias_gelu(const void* x, const void* bias, void* out, int64_t rows, int64_t cols, int dtype, void* stream) {
  if (rows < 0 || cols < 0 || cols > 0x7fffffff) return NTB200_INVALID_ARG;
  if (rows == 0 || cols == 0) return NTB200_OK;
  if (x == nullptr || out == nullptr) return NTB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case NTB200_F32: return ntb200::launch_bias_gelu<NTB200_F32>(x, bias, out, rows, cols, st);
    case NTB200_F16: return ntb200::launch_bias_gelu<NTB200_F16>(x, bias, out, rows, cols, st);
    case NTB200_BF16: return ntb200::launch_bias_gelu<NTB200_BF16>(x, bias, out, rows, cols, st);
    default: return NTB200_UNSUPPORTED_DTYPE;
  }
}

}  // extern "C"

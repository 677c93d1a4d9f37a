// mma.sync building blocks of the attention kernels (fragment loads, swizzled shared-memory tiles, cp.async) and the
// warp-per-(sequence, head) kernel for sequences of at most 32 tokens, shared by attention.cu (stand-alone launch) and
// attention_tcgen05.cu (the same warps run beside the block that builds the tensor-memory kernel's work list).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace ntb200 {
namespace {

constexpr int64_t kTinyMaxLen = 32;  // longest sequence the warp-per-(sequence, head) kernel takes

template <typename T>
struct MmaOp;
template <>
struct MmaOp<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <>
struct MmaOp<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float x, float y) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// byte offset of 16-byte chunk `c` of row `r` in a [rows][D] two-byte tile; the chunk index is XOR-swizzled with
// the row so that the eight rows one ldmatrix phase reads fall into eight different 16-byte bank groups
template <int D>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
  if (D == 32) return (uint32_t)(r * 64 + ((c ^ ((r >> 1) & 3)) << 4));
  if (D == 64) return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4));
  return (uint32_t)(r * 256 + ((((c & 7) ^ (r & 7)) | (c & 8)) << 4));
}

// ------------------------------------------------------- short sequences: one warp per (sequence, head)
// When no sequence of the batch is longer than kR (16 or 32) tokens, a (sequence, head) pair is one or two 16-row MMA
// tiles and a tile per CTA (or a 128-row tensor-memory tile per work item) would spend its time on rows that do not
// exist: the time of the larger kernels then follows the number of sequences, not of tokens.  Here every WARP owns one
// (sequence, head): it stages the Q, K and V rows of the pair in its own slice of shared memory (16-byte cp.async,
// whole 16-row groups, rows past the end zero-filled), forms S = Q K^T with mma.sync.m16n8k16, applies one softmax over
// the (at most kR) keys in registers and multiplies by V.  A warp touches the rows of its own sequence only, so a
// NaN / Inf stays inside the sequence that holds it.  Sequences longer than kR are not computed (the caller passes the
// longest length); query rows of a sequence without keys are zeroed.
__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// The work of one warp: (sequence, head) number w of the flattened list; warp_smem = this warp's 3 * kR * kD * 2 bytes.
template <typename T, int kD, int kR>
__device__ __forceinline__ void attn_tiny_warp(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk,
                                               const T* __restrict__ v, int64_t ldv, T* __restrict__ out,
                                               const int64_t* __restrict__ offsets_q, const int64_t* __restrict__ offsets_k,
                                               int64_t batch, int H, float scale_log2e, int64_t w, uint32_t warp_smem) {
  constexpr uint32_t kTileBytes = kR * kD * 2;
  constexpr int kChunks = kD / 8;   // 16-byte chunks per row
  constexpr int kGroups = kR / 16;  // 16-key groups (and 16-query tiles) at most
  const int lane = threadIdx.x & 31;
  const int64_t b = w / H;
  if (b >= batch) return;
  const int h = (int)(w - b * H);
  const int64_t E = (int64_t)H * kD;
  const int64_t oq = offsets_q[b], ok = offsets_k[b];
  const int64_t Lq64 = (offsets_q[b + 1] - oq) / E, L64 = (offsets_k[b + 1] - ok) / E;
  if (Lq64 <= 0 || Lq64 > kR || L64 > kR) return;
  const int Lq = (int)Lq64, L = (int)L64;
  T* obase = out + (oq / E) * E + (int64_t)h * kD;
  if (L <= 0) {  // no keys: an empty softmax, the rows are zeros
    for (int i = lane; i < Lq * (kD / 2); i += 32) reinterpret_cast<uint32_t*>(obase + (int64_t)(i / (kD / 2)) * E)[i % (kD / 2)] = 0u;
    return;
  }
  const T* qbase = q + (oq / E) * ldq + (int64_t)h * kD;
  const T* kbase = k + (ok / E) * ldk + (int64_t)h * kD;
  const T* vbase = v + (ok / E) * ldv + (int64_t)h * kD;
  const uint32_t sq = warp_smem;
  const uint32_t sk = sq + kTileBytes, sv = sk + kTileBytes;
  const int rows_q = (Lq + 15) & ~15, rows_k = (L + 15) & ~15;
  for (int idx = lane; idx < rows_q * kChunks; idx += 32) {
    const int r = idx / kChunks, c = idx % kChunks;
    const bool valid = r < Lq;
    cp_async_16_zfill(sq + tile_off<kD>(r, c), qbase + (int64_t)(valid ? r : 0) * ldq + c * 8, valid ? 16u : 0u);
  }
  for (int idx = lane; idx < rows_k * kChunks; idx += 32) {
    const int r = idx / kChunks, c = idx % kChunks;
    const bool valid = r < L;
    cp_async_16_zfill(sk + tile_off<kD>(r, c), kbase + (int64_t)(valid ? r : 0) * ldk + c * 8, valid ? 16u : 0u);
    cp_async_16_zfill(sv + tile_off<kD>(r, c), vbase + (int64_t)(valid ? r : 0) * ldv + c * 8, valid ? 16u : 0u);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncwarp();

  constexpr int KS = kD / 16, NO = kD / 8;
  const int nkg = rows_k >> 4;  // groups of 16 keys staged (the rest of the tiles is not initialised and never read)
  for (int qt = 0; qt * 16 < Lq; ++qt) {
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) ldmatrix_x4(qf[ks], sq + tile_off<kD>(qt * 16 + (lane & 15), ks * 2 + (lane >> 4)));
    float s[2 * kGroups][4];  // n-tiles of 8 keys
#pragma unroll
    for (int i = 0; i < 2 * kGroups; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int np = 0; np < kGroups; ++np) {
        if (np < nkg) {
          uint32_t kf[4];
          ldmatrix_x4(kf, sk + tile_off<kD>(np * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
          MmaOp<T>::mma(s[np * 2], qf[ks], kf[0], kf[1]);
          MmaOp<T>::mma(s[np * 2 + 1], qf[ks], kf[2], kf[3]);
        }
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2 * kGroups; ++nt) {
      const int key = nt * 8 + 2 * (lane & 3);
      if (key >= L) s[nt][0] = s[nt][2] = -INFINITY;
      if (key + 1 >= L) s[nt][1] = s[nt][3] = -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = mx0 * scale_log2e, mn1 = mx1 * scale_log2e;
    float l0 = 0.0f, l1 = 0.0f;
    uint32_t pf[kGroups][4];  // P as A fragments: k-steps of 16 keys
#pragma unroll
    for (int nt = 0; nt < 2 * kGroups; ++nt) {
      const float p0 = exp2f(fmaf(s[nt][0], scale_log2e, -mn0));
      const float p1 = exp2f(fmaf(s[nt][1], scale_log2e, -mn0));
      const float p2 = exp2f(fmaf(s[nt][2], scale_log2e, -mn1));
      const float p3 = exp2f(fmaf(s[nt][3], scale_log2e, -mn1));
      l0 += p0 + p1;
      l1 += p2 + p3;
      pf[nt >> 1][(nt & 1) * 2] = MmaOp<T>::pack(p0, p1);
      pf[nt >> 1][(nt & 1) * 2 + 1] = MmaOp<T>::pack(p2, p3);
    }
    float o[NO][4];
#pragma unroll
    for (int i = 0; i < NO; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < kGroups; ++ks) {
      if (ks < nkg) {
#pragma unroll
        for (int np = 0; np < NO / 2; ++np) {
          uint32_t vf[4];
          ldmatrix_x4_trans(vf, sv + tile_off<kD>(ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), np * 2 + (lane >> 4)));
          MmaOp<T>::mma(o[np * 2], pf[ks], vf[0], vf[1]);
          MmaOp<T>::mma(o[np * 2 + 1], pf[ks], vf[2], vf[3]);
        }
      }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    const int r0 = qt * 16 + (lane >> 2), r1 = r0 + 8;
    uint32_t* orow0 = reinterpret_cast<uint32_t*>(obase + (int64_t)r0 * E);
    uint32_t* orow1 = reinterpret_cast<uint32_t*>(obase + (int64_t)r1 * E);
#pragma unroll
    for (int nt = 0; nt < NO; ++nt) {
      const int col2 = nt * 4 + (lane & 3);  // index in 32-bit pairs
      if (r0 < Lq) orow0[col2] = MmaOp<T>::pack(o[nt][0] * i0, o[nt][1] * i0);
      if (r1 < Lq) orow1[col2] = MmaOp<T>::pack(o[nt][2] * i1, o[nt][3] * i1);
    }
  }
}

template <typename T, int kD, int kR, int kWarps>
__global__ void __launch_bounds__(kWarps * 32)
attn_tiny_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk, const T* __restrict__ v, int64_t ldv,
                 T* __restrict__ out, const int64_t* __restrict__ offsets_q, const int64_t* __restrict__ offsets_k, int64_t batch,
                 int H, float scale_log2e) {
  extern __shared__ __align__(128) uint8_t tiny_smem[];  // per warp: Q, K and V tiles of kR x kD each
  const int warp = threadIdx.x >> 5;
  attn_tiny_warp<T, kD, kR>(q, ldq, k, ldk, v, ldv, out, offsets_q, offsets_k, batch, H, scale_log2e,
                            (int64_t)blockIdx.x * kWarps + warp,
                            (uint32_t)__cvta_generic_to_shared(tiny_smem) + (uint32_t)warp * (3u * kR * kD * 2u));
}

}  // namespace
}  // namespace ntb200

// Shared device/host helpers for the ntb200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "ntb200.h"

namespace ntb200 {

// Number of SMs on a B200; grids of persistent kernels are sized in multiples of it.
constexpr int kNumSMs = 148;

// ---------------------------------------------------------------------------------
// Division of a 31-bit dividend by a launch-constant 30-bit divisor with one
// multiply-high, one add and one shift (Granlund & Montgomery, "Division by invariant
// integers using multiplication", PLDI 1994, round-up variant).
// Valid for 1 <= d <= 2^30 and n < 2^31.
struct FastDiv {
  uint32_t d;
  uint32_t mul;
  uint32_t shift;
};

inline FastDiv make_fastdiv(uint64_t d64) {
  FastDiv f;
  uint32_t d = (uint32_t)d64;
  if (d == 0) d = 1;
  uint32_t shift = 0;
  while (shift < 32 && (1ull << shift) < d) ++shift;
  uint64_t magic = ((1ull << 32) * ((1ull << shift) - d)) / d + 1;
  f.d = d;
  f.mul = (uint32_t)magic;
  f.shift = shift;
  return f;
}

__host__ __device__ __forceinline__ uint32_t fastdiv(uint32_t n, const FastDiv& f) {
#ifdef __CUDA_ARCH__
  return (__umulhi(n, f.mul) + n) >> f.shift;
#else
  return (uint32_t)((((uint64_t)n * f.mul) >> 32) + n) >> f.shift;
#endif
}

// Index arithmetic policy: 32-bit + FastDiv when one padded entry has < 2^30 elements,
// true 64-bit division otherwise.
template <bool BIG>
struct IdxPolicy;
template <>
struct IdxPolicy<false> {
  using T = uint32_t;
  static __device__ __forceinline__ T div(T n, const FastDiv& f, uint64_t) { return fastdiv(n, f); }
};
template <>
struct IdxPolicy<true> {
  using T = uint64_t;
  static __device__ __forceinline__ T div(T n, const FastDiv&, uint64_t d) { return n / d; }
};

// quotient/remainder of two non-negative 64-bit values, 32-bit fast path when both fit
__device__ __forceinline__ void divmod_u64(uint64_t n, uint64_t d, uint64_t& q, uint64_t& r) {
  if (((n | d) >> 32) == 0) {
    uint32_t qq = (uint32_t)n / (uint32_t)d;
    q = qq;
    r = (uint32_t)n - qq * (uint32_t)d;
  } else {
    q = n / d;
    r = n - q * d;
  }
}

template <int ES>
struct ElemBits;
template <>
struct ElemBits<1> { using T = uint8_t; };
template <>
struct ElemBits<2> { using T = uint16_t; };
template <>
struct ElemBits<4> { using T = uint32_t; };
template <>
struct ElemBits<8> { using T = uint64_t; };

// largest b in [lo, hi] with offsets[b] <= e (requires offsets[lo] <= e)
__device__ __forceinline__ int64_t find_entry(const int64_t* __restrict__ offsets, int64_t lo, int64_t hi, int64_t e) {
  while (lo < hi) {
    const int64_t mid = (lo + hi + 1) >> 1;
    if (offsets[mid] <= e) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// The same search by a whole warp: 32 probes per step instead of one, so a batch of 4096 entries takes three
// dependent loads instead of twelve (every lane returns the result; requires offsets[lo] <= e).
__device__ __forceinline__ int64_t find_entry_warp(const int64_t* __restrict__ offsets, int64_t lo, int64_t hi, int64_t e) {
  const int lane = threadIdx.x & 31;
  while (hi > lo) {
    const int64_t span = hi - lo;                 // candidates lo + 1 .. hi
    const int64_t step = (span + 31) / 32;        // probe lo + step, lo + 2 step, ... (clamped to hi)
    int64_t probe = lo + step * (lane + 1);
    probe = probe > hi ? hi : probe;
    const unsigned le = __ballot_sync(0xffffffffu, offsets[probe] <= e);
    if (le == 0) {                                // the answer lies below the first probe
      hi = lo + step - 1;
    } else {
      const int top = 31 - __clz(le);             // last probe that is still <= e
      int64_t nlo = lo + step * (top + 1);
      nlo = nlo > hi ? hi : nlo;
      const int64_t nhi = nlo + step - 1;
      lo = nlo;
      hi = nhi > hi ? hi : nhi;
    }
  }
  return lo;
}

// 16-byte global accesses of the copy kernels.  Measured on B200 at the 4096 x (L_i, 1024) bf16 workload: default-cached
// loads and stores beat the streaming (.cs) forms (pad 6.62 vs 6.22 TB/s, unpad 6.31 vs 5.72 TB/s).
__device__ __forceinline__ uint4 ld_global_16_stream(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st_global_16_stream(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

// The 16 bytes at `sp` for 1- and 2-byte elements whose address is not 16-byte aligned: five aligned 4-byte words
// realigned with funnel shifts instead of sixteen or eight element loads.  Reads up to 3 bytes before `sp` (inside the
// aligned word that holds its first byte) and up to 3 bytes after sp + 16 (inside the word that holds its last byte);
// `limit` is the end of the source buffer, and a vector whose last word would pass it takes the element loads.
// Used by the pad kernels only: in the unpad kernels the same form measured slower (it keeps fewer loads in flight).
template <int ES>
__device__ __forceinline__ uint4 load16_realign(const void* sp, const void* limit) {
  static_assert(ES <= 2, "1- and 2-byte elements");
  const uintptr_t a = reinterpret_cast<uintptr_t>(sp);
  const uintptr_t w0 = a & ~uintptr_t(3);
  if (w0 + 20 <= reinterpret_cast<uintptr_t>(limit)) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(w0);
    const uint32_t c0 = w[0], c1 = w[1], c2 = w[2], c3 = w[3], c4 = w[4];
    const uint32_t shift = (uint32_t)(a & 3) * 8;  // (a funnel shift by 0 returns the low word)
    return make_uint4(__funnelshift_r(c0, c1, shift), __funnelshift_r(c1, c2, shift), __funnelshift_r(c2, c3, shift),
                      __funnelshift_r(c3, c4, shift));
  }
  union {
    uint4 v;
    uint8_t b1[16];
    uint16_t b2[8];
  } out;
  if (ES == 1) {
#pragma unroll
    for (int k = 0; k < 16; ++k) out.b1[k] = reinterpret_cast<const uint8_t*>(sp)[k];
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) out.b2[k] = reinterpret_cast<const uint16_t*>(sp)[k];
  }
  return out.v;
}

// One-time, per-device host set-up (cudaFuncSetAttribute and occupancy queries apply to the current device only, so
// a process that drives several GPUs must repeat them on each).  `done` is an array of kMaxDevices flags; `setup`
// runs with the calling thread's current device and returns false on failure.  Two threads racing on the same
// device may both run `setup`, which is idempotent.
constexpr int kMaxDevices = 64;
template <typename F>
inline bool once_per_device(std::atomic<int>* done, F&& setup) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return false;
  if (done[dev].load(std::memory_order_acquire) != 0) return true;
  if (!setup()) return false;
  done[dev].store(1, std::memory_order_release);
  return true;
}

inline int status_from_cuda(cudaError_t e) { return e == cudaSuccess ? NTB200_OK : NTB200_LAUNCH_FAILED; }

}  // namespace ntb200

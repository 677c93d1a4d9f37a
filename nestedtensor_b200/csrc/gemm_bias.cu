// C[M,N] = A[M,K] * W[N,K]^T + bias[N] on the packed token buffer of a nested tensor: the QKV and
// output projections of self-attention.  Tokens of all sequences are contiguous, so the "grouped
// varlen" projection is one M = sum(L_i) GEMM whose last row tile is predicated.
//
// Two code paths in one backend:
//   * fp16 / bf16, K % 8 == 0, N % 8 == 0: persistent warp-specialised tcgen05 kernel — TMA (128-byte
//     swizzle, no multicast) feeds a 4-stage shared-memory ring, one thread issues
//     tcgen05.mma.cta_group::1 (128 x 256 x 16) into two 256-column TMEM accumulators, eight epilogue warps
//     drain one accumulator (tcgen05.ld), add the bias and store while the other is being filled;
//   * everything else (fp32, odd shapes): a tiled SIMT kernel with fp32 accumulation.
// Replaces NestedTensor_matmul's packed fast path (nestedtensor/csrc/matmul.cpp:12-45, one cuBLAS GEMM)
// plus the separate bias pass of NestedTensor_add_Tensor (nestedtensor/csrc/BinaryOps.cpp:97-107).

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "attention_internal.cuh"
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ntb200 {
namespace {

// Set by a kernel whose bounded wait ran out (bit 0: producer, 1: MMA issuer, 2: epilogue).
__device__ int g_gemm_error = 0;

// ------------------------------------------------------------------------ tcgen05 path
constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4;
constexpr int kABytes = kBM * kBK * 2;            // 16 KB
constexpr int kBBytes = kBN * kBK * 2;            // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;    // 48 KB
constexpr int kAccCols = kBN;                     // fp32 accumulator columns per stage
constexpr int kTmemCols = 2 * kAccCols;           // 512: the whole TMEM, two accumulator stages
constexpr int kEpiWarps = 8;                      // two warps per tensor-memory lane quarter, 128 columns each
constexpr int kEpiThreads = 32 * kEpiWarps;
constexpr int kGemmThreads = 64 + kEpiThreads;    // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
constexpr int kCtrlBytes = 256 + kBN * 4;         // barriers + tmem slot + abort flag, bias tile
constexpr int kGemmSmem = 1024 + kStages * kStageBytes + kCtrlBytes;

struct Ctrl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint64_t done;
  uint32_t tmem_base;
  volatile int abort;
};
static_assert(sizeof(Ctrl) <= 256, "control block");

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = ptx::globaltimer_ns();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
      if (ptx::mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) return false;
  }
}

template <int FMT>
struct OutPack;
template <>
struct OutPack<0> {  // fp16
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float load(const void* p, int i) { return __half2float(reinterpret_cast<const __half*>(p)[i]); }
  static __device__ __forceinline__ float lo(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w & 0xffffu))); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }
};
template <>
struct OutPack<1> {  // bf16
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float load(const void* p, int i) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  }
  static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
};

// tanh form of GELU (the one the reference's fused kernels use, nestedtensor/csrc/cuda/cuda_kernels.cu:29-36)
// with the hardware tanh approximation (relative error 2^-11, below the 16-bit output rounding).
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (x + 0.044715f * x * x * x)));
  return 0.5f * x * (1.0f + t);
}

// 32 accumulator columns of one output row: + bias, optional GELU, optional + residual (the same 32 columns
// of the residual row, already in registers: the caller loads them a chunk ahead), packed to 16 bits, stored.  With `wide` (row stride and base
// 32-byte aligned) each store is one full 32-byte sector (st.global.v8); a warp-wide 16-byte store per row
// would touch every sector twice.
// The thread's own 64 bytes of the residual row for one 32-column chunk (zeros past the matrix edge).
__device__ __forceinline__ void load_res32(const uint16_t* res, int n_left, bool live, uint4 (&q)[4]) {
#pragma unroll
  for (int g = 0; g < 4; ++g)
    q[g] = (live && g * 8 < n_left) ? *reinterpret_cast<const uint4*>(res + g * 8) : make_uint4(0, 0, 0, 0);
}

// Pulls this thread's 128 columns (256 bytes) of the residual row towards L2 while the tile is still being
// accumulated, so that the loads in the epilogue find it there.
__device__ __forceinline__ void prefetch_res_l2(const uint16_t* rrow, bool live, int c_begin, int n_left) {
  if (rrow == nullptr || !live) return;
  if (c_begin < n_left) asm volatile("prefetch.global.L2 [%0];" ::"l"(rrow + c_begin));
  if (c_begin + 64 < n_left) asm volatile("prefetch.global.L2 [%0];" ::"l"(rrow + c_begin + 64));
}

template <int FMT>
__device__ __forceinline__ void store_chunk32(uint16_t* dst, const uint32_t (&r)[32], const float* bias32, int n_left,
                                              bool wide, int act, const uint4 (&res)[4], bool has_res) {
  float v[32];
#pragma unroll
  for (int k = 0; k < 32; ++k) v[k] = __uint_as_float(r[k]) + bias32[k];
  if (act == 1) {
    // tanh GELU on packed fp32 pairs: 0.5 x (1 + tanh(k x (1 + c x^2))), six packed FMA-pipe instructions and two
    // MUFU tanh per pair
    const uint64_t c2 = ptx::f32x2_pack(0.044715f, 0.044715f), one2 = ptx::f32x2_pack(1.0f, 1.0f);
    const uint64_t k2 = ptx::f32x2_pack(0.7978845608028654f, 0.7978845608028654f), half2 = ptx::f32x2_pack(0.5f, 0.5f);
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const uint64_t x = ptx::f32x2_pack(v[2 * k], v[2 * k + 1]);
      const uint64_t x2 = ptx::f32x2_fma(x, x, 0ull);
      const uint64_t arg = ptx::f32x2_fma(ptx::f32x2_fma(x, ptx::f32x2_fma(x2, c2, one2), 0ull), k2, 0ull);
      float a0, a1, t0, t1;
      ptx::f32x2_unpack(arg, a0, a1);
      asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(a0));
      asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(a1));
      const uint64_t hx = ptx::f32x2_fma(x, half2, 0ull);
      ptx::f32x2_unpack(ptx::f32x2_fma(hx, ptx::f32x2_pack(t0, t1), hx), v[2 * k], v[2 * k + 1]);
    }
  } else if (act == 2) {
#pragma unroll
    for (int k = 0; k < 32; ++k) v[k] = fmaxf(v[k], 0.0f);
  }
  if (has_res) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint32_t w[4] = {res[g].x, res[g].y, res[g].z, res[g].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[g * 8 + 2 * k] += OutPack<FMT>::lo(w[k]);
        v[g * 8 + 2 * k + 1] += OutPack<FMT>::hi(w[k]);
      }
    }
  }
  uint32_t p[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) p[k] = OutPack<FMT>::pack(v[2 * k], v[2 * k + 1]);
  if (wide) {
#pragma unroll
    for (int g = 0; g < 2; ++g)
      if (g * 16 < n_left)
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + g * 16), "r"(p[g * 8 + 0]),
                     "r"(p[g * 8 + 1]), "r"(p[g * 8 + 2]), "r"(p[g * 8 + 3]), "r"(p[g * 8 + 4]), "r"(p[g * 8 + 5]),
                     "r"(p[g * 8 + 6]), "r"(p[g * 8 + 7])
                     : "memory");
  } else {
#pragma unroll
    for (int g = 0; g < 4; ++g)
      if (g * 8 < n_left) *reinterpret_cast<uint4*>(dst + g * 8) = make_uint4(p[g * 4], p[g * 4 + 1], p[g * 4 + 2], p[g * 4 + 3]);
  }
}

template <int FMT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bias_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const void* __restrict__ bias, const void* __restrict__ residual, int act, void* __restrict__ C,
                         int M, int N, int K) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + kStages * kStageBytes);
  float* s_bias = reinterpret_cast<float*>(smem + kStages * kStageBytes + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (M + kBM - 1) / kBM, num_n = (N + kBN - 1) / kBN, num_k = (K + kBK - 1) / kBK;
  const int num_tiles = num_m * num_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctrl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&ctrl->tfull[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->tempty[a]), kEpiWarps);
    }
    ptx::mbar_init(ptx::smem_u32(&ctrl->done), 1);
    ctrl->abort = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&ctrl->tmem_base), kTmemCols);
    ptx::tmem_relinquish();
    ptx::tc_fence_before_sync();
  }
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = ctrl->tmem_base;
  const uint32_t smem_base = ptx::smem_u32(smem);

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (ptx::elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / num_n) * kBM, n0 = (tile % num_n) * kBN;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1;
          if (!wait_or_abort(ptx::smem_u32(&ctrl->empty[s]), ph ^ 1, &ctrl->abort)) {
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&ctrl->full[s]);
          ptx::mbar_arrive_expect_tx(full, kStageBytes);
          ptx::tma_load_2d(smem_base + s * kStageBytes, &map_a, full, kb * kBK, m0);
          ptx::tma_load_2d(smem_base + s * kStageBytes + kABytes, &map_w, full, kb * kBK, n0);
        }
      }
      if (!ok) {
        ctrl->abort = 1;
        atomicOr(&g_gemm_error, 1);
      }
      // drain: every load issued must have landed before this CTA's shared memory is released
      const uint32_t first = it > (uint32_t)kStages ? it - kStages : 0;
      for (uint32_t i = first; i < it; ++i)
        ptx::mbar_wait(ptx::smem_u32(&ctrl->full[i % kStages]), (i / kStages) & 1);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::umma_idesc_f16(FMT, kBM, kBN);
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_iter) {
        const uint32_t acc = tile_iter & 1;
        if (!wait_or_abort(ptx::smem_u32(&ctrl->tempty[acc]), ((tile_iter >> 1) & 1) ^ 1, &ctrl->abort)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1;
          if (!wait_or_abort(ptx::smem_u32(&ctrl->full[s]), ph, &ctrl->abort)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = smem_base + s * kStageBytes, b_addr = a_addr + kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            ptx::umma_f16(d_tmem, ptx::umma_desc_kmajor_sw128(a_addr + k * 32), ptx::umma_desc_kmajor_sw128(b_addr + k * 32),
                          idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(ptx::smem_u32(&ctrl->empty[s]));  // frees the stage when these MMAs retire
        }
        if (ok) ptx::umma_commit(ptx::smem_u32(&ctrl->tfull[acc]));
      }
      if (!ok) {
        ctrl->abort = 1;
        atomicOr(&g_gemm_error, 2);
      }
      // all MMAs must have retired before TMEM is freed
      ptx::umma_commit(ptx::smem_u32(&ctrl->done));
      ptx::mbar_wait(ptx::smem_u32(&ctrl->done), 0);
    }
  } else {
    // ---------------------------------------------------------------- epilogue (256 threads)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int et = threadIdx.x - 64;
    const bool wide = (N % 16 == 0) && (reinterpret_cast<uintptr_t>(C) % 32 == 0);
    uint32_t tile_iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_iter) {
      const int m0 = (tile / num_n) * kBM, n0 = (tile % num_n) * kBN;
      const uint32_t acc = tile_iter & 1;
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");  // previous tile's bias reads are done
      for (int i = et; i < kBN; i += kEpiThreads) {
        const int n = n0 + i;
        s_bias[i] = (bias != nullptr && n < N) ? OutPack<FMT>::load(bias, n) : 0.0f;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      const int row = m0 + q * 32 + lane;
      uint16_t* crow = reinterpret_cast<uint16_t*>(C) + (size_t)row * N + n0;
      const uint16_t* rrow = residual != nullptr ? reinterpret_cast<const uint16_t*>(residual) + (size_t)row * N + n0 : nullptr;
      prefetch_res_l2(rrow, row < M, ((warp - 2) >> 2) * (kBN / 2), N - n0);  // while the main loop of this tile still runs
      if (ok && !wait_or_abort(ptx::smem_u32(&ctrl->tfull[acc]), (tile_iter >> 1) & 1, &ctrl->abort)) ok = false;
      if (!ok) continue;  // keep taking the named barriers with the other epilogue warps
      ptx::tc_fence_after_sync();
      // two register buffers: the tensor-memory load of the next 32 columns runs under the bias add, the
      // packing and the stores of the current ones
      const uint32_t tacc = tmem_base + acc * kAccCols + ((uint32_t)(q * 32) << 16);
      uint32_t ra[32], rb[32];
      uint4 qa[4], qb[4];  // the residual of the same chunks, loaded together with the accumulator
      const bool has_res = rrow != nullptr, res_live = has_res && row < M;
      const int c_begin = ((warp - 2) >> 2) * (kBN / 2), c_end = c_begin + kBN / 2;  // this warp's 128 columns
      if (n0 + c_begin < N) {
        ptx::tmem_ld_32x32b_x32(tacc + c_begin, ra);
        if (has_res) load_res32(rrow + c_begin, N - (n0 + c_begin), res_live, qa);
      }
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 64) {
        if (n0 + c >= N) break;
        ptx::tmem_ld_wait();
        const bool second = n0 + c + 32 < N;
        if (second) {
          ptx::tmem_ld_32x32b_x32(tacc + c + 32, rb);
          if (has_res) load_res32(rrow + c + 32, N - (n0 + c + 32), res_live, qb);
        }
        if (row < M) store_chunk32<FMT>(crow + c, ra, s_bias + c, N - (n0 + c), wide, act, qa, has_res);
        if (!second) break;
        ptx::tmem_ld_wait();
        if (c + 64 < c_end && n0 + c + 64 < N) {
          ptx::tmem_ld_32x32b_x32(tacc + c + 64, ra);
          if (has_res) load_res32(rrow + c + 64, N - (n0 + c + 64), res_live, qa);
        }
        if (row < M) store_chunk32<FMT>(crow + c + 32, rb, s_bias + c + 32, N - (n0 + c + 32), wide, act, qb, has_res);
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctrl->tempty[acc]));
    }
    if (!ok && lane == 0) {
      ctrl->abort = 1;
      atomicOr(&g_gemm_error, 4);
    }
  }

  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------- tcgen05 path, CTA pairs (cta_group::2)
// A cluster of two CTAs computes a 256 x 256 tile: CTA r loads rows [r*128, r*128+128) of the A tile and
// rows [r*128, r*128+128) of the W tile (half of N) into its own shared memory; one thread of CTA 0 issues
// tcgen05.mma.cta_group::2 (M = 256), which reads both CTAs' operands and writes each CTA's 128 accumulator
// rows into that CTA's tensor memory.  Per FLOP this moves 1.5x fewer bytes from L2 into the SMs than the
// single-CTA 128 x 256 tile.  No load is multicast: every CTA fetches what it needs itself, the TMA
// completion bytes of both CTAs land on CTA 0's barrier, and CTA 0 releases stages / publishes
// accumulators with one commit per CTA.
constexpr int k2Stages = 6;
constexpr int k2HalfBytes = 128 * kBK * 2;          // 16 KB: 128 rows x 64 columns
constexpr int k2StageBytes = 2 * k2HalfBytes;       // A half + W half
constexpr int k2Smem = 1024 + k2Stages * k2StageBytes + kCtrlBytes;

struct Ctrl2 {
  uint64_t full[k2Stages];    // used in CTA 0: bytes of both CTAs
  uint64_t empty[k2Stages];   // one per CTA
  uint64_t tfull[2];          // one per CTA
  uint64_t tempty[2];         // used in CTA 0: the epilogue warps of both CTAs arrive
  uint64_t done;
  uint64_t rfull[4];          // RES: residual box landed (bytes), one per 64-column box of this CTA's 128 x 256 tile
  uint64_t rempty[4];         // RES: the four warps that read a box are done with it
  uint32_t tmem_base;
  volatile int abort;
};
static_assert(sizeof(Ctrl2) <= 256, "control block");
// RES (a residual matrix is added in the epilogue): the residual tile of each CTA, 128 rows x 256 columns, is staged
// in shared memory by TMA as four 128 x 64 boxes (16 KB each, 128-byte swizzle) instead of per-thread 64-byte row
// reads; it takes the place of one main-loop stage and a bit.  Each group of four epilogue warps (128 columns) owns
// two boxes; the first warp's lane 0 reloads a box for the CTA's next tile as soon as the four warps have released
// it, so the load of box h for tile i + 1 runs under the epilogue of the other box and the next main loop.
constexpr int k2ResBoxBytes = 128 * 64 * 2;
constexpr int k2ResBytes = 4 * k2ResBoxBytes;
constexpr int k2StagesRes = k2Stages - 1;
constexpr int k2SmemRes = 1024 + k2StagesRes * k2StageBytes + k2ResBytes + kCtrlBytes;
static_assert(k2SmemRes <= 232448, "shared memory of the residual variant");

// The thread's 64 bytes (32 columns) of row r of a swizzled 128 x 64 residual box: 16-byte units u0 .. u0 + 3.
__device__ __forceinline__ void load_res_smem(uint32_t box, int r, int u0, uint4 (&q)[4]) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const uint32_t addr = box + (uint32_t)r * 128u + ((uint32_t)((u0 + g) ^ (r & 7)) << 4);
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(q[g].x), "=r"(q[g].y), "=r"(q[g].z), "=r"(q[g].w) : "r"(addr));
  }
}

template <int FMT, bool RES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bias_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                              const __grid_constant__ CUtensorMap map_r, const void* __restrict__ bias,
                              const void* __restrict__ residual, int act, void* __restrict__ C, int M, int N, int K) {
  constexpr int k2Stages = RES ? k2StagesRes : ntb200::k2Stages;  // (shadows the namespace constant below)
  constexpr int kResOff = k2Stages * k2StageBytes;                // residual boxes (RES), then the control block
  constexpr int kCtrlOff = kResOff + (RES ? k2ResBytes : 0);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctrl2* ctrl = reinterpret_cast<Ctrl2*>(smem + kCtrlOff);
  float* s_bias = reinterpret_cast<float*>(smem + kCtrlOff + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_m = (M + 255) / 256, num_n = (N + 255) / 256, num_k = (K + kBK - 1) / kBK;
  const int num_tiles = num_m * num_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < k2Stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctrl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&ctrl->tfull[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->tempty[a]), 2 * kEpiWarps);
    }
    ptx::mbar_init(ptx::smem_u32(&ctrl->done), 1);
    if (RES) {
      for (int j = 0; j < 4; ++j) {
        ptx::mbar_init(ptx::smem_u32(&ctrl->rfull[j]), 1);
        ptx::mbar_init(ptx::smem_u32(&ctrl->rempty[j]), 4);
      }
      ptx::prefetch_tensormap(&map_r);
    }
    ctrl->abort = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(&ctrl->tmem_base), kTmemCols);
    ptx::tmem_relinquish_pair();
    ptx::tc_fence_before_sync();
  }
  // both CTAs' barriers exist before either signals the other
  ptx::cluster_arrive();
  ptx::cluster_wait();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = ctrl->tmem_base;
  const uint32_t smem_base = ptx::smem_u32(smem);

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (ptx::elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile / num_n) * 256 + (int)rank * 128, n0 = (tile % num_n) * 256 + (int)rank * 128;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const uint32_t s = it % k2Stages, ph = (it / k2Stages) & 1;
          if (!wait_or_abort(ptx::smem_u32(&ctrl->empty[s]), ph ^ 1, &ctrl->abort)) {
            ok = false;
            break;
          }
          const uint32_t full_local = ptx::smem_u32(&ctrl->full[s]);
          const uint32_t full_leader = ptx::mapa_shared(full_local, 0);
          if (rank == 0) ptx::mbar_arrive_expect_tx(full_local, 2 * k2StageBytes);
          ptx::tma_load_2d_pair(smem_base + s * k2StageBytes, &map_a, full_leader, kb * kBK, m0);
          ptx::tma_load_2d_pair(smem_base + s * k2StageBytes + k2HalfBytes, &map_w, full_leader, kb * kBK, n0);
        }
      }
      if (!ok) {
        ctrl->abort = 1;
        atomicOr(&g_gemm_error, 1);
      }
      if (rank == 0) {  // CTA 0 sees the landing of both CTAs' loads on its own barriers
        const uint32_t first = it > (uint32_t)k2Stages ? it - k2Stages : 0;
        for (uint32_t i = first; i < it; ++i) ptx::mbar_wait(ptx::smem_u32(&ctrl->full[i % k2Stages]), (i / k2Stages) & 1);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (CTA 0 only)
    if (rank == 0 && ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::umma_idesc_f16(FMT, 256, kBN);
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tile_iter) {
        const uint32_t acc = tile_iter & 1;
        if (!wait_or_abort(ptx::smem_u32(&ctrl->tempty[acc]), ((tile_iter >> 1) & 1) ^ 1, &ctrl->abort)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const uint32_t s = it % k2Stages, ph = (it / k2Stages) & 1;
          if (!wait_or_abort(ptx::smem_u32(&ctrl->full[s]), ph, &ctrl->abort)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = smem_base + s * k2StageBytes, b_addr = a_addr + k2HalfBytes;
          const uint64_t da = ptx::umma_desc_kmajor_sw128(a_addr), db = ptx::umma_desc_kmajor_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) ptx::umma_f16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          // free the stage in both CTAs once these MMAs retire
          const uint32_t e = ptx::smem_u32(&ctrl->empty[s]);
          ptx::umma_commit_pair(e);
          ptx::umma_commit_pair(ptx::mapa_shared(e, 1));
        }
        if (ok) {
          const uint32_t t = ptx::smem_u32(&ctrl->tfull[acc]);
          ptx::umma_commit_pair(t);
          ptx::umma_commit_pair(ptx::mapa_shared(t, 1));
        }
      }
      if (!ok) {
        ctrl->abort = 1;
        atomicOr(&g_gemm_error, 2);
      }
      ptx::umma_commit_pair(ptx::smem_u32(&ctrl->done));
      ptx::mbar_wait(ptx::smem_u32(&ctrl->done), 0);
    }
  } else {
    // ---------------------------------------------------------------- epilogue (256 threads per CTA)
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    const bool wide = (N % 16 == 0) && (reinterpret_cast<uintptr_t>(C) % 32 == 0);
    uint32_t tile_iter = 0;
    bool ok = true;
    uint32_t res_issued[2] = {0, 0}, res_landed[2] = {0, 0};  // RES, loader thread: loads issued / seen landed per box
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++tile_iter) {
      const int m0 = (tile / num_n) * 256 + (int)rank * 128, n0 = (tile % num_n) * 256;
      const uint32_t acc = tile_iter & 1;
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      for (int i = et; i < kBN; i += kEpiThreads) {
        const int n = n0 + i;
        s_bias[i] = (bias != nullptr && n < N) ? OutPack<FMT>::load(bias, n) : 0.0f;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      const int row = m0 + q * 32 + lane;
      uint16_t* crow = reinterpret_cast<uint16_t*>(C) + (size_t)row * N + n0;
      if constexpr (RES) {
        const int g = (warp - 2) >> 2;                          // column group: boxes 2g and 2g + 1
        const bool loader = ((warp - 2) & 3) == 0 && lane == 0;  // reloads the group's boxes
        const int c_begin = g * (kBN / 2);
        const uint32_t box0 = smem_base + kResOff + (uint32_t)(2 * g) * k2ResBoxBytes;
        const int next_tile = tile + num_pairs;
        if (tile_iter == 0 && loader) {  // the first tile's boxes (later ones are loaded a tile ahead, below)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t bar = ptx::smem_u32(&ctrl->rfull[2 * g + h]);
            ptx::mbar_arrive_expect_tx(bar, k2ResBoxBytes);
            ptx::tma_load_2d(box0 + h * k2ResBoxBytes, &map_r, bar, n0 + c_begin + 64 * h, m0);
            res_issued[h] = 1;
          }
        }
        __syncwarp();
        if (ok && !wait_or_abort(ptx::smem_u32(&ctrl->tfull[acc]), (tile_iter >> 1) & 1, &ctrl->abort)) ok = false;
        if (!ok) continue;  // (aborted: nobody issues or awaits anything further; the loads in flight are drained below)
        ptx::tc_fence_after_sync();
        const uint32_t tacc = tmem_base + acc * kAccCols + ((uint32_t)(q * 32) << 16);
        const int r_loc = q * 32 + lane;
        uint32_t ra[32], rb[32];
        uint4 qa[4], qb[4];
        if (n0 + c_begin < N) ptx::tmem_ld_32x32b_x32(tacc + c_begin, ra);
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          const int c = c_begin + 64 * h;
          const uint32_t box = box0 + h * k2ResBoxBytes;
          if (!wait_or_abort(ptx::smem_u32(&ctrl->rfull[2 * g + h]), tile_iter & 1, &ctrl->abort)) ok = false;
          else res_landed[h] = tile_iter + 1;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            ptx::tmem_ld_wait();  // (a tensor-memory load may be in flight)
            break;
          }
          if (n0 + c < N) {  // (uniform over the group)
            ptx::tmem_ld_wait();
            const bool second = n0 + c + 32 < N;
            if (second) ptx::tmem_ld_32x32b_x32(tacc + c + 32, rb);
            load_res_smem(box, r_loc, 0, qa);
            if (row < M) store_chunk32<FMT>(crow + c, ra, s_bias + c, N - (n0 + c), wide, act, qa, true);
            if (second) {
              ptx::tmem_ld_wait();
              if (h == 0 && n0 + c + 64 < N) ptx::tmem_ld_32x32b_x32(tacc + c + 64, ra);
              load_res_smem(box, r_loc, 4, qb);
              if (row < M) store_chunk32<FMT>(crow + c + 32, rb, s_bias + c + 32, N - (n0 + c + 32), wide, act, qb, true);
            }
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctrl->rempty[2 * g + h]));
          if (loader && next_tile < num_tiles) {  // the same box of the CTA's next tile, once all four warps left it
            if (wait_or_abort(ptx::smem_u32(&ctrl->rempty[2 * g + h]), tile_iter & 1, &ctrl->abort)) {
              const int nm0 = (next_tile / num_n) * 256 + (int)rank * 128, nn0 = (next_tile % num_n) * 256;
              const uint32_t bar = ptx::smem_u32(&ctrl->rfull[2 * g + h]);
              ptx::mbar_arrive_expect_tx(bar, k2ResBoxBytes);
              ptx::tma_load_2d(box, &map_r, bar, nn0 + c, nm0);
              res_issued[h] = tile_iter + 2;
            } else {
              ctrl->abort = 1;
            }
          }
          __syncwarp();
        }
        if (!ok) continue;
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(ptx::smem_u32(&ctrl->tempty[acc]), 0));
        continue;
      }
      const uint16_t* rrow = residual != nullptr ? reinterpret_cast<const uint16_t*>(residual) + (size_t)row * N + n0 : nullptr;
      prefetch_res_l2(rrow, row < M, ((warp - 2) >> 2) * (kBN / 2), N - n0);  // while the main loop of this tile still runs
      if (ok && !wait_or_abort(ptx::smem_u32(&ctrl->tfull[acc]), (tile_iter >> 1) & 1, &ctrl->abort)) ok = false;
      if (!ok) continue;
      ptx::tc_fence_after_sync();
      // two register buffers: the tensor-memory load of the next 32 columns runs under the bias add, the
      // packing and the stores of the current ones
      const uint32_t tacc = tmem_base + acc * kAccCols + ((uint32_t)(q * 32) << 16);
      uint32_t ra[32], rb[32];
      uint4 qa[4], qb[4];  // the residual of the same chunks, loaded together with the accumulator
      const bool has_res = rrow != nullptr, res_live = has_res && row < M;
      const int c_begin = ((warp - 2) >> 2) * (kBN / 2), c_end = c_begin + kBN / 2;  // this warp's 128 columns
      if (n0 + c_begin < N) {
        ptx::tmem_ld_32x32b_x32(tacc + c_begin, ra);
        if (has_res) load_res32(rrow + c_begin, N - (n0 + c_begin), res_live, qa);
      }
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 64) {
        if (n0 + c >= N) break;
        ptx::tmem_ld_wait();
        const bool second = n0 + c + 32 < N;
        if (second) {
          ptx::tmem_ld_32x32b_x32(tacc + c + 32, rb);
          if (has_res) load_res32(rrow + c + 32, N - (n0 + c + 32), res_live, qb);
        }
        if (row < M) store_chunk32<FMT>(crow + c, ra, s_bias + c, N - (n0 + c), wide, act, qa, has_res);
        if (!second) break;
        ptx::tmem_ld_wait();
        if (c + 64 < c_end && n0 + c + 64 < N) {
          ptx::tmem_ld_32x32b_x32(tacc + c + 64, ra);
          if (has_res) load_res32(rrow + c + 64, N - (n0 + c + 64), res_live, qa);
        }
        if (row < M) store_chunk32<FMT>(crow + c + 32, rb, s_bias + c + 32, N - (n0 + c + 32), wide, act, qb, has_res);
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      // the accumulator stage is free when the epilogue warps of BOTH CTAs have read it: all arrive at CTA 0
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa_shared(ptx::smem_u32(&ctrl->tempty[acc]), 0));
    }
    if (!ok && lane == 0) {
      ctrl->abort = 1;
      atomicOr(&g_gemm_error, 4);
    }
    if (RES) {  // after an abort: a residual box still in flight must land before the shared memory is released
#pragma unroll
      for (int h = 0; h < 2; ++h)
        if (res_issued[h] > res_landed[h])
          ptx::mbar_wait(ptx::smem_u32(&ctrl->rfull[2 * ((warp - 2) >> 2) + h]), (res_issued[h] - 1) & 1);
    }
  }

  // neither CTA may free tensor memory or leave (its barriers are signalled remotely) before both are done
  ptx::tc_fence_before_sync();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// row-major [rows, cols] two-byte matrix, box = box_rows x 64 columns, 128-byte swizzle, zero fill
bool make_map_2d(CUtensorMap* map, const void* base, int dtype, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return false;
  const cuuint64_t gdim[2] = {cols, rows};
  const cuuint64_t gstride[1] = {cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == NTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int FMT>
int launch_tcgen05(const void* A, const void* W, const void* bias, const void* residual, int act, void* C, int M, int N, int K,
                   int dtype, cudaStream_t st) {
  CUtensorMap map_a, map_w;
  if (!make_map_2d(&map_a, A, dtype, (uint64_t)M, (uint64_t)K, kBM)) return NTB200_LAUNCH_FAILED;
  if (!make_map_2d(&map_w, W, dtype, (uint64_t)N, (uint64_t)K, kBN)) return NTB200_LAUNCH_FAILED;
  static std::atomic<int> attr_set[kMaxDevices];
  if (!once_per_device(attr_set, [] {
        return cudaFuncSetAttribute(gemm_bias_tcgen05_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem) ==
               cudaSuccess;
      }))
    return NTB200_LAUNCH_FAILED;
  const int num_tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
  int dev = 0, sms = kNumSMs;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = num_tiles < sms ? num_tiles : sms;
  gemm_bias_tcgen05_kernel<FMT><<<grid, kGemmThreads, kGemmSmem, st>>>(map_a, map_w, bias, residual, act, C, M, N, K);
  return status_from_cuda(cudaGetLastError());
}

template <int FMT, bool RES>
int launch_tcgen05_pair(const void* A, const void* W, const void* bias, const void* residual, int act, void* C, int M, int N,
                        int K, int dtype, cudaStream_t st) {
  constexpr int smem_bytes = RES ? k2SmemRes : k2Smem;
  CUtensorMap map_a, map_w, map_r;
  if (!make_map_2d(&map_a, A, dtype, (uint64_t)M, (uint64_t)K, 128)) return NTB200_LAUNCH_FAILED;
  if (!make_map_2d(&map_w, W, dtype, (uint64_t)N, (uint64_t)K, 128)) return NTB200_LAUNCH_FAILED;
  if (RES) {
    if (!make_map_2d(&map_r, residual, dtype, (uint64_t)M, (uint64_t)N, 128)) return NTB200_LAUNCH_FAILED;
  } else {
    map_r = map_a;  // (not read)
  }
  static std::atomic<int> attr_set[kMaxDevices];
  if (!once_per_device(attr_set, [] {
        return cudaFuncSetAttribute(gemm_bias_tcgen05_pair_kernel<FMT, RES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    smem_bytes) == cudaSuccess;
      }))
    return NTB200_LAUNCH_FAILED;
  const int num_tiles = ((M + 255) / 256) * ((N + 255) / 256);
  int dev = 0, sms = kNumSMs;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // how many CTA pairs can be resident at once (GPCs with an odd SM count leave one SM without a partner)
  static std::atomic<int> max_pairs_of[kMaxDevices];
  if (dev < 0 || dev >= kMaxDevices) return NTB200_LAUNCH_FAILED;
  int max_pairs = max_pairs_of[dev].load(std::memory_order_relaxed);
  if (max_pairs == 0) {
    cfg.gridDim = dim3(2 * (sms / 2));
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_bias_tcgen05_pair_kernel<FMT, RES>, &cfg) == cudaSuccess && n > 0) max_pairs = n;
    else max_pairs = sms / 2;
    (void)cudaGetLastError();
    max_pairs_of[dev].store(max_pairs, std::memory_order_relaxed);
  }
  const int pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
  cfg.gridDim = dim3(2 * pairs);
  if (cudaLaunchKernelEx(&cfg, gemm_bias_tcgen05_pair_kernel<FMT, RES>, map_a, map_w, map_r, bias, residual, act, C, M, N, K) !=
      cudaSuccess) {
    (void)cudaGetLastError();
    return NTB200_LAUNCH_FAILED;
  }
  return status_from_cuda(cudaGetLastError());
}

// --------------------------------------------------------------------------- SIMT path
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

constexpr int kSimtTile = 64, kSimtK = 16;

template <typename T>
__global__ void __launch_bounds__(256) gemm_bias_simt_kernel(const T* __restrict__ A, const T* __restrict__ W,
                                                             const T* __restrict__ bias, const T* __restrict__ residual,
                                                             int act, T* __restrict__ C, int64_t M, int64_t N, int64_t K) {
  __shared__ float sA[kSimtK][kSimtTile + 1];
  __shared__ float sW[kSimtK][kSimtTile + 1];
  const int64_t m0 = (int64_t)blockIdx.y * kSimtTile, n0 = (int64_t)blockIdx.x * kSimtTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += kSimtK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int r = idx >> 4, kk = idx & 15;
      const int64_t k = k0 + kk;
      sA[kk][r] = (m0 + r < M && k < K) ? Cvt<T>::to_f(A[(m0 + r) * K + k]) : 0.0f;
      sW[kk][r] = (n0 + r < N && k < K) ? Cvt<T>::to_f(W[(n0 + r) * K + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSimtK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = sA[kk][ty * 4 + i];
        w[i] = sW[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n < N) {
        float v = acc[i][j] + (bias != nullptr ? Cvt<T>::to_f(bias[n]) : 0.0f);
        if (act == 1) v = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        if (act == 2) v = fmaxf(v, 0.0f);
        if (residual != nullptr) v += Cvt<T>::to_f(residual[m * N + n]);
        C[m * N + n] = Cvt<T>::from_f(v);
      }
    }
  }
}

template <typename T>
int launch_simt(const void* A, const void* W, const void* bias, const void* residual, int act, void* C, int64_t M, int64_t N,
                int64_t K, cudaStream_t st) {
  const int64_t gx = (N + kSimtTile - 1) / kSimtTile, gy = (M + kSimtTile - 1) / kSimtTile;
  if (gx > 0x7fffffffll || gy > 65535) return NTB200_UNSUPPORTED_SHAPE;
  dim3 grid((unsigned)gx, (unsigned)gy);
  gemm_bias_simt_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(A), static_cast<const T*>(W),
                                                 static_cast<const T*>(bias), static_cast<const T*>(residual), act,
                                                 static_cast<T*>(C), M, N, K);
  return status_from_cuda(cudaGetLastError());
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int gemm_error_flags_read_and_clear() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
  }
  return v;
}

}  // namespace ntb200

using namespace ntb200;

extern "C" {

int ntb200_gemm_bias_act(const void* A, const void* W, const void* bias, const void* residual, void* C, int64_t M, int64_t N,
                         int64_t K, int dtype, int act, int force_simt, void* stream) {
  if (M < 0 || N < 0 || K < 0 || act < 0 || act > 2) return NTB200_INVALID_ARG;
  if (dtype != NTB200_F32 && dtype != NTB200_F16 && dtype != NTB200_BF16) return NTB200_UNSUPPORTED_DTYPE;
  if (M == 0 || N == 0) return NTB200_OK;
  if (A == nullptr || W == nullptr || C == nullptr) return NTB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // force_simt: 0 = best available, 1 = SIMT, 2 = single-CTA tcgen05 kernel, 3 = CTA-pair tcgen05 kernel,
  // 4 = CTA-pair kernel that reads the residual rows per thread whatever K is (for comparisons)
  const bool tc = force_simt != 1 && dtype != NTB200_F32 && K >= 8 && (K % 8) == 0 && (N % 8) == 0 && aligned16(A) && aligned16(W) &&
                  aligned16(C) && (residual == nullptr || aligned16(residual)) && M < (1ll << 31) - 256 && N < (1ll << 31) - 256 && K < (1ll << 31) - kBK;
  if ((force_simt == 2 || force_simt == 3 || force_simt == 4) && !tc) return NTB200_UNSUPPORTED_SHAPE;
  if (force_simt < 0 || force_simt > 4) return NTB200_INVALID_ARG;
  if (tc) {
    const bool pair = force_simt == 3 || force_simt == 4 || (force_simt == 0 && M > 128);
    // The residual tile comes through shared memory (at the price of one main-loop stage) while the main loop of a
    // tile is short; from K = 2048 on the per-thread row reads of the other variant hide under it (K = 4096: 2 % faster).
    if (pair && residual != nullptr && K < 2048 && force_simt != 4) {
      if (dtype == NTB200_F16) return launch_tcgen05_pair<0, true>(A, W, bias, residual, act, C, (int)M, (int)N, (int)K, dtype, st);
      return launch_tcgen05_pair<1, true>(A, W, bias, residual, act, C, (int)M, (int)N, (int)K, dtype, st);
    }
    if (pair) {
      if (dtype == NTB200_F16) return launch_tcgen05_pair<0, false>(A, W, bias, residual, act, C, (int)M, (int)N, (int)K, dtype, st);
      return launch_tcgen05_pair<1, false>(A, W, bias, residual, act, C, (int)M, (int)N, (int)K, dtype, st);
    }
    if (dtype == NTB200_F16) return launch_tcgen05<0>(A, W, bias, residual, act, C, (int)M, (int)N, (int)K, dtype, st);
    return launch_tcgen05<1>(A, W, bias, residual, act, C, (int)M, (int)N, (int)K, dtype, st);
  }
  const size_t es = dtype == NTB200_F32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(A) % es) || (reinterpret_cast<uintptr_t>(W) % es) || (reinterpret_cast<uintptr_t>(C) % es) ||
      (reinterpret_cast<uintptr_t>(residual) % es))
    return NTB200_MISALIGNED;
  switch (dtype) {
    case NTB200_F32: return launch_simt<float>(A, W, bias, residual, act, C, M, N, K, st);
    case NTB200_F16: return launch_simt<__half>(A, W, bias, residual, act, C, M, N, K, st);
    case NTB200_BF16: return launch_simt<__nv_bfloat16>(A, W, bias, residual, act, C, M, N, K, st);
  }
  return NTB200_UNSUPPORTED_DTYPE;
}

int ntb200_gemm_bias(const void* A, const void* W, const void* bias, void* C, int64_t M, int64_t N, int64_t K, int dtype,
                     int force_simt, void* stream) {
  return ntb200_gemm_bias_act(A, W, bias, nullptr, C, M, N, K, dtype, 0, force_simt, stream);
}

int ntb200_device_error_flags(void) {
  const int g = gemm_error_flags_read_and_clear();
  const int a = attn_tcgen05_error_flags_read_and_clear();
  const int c = construct_error_flags_read_and_clear();
  if (g < 0 || a < 0 || c < 0) return -1;
  return g | (a << 8) | (c << 16);
}

}  // extern "C"

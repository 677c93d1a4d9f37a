// Variable-length self-attention on tcgen05 tensor cores, head_dim 64, fp16 / bf16.
//
// One CTA = one (sequence, head, 128-query tile).  For every block of 128 keys:
//     S[128 x n]   = Q K^T          tcgen05.mma, both operands K-major in shared memory (TMA, 128-B swizzle)
//     P            = exp2(scale*log2e*S - m)   one softmax thread per query ROW (TMEM lane = row, so no
//                                   cross-thread reduction); P is written back over S as packed 16-bit
//     O[128 x 64] += P V            tcgen05.mma with A = P read from tensor memory, B = V tile as MN-major
// S / P (128 columns) and O (64 columns) live in tensor memory (256 columns per CTA, two CTAs per SM so
// one CTA's softmax overlaps the other's MMAs).  Q, K and V tiles come straight out of the packed token
// matrices through 2-D tensor maps (row = token, column = head): for self-attention the three maps are one map over
// the [T, 3E] projection output with column offsets 0 / E / 2E; for cross-attention (queries of sequence b over the
// keys / values of sequence b of another nested tensor) they are maps over the [Tq, E] query projection and the
// key / value projections.  Padded tokens are never materialised; rows past the end of a sequence belong to the next
// sequence (or are zero-filled past the end of the buffer) and are masked / cleared / never stored.
// The list of (sequence, query tile) work items is built on the device, longest sequences first.
// Every wait is bounded; a wait that runs out sets an error flag, the CTA drains and frees its TMEM.
// Replaces steps 2-8 of bt_min_mha (nestedtensor/csrc/cuda/mha.cpp:59-105).

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "attention_internal.cuh"
#include "attention_tiny.cuh"
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ntb200 {
namespace {

__device__ int g_attn_error = 0;  // bit 0 producer, 1 MMA issuer, 2 softmax

constexpr int kQT = 128;   // query rows per CTA (TMEM lanes)
constexpr int kKV = 128;   // keys per block
constexpr int kHD = 64;    // head dim
constexpr int kTile = kQT * kHD * 2;  // 16 KB: one 128 x 64 two-byte tile
constexpr int kStages = 2;
// Of the 16 key pairs of a 32-key chunk, pair 2k+1 is exponentiated by the polynomial when bit k is set
// (0xff: half of all exponentials, 0xaa: a quarter, 0: none), the others on the MUFU unit.  A quarter measured
// best on B200 at the BERT-large batch (none: +1 %, half: +6 %).
constexpr unsigned kPolyPairs = 0xaa;
// A row's reference maximum is raised (and its running output rescaled) only when a block's maximum exceeds it
// by more than this many powers of two.
constexpr float kLazyRescale = 8.0f;
constexpr int kTmemCols = 256;        // S: columns [0,128), P: [128,192), O: [192,256)
constexpr int kPCol = 128;
constexpr int kOCol = 192;
constexpr int kAttnThreads = 256;     // warps 0-3 softmax, warp 4 TMA, warp 5 MMA, warps 6-7 idle
// Register exchange of setmaxnreg.  A request for more registers than the other warps of the CTA give back blocks for
// ever (it is not one of the bounded waits), so the two counts must add up to twice the count the kernel is launched
// with: 128 at two 256-thread CTAs per SM.  With eight warps every SM sub-partition hosts one softmax warp and one
// control / idle warp of the CTA, so the exchange also balances per sub-partition.
constexpr int kRegLaunch = 65536 / (2 * kAttnThreads);
constexpr int kRegSoftmax = 208;
constexpr int kRegControl = 48;
static_assert(kRegSoftmax + kRegControl == 2 * kRegLaunch && kRegLaunch % 8 == 0, "setmaxnreg exchange must balance");
constexpr int kAttnSmem = 1024 + kTile * (2 + 2 * kStages) + 256;  // 2 Q buffers + 2 stages of (K, V)

struct Ctrl {
  uint64_t full_k[kStages];   // K tile (plus Q with the first block of an item) landed
  uint64_t empty_k[kStages];  // QK^T of that stage retired: K (and the Q buffer two items back) reusable
  uint64_t full_v[kStages];
  uint64_t empty_v[kStages];  // PV of that stage retired (and the softmax warps have stored its P)
  uint64_t s_ready;
  uint64_t s_free;
  uint64_t p_ready;
  uint64_t o_ready;
  uint64_t done;
  uint32_t tmem_base;
  volatile int abort;
};

static_assert(sizeof(Ctrl) <= 256, "control block exceeds its shared-memory slot");

__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = ptx::globaltimer_ns();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (ptx::mbar_try_wait_suspend(bar, parity, 20000u)) return true;
    if (*abort_flag) return false;
    if (ptx::globaltimer_ns() - t0 > ptx::kWaitLimitNs) return false;
  }
}

template <int FMT>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (FMT == 0) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// ------------------------------------------------------------------ work list
// items[i] = (first query token of the tile, valid query rows in the tile, first key token of the sequence, number
// of keys) for every 128-query tile, ordered by decreasing number of key blocks so that the longest items start
// first; *count = number of items.  Sequences without queries or without keys produce no item; the output rows of a
// sequence without keys are zeroed here (an empty softmax).  Sequences of at most skip_short queries and keys produce
// no item either: the caller has given them to the warp-per-(sequence, head) kernel.  One block.
constexpr int kListThreads = 1024;
constexpr int kBuckets = 9;  // key blocks 1..8+, (0 unused)

template <bool SELF>  // SELF: queries and keys are the same sequences, so none has queries without keys
__device__ __forceinline__ void build_items_block(const int64_t* __restrict__ offsets_q, const int64_t* __restrict__ offsets_k,
                                                  int64_t batch, int64_t row_elems, int4* __restrict__ items,
                                                  int* __restrict__ count, int64_t capacity, uint16_t* __restrict__ out,
                                                  int skip_short) {
  const int nthreads = (int)blockDim.x;  // 1024 alone, 256 beside the short-sequence warps
  __shared__ int s_cnt[kBuckets];
  __shared__ int s_base[kBuckets];
  if (threadIdx.x < kBuckets) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  for (int64_t b = threadIdx.x; b < batch; b += nthreads) {
    const int64_t Lq = (offsets_q[b + 1] - offsets_q[b]) / row_elems, Lk = (offsets_k[b + 1] - offsets_k[b]) / row_elems;
    if (Lq <= 0 || Lk <= 0 || (Lq <= skip_short && Lk <= skip_short)) continue;
    const int nq = (int)((Lq + kQT - 1) / kQT);
    int nb = (int)((Lk + kKV - 1) / kKV);
    nb = nb >= kBuckets ? kBuckets - 1 : nb;
    atomicAdd(&s_cnt[nb], nq);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int k = kBuckets - 1; k >= 1; --k) {
      s_base[k] = acc;
      acc += s_cnt[k];
    }
    *count = acc < capacity ? acc : (int)capacity;
  }
  __syncthreads();
  for (int64_t b = threadIdx.x; b < batch; b += nthreads) {
    const int64_t Lq = (offsets_q[b + 1] - offsets_q[b]) / row_elems, Lk = (offsets_k[b + 1] - offsets_k[b]) / row_elems;
    if (Lq <= 0 || Lk <= 0 || (Lq <= skip_short && Lk <= skip_short)) continue;
    const int nq = (int)((Lq + kQT - 1) / kQT);
    int nb = (int)((Lk + kKV - 1) / kKV);
    nb = nb >= kBuckets ? kBuckets - 1 : nb;
    const int pos = atomicAdd(&s_base[nb], nq);
    const int tq0 = (int)(offsets_q[b] / row_elems), tk0 = (int)(offsets_k[b] / row_elems);
    for (int t = 0; t < nq; ++t) {
      const int64_t rows = Lq - (int64_t)t * kQT < kQT ? Lq - (int64_t)t * kQT : kQT;
      if (pos + t < capacity) items[pos + t] = make_int4(tq0 + t * kQT, (int)rows, tk0, (int)Lk);
    }
  }
  if (SELF) return;
  // Queries whose key sequence is empty get zeros (self-attention never has any: Lq == Lk).  The sequences are found in
  // parallel and listed in shared memory; the block then clears their rows together.
  __shared__ int s_nempty;
  __shared__ int s_empty[kListThreads];
  if (threadIdx.x == 0) s_nempty = 0;
  __syncthreads();
  for (int64_t b = threadIdx.x; b < batch; b += nthreads) {
    if (offsets_k[b + 1] > offsets_k[b] || offsets_q[b + 1] == offsets_q[b]) continue;
    const int pos = atomicAdd(&s_nempty, 1);
    if (pos < kListThreads) {
      s_empty[pos] = (int)b;
    } else {  // more than the list holds: this thread clears the rows itself
      for (int64_t e = offsets_q[b]; e < offsets_q[b + 1]; ++e) out[e] = 0;
    }
  }
  __syncthreads();
  const int n_listed = s_nempty < kListThreads ? s_nempty : kListThreads;
  for (int i = 0; i < n_listed; ++i) {
    const int64_t e0 = offsets_q[s_empty[i]], e1 = offsets_q[s_empty[i] + 1];
    for (int64_t e = e0 + threadIdx.x; e < e1; e += nthreads) out[e] = 0;
  }
}

__global__ void __launch_bounds__(kListThreads) build_items_kernel(const int64_t* __restrict__ offsets_q,
                                                                   const int64_t* __restrict__ offsets_k, int64_t batch,
                                                                   int64_t row_elems, int4* __restrict__ items,
                                                                   int* __restrict__ count, int64_t capacity,
                                                                   uint16_t* __restrict__ out) {
  build_items_block<false>(offsets_q, offsets_k, batch, row_elems, items, count, capacity, out, 0);
}

// The same list for self-attention on the default path, in one launch with the short sequences: block 0 builds the list
// without the sequences of at most kTinyMaxLen tokens, and every warp of the other blocks computes one (sequence, head)
// of those sequences by itself (attn_tiny_warp; it returns at once for a longer sequence).  The short sequences thus
// cost no launch of their own, and which kernel computes a sequence depends on its own length only.
constexpr int kPrepWarps = 8;
constexpr int kPrepSmem = kPrepWarps * 3 * (int)kTinyMaxLen * kHD * 2;  // 96 KB: Q, K, V tiles of 32 x 64 per warp

template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32)
prepare_self_attention_kernel(const int64_t* __restrict__ offsets, int64_t batch, int64_t row_elems, int4* __restrict__ items,
                              int* __restrict__ count, int64_t capacity, const T* __restrict__ qkv, T* __restrict__ out, int H,
                              float scale_log2e) {
  extern __shared__ __align__(128) uint8_t prep_smem[];
  if (blockIdx.x == 0) {
    build_items_block<true>(offsets, offsets, batch, row_elems, items, count, capacity, reinterpret_cast<uint16_t*>(out), (int)kTinyMaxLen);
    return;
  }
  const int warp = threadIdx.x >> 5;
  attn_tiny_warp<T, kHD, (int)kTinyMaxLen>(qkv, 3 * row_elems, qkv + row_elems, 3 * row_elems, qkv + 2 * row_elems, 3 * row_elems, out,
                                           offsets, offsets, batch, H, scale_log2e, ((int64_t)blockIdx.x - 1) * kPrepWarps + warp,
                                           (uint32_t)__cvta_generic_to_shared(prep_smem) + (uint32_t)warp * (uint32_t)(kPrepSmem / kPrepWarps));
}

// ------------------------------------------------------------------ attention
// Persistent: CTA c works on items c, c + gridDim.x, ... of the flattened (work item, head) list.  All
// barriers run on one global block counter g (one phase per 128-key block).
//   warps 0-3  softmax warpgroup (one thread per query row; registers raised with setmaxnreg so a whole
//              128-key row of S lives in registers: S is read from tensor memory ONCE per block)
//   warp 4     TMA producer   warp 5  MMA issuer (also clears V rows past a sequence's end)   warps 6-7  idle
// Tensor memory (256 columns): S [0,128) fp32, P [128,192) packed 16-bit, O [192,256) fp32.  P has its own
// columns, so QK^T of block g+1 is issued as soon as the softmax warps have read S of block g
// (s_free), before PV of block g: the tensor pipe works under the softmax of the same CTA.
// Two 256-thread CTAs per SM at 128 registers per thread; the control warpgroup then drops to 48 and the
// softmax warpgroup rises to 208.
// The output of an item is written during the FIRST block of the next item (after that block's row maximum,
// 16 columns at a time so that it fits beside the live S row): its last PV retires while the next S is loaded
// and reduced, instead of being waited for.  The softmax warps sit at their register budget; this only pays
// because the write needs about 30 registers (it spilled, and lost 20 %, before the row sums were cut to two
// packed accumulators).
template <int FMT>
__global__ void __launch_bounds__(kAttnThreads, 2)
attn_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, int col_q, int col_k, int col_v, void* __restrict__ out,
                    const int4* __restrict__ items, const int* __restrict__ count, int H, float scale_log2e) {
  const int n_items = *count;
  if ((int64_t)blockIdx.x >= (int64_t)n_items * H) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + kTile * (2 + 2 * kStages));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t E = (int64_t)H * kHD;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctrl->full_k[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->empty_k[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->full_v[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->empty_v[s]), 5);  // PV commit + the four softmax warps
    }
    ptx::mbar_init(ptx::smem_u32(&ctrl->s_ready), 1);
    ptx::mbar_init(ptx::smem_u32(&ctrl->s_free), 4);
    ptx::mbar_init(ptx::smem_u32(&ctrl->p_ready), 4);
    ptx::mbar_init(ptx::smem_u32(&ctrl->o_ready), 1);
    ptx::mbar_init(ptx::smem_u32(&ctrl->done), 1);
    ctrl->abort = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
  }
  if (warp == 5) {
    ptx::tmem_alloc(ptx::smem_u32(&ctrl->tmem_base), kTmemCols);
    ptx::tmem_relinquish();
    ptx::tc_fence_before_sync();
  }
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = ctrl->tmem_base;
  const uint32_t s_q = ptx::smem_u32(smem);          // two Q buffers
  const uint32_t s_k = s_q + 2 * kTile;              // K ring: stage s at s_k + s*kTile
  const uint32_t s_v = s_k + kStages * kTile;        // V ring: stage s at s_v + s*kTile

  // One 16-byte record per work item; every role fetches the record of its NEXT item while it works on
  // the current one, so the load latency never sits on a critical path.
  struct Item {
    int tq, rows, h, L, tok0, n_blk;  // first query token and valid rows of the tile; keys: first token and count
  };
  // Position in the flattened (work item, head) list; a CTA steps through it by gridDim.x without a
  // division per item.
  struct Pos {
    int item, h;
  };
  const int step_items = (int)(gridDim.x / (unsigned)H), step_heads = (int)(gridDim.x % (unsigned)H);
  const Pos first = {(int)(blockIdx.x / (unsigned)H), (int)(blockIdx.x % (unsigned)H)};
  auto next = [&](Pos p) {
    p.item += step_items;
    p.h += step_heads;
    if (p.h >= H) {
      p.h -= H;
      ++p.item;
    }
    return p;
  };
  auto fetch = [&](const Pos& p) { return p.item < n_items ? __ldg(items + p.item) : make_int4(0, 1, 0, 1); };
  auto decode = [&](const Pos& p, const int4& w) {
    Item it;
    it.h = p.h;
    it.tq = w.x;
    it.rows = w.y;
    it.tok0 = w.z;
    it.L = w.w;
    it.n_blk = (w.w + kKV - 1) / kKV;
    return it;
  };

  if (warp >= 4) {
    ptx::setmaxnreg_dec<kRegControl>();
    if (warp == 4 && ptx::elect_one()) {
      // ------------------------------------------------------------ TMA producer
      bool ok = true;
      uint32_t g = 0, n = 0;
      int4 rec = fetch(first);
      for (Pos i = first; i.item < n_items && ok; i = next(i), ++n) {
        const Item it = decode(i, rec);
        rec = fetch(next(i));
        for (int j = 0; j < it.n_blk; ++j, ++g) {
          const uint32_t s = g % kStages, ph = (g / kStages) & 1;
          // K (and Q) as soon as the QK^T that last read this stage has retired ...
          if (!wait_or_abort(ptx::smem_u32(&ctrl->empty_k[s]), ph ^ 1, &ctrl->abort)) {
            ok = false;
            break;
          }
          const uint32_t fk = ptx::smem_u32(&ctrl->full_k[s]);
          ptx::mbar_arrive_expect_tx(fk, (j == 0 ? 2 : 1) * kTile);
          // Q buffer n&1 was last read by item n-2, all of whose QK^T precede the release of this stage
          if (j == 0) ptx::tma_load_2d(s_q + (n & 1) * kTile, &map_q, fk, col_q + it.h * kHD, it.tq);
          ptx::tma_load_2d(s_k + s * kTile, &map_k, fk, col_k + it.h * kHD, it.tok0 + j * kKV);
          // ... V only once the PV that last read its stage has retired
          if (!wait_or_abort(ptx::smem_u32(&ctrl->empty_v[s]), ph ^ 1, &ctrl->abort)) {
            ok = false;
            ++g;  // the K load of this block was issued: include it in the drain below
            break;
          }
          const uint32_t fv = ptx::smem_u32(&ctrl->full_v[s]);
          ptx::mbar_arrive_expect_tx(fv, kTile);
          ptx::tma_load_2d(s_v + s * kTile, &map_v, fv, col_v + it.h * kHD, it.tok0 + j * kKV);
        }
      }
      if (!ok) {
        ctrl->abort = 1;
        atomicOr(&g_attn_error, 1);
      }
      // every issued load must land before exit (a V load that was never issued after an abort cannot
      // complete; that wait is bounded and runs out)
      const uint32_t first = g > (uint32_t)kStages ? g - kStages : 0;
      for (uint32_t k = first; k < g; ++k) {
        ptx::mbar_wait(ptx::smem_u32(&ctrl->full_k[k % kStages]), (k / kStages) & 1);
        if (ok) ptx::mbar_wait(ptx::smem_u32(&ctrl->full_v[k % kStages]), (k / kStages) & 1);
      }
    } else if (warp == 5 && ptx::elect_one()) {
      // ------------------------------------------------------------ MMA issuer
      bool ok = true;
      const uint32_t t_s = tmem_base, t_p = tmem_base + kPCol, t_o = tmem_base + kOCol;
      constexpr uint32_t idesc_pv = ptx::umma_idesc_f16(FMT, kQT, kHD, 0, 1);  // B = V is MN-major
      const uint64_t desc_q0 = ptx::umma_desc_kmajor_sw128(s_q);
      const uint64_t desc_k0 = ptx::umma_desc_kmajor_sw128(s_k);
      const uint64_t desc_v0 = ptx::umma_desc_mnmajor_sw128(s_v);
      // cursor A: the block whose QK^T is issued next (runs one block ahead of cursor B: PV)
      Pos ia = first;
      uint32_t ga = 0, na = 0;
      int ja = 0;
      Item a = decode(ia, fetch(ia));
      int4 rec_a = fetch(next(ia));
      auto issue_qk = [&]() -> bool {
        const uint32_t s = ga % kStages, ph = (ga / kStages) & 1;
        if (!wait_or_abort(ptx::smem_u32(&ctrl->full_k[s]), ph, &ctrl->abort)) return false;
        ptx::tc_fence_after_sync();
        int nvalid = a.L - ja * kKV;
        nvalid = nvalid > kKV ? kKV : nvalid;
        const uint32_t idesc_qk = ptx::umma_idesc_f16(FMT, kQT, (nvalid + 15) & ~15);
        const uint64_t dq = desc_q0 + (uint64_t)((na & 1) * (kTile >> 4));
        const uint64_t dk = desc_k0 + (uint64_t)(s * (kTile >> 4));
#pragma unroll
        for (int k = 0; k < kHD / 16; ++k) ptx::umma_f16(t_s, dq + 2 * k, dk + 2 * k, idesc_qk, k != 0 ? 1u : 0u);
        ptx::umma_commit(ptx::smem_u32(&ctrl->empty_k[s]));
        ptx::umma_commit(ptx::smem_u32(&ctrl->s_ready));
        ++ga;
        if (++ja == a.n_blk) {
          ja = 0;
          ++na;
          ia = next(ia);
          a = decode(ia, rec_a);
          rec_a = fetch(next(ia));
        }
        return true;
      };
      ok = issue_qk();
      uint32_t gb = 0;
      int4 rec_b = fetch(first);
      for (Pos ib = first; ib.item < n_items && ok; ib = next(ib)) {
        const Item b = decode(ib, rec_b);
        rec_b = fetch(next(ib));
        for (int jb = 0; jb < b.n_blk && ok; ++jb, ++gb) {
          // S of block gb is in the softmax warps' registers: the next QK^T may overwrite it
          if (ia.item < n_items) {
            if (!wait_or_abort(ptx::smem_u32(&ctrl->s_free), gb & 1, &ctrl->abort)) { ok = false; break; }
            if (!issue_qk()) { ok = false; break; }
          }
          const uint32_t s = gb % kStages;
          int nvalid = b.L - jb * kKV;
          nvalid = nvalid > kKV ? kKV : nvalid;
          if ((nvalid & 15) != 0) {
            // The last 16-key step of a ragged block multiplies P (exactly zero there) with V rows that belong to the
            // NEXT sequence: 0 x NaN or 0 x Inf in such a row would reach this sequence's output.  While the softmax
            // warps are still busy with this block, this thread clears those rows of the landed V tile, so that a
            // non-finite value stays inside the sequence that holds it (the reference pads every sequence with zeros).
            if (!wait_or_abort(ptx::smem_u32(&ctrl->full_v[s]), (gb / kStages) & 1, &ctrl->abort)) { ok = false; break; }
            const int r_end = (nvalid + 15) & ~15;
            for (int r = nvalid; r < r_end; ++r) {
              const uint32_t addr = s_v + s * kTile + (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
#pragma unroll
              for (int c = 0; c < 8; ++c)
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr + c * 16), "r"(0u) : "memory");
            }
            ptx::fence_proxy_async();  // make the generic-proxy stores visible to the tensor core's reads
          }
          if (!wait_or_abort(ptx::smem_u32(&ctrl->p_ready), gb & 1, &ctrl->abort)) { ok = false; break; }
          if (!wait_or_abort(ptx::smem_u32(&ctrl->full_v[s]), (gb / kStages) & 1, &ctrl->abort)) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const int ksteps = (nvalid + 15) >> 4;
          const uint64_t dv = desc_v0 + (uint64_t)(s * (kTile >> 4));
#pragma unroll
          for (int ks = 0; ks < kKV / 16; ++ks) {
            if (ks < ksteps)
              ptx::umma_f16_ts(t_o, t_p + ks * 8, dv + (uint64_t)(ks * (2048 >> 4)), idesc_pv, (jb | ks) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(ptx::smem_u32(&ctrl->empty_v[s]));
          ptx::umma_commit(ptx::smem_u32(&ctrl->o_ready));
        }
      }
      if (!ok) {
        ctrl->abort = 1;
        atomicOr(&g_attn_error, 2);
      }
      // every MMA issued must have retired before tensor memory is freed
      ptx::umma_commit(ptx::smem_u32(&ctrl->done));
      ptx::mbar_wait(ptx::smem_u32(&ctrl->done), 0);
    }
  } else {
    // ------------------------------------------------------------ softmax, one thread per query row
    ptx::setmaxnreg_inc<kRegSoftmax>();
    const int q = warp;                              // TMEM lane quarter of this warp
    const int row = q * 32 + lane;                   // row inside the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr, t_p = tmem_base + kPCol + lane_addr, t_o = tmem_base + kOCol + lane_addr;
    bool ok = true;
    uint32_t g = 0;

    // State of the item whose output is still to be written (by write_pending, during the next item).
    struct Pending {
      bool any;          // an item is waiting for its output
      bool warp_active;  // this warp owns valid rows of it
      float inv;         // 1 / softmax denominator of this thread's row
      int rows;          // valid rows in the tile
      int64_t out_row0;  // element offset of (first token of the tile, head) in the output
    } pend = {false, false, 0.0f, 0, 0};
    auto write_pending = [&]() {
      // each thread normalises its own row and stores it 32 bytes (one full sector) at a time, 16 accumulator
      // columns per step so that it fits beside a live S row
      if (pend.warp_active) {
        const bool live = row < pend.rows;  // (the tensor-memory loads are warp-wide: only the store is per row)
        const float inv = pend.inv;
        uint16_t* orow = reinterpret_cast<uint16_t*>(out) + pend.out_row0 + (int64_t)row * E;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r0[16];
          ptx::tmem_ld_32x32b_x16(t_o + c * 16, r0);
          ptx::tmem_ld_wait();
          if (live)
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(orow + c * 16),
                       "r"(pack2<FMT>(__uint_as_float(r0[0]) * inv, __uint_as_float(r0[1]) * inv)),
                       "r"(pack2<FMT>(__uint_as_float(r0[2]) * inv, __uint_as_float(r0[3]) * inv)),
                       "r"(pack2<FMT>(__uint_as_float(r0[4]) * inv, __uint_as_float(r0[5]) * inv)),
                       "r"(pack2<FMT>(__uint_as_float(r0[6]) * inv, __uint_as_float(r0[7]) * inv)),
                       "r"(pack2<FMT>(__uint_as_float(r0[8]) * inv, __uint_as_float(r0[9]) * inv)),
                       "r"(pack2<FMT>(__uint_as_float(r0[10]) * inv, __uint_as_float(r0[11]) * inv)),
                       "r"(pack2<FMT>(__uint_as_float(r0[12]) * inv, __uint_as_float(r0[13]) * inv)),
                       "r"(pack2<FMT>(__uint_as_float(r0[14]) * inv, __uint_as_float(r0[15]) * inv))
                       : "memory");
        }
      }
      pend.any = false;
    };
    int4 rec = fetch(first);
    for (Pos i = first; i.item < n_items; i = next(i)) {
      const Item it = decode(i, rec);
      rec = fetch(next(i));
      const bool warp_active = q * 32 < it.rows;  // warp-uniform
      float m = -INFINITY, l = 0.0f;
      for (int j = 0; j < it.n_blk; ++j, ++g) {
        if (ok && !wait_or_abort(ptx::smem_u32(&ctrl->s_ready), g & 1, &ctrl->abort)) ok = false;
        int nvalid = it.L - j * kKV;
        nvalid = nvalid > kKV ? kKV : nvalid;
        const int nchunks = (nvalid + 31) >> 5;
        uint32_t sv[4][32];  // the whole row of S (up to 128 keys) in registers
        if (ok && warp_active) {
          ptx::tc_fence_after_sync();
          ptx::tmem_ld_32x32b_x32(t_s, sv[0]);
          if (nchunks > 1) ptx::tmem_ld_32x32b_x32(t_s + 32, sv[1]);
          if (nchunks > 2) ptx::tmem_ld_32x32b_x32(t_s + 64, sv[2]);
          if (nchunks > 3) ptx::tmem_ld_32x32b_x32(t_s + 96, sv[3]);
          ptx::tmem_ld_wait();
        }
        // S has been consumed: the MMA warp may issue the next block's QK^T
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctrl->s_free));
        float m_new = m, corr = 1.0f;
        bool any_up = false;
        if (ok && warp_active) {
          // Keys past the end of the sequence become -inf once, here, so that the maximum and the exponentials
          // below need no per-element predicate (only the last 32-key chunk of a block can be ragged).
          // (Written as a loop of zero or one trips: as a plain `if` the compiler predicates the 128 selects and
          // issues them for every block, ragged or not - about 230 cycles per block on the measured build.)
#pragma unroll 1
          for (int ragged = (nvalid & 31) != 0 ? 1 : 0; ragged > 0; --ragged) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              // (a range test, not "c == nchunks - 1": the latter is turned into a run-time index and sends the
              // row to local memory)
              if (nvalid > c * 32 && nvalid < (c + 1) * 32) {
#pragma unroll
                for (int k = 0; k < 32; ++k) sv[c][k] = (c * 32 + k >= nvalid) ? 0xff800000u : sv[c][k];
              }
            }
          }
          // row maximum, four independent chains of three-input maxima
          float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c < nchunks) {
#pragma unroll
              for (int k = 0; k < 32; k += 8) {
                mx0 = ptx::fmax3(mx0, __uint_as_float(sv[c][k]), __uint_as_float(sv[c][k + 1]));
                mx1 = ptx::fmax3(mx1, __uint_as_float(sv[c][k + 2]), __uint_as_float(sv[c][k + 3]));
                mx2 = ptx::fmax3(mx2, __uint_as_float(sv[c][k + 4]), __uint_as_float(sv[c][k + 5]));
                mx3 = ptx::fmax3(mx3, __uint_as_float(sv[c][k + 6]), __uint_as_float(sv[c][k + 7]));
              }
            }
          }
          const float mxs = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2e;
          if (j == 0) {
            m_new = mxs;  // the first block of an item: O is overwritten and the row sum starts at zero
          } else {
            // Lazy rescaling: while no row of the warp exceeds its reference maximum by more than kLazyRescale, the
            // reference stays and P simply grows up to 2^kLazyRescale, which fp32 sums and 16-bit P hold without
            // loss; the final division by the row sum cancels the offset.
            any_up = __any_sync(0xffffffffu, mxs > m + kLazyRescale);
            if (any_up) {
              m_new = fmaxf(m, mxs);
              corr = ptx::ex2_approx(m - m_new);
            }
          }
        }
        // PV of the previous block must have retired before P is overwritten / O is rescaled
        if (ok && g > 0 && !wait_or_abort(ptx::smem_u32(&ctrl->o_ready), (g - 1) & 1, &ctrl->abort)) ok = false;
        if (ok && j == 0 && pend.any) {
          // Output of the previous item, written while this item's first block is already in flight: its last
          // PV retired during the work above, and this item's first PV (which overwrites O) cannot be issued
          // before these warps arrive at p_ready below.
          ptx::tc_fence_after_sync();
          write_pending();
        }
        if (ok && warp_active) {
          ptx::tc_fence_after_sync();
          if (any_up) {
            // rescale the running output (only when some row of the warp raised its reference maximum)
#pragma unroll
            for (int c = 0; c < 4; ++c) {  // 16 columns at a time: the S row stays live in registers
              uint32_t r0[16];
              ptx::tmem_ld_32x32b_x16(t_o + c * 16, r0);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 16; ++k) r0[k] = __float_as_uint(__uint_as_float(r0[k]) * corr);
              ptx::tmem_st_32x32b_x16(t_o + c * 16, r0);
            }
          }
          // P = exp2(S*scale*log2e - m_new), packed two per column.  A quarter of the exponentials go through
          // a polynomial on the FMA pipe instead of the MUFU unit (16 results per clock per SM); measured at
          // the BERT-large workload a quarter beats none, three eighths and a half, because the polynomial
          // costs about five issue slots per value.  Scaling, polynomial and row sum run on packed fp32 pairs.
          const uint64_t sc2 = ptx::f32x2_pack(scale_log2e, scale_log2e);
          const uint64_t nm2 = ptx::f32x2_pack(-m_new, -m_new);
          uint64_t acc0 = 0, acc1 = 0;  // packed partial row sums (four independent chains)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c < nchunks) {
              uint32_t pk[16];
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const uint64_t xa = ptx::f32x2_fma(ptx::f32x2_pack(__uint_as_float(sv[c][4 * k]), __uint_as_float(sv[c][4 * k + 1])), sc2, nm2);
                const uint64_t xb = ptx::f32x2_fma(ptx::f32x2_pack(__uint_as_float(sv[c][4 * k + 2]), __uint_as_float(sv[c][4 * k + 3])), sc2, nm2);
                float a0, a1, b0, b1;
                ptx::f32x2_unpack(xa, a0, a1);
                ptx::f32x2_unpack(xb, b0, b1);
                const float p0 = ptx::ex2_approx(a0), p1 = ptx::ex2_approx(a1);
                float p2, p3;
                if ((kPolyPairs >> k) & 1) {
                  ptx::ex2_poly_x2(ptx::f32x2_pack(fmaxf(b0, -126.0f), fmaxf(b1, -126.0f)), p2, p3);
                } else {
                  p2 = ptx::ex2_approx(b0);
                  p3 = ptx::ex2_approx(b1);
                }
                acc0 = ptx::f32x2_add(acc0, ptx::f32x2_pack(p0, p1));
                acc1 = ptx::f32x2_add(acc1, ptx::f32x2_pack(p2, p3));
                pk[2 * k] = pack2<FMT>(p0, p1);
                pk[2 * k + 1] = pack2<FMT>(p2, p3);
              }
              ptx::tmem_st_32x32b_x16(t_p + c * 16, pk);
            }
          }
          float rs, rs_hi;
          ptx::f32x2_unpack(ptx::f32x2_add(acc0, acc1), rs, rs_hi);
          rs += rs_hi;
          l = l * corr + rs;
          m = m_new;
          ptx::tmem_st_wait();
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(ptx::smem_u32(&ctrl->p_ready));
          ptx::mbar_arrive(ptx::smem_u32(&ctrl->empty_v[g % kStages]));
        }
      }
      // the output of this item is written during the next item's first block (or after the loop)
      pend.any = true;
      pend.warp_active = warp_active;
      pend.inv = 1.0f / l;
      pend.rows = it.rows;
      pend.out_row0 = (int64_t)it.tq * E + (int64_t)it.h * kHD;
    }
    if (ok && pend.any) {  // the last item of this CTA
      if (!wait_or_abort(ptx::smem_u32(&ctrl->o_ready), (g - 1) & 1, &ctrl->abort)) ok = false;
      if (ok) {
        ptx::tc_fence_after_sync();
        write_pending();
      }
    }
    if (!ok && lane == 0) {
      ctrl->abort = 1;
      atomicOr(&g_attn_error, 4);
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

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

// One source of 128-row x 64-column tiles: a row-major [rows, cols] two-byte matrix with row stride `ld` elements.
struct TileSource {
  const void* base;
  int64_t rows, cols, ld;
};

bool make_tile_map(CUtensorMap* map, const TileSource& src, int dtype) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return false;
  const cuuint64_t gdim[2] = {(cuuint64_t)src.cols, (cuuint64_t)src.rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)(src.ld * 2)};
  const cuuint32_t box[2] = {(cuuint32_t)kHD, (cuuint32_t)kQT};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == NTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(map, dt, 2, const_cast<void*>(src.base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int FMT>
int launch(const TileSource& q, int col_q, const TileSource& k, int col_k, const TileSource& v, int col_v, void* out,
           const int64_t* offsets_q, const int64_t* offsets_k, int64_t batch, int64_t q_tokens, int H, float scaling, int dtype,
           void* workspace, cudaStream_t st, int skip_short) {  // skip_short > 0: self-attention only
  const int64_t E = (int64_t)H * kHD;
  CUtensorMap map_q, map_k, map_v;
  if (!make_tile_map(&map_q, q, dtype) || !make_tile_map(&map_k, k, dtype) || !make_tile_map(&map_v, v, dtype))
    return NTB200_LAUNCH_FAILED;
  static std::atomic<int> attr_set[kMaxDevices];
  if (!once_per_device(attr_set, [] {
        return cudaFuncSetAttribute(attn_tcgen05_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem) == cudaSuccess;
      }))
    return NTB200_LAUNCH_FAILED;
  const int64_t capacity = attn_tcgen05_item_capacity(batch, q_tokens);
  int* count = static_cast<int*>(workspace);
  int4* items = reinterpret_cast<int4*>(static_cast<uint8_t*>(workspace) + 16);
  if (skip_short > 0) {
    // self-attention on the default path (q, k and v are column blocks of one [T, 3E] matrix, offsets_q == offsets_k)
    using T16 = typename std::conditional<FMT == 0, __half, __nv_bfloat16>::type;
    static std::atomic<int> prep_set[kMaxDevices];
    if (!once_per_device(prep_set, [] {
          return cudaFuncSetAttribute(prepare_self_attention_kernel<T16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrepSmem) == cudaSuccess;
        }))
      return NTB200_LAUNCH_FAILED;
    const int64_t blocks = 1 + (batch * H + kPrepWarps - 1) / kPrepWarps;
    if (blocks > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
    prepare_self_attention_kernel<T16><<<(unsigned)blocks, kPrepWarps * 32, kPrepSmem, st>>>(
        offsets_q, batch, E, items, count, capacity, static_cast<const T16*>(q.base), static_cast<T16*>(out), H, scaling * 1.4426950408889634f);
  } else {
    build_items_kernel<<<1, kListThreads, 0, st>>>(offsets_q, offsets_k, batch, E, items, count, capacity, static_cast<uint16_t*>(out));
  }
  int dev = 0, sms = kNumSMs;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int64_t grid = 2ll * sms;  // two resident CTAs per SM, each loops over its share of the items
  if (grid > capacity * H) grid = capacity * H;
  attn_tcgen05_kernel<FMT><<<(unsigned)grid, kAttnThreads, kAttnSmem, st>>>(map_q, map_k, map_v, col_q, col_k, col_v, out, items, count, H,
                                                                            scaling * 1.4426950408889634f);
  return status_from_cuda(cudaGetLastError());
}

}  // namespace

int64_t attn_tcgen05_item_capacity(int64_t batch, int64_t total_tokens) { return batch + total_tokens / kQT + 1; }

size_t attn_tcgen05_workspace_bytes(int64_t batch, int64_t total_tokens) {
  return 16 + sizeof(int4) * (size_t)attn_tcgen05_item_capacity(batch, total_tokens);
}

bool attn_tcgen05_supported(int64_t batch, int64_t total_tokens, int num_heads, int head_dim, int dtype) {
  return head_dim == kHD && (dtype == NTB200_F16 || dtype == NTB200_BF16) && num_heads <= 65535 &&
         total_tokens < (1ll << 31) - kQT && 3ll * num_heads * kHD < (1ll << 31) &&
         attn_tcgen05_item_capacity(batch, total_tokens) < (1ll << 31);
}

int attn_tcgen05_launch(const void* qkv, void* out, const int64_t* offsets, int64_t batch, int64_t total_tokens, int H,
                        float scaling, int dtype, void* workspace, cudaStream_t st, int skip_short) {
  const int64_t E = (int64_t)H * kHD;
  const TileSource src = {qkv, total_tokens, 3 * E, 3 * E};  // one map, three column offsets
  if (dtype == NTB200_F16)
    return launch<0>(src, 0, src, (int)E, src, (int)(2 * E), out, offsets, offsets, batch, total_tokens, H, scaling, dtype, workspace, st,
                     skip_short);
  return launch<1>(src, 0, src, (int)E, src, (int)(2 * E), out, offsets, offsets, batch, total_tokens, H, scaling, dtype, workspace, st,
                   skip_short);
}

int attn_tcgen05_cross_launch(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, void* out,
                              const int64_t* offsets_q, const int64_t* offsets_k, int64_t batch, int64_t q_tokens, int64_t k_tokens,
                              int H, float scaling, int dtype, void* workspace, cudaStream_t st) {
  const int64_t E = (int64_t)H * kHD;
  const TileSource sq = {q, q_tokens, E, ldq}, sk = {k, k_tokens, E, ldk}, sv = {v, k_tokens, E, ldv};
  if (dtype == NTB200_F16)
    return launch<0>(sq, 0, sk, 0, sv, 0, out, offsets_q, offsets_k, batch, q_tokens, H, scaling, dtype, workspace, st, 0);
  return launch<1>(sq, 0, sk, 0, sv, 0, out, offsets_q, offsets_k, batch, q_tokens, H, scaling, dtype, workspace, st, 0);
}

int attn_tcgen05_error_flags_read_and_clear() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
  }
  return v;
}

}  // namespace ntb200

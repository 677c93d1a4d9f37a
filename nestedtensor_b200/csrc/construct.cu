// The step before the ragged path: building the packed buffer.
//
//   pack_pointers   out[offsets[b] + i] = src_b[i]   B separately allocated device tensors -> one buffer, one launch
//   embedding       out[t, :] = weight[index[t], :]  on the packed index buffer of a nested tensor
//
// Both stream every byte once (HBM-bound).  pack_pointers replaces the per-constituent copy loop of the
// packed storage constructor (nestedtensor/csrc/storage/Packed.h:75-98, nestedtensor/csrc/creation.cpp:191-222);
// embedding replaces the packed fast path of NestedTensor_embedding (nestedtensor/csrc/functions.cpp:29-56,
// at::embedding on the index buffer).

#include "common.cuh"

namespace ntb200 {
namespace {

__device__ int g_construct_error = 0;  // bit 0: an embedding index was out of range (its row was zero-filled)

constexpr int kPackThreads = 256, kPackVecs = 8;  // 32 KB of output per tile, as in the pad / unpad kernels
constexpr int kPackEnt = 128;                      // entries per tile kept in shared memory

// Flat walk over 16-byte vectors of the OUTPUT.  A vector that lies inside one constituent whose source is
// 16-byte aligned at that point is one 16-byte load; any other vector is assembled element by element
// (it crosses constituents, or its source is not aligned).  The tile first narrows the range of entries it
// can touch (two searches, through shared memory), so the per-vector search is over a handful of entries.
template <int ES>
__global__ void __launch_bounds__(kPackThreads)
pack_pointers_kernel(const void* const* __restrict__ srcs, const int64_t* __restrict__ offsets, int64_t batch,
                     void* __restrict__ out, int64_t total_elems) {
  using T = typename ElemBits<ES>::T;
  constexpr int EPV = 16 / ES;
  __shared__ int64_t s_range[2];
  __shared__ int64_t s_off[kPackEnt + 1];     // offsets and sources of the tile's entries (when at most kPackEnt)
  __shared__ const void* s_src[kPackEnt];
  const int64_t n_vec = (total_elems + EPV - 1) / EPV;
  const int64_t tile0 = (int64_t)blockIdx.x * (kPackThreads * kPackVecs);
  if (threadIdx.x < 64) {  // warp 0: the tile's first entry, warp 1: its last one (32 probes per search step)
    int64_t e = (threadIdx.x < 32 ? tile0 : tile0 + kPackThreads * kPackVecs - 1) * EPV;
    e = e < total_elems ? e : total_elems - 1;
    const int64_t found = find_entry_warp(offsets, 0, batch - 1, e);
    if ((threadIdx.x & 31) == 0) s_range[threadIdx.x >> 5] = found;
  }
  __syncthreads();
  const int64_t lo = s_range[0], hi = s_range[1];
  const bool cached = hi - lo < kPackEnt;
  if (cached && threadIdx.x <= hi - lo + 1) s_off[threadIdx.x] = offsets[lo + threadIdx.x];
  if (cached && threadIdx.x <= hi - lo) s_src[threadIdx.x] = srcs[lo + threadIdx.x];
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kPackVecs; ++j) {
    const int64_t v = tile0 + (int64_t)j * kPackThreads + threadIdx.x;
    if (v >= n_vec) break;
    const int64_t e0 = v * EPV;
    int64_t b, first, end_b;
    const void* base;
    if (cached) {
      int l = 0, h = (int)(hi - lo);
      while (l < h) {
        const int mid = (l + h + 1) >> 1;
        if (s_off[mid] <= e0) l = mid;
        else h = mid - 1;
      }
      b = lo + l;
      first = s_off[l];
      end_b = s_off[l + 1];
      base = s_src[l];
    } else {
      b = find_entry(offsets, lo, hi, e0);
      first = offsets[b];
      end_b = offsets[b + 1];
      base = srcs[b];
    }
    const T* src = static_cast<const T*>(base) + (e0 - first);
    if (e0 + EPV <= end_b && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
      st_global_16_stream(static_cast<T*>(out) + e0, ld_global_16_stream(src));
    } else {
      T* dst = static_cast<T*>(out) + e0;
      int64_t nxt = end_b;
#pragma unroll
      for (int k = 0; k < EPV; ++k) {
        const int64_t e = e0 + k;
        if (e >= total_elems) break;
        while (e >= nxt) {  // empty constituents are skipped here
          ++b;
          nxt = offsets[b + 1];
        }
        dst[k] = static_cast<const T*>(srcs[b])[e - offsets[b]];
      }
    }
  }
}

constexpr int kEmbThreads = 256;

// One warp per output row (token); 16-byte vectors when the row size and both bases allow it.
template <typename IDX, bool VEC>
__global__ void __launch_bounds__(kEmbThreads)
embedding_kernel(const void* __restrict__ weight, const IDX* __restrict__ index, void* __restrict__ out, int64_t tokens,
                 int64_t vocab, int64_t row_bytes) {
  const int64_t t = (int64_t)blockIdx.x * (kEmbThreads / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const int64_t i = (int64_t)index[t];
  const bool ok = i >= 0 && i < vocab;
  if (!ok && lane == 0) atomicOr(&g_construct_error, 1);
  const uint8_t* src = static_cast<const uint8_t*>(weight) + (ok ? i : 0) * row_bytes;
  uint8_t* dst = static_cast<uint8_t*>(out) + t * row_bytes;
  if (VEC) {
    const int64_t nv = row_bytes >> 4;
    for (int64_t v = lane; v < nv; v += 32) {
      uint4 x = make_uint4(0, 0, 0, 0);
      if (ok) x = ld_global_16_stream(src + (v << 4));
      st_global_16_stream(dst + (v << 4), x);
    }
  } else {
    for (int64_t k = lane; k < row_bytes; k += 32) dst[k] = ok ? src[k] : (uint8_t)0;
  }
}

}  // namespace

int construct_error_flags_read_and_clear() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_construct_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_construct_error, &zero, sizeof(int));
  }
  return v;
}

}  // namespace ntb200

using namespace ntb200;

extern "C" {

int ntb200_pack_pointers(const void* const* srcs, const int64_t* offsets, int64_t batch, void* out, int64_t total_elems,
                         int elem_size, void* stream) {
  if (batch < 0 || total_elems < 0) return NTB200_INVALID_ARG;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return NTB200_UNSUPPORTED_DTYPE;
  if (batch == 0 || total_elems == 0) return NTB200_OK;
  if (srcs == nullptr || offsets == nullptr || out == nullptr) return NTB200_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(out) & 15) return NTB200_MISALIGNED;
  const int64_t epv = 16 / elem_size;
  const int64_t n_vec = (total_elems + epv - 1) / epv;
  const int64_t grid = (n_vec + kPackThreads * kPackVecs - 1) / (kPackThreads * kPackVecs);
  if (grid > 0x7fffffff) return NTB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (elem_size) {
    case 1: pack_pointers_kernel<1><<<(unsigned)grid, kPackThreads, 0, st>>>(srcs, offsets, batch, out, total_elems); break;
    case 2: pack_pointers_kernel<2><<<(unsigned)grid, kPackThreads, 0, st>>>(srcs, offsets, batch, out, total_elems); break;
    case 4: pack_pointers_kernel<4><<<(unsigned)grid, kPackThreads, 0, st>>>(srcs, offsets, batch, out, total_elems); break;
    default: pack_pointers_kernel<8><<<(unsigned)grid, kPackThreads, 0, st>>>(srcs, offsets, batch, out, total_elems); break;
  }
  return status_from_cuda(cudaGetLastError());
}

int ntb200_embedding(const void* weight, const void* index, int index_bytes, void* out, int64_t tokens, int64_t vocab,
                     int64_t embed_dim, int elem_size, void* stream) {
  if (tokens < 0 || vocab < 0 || embed_dim < 0 || (index_bytes != 4 && index_bytes != 8)) return NTB200_INVALID_ARG;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return NTB200_UNSUPPORTED_DTYPE;
  if (tokens == 0 || embed_dim == 0) return NTB200_OK;
  if (weight == nullptr || index == nullptr || out == nullptr || vocab == 0) return NTB200_INVALID_ARG;
  const int64_t row_bytes = embed_dim * elem_size;
  const bool vec = (row_bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(weight) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  const int64_t grid = (tokens + kEmbThreads / 32 - 1) / (kEmbThreads / 32);
  if (grid > 0x7fffffff) return NTB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define NTB200_EMB(IDX, VEC) \
  embedding_kernel<IDX, VEC><<<(unsigned)grid, kEmbThreads, 0, st>>>(weight, static_cast<const IDX*>(index), out, tokens, vocab, row_bytes)
  if (index_bytes == 8) {
    if (vec) NTB200_EMB(int64_t, true);
    else NTB200_EMB(int64_t, false);
  } else {
    if (vec) NTB200_EMB(int32_t, true);
    else NTB200_EMB(int32_t, false);
  }
#undef NTB200_EMB
  return status_from_cuda(cudaGetLastError());
}

}  // extern "C"

// ---------------------------------------------------------------------- ragged 2-D transposes (NCHW <-> NHWC)
// Constituent b is a row-major [rows_b x cols_b] matrix with one regular extent R and one ragged extent n_b
// (channels x pixels or pixels x channels); the output holds its transpose at the same element offset.
// Replaces transpose_nchw_nhwc / transpose_nhwc_nchw (nestedtensor/csrc/cuda/transpose.cu:10-238,
// nestedtensor/csrc/transpose.cpp:87-202) without their host-built block-offset tables: the grid is
// (tiles of the largest constituent, batch) and blocks past a constituent's last tile exit.
namespace ntb200 {
namespace {

constexpr int kTrTile = 64;

template <typename T>
__global__ void __launch_bounds__(256)
transpose_ragged_kernel(const T* __restrict__ in, T* __restrict__ out, const int64_t* __restrict__ offsets, int64_t regular,
                        int regular_is_rows) {
  __shared__ T tile[kTrTile][kTrTile + 1];
  const int64_t b = blockIdx.y;
  const int64_t off = offsets[b];
  const int64_t n = (offsets[b + 1] - off) / regular;  // ragged extent
  const int64_t rows = regular_is_rows ? regular : n, cols = regular_is_rows ? n : regular;
  const int64_t tiles_reg = (regular + kTrTile - 1) / kTrTile;
  const int64_t t_rag = blockIdx.x / tiles_reg, t_reg = blockIdx.x % tiles_reg;
  if (t_rag * kTrTile >= n) return;
  const int64_t r0 = (regular_is_rows ? t_reg : t_rag) * kTrTile, c0 = (regular_is_rows ? t_rag : t_reg) * kTrTile;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const T* src = in + off;
  T* dst = out + off;
#pragma unroll
  for (int i = 0; i < kTrTile; i += 8) {
    const int64_t r = r0 + ty + i;
#pragma unroll
    for (int j = 0; j < kTrTile; j += 32) {
      const int64_t c = c0 + tx + j;
      if (r < rows && c < cols) tile[ty + i][tx + j] = src[r * cols + c];
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kTrTile; i += 8) {
    const int64_t c = c0 + ty + i;  // output row
#pragma unroll
    for (int j = 0; j < kTrTile; j += 32) {
      const int64_t r = r0 + tx + j;  // output column
      if (r < rows && c < cols) dst[c * rows + r] = tile[tx + j][ty + i];
    }
  }
}

// The same transpose when a row of `regular` elements is a whole number of 16-byte vectors (C * element size
// a multiple of 16, always so for fp16 / bf16 feature maps with C % 8 == 0): the side on which the regular
// extent is contiguous moves 16 bytes per thread, the ragged side (rows of n_b elements at any phase) stays
// element-wise but coalesced.  The tile lives in shared memory as [ragged][regular] 32-bit words with an odd
// word stride: the vector side touches it with four 32-bit accesses per vector and the element side with one
// element per thread over 32 consecutive ragged positions, both free of bank conflicts for 2-byte elements
// (at most two-way for 1- and 4-byte ones).
constexpr int kTrRag = 128;  // ragged-extent tile of the vector kernel (more bytes in flight per CTA)

template <typename T, bool REG_IS_ROWS>
__global__ void __launch_bounds__(256)
transpose_ragged_vec_kernel(const T* __restrict__ in, T* __restrict__ out, const int64_t* __restrict__ offsets, int64_t regular) {
  constexpr int VE = 16 / (int)sizeof(T);               // elements per vector
  constexpr int kVecPerRow = kTrTile / VE;              // vectors covering the tile's regular extent
  constexpr int kWords = kTrTile * (int)sizeof(T) / 4;  // 32-bit words of one ragged position's slice
  constexpr int kStride = (kWords + 1) * 4 / (int)sizeof(T);  // elements per tile row: an odd number of words
  constexpr int kPerThread = kTrTile / (256 / kTrRag);        // element-side accesses per thread
  constexpr int kVecPerThread = (kTrRag * kVecPerRow) / 256;  // vector-side accesses per thread
  __shared__ __align__(16) T tile[kTrRag][kStride];           // [ragged][regular]
  const int64_t b = blockIdx.y;
  const int64_t off = offsets[b];
  const int64_t n = (offsets[b + 1] - off) / regular;
  const int64_t tiles_reg = (regular + kTrTile - 1) / kTrTile;
  const int64_t t_rag = blockIdx.x / tiles_reg, t_reg = blockIdx.x % tiles_reg;
  if (t_rag * kTrRag >= n) return;
  const int64_t p0 = t_rag * kTrRag, c0 = t_reg * kTrTile;
  const T* src = in + off;
  T* dst = out + off;
  const int px_l = threadIdx.x & (kTrRag - 1), cy = threadIdx.x / kTrRag;  // element-wise side: 128 ragged x 2 regular
  // The element-wise side costs one compare, one pointer step, one global and one shared access per element:
  // thread (px_l, cy) owns regular positions cy, cy + kRegStep, ... of ragged position p0 + px_l, walks them with
  // a pointer that advances kRegStep rows of n elements, and tests i * kRegStep against `lim`, the count of
  // valid regular positions from cy on (0 when its ragged position lies past the constituent's end).
  constexpr int kRegStep = 256 / kTrRag;
  const int64_t step = (int64_t)kRegStep * n;
  const int64_t reg_left = regular - c0 - cy;
  const int lim = (p0 + px_l < n && reg_left > 0) ? (int)(reg_left < kTrTile ? reg_left : kTrTile) : 0;
  // every global load of a phase is issued before the first shared-memory store that depends on one
  if (REG_IS_ROWS) {  // in [regular][n] -> out [n][regular]
    constexpr int kBatch = kPerThread / 2;  // loads in flight per thread (two batches keep the register count down)
    const T* p = src + (c0 + cy) * n + p0 + px_l;
#pragma unroll
    for (int h = 0; h < kPerThread; h += kBatch) {
      T vals[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        vals[i] = ((h + i) * kRegStep < lim) ? *p : T(0);
        p += step;
      }
#pragma unroll
      for (int i = 0; i < kBatch; ++i) tile[px_l][cy + (h + i) * kRegStep] = vals[i];
    }
  } else {  // in [n][regular] -> out [regular][n]
    uint4 x[kVecPerThread];
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
      const int idx = k * 256 + threadIdx.x;
      const int pl = idx / kVecPerRow, v = idx % kVecPerRow;
      const int64_t px = p0 + pl, c = c0 + v * VE;
      x[k] = (px < n && c < regular) ? *reinterpret_cast<const uint4*>(src + px * regular + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
      const int idx = k * 256 + threadIdx.x;
      const int pl = idx / kVecPerRow, v = idx % kVecPerRow;
      uint32_t* w = reinterpret_cast<uint32_t*>(&tile[pl][v * VE]);
      w[0] = x[k].x;
      w[1] = x[k].y;
      w[2] = x[k].z;
      w[3] = x[k].w;
    }
  }
  __syncthreads();
  if (REG_IS_ROWS) {
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
      const int idx = k * 256 + threadIdx.x;
      const int pl = idx / kVecPerRow, v = idx % kVecPerRow;
      const int64_t px = p0 + pl, c = c0 + v * VE;
      if (px < n && c < regular) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&tile[pl][v * VE]);
        *reinterpret_cast<uint4*>(dst + px * regular + c) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  } else {
    T* q = dst + (c0 + cy) * n + p0 + px_l;
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      if (i * kRegStep < lim) *q = tile[px_l][cy + i * kRegStep];
      q += step;
    }
  }
}

// 2-byte elements (fp16 / bf16 feature maps): the ragged side moves aligned PAIRS of pixels, 4 bytes per thread and
// access, which halves its load/store instructions and doubles the bytes a thread keeps in flight.  The tile lives
// in shared memory as [regular][pixel pair] 32-bit words (one word = two neighbouring pixels of one channel) with
// an odd word stride: the pair side touches consecutive words, the vector side reads, per pixel pair and group of
// eight channels, eight words and regroups them into the two 16-byte vectors of the two pixels with byte permutes;
// both are free of bank conflicts.  A pair is 4-byte aligned in global memory unless the constituent has an odd
// number of pixels AND the channel index is odd; the channel parity is fixed per thread, so that case (and a last
// single pixel) falls back to two 2-byte accesses without divergence inside a warp.
constexpr int kPairPx = 128;                // pixels per tile
constexpr int kPairWords = kPairPx / 2 + 1;  // words per channel row of the tile (odd)

template <bool REG_IS_ROWS>
__global__ void __launch_bounds__(256)
transpose_ragged_pair_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, const int64_t* __restrict__ offsets,
                             int64_t regular) {
  __shared__ uint32_t tile[kTrTile][kPairWords];  // [channel][pixel pair]
  const int64_t b = blockIdx.y;
  const int64_t off = offsets[b];
  const int64_t n = (offsets[b + 1] - off) / regular;
  const int64_t tiles_reg = (regular + kTrTile - 1) / kTrTile;
  const int64_t t_rag = blockIdx.x / tiles_reg, t_reg = blockIdx.x % tiles_reg;
  if (t_rag * kPairPx >= n) return;
  const int64_t p0 = t_rag * kPairPx, c0 = t_reg * kTrTile;
  const uint16_t* src = in + off;
  uint16_t* dst = out + off;
  // pair side: thread (pp, cy) owns pixel pair pp of channels c0 + cy, c0 + cy + 4, ...
  constexpr int kChStep = 4, kPerThread = kTrTile / kChStep;
  const int pp = threadIdx.x & 63, cy = threadIdx.x >> 6;
  const int64_t px = p0 + 2 * pp;
  const int n_here = px + 1 < n ? 2 : (px < n ? 1 : 0);
  const bool aligned = !((n & 1) && (cy & 1));  // (off, p0 and c0 are even)
  const int64_t ch_left = regular - c0 - cy;
  const int lim = n_here > 0 && ch_left > 0 ? (int)(ch_left < kTrTile ? ch_left : kTrTile) : 0;  // valid while i * 4 < lim
  const int64_t step = (int64_t)kChStep * n;
  // vector side: item (pixel pair q, channel group v): a pixel's eight channel groups on eight neighbouring lanes
  // (128-byte rows of the channel-contiguous matrix), four pixel pairs per warp
  auto item = [&](int k, int& q, int& v) {
    const int idx = k * 256 + threadIdx.x;
    v = idx & 7;
    q = idx >> 3;
  };
  // word column of pixel pair q in channel row c: pairs of the upper 32 channel rows sit four words off, which keeps
  // the eight channel groups of the vector side (rows 8 v + m, a stride of 8 * 65 words = 8 banks) on distinct banks
  auto col = [](int c, int q) { return q ^ ((c >> 5) << 2); };
  if (REG_IS_ROWS) {  // in [regular][n] -> out [n][regular]
    // (the choice between word and half-word accesses is made once, outside the unrolled loops, so that every
    // load of the thread is issued before the first shared-memory store)
    const uint16_t* p = src + (c0 + cy) * n + px;
    if (aligned && n_here == 2) {
      uint32_t w[kPerThread];
#pragma unroll
      for (int i = 0; i < kPerThread; ++i) {
        w[i] = (i * kChStep < lim) ? *reinterpret_cast<const uint32_t*>(p) : 0u;
        p += step;
      }
#pragma unroll
      for (int i = 0; i < kPerThread; ++i) tile[cy + i * kChStep][col(cy + i * kChStep, pp)] = w[i];
    } else {
      constexpr int kBatch = kPerThread / 2;  // the same number of registers as the word path
#pragma unroll
      for (int h = 0; h < kPerThread; h += kBatch) {
        uint16_t lo[kBatch], hi[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
          lo[i] = ((h + i) * kChStep < lim) ? p[0] : (uint16_t)0;
          hi[i] = ((h + i) * kChStep < lim && n_here == 2) ? p[1] : (uint16_t)0;
          p += step;
        }
#pragma unroll
        for (int i = 0; i < kBatch; ++i) tile[cy + (h + i) * kChStep][col(cy + (h + i) * kChStep, pp)] = (uint32_t)lo[i] | ((uint32_t)hi[i] << 16);
      }
    }
  } else {  // in [n][regular] -> out [regular][n]
    uint4 x0[2], x1[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      int q, v;
      item(k, q, v);
      const int64_t q0 = p0 + 2 * q, c = c0 + v * 8;
      x0[k] = (q0 < n && c < regular) ? *reinterpret_cast<const uint4*>(src + q0 * regular + c) : make_uint4(0, 0, 0, 0);
      x1[k] = (q0 + 1 < n && c < regular) ? *reinterpret_cast<const uint4*>(src + (q0 + 1) * regular + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      int q, v;
      item(k, q, v);
      const uint32_t a[4] = {x0[k].x, x0[k].y, x0[k].z, x0[k].w}, c[4] = {x1[k].x, x1[k].y, x1[k].z, x1[k].w};
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        tile[v * 8 + 2 * m][col(v * 8, q)] = __byte_perm(a[m], c[m], 0x5410);      // channel 2m: low halves of both pixels
        tile[v * 8 + 2 * m + 1][col(v * 8, q)] = __byte_perm(a[m], c[m], 0x7632);  // channel 2m + 1: high halves
      }
    }
  }
  __syncthreads();
  if (REG_IS_ROWS) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      int q, v;
      item(k, q, v);
      uint32_t w[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) w[m] = tile[v * 8 + m][col(v * 8, q)];
      const int64_t q0 = p0 + 2 * q, c = c0 + v * 8;
      if (c < regular) {
        if (q0 < n)
          *reinterpret_cast<uint4*>(dst + q0 * regular + c) =
              make_uint4(__byte_perm(w[0], w[1], 0x5410), __byte_perm(w[2], w[3], 0x5410), __byte_perm(w[4], w[5], 0x5410),
                         __byte_perm(w[6], w[7], 0x5410));
        if (q0 + 1 < n)
          *reinterpret_cast<uint4*>(dst + (q0 + 1) * regular + c) =
              make_uint4(__byte_perm(w[0], w[1], 0x7632), __byte_perm(w[2], w[3], 0x7632), __byte_perm(w[4], w[5], 0x7632),
                         __byte_perm(w[6], w[7], 0x7632));
      }
    }
  } else {
    uint16_t* q = dst + (c0 + cy) * n + px;
    uint32_t w[kPerThread];
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) w[i] = tile[cy + i * kChStep][col(cy + i * kChStep, pp)];
    if (aligned && n_here == 2) {
#pragma unroll
      for (int i = 0; i < kPerThread; ++i) {
        if (i * kChStep < lim) *reinterpret_cast<uint32_t*>(q) = w[i];
        q += step;
      }
    } else {
#pragma unroll
      for (int i = 0; i < kPerThread; ++i) {
        if (i * kChStep < lim) {
          q[0] = (uint16_t)w[i];
          if (n_here == 2) q[1] = (uint16_t)(w[i] >> 16);
        }
        q += step;
      }
    }
  }
}

// The same transpose for a SMALL regular extent (RGB / RGBA images, a few channels): the 64-channel tiles of the kernels
// above would be all but empty.  A block takes kSmallThreads * PPT consecutive pixels of one constituent; on the
// pixel-major side these are one contiguous run of pixels * C elements, moved by the whole block in element order, and
// on the channel-major side C runs of pixels, PPT elements per thread and channel (PPT loads in flight per thread and
// channel: with one, the kernel is bound by latency); the two meet in shared memory.  There a pixel's C elements are
// consecutive, which for an even C puts the threads of a warp up to 16 ways onto the same banks on the channel-major
// side; an even C of 4 or more therefore gets one element of padding per pixel, and the element-order side steps its
// (pixel, channel) position along with the linear index instead of dividing.
constexpr int kSmallThreads = 256;
constexpr int64_t kSmallRegularMax = 24;    // ... and at most kSmallPixelBytes per pixel (measured: from 32 channels on the tile kernels are level or ahead)
constexpr int64_t kSmallPixelBytes = 192;  // (padding included: 256 pixels of a block then fill 48 KB)

// MODE 0: C odd or below 4, no padding, linear slots; 1: C a power of two (pixel and channel of a linear index are a
// shift and a mask); 2: any other even C (pixel and channel stepped along with the index)
template <typename T, bool REG_IS_ROWS, int PPT, int MODE>
__global__ void __launch_bounds__(kSmallThreads)
transpose_small_regular_kernel(const T* __restrict__ in, T* __restrict__ out, const int64_t* __restrict__ offsets, int regular) {
  extern __shared__ __align__(16) uint8_t small_smem[];
  T* sm = reinterpret_cast<T*>(small_smem);
  constexpr int kPx = kSmallThreads * PPT;
  const int64_t off = offsets[blockIdx.y];
  const int64_t n = (offsets[blockIdx.y + 1] - off) / regular;  // pixels
  const int64_t p0 = (int64_t)blockIdx.x * kPx;
  if (p0 >= n) return;
  const int np = n - p0 < kPx ? (int)(n - p0) : kPx;
  const int C = regular, t = threadIdx.x;
  const int S = MODE == 0 ? C : C + 1;  // shared-memory pixel stride
  // element-order side: linear index i = t, t + 256, ... as (pixel q, channel r)
  const int sh = 31 - __clz(C);  // MODE 1
  int q = 0, r = 0, dq = 0, dr = 0;  // MODE 2: advanced by (256 / C, 256 % C)
  if (MODE == 2) {
    q = t / C, r = t - q * C;
    dq = kSmallThreads / C, dr = kSmallThreads - dq * C;
  }
  auto slot = [&](int i) { return MODE == 0 ? i : (MODE == 1 ? (i >> sh) * S + (i & (C - 1)) : q * S + r); };
  auto advance = [&]() {
    if (MODE == 2) {
      q += dq;
      r += dr;
      if (r >= C) {
        r -= C;
        ++q;
      }
    }
  };
  const T* src = in + off;
  T* dst = out + off;
  if (REG_IS_ROWS) {  // [C x n] -> [n x C]
    const T* s = src + p0 + t;
#pragma unroll 2
    for (int c = 0; c < C; ++c) {
      T v[PPT];
#pragma unroll
      for (int k = 0; k < PPT; ++k) v[k] = t + k * kSmallThreads < np ? s[(int64_t)c * n + k * kSmallThreads] : T(0);
#pragma unroll
      for (int k = 0; k < PPT; ++k)
        if (t + k * kSmallThreads < np) sm[(t + k * kSmallThreads) * S + c] = v[k];
    }
    __syncthreads();
    T* d = dst + p0 * C;
    for (int i = t; i < np * C; i += kSmallThreads, advance()) d[i] = sm[slot(i)];
  } else {  // [n x C] -> [C x n]
    const T* s = src + p0 * C;
    for (int i = t; i < np * C; i += kSmallThreads, advance()) sm[slot(i)] = s[i];
    __syncthreads();
    T* d = dst + p0 + t;
#pragma unroll 2
    for (int c = 0; c < C; ++c) {
#pragma unroll
      for (int k = 0; k < PPT; ++k)
        if (t + k * kSmallThreads < np) d[(int64_t)c * n + k * kSmallThreads] = sm[(t + k * kSmallThreads) * S + c];
    }
  }
}

constexpr int small_mode(int64_t regular) { return (regular < 4 || (regular & 1)) ? 0 : ((regular & (regular - 1)) == 0 ? 1 : 2); }
constexpr int64_t small_stride(int64_t regular) { return small_mode(regular) == 0 ? regular : regular + 1; }

template <typename T, int PPT, int MODE>
void launch_transpose_small_m(const void* in, void* out, const int64_t* offsets, int64_t nb, int64_t regular, int regular_is_rows,
                              int64_t max_ragged, cudaStream_t st) {
  constexpr int kPx = kSmallThreads * PPT;
  dim3 grid((unsigned)((max_ragged + kPx - 1) / kPx), (unsigned)nb);
  const size_t smem = (size_t)kPx * (size_t)small_stride(regular) * sizeof(T);  // at most 48 KB
  if (regular_is_rows)
    transpose_small_regular_kernel<T, true, PPT, MODE><<<grid, kSmallThreads, smem, st>>>(static_cast<const T*>(in), static_cast<T*>(out), offsets, (int)regular);
  else
    transpose_small_regular_kernel<T, false, PPT, MODE><<<grid, kSmallThreads, smem, st>>>(static_cast<const T*>(in), static_cast<T*>(out), offsets, (int)regular);
}

template <typename T, int PPT>
void launch_transpose_small(const void* in, void* out, const int64_t* offsets, int64_t nb, int64_t regular, int regular_is_rows,
                            int64_t max_ragged, cudaStream_t st) {
  switch (small_mode(regular)) {
    case 0: return launch_transpose_small_m<T, PPT, 0>(in, out, offsets, nb, regular, regular_is_rows, max_ragged, st);
    case 1: return launch_transpose_small_m<T, PPT, 1>(in, out, offsets, nb, regular, regular_is_rows, max_ragged, st);
    default: return launch_transpose_small_m<T, PPT, 2>(in, out, offsets, nb, regular, regular_is_rows, max_ragged, st);
  }
}

template <typename T>
int launch_transpose_ragged(const void* in, void* out, const int64_t* offsets, int64_t batch, int64_t regular,
                            int regular_is_rows, int64_t max_ragged, cudaStream_t st) {
  const bool vec = sizeof(T) < 8 && (regular * (int64_t)sizeof(T)) % 16 == 0 &&
                   ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (regular <= kSmallRegularMax && small_stride(regular) * (int64_t)sizeof(T) <= kSmallPixelBytes) {
    if ((max_ragged + kSmallThreads - 1) / kSmallThreads > 0x7fffffff) return NTB200_UNSUPPORTED_SHAPE;
    const int64_t pixel_bytes = small_stride(regular) * (int64_t)sizeof(T);  // 1024 / 512 / 256 pixels per block: what fits 48 KB of shared memory
    for (int64_t b0 = 0; b0 < batch; b0 += 65535) {  // gridDim.y limit
      const int64_t nb = batch - b0 < 65535 ? batch - b0 : 65535;
      if (pixel_bytes <= 48)
        launch_transpose_small<T, 4>(in, out, offsets + b0, nb, regular, regular_is_rows, max_ragged, st);
      else if (pixel_bytes <= 96)
        launch_transpose_small<T, 2>(in, out, offsets + b0, nb, regular, regular_is_rows, max_ragged, st);
      else
        launch_transpose_small<T, 1>(in, out, offsets + b0, nb, regular, regular_is_rows, max_ragged, st);
    }
    return status_from_cuda(cudaGetLastError());
  }
  const int64_t rag_tile = vec ? kTrRag : kTrTile;
  const int64_t tiles = ((regular + kTrTile - 1) / kTrTile) * ((max_ragged + rag_tile - 1) / rag_tile);
  if (tiles > 0x7fffffff) return NTB200_UNSUPPORTED_SHAPE;
  for (int64_t b0 = 0; b0 < batch; b0 += 65535) {  // gridDim.y limit
    const int64_t nb = batch - b0 < 65535 ? batch - b0 : 65535;
    dim3 grid((unsigned)tiles, (unsigned)nb);
    if constexpr (sizeof(T) == 2) {
      if (vec) {  // (kPairPx == kTrRag: the same grid)
        if (regular_is_rows)
          transpose_ragged_pair_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out), offsets + b0, regular);
        else
          transpose_ragged_pair_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out), offsets + b0, regular);
        continue;
      }
    }
    if constexpr (sizeof(T) < 8) {
      if (vec && regular_is_rows) {
        transpose_ragged_vec_kernel<T, true><<<grid, 256, 0, st>>>(static_cast<const T*>(in), static_cast<T*>(out), offsets + b0, regular);
        continue;
      }
      if (vec) {
        transpose_ragged_vec_kernel<T, false><<<grid, 256, 0, st>>>(static_cast<const T*>(in), static_cast<T*>(out), offsets + b0, regular);
        continue;
      }
    }
    transpose_ragged_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(in), static_cast<T*>(out), offsets + b0, regular,
                                                     regular_is_rows);
  }
  return status_from_cuda(cudaGetLastError());
}

}  // namespace
}  // namespace ntb200

extern "C" int ntb200_transpose_ragged(const void* in, void* out, const int64_t* offsets, int64_t batch, int64_t regular,
                                       int regular_is_rows, int64_t max_ragged, int elem_size, void* stream) {
  using namespace ntb200;
  if (batch < 0 || regular < 0 || max_ragged < 0) return NTB200_INVALID_ARG;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return NTB200_UNSUPPORTED_DTYPE;
  if (batch == 0 || regular == 0 || max_ragged == 0) return NTB200_OK;
  if (in == nullptr || out == nullptr || offsets == nullptr || in == out) return NTB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (elem_size) {
    case 1: return launch_transpose_ragged<uint8_t>(in, out, offsets, batch, regular, regular_is_rows, max_ragged, st);
    case 2: return launch_transpose_ragged<uint16_t>(in, out, offsets, batch, regular, regular_is_rows, max_ragged, st);
    case 4: return launch_transpose_ragged<uint32_t>(in, out, offsets, batch, regular, regular_is_rows, max_ragged, st);
    default: return launch_transpose_ragged<uint64_t>(in, out, offsets, batch, regular, regular_is_rows, max_ragged, st);
  }
}

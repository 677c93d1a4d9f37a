// Ragged <-> dense copy kernels, validity masks and size recovery for nested tensors.
//
// Design (B200, HBM-bound byte movers):
//   * every kernel walks its OUTPUT as a flat array of 16-byte vectors, so stores are
//     always full-width and aligned whatever the row pitch; the matching input address is
//     derived per vector with launch-constant multiply-shift division (no per-element / or %);
//   * 64-bit element indices everywhere (a (4096,1024,1024) bf16 output has 2^32 elements);
//   * loads fall back to element-wise only where source and destination differ in
//     16-byte phase (ragged rows of odd length) or at row / entry edges;
//   * with two or three ragged dimensions and long innermost rows (images) a warp takes one innermost
//     row instead: the row is located once and its vectors need no division (pad_rows_kernel,
//     unpad_rows_kernel, scan_rows_kernel).
// The reference's counterparts are add_padding_{1,2,3}, remove_padding_2 / remove_padding and
// add_padding_mask in nestedtensor/csrc/cuda/padding.cu:10-414 (scalar strided copies with int
// indices, one thread per sequence for the mask variant).

#include "common.cuh"

namespace ntb200 {
namespace {

// Tile shape of the copy kernels, fixed after a sweep on B200 at the 4096 x (L_i, 1024) bf16 batch: 256 threads x 8
// 16-byte vectors = 32 KB per tile, all loads of a tile issued before its stores.
constexpr int kThreads = 256;
constexpr int kVecPerThread = 8;

// ------------------------------------------------------------------------------ pad
struct PadParams {
  const void* src;
  void* dst;
  const int64_t* offsets;
  const int64_t* sizes;
  int64_t size_stride;
  int64_t batch;
  int64_t total;    // batch * P output elements
  uint64_t P;       // padded elements per entry
  uint64_t m[3];    // padded extents, outer -> inner (first ND used)
  FastDiv divP;     // by P
  FastDiv div1;     // ND==2: by m[1];  ND==3: by m[1]*m[2]
  FastDiv div2;     // ND==3: by m[2]
  uint64_t pad_bits;
  int64_t inner;    // contiguous elements per innermost index (folded regular trailing dims);
                    // m[ND-1] is already multiplied by it, sizes[.][ND-1] is not
  uint8_t* mask;    // FUSE kernels: one byte per output element (1 inside a constituent), same shape as dst
};

// Validity bytes of one output vector: the n low bytes of the result are 0x01 (n in [0, 8]).
__device__ __forceinline__ uint64_t ones_bytes(int n) {
  return n >= 8 ? 0x0101010101010101ull : (0x0101010101010101ull & ((1ull << (8 * n)) - 1ull));
}
// Store the VE validity bytes of a vector (VE = 2, 4, 8 or 16) with one aligned store.
template <int VE>
__device__ __forceinline__ void store_mask_vec(uint8_t* p, uint64_t lo, uint64_t hi) {
  if (VE == 2) *reinterpret_cast<uint16_t*>(p) = (uint16_t)lo;
  else if (VE == 4) *reinterpret_cast<uint32_t*>(p) = (uint32_t)lo;
  else if (VE == 8) *reinterpret_cast<uint64_t*>(p) = lo;
  else *reinterpret_cast<uint4*>(p) = make_uint4((uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)hi, (uint32_t)(hi >> 32));
}

// ---- one ragged dimension (sequences (L_i, D), the common case): everything inline.  For ND = 1 the
// boundary path needs no division, the whole kernel stays small and needs only 32 registers (full
// occupancy), which measured 5 % faster at configuration 2 than the two-pass kernel below.
// Value of output element r of entry b (entry edges).
template <int ES, int ND, bool MASK, bool BIG>
__device__ __forceinline__ typename ElemBits<ES>::T pad1_elem(const PadParams& p, int64_t b, uint64_t r) {
  using E = typename ElemBits<ES>::T;
  using IP = IdxPolicy<BIG>;
  using I = typename IP::T;
  const int64_t* s = p.sizes + b * p.size_stride;
  bool valid;
  int64_t lin;
  if (ND == 1) {
    valid = (int64_t)r < s[0] * p.inner;
    lin = (int64_t)r;
  } else if (ND == 2) {
    I i0 = IP::div((I)r, p.div1, p.m[1]);
    I c = (I)r - i0 * (I)p.m[1];
    int64_t s1 = s[1] * p.inner;
    valid = (int64_t)i0 < s[0] && (int64_t)c < s1;
    lin = (int64_t)i0 * s1 + (int64_t)c;
  } else {
    const uint64_t m12 = p.m[1] * p.m[2];
    I i0 = IP::div((I)r, p.div1, m12);
    I rem = (I)r - i0 * (I)m12;
    I i1 = IP::div(rem, p.div2, p.m[2]);
    I c = rem - i1 * (I)p.m[2];
    int64_t s1 = s[1], s2 = s[2] * p.inner;
    valid = (int64_t)i0 < s[0] && (int64_t)i1 < s1 && (int64_t)c < s2;
    lin = ((int64_t)i0 * s1 + (int64_t)i1) * s2 + (int64_t)c;
  }
  if (MASK) return (E)(valid ? 1 : 0);
  if (!valid) return (E)p.pad_bits;
  return reinterpret_cast<const E*>(p.src)[p.offsets[b] + lin];
}

// FUSE: besides the data, write the validity mask of the same shape (one byte per output element) in the same pass.
template <int ES, bool MASK, bool BIG, bool FUSE = false>
__global__ void __launch_bounds__(kThreads) pad1_kernel(const PadParams p) {
  constexpr int ND = 1;
  using E = typename ElemBits<ES>::T;
  using IP = IdxPolicy<BIG>;
  using I = typename IP::T;
  constexpr int VE = 16 / ES;
  constexpr uint32_t kTileElems = kThreads * kVecPerThread * VE;

  const int64_t tile_e0 = (int64_t)blockIdx.x * kTileElems;
  const uint64_t b0 = (uint64_t)tile_e0 / p.P;
  const I r0 = (I)((uint64_t)tile_e0 - b0 * p.P);
  const E padv = (E)p.pad_bits;
  E* __restrict__ dst = reinterpret_cast<E*>(p.dst);
  const E* __restrict__ src = reinterpret_cast<const E*>(p.src);
  // end of the ragged buffer (read only by the realigning loads of 1- and 2-byte elements)
  const E* src_limit = (MASK || ES > 2) ? nullptr : src + p.offsets[p.batch];

#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    const uint32_t rel = (uint32_t)(u * kThreads + threadIdx.x) * VE;
    const int64_t e = tile_e0 + rel;
    if (e >= p.total) break;
    const I t = r0 + (I)rel;
    const I qb = IP::div(t, p.divP, p.P);
    const I r = t - qb * (I)p.P;
    const int64_t b = (int64_t)b0 + (int64_t)qb;

    union {
      uint4 v;
      E e[VE];
    } out;

    // locate the innermost row holding element r
    const int64_t* s = p.sizes + b * p.size_stride;
    I c;
    uint64_t row_len;
    bool outer_valid;
    int64_t s_last, src_row;
    if (ND == 1) {
      c = r;
      row_len = p.P;
      outer_valid = true;
      s_last = s[0] * p.inner;
      src_row = MASK ? 0 : p.offsets[b];
    } else if (ND == 2) {
      I i0 = IP::div(r, p.div1, p.m[1]);
      c = r - i0 * (I)p.m[1];
      row_len = p.m[1];
      outer_valid = (int64_t)i0 < s[0];
      s_last = s[1] * p.inner;
      src_row = MASK ? 0 : p.offsets[b] + (int64_t)i0 * s_last;
    } else {
      const uint64_t m12 = p.m[1] * p.m[2];
      I i0 = IP::div(r, p.div1, m12);
      I rem = r - i0 * (I)m12;
      I i1 = IP::div(rem, p.div2, p.m[2]);
      c = rem - i1 * (I)p.m[2];
      row_len = p.m[2];
      int64_t s1 = s[1];
      outer_valid = (int64_t)i0 < s[0] && (int64_t)i1 < s1;
      s_last = s[2] * p.inner;
      src_row = MASK ? 0 : p.offsets[b] + ((int64_t)i0 * s1 + (int64_t)i1) * s_last;
    }

    uint64_t mlo = 0, mhi = 0;  // FUSE: validity bytes of this vector
    if ((uint64_t)c + VE <= row_len) {
      // the whole vector lies in one innermost row
      int64_t nvalid = outer_valid ? (s_last - (int64_t)c) : 0;
      nvalid = nvalid < 0 ? 0 : (nvalid > VE ? VE : nvalid);
      if (FUSE) {
        mlo = ones_bytes((int)nvalid);
        if (VE == 16) mhi = ones_bytes((int)nvalid - 8 > 0 ? (int)nvalid - 8 : 0);
      }
      if (nvalid == VE) {
        if (MASK) {
#pragma unroll
          for (int k = 0; k < VE; ++k) out.e[k] = (E)1;
        } else {
          const E* sp = src + src_row + (int64_t)c;
          if ((reinterpret_cast<uintptr_t>(sp) & 15) == 0) {
            out.v = ld_global_16_stream(sp);
          } else if constexpr (ES <= 2) {
            out.v = load16_realign<ES>(sp, src_limit);
          } else {
#pragma unroll
            for (int k = 0; k < VE; ++k) out.e[k] = sp[k];
          }
        }
      } else if (nvalid == 0) {
#pragma unroll
        for (int k = 0; k < VE; ++k) out.e[k] = MASK ? (E)0 : padv;
      } else {
        const E* sp = src + src_row + (int64_t)c;
#pragma unroll
        for (int k = 0; k < VE; ++k) {
          if (k < nvalid) out.e[k] = MASK ? (E)1 : sp[k];
          else out.e[k] = MASK ? (E)0 : padv;
        }
      }
    } else {
      // the vector crosses a row (possibly an entry) boundary: one element at a time
#pragma unroll
      for (int k = 0; k < VE; ++k) {
        uint64_t rk = (uint64_t)r + k;
        int64_t bk = b;
        while (rk >= p.P) {
          rk -= p.P;
          ++bk;
        }
        out.e[k] = (e + k < p.total) ? pad1_elem<ES, 1, MASK, BIG>(p, bk, rk) : (E)0;
        if (FUSE && e + k < p.total && (int64_t)rk < p.sizes[bk * p.size_stride] * p.inner) {
          if (k < 8) mlo |= 1ull << (8 * (k & 7));
          else mhi |= 1ull << (8 * (k & 7));
        }
      }
    }

    if (e + VE <= p.total) {
      st_global_16_stream(dst + e, out.v);
      if (FUSE) store_mask_vec<VE>(p.mask + e, mlo, mhi);
    } else {
#pragma unroll
      for (int k = 0; k < VE; ++k)
        if (e + k < p.total) {
          dst[e + k] = out.e[k];
          if (FUSE) p.mask[e + k] = (uint8_t)(((k < 8 ? mlo : mhi) >> (8 * (k & 7))) & 1);
        }
    }
  }
}

// Row position of output element r of entry b.
template <int ND, bool MASK, bool BIG>
struct PadPos {
  typename IdxPolicy<BIG>::T c;  // column inside the innermost padded row
  uint64_t row_len;              // padded length of that row
  uint64_t w0, w1;               // outer indices of the row
  bool outer_valid;              // the row exists in the constituent
  int64_t s_last;                // valid length of the row
  int64_t src_row;               // source element index of the row's first element
};

template <int ND, bool MASK, bool BIG>
__device__ __forceinline__ PadPos<ND, MASK, BIG> pad_locate(const PadParams& p, int64_t b, typename IdxPolicy<BIG>::T r) {
  using IP = IdxPolicy<BIG>;
  using I = typename IP::T;
  PadPos<ND, MASK, BIG> q;
  const int64_t* s = p.sizes + b * p.size_stride;
  q.w0 = q.w1 = 0;
  if (ND == 1) {
    q.c = r;
    q.row_len = p.P;
    q.outer_valid = true;
    q.s_last = s[0] * p.inner;
    q.src_row = MASK ? 0 : p.offsets[b];
  } else if (ND == 2) {
    const I i0 = IP::div(r, p.div1, p.m[1]);
    q.c = r - i0 * (I)p.m[1];
    q.row_len = p.m[1];
    q.outer_valid = (int64_t)i0 < s[0];
    q.s_last = s[1] * p.inner;
    q.src_row = MASK ? 0 : p.offsets[b] + (int64_t)i0 * q.s_last;
    q.w0 = (uint64_t)i0;
  } else {
    const uint64_t m12 = p.m[1] * p.m[2];
    const I i0 = IP::div(r, p.div1, m12);
    const I rem = r - i0 * (I)m12;
    const I i1 = IP::div(rem, p.div2, p.m[2]);
    q.c = rem - i1 * (I)p.m[2];
    q.row_len = p.m[2];
    const int64_t s1 = s[1];
    q.outer_valid = (int64_t)i0 < s[0] && (int64_t)i1 < s1;
    q.s_last = s[2] * p.inner;
    q.src_row = MASK ? 0 : p.offsets[b] + ((int64_t)i0 * s1 + (int64_t)i1) * q.s_last;
    q.w0 = (uint64_t)i0;
    q.w1 = (uint64_t)i1;
  }
  return q;
}

// One tile = kThreads * kVecPerThread output vectors.  Pass 1 (fully unrolled, branch-light) handles every
// vector that lies inside one innermost row and only FLAGS the others; pass 2 is a single compact loop over
// the flagged vectors (row / entry boundaries, the ragged tail of the output) that walks element by element
// while carrying the indices over the boundary.  Keeping the boundary code out of the unrolled body keeps
// the kernels small: a warp takes the boundary path whenever one of its 32 vectors needs it.
template <int ES, int ND, bool MASK, bool BIG, bool FUSE = false>
__global__ void __launch_bounds__(kThreads) pad_kernel(const PadParams p) {
  using E = typename ElemBits<ES>::T;
  using IP = IdxPolicy<BIG>;
  using I = typename IP::T;
  constexpr int VE = 16 / ES;
  constexpr uint32_t kTileElems = kThreads * kVecPerThread * VE;

  const int64_t tile_e0 = (int64_t)blockIdx.x * kTileElems;
  const uint64_t b0 = (uint64_t)tile_e0 / p.P;
  const I r0 = (I)((uint64_t)tile_e0 - b0 * p.P);
  const E padv = (E)p.pad_bits;
  E* __restrict__ dst = reinterpret_cast<E*>(p.dst);
  const E* __restrict__ src = reinterpret_cast<const E*>(p.src);
  // end of the ragged buffer (read only by the realigning loads of 1- and 2-byte elements)
  const E* src_limit = (MASK || ES > 2) ? nullptr : src + p.offsets[p.batch];
  union Vec {
    uint4 v;
    E e[VE];
  };
  uint32_t boundary = 0, ready = 0;
  Vec val[kVecPerThread];
  uint8_t nval[FUSE ? kVecPerThread : 1];  // FUSE: valid elements of each located vector (they form a prefix)

  // pass 1a: locate every vector of the tile and issue all its loads back to back
#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    const uint32_t rel = (uint32_t)(u * kThreads + threadIdx.x) * VE;
    const int64_t e = tile_e0 + rel;
    if (e >= p.total) break;
    const I t = r0 + (I)rel;
    const I qb = IP::div(t, p.divP, p.P);
    const I r = t - qb * (I)p.P;
    const int64_t b = (int64_t)b0 + (int64_t)qb;
    const PadPos<ND, MASK, BIG> q = pad_locate<ND, MASK, BIG>(p, b, r);
    if ((uint64_t)q.c + VE > q.row_len || e + VE > p.total) {
      boundary |= 1u << u;
      continue;
    }
    ready |= 1u << u;
    Vec& out = val[u];
    int64_t nvalid = q.outer_valid ? (q.s_last - (int64_t)q.c) : 0;
    nvalid = nvalid < 0 ? 0 : (nvalid > VE ? VE : nvalid);
    if (FUSE) nval[u] = (uint8_t)nvalid;
    if (nvalid == VE) {
      if (MASK) {
#pragma unroll
        for (int k = 0; k < VE; ++k) out.e[k] = (E)1;
      } else {
        const E* sp = src + q.src_row + (int64_t)q.c;
        if ((reinterpret_cast<uintptr_t>(sp) & 15) == 0) {
          out.v = ld_global_16_stream(sp);
        } else if constexpr (ES <= 2) {
          out.v = load16_realign<ES>(sp, src_limit);
        } else {
#pragma unroll
          for (int k = 0; k < VE; ++k) out.e[k] = sp[k];
        }
      }
    } else if (nvalid == 0) {
#pragma unroll
      for (int k = 0; k < VE; ++k) out.e[k] = MASK ? (E)0 : padv;
    } else {
      const E* sp = src + q.src_row + (int64_t)q.c;
#pragma unroll
      for (int k = 0; k < VE; ++k) {
        if (k < nvalid) out.e[k] = MASK ? (E)1 : sp[k];
        else out.e[k] = MASK ? (E)0 : padv;
      }
    }
  }
  // pass 1b: the stores
#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    if (ready & (1u << u)) st_global_16_stream(dst + tile_e0 + (uint32_t)(u * kThreads + threadIdx.x) * VE, val[u].v);
  }
  if (FUSE) {
#pragma unroll
    for (int u = 0; u < kVecPerThread; ++u) {
      if (ready & (1u << u)) {
        const int nv = nval[u];
        store_mask_vec<VE>(p.mask + tile_e0 + (uint32_t)(u * kThreads + threadIdx.x) * VE, ones_bytes(nv),
                           VE == 16 ? ones_bytes(nv - 8 > 0 ? nv - 8 : 0) : 0ull);
      }
    }
  }

  // pass 2: the flagged vectors
#pragma unroll 1
  while (boundary != 0) {
    const int u = __ffs(boundary) - 1;
    boundary &= boundary - 1;
    const uint32_t rel = (uint32_t)(u * kThreads + threadIdx.x) * VE;
    const int64_t e = tile_e0 + rel;
    const I t = r0 + (I)rel;
    const I qb = IP::div(t, p.divP, p.P);
    const I r = t - qb * (I)p.P;
    int64_t bb = (int64_t)b0 + (int64_t)qb;
    PadPos<ND, MASK, BIG> q = pad_locate<ND, MASK, BIG>(p, bb, r);
    uint64_t cc = (uint64_t)q.c;
    Vec out;
    uint64_t mlo = 0, mhi = 0;
#pragma unroll
    for (int k = 0; k < VE; ++k) {
      const bool in_range = e + k < p.total;
      const bool v = in_range && q.outer_valid && (int64_t)cc < q.s_last;
      out.e[k] = v ? (MASK ? (E)1 : src[q.src_row + (int64_t)cc]) : (MASK || !in_range ? (E)0 : padv);
      if (FUSE && v) {
        if (k < 8) mlo |= 1ull << (8 * (k & 7));
        else mhi |= 1ull << (8 * (k & 7));
      }
      if (++cc == q.row_len) {
        cc = 0;
        bool next_entry = false;
        if (ND == 1) {
          next_entry = true;
        } else if (ND == 2) {
          if (++q.w0 == p.m[0]) {
            q.w0 = 0;
            next_entry = true;
          }
        } else {
          if (++q.w1 == p.m[1]) {
            q.w1 = 0;
            if (++q.w0 == p.m[0]) {
              q.w0 = 0;
              next_entry = true;
            }
          }
        }
        if (next_entry) ++bb;
        if (bb < p.batch) {
          const int64_t* sn = p.sizes + bb * p.size_stride;
          if (ND == 1) {
            q.s_last = sn[0] * p.inner;
            q.src_row = MASK ? 0 : p.offsets[bb];
          } else if (ND == 2) {
            q.outer_valid = (int64_t)q.w0 < sn[0];
            q.s_last = sn[1] * p.inner;
            q.src_row = MASK ? 0 : p.offsets[bb] + (int64_t)q.w0 * q.s_last;
          } else {
            const int64_t s1 = sn[1];
            q.outer_valid = (int64_t)q.w0 < sn[0] && (int64_t)q.w1 < s1;
            q.s_last = sn[2] * p.inner;
            q.src_row = MASK ? 0 : p.offsets[bb] + ((int64_t)q.w0 * s1 + (int64_t)q.w1) * q.s_last;
          }
        } else {
          q.outer_valid = false;
        }
      }
    }
    if (e + VE <= p.total) {
      st_global_16_stream(dst + e, out.v);
      if (FUSE) store_mask_vec<VE>(p.mask + e, mlo, mhi);
    } else {
#pragma unroll
      for (int k = 0; k < VE; ++k)
        if (e + k < p.total) {
          dst[e + k] = out.e[k];
          if (FUSE) p.mask[e + k] = (uint8_t)(((k < 8 ? mlo : mhi) >> (8 * (k & 7))) & 1);
        }
    }
  }
}

// ---------------------------------------------------------------------------- unpad
struct UnpadParams {
  const void* src;
  void* dst;
  const int64_t* offsets;
  const int64_t* sizes;
  int64_t size_stride;
  int64_t batch;
  int64_t total;  // offsets[batch]
  uint64_t P;
  uint64_t m[3];  // m[ND-1] already multiplied by inner
  int64_t inner;
};

// source index (in the padded tensor) of element r of entry b, and the number of
// elements left in that innermost row starting at r
template <int ND>
__device__ __forceinline__ void unpad_locate(const UnpadParams& p, int64_t b, uint64_t r, int64_t& src_idx,
                                             int64_t& run, uint64_t& w0, uint64_t& w1) {
  const int64_t* s = p.sizes + b * p.size_stride;
  const int64_t base = b * (int64_t)p.P;
  w0 = w1 = 0;
  if (ND == 1) {
    src_idx = base + (int64_t)r;
    run = s[0] * p.inner - (int64_t)r;
  } else if (ND == 2) {
    uint64_t c;
    const uint64_t s1 = (uint64_t)(s[1] * p.inner);
    divmod_u64(r, s1, w0, c);
    src_idx = base + (int64_t)(w0 * p.m[1] + c);
    run = (int64_t)(s1 - c);
  } else {
    uint64_t rem, c;
    const uint64_t s1 = (uint64_t)s[1], s2 = (uint64_t)(s[2] * p.inner);
    divmod_u64(r, s1 * s2, w0, rem);
    divmod_u64(rem, s2, w1, c);
    src_idx = base + (int64_t)((w0 * p.m[1] + w1) * p.m[2] + c);
    run = (int64_t)(s2 - c);
  }
}

// The divisors of unpad_locate are per entry (its own row and plane lengths), so they cannot be turned into
// multiply-shift pairs on the host the way the padded extents are.  A tile touches few entries: the block
// builds the pairs for the first kUnpadEnt of them in shared memory once, and a vector whose entry is in the
// table (and small enough for 32-bit arithmetic) locates itself without a division.
constexpr int kUnpadEnt = 8;
constexpr int kUnpadOff = 128;  // entries per tile whose offsets are kept in shared memory
struct UnpadEnt {
  FastDiv f_plane, f_row;  // divide by s12 (3 ragged dims only) and by s2
  uint32_t s12, s2;        // elements of one valid plane / of one valid innermost row
  uint32_t ok;
};

__device__ __forceinline__ FastDiv make_fastdiv_device(uint32_t d) {
  FastDiv f;
  if (d == 0) d = 1;
  const uint32_t shift = d <= 1 ? 0 : 32 - __clz(d - 1);  // smallest shift with 2^shift >= d
  f.d = d;
  f.mul = (uint32_t)(((1ull << 32) * ((1ull << shift) - d)) / d + 1);
  f.shift = shift;
  return f;
}

template <int ND>
__device__ __forceinline__ UnpadEnt unpad_entry_divisors(const UnpadParams& p, int64_t b) {
  UnpadEnt en;
  en.ok = 0;
  en.s12 = en.s2 = 1;
  en.f_plane = en.f_row = FastDiv{1, 1, 0};
  const int64_t* s = p.sizes + b * p.size_stride;
  const uint64_t s2 = (uint64_t)(s[ND - 1] * p.inner);
  const uint64_t s12 = (ND == 3 ? (uint64_t)s[1] : 1ull) * s2;
  const uint64_t count = (uint64_t)(p.offsets[b + 1] - p.offsets[b]);
  if (s12 > 0 && s12 < (1ull << 30) && count < (1ull << 30)) {
    en.ok = 1;
    en.s12 = (uint32_t)s12;
    en.s2 = (uint32_t)s2;
    en.f_plane = make_fastdiv_device((uint32_t)s12);
    en.f_row = make_fastdiv_device((uint32_t)s2);
  }
  return en;
}

// unpad_locate for an entry of the table: r < 2^30 and both divisors < 2^30
template <int ND>
__device__ __forceinline__ void unpad_locate_fast(const UnpadParams& p, const UnpadEnt& en, int64_t b, uint32_t r,
                                                  int64_t& src_idx, int64_t& run, uint64_t& w0, uint64_t& w1) {
  const int64_t base = b * (int64_t)p.P;
  if (ND == 2) {
    const uint32_t i0 = fastdiv(r, en.f_row);
    const uint32_t c = r - i0 * en.s2;
    w0 = i0;
    w1 = 0;
    src_idx = base + (int64_t)((uint64_t)i0 * p.m[1] + c);
    run = (int64_t)(en.s2 - c);
  } else {
    const uint32_t i0 = fastdiv(r, en.f_plane);
    const uint32_t rem = r - i0 * en.s12;
    const uint32_t i1 = fastdiv(rem, en.f_row);
    const uint32_t c = rem - i1 * en.s2;
    w0 = i0;
    w1 = i1;
    src_idx = base + (int64_t)(((uint64_t)i0 * p.m[1] + i1) * p.m[2] + c);
    run = (int64_t)(en.s2 - c);
  }
}

// Same two-pass structure as pad_kernel: pass 1 copies every output vector whose 16 bytes come from one
// source row, pass 2 walks the flagged ones (end of a source row or entry, ragged tail).
template <int ES, int ND>
__global__ void __launch_bounds__(kThreads) unpad_kernel(const UnpadParams p) {
  using E = typename ElemBits<ES>::T;
  constexpr int VE = 16 / ES;
  constexpr uint32_t kTileElems = kThreads * kVecPerThread * VE;
  __shared__ int64_t s_range[2];
  __shared__ UnpadEnt s_ent[ND >= 2 ? kUnpadEnt : 1];

  __shared__ int64_t s_off[kUnpadOff + 1];  // offsets of the tile's entries (when there are at most kUnpadOff)
  const int64_t tile_e0 = (int64_t)blockIdx.x * kTileElems;
  if (threadIdx.x < 64) {  // warp 0 finds the tile's first entry, warp 1 its last one
    int64_t tile_last = tile_e0 + kTileElems - 1;
    if (tile_last > p.total - 1) tile_last = p.total - 1;
    const int64_t found = find_entry_warp(p.offsets, 0, p.batch - 1, threadIdx.x < 32 ? tile_e0 : tile_last);
    if ((threadIdx.x & 31) == 0) s_range[threadIdx.x >> 5] = found;
  }
  __syncthreads();
  const int64_t blo = s_range[0], bhi = s_range[1];
  const bool off_cached = bhi - blo < kUnpadOff;
  if (off_cached && threadIdx.x <= bhi - blo + 1) s_off[threadIdx.x] = p.offsets[blo + threadIdx.x];
  if (ND >= 2) {
    if (threadIdx.x < kUnpadEnt && blo + threadIdx.x <= bhi) s_ent[threadIdx.x] = unpad_entry_divisors<ND>(p, blo + threadIdx.x);
  }
  __syncthreads();
  // entry of output element e (inside this tile) and its first element
  auto entry_of = [&](int64_t e, int64_t& first) {
    if (off_cached) {
      int lo = 0, hi = (int)(bhi - blo);
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_off[mid] <= e) lo = mid;
        else hi = mid - 1;
      }
      first = s_off[lo];
      return blo + lo;
    }
    const int64_t b = find_entry(p.offsets, blo, bhi, e);
    first = p.offsets[b];
    return b;
  };
  E* __restrict__ dst = reinterpret_cast<E*>(p.dst);
  const E* __restrict__ src = reinterpret_cast<const E*>(p.src);
  union Vec {
    uint4 v;
    E e[VE];
  };
  uint32_t boundary = 0, ready = 0;
  Vec val[kVecPerThread];

  // pass 1a: locate and load
#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    const int64_t e = tile_e0 + (int64_t)(u * kThreads + threadIdx.x) * VE;
    if (e >= p.total) break;
    int64_t first;
    const int64_t b = entry_of(e, first);
    int64_t src_idx, run;
    uint64_t w0, w1;
    const int64_t ei = b - blo;
    if (ND >= 2 && ei < kUnpadEnt && s_ent[ei].ok) {
      unpad_locate_fast<ND>(p, s_ent[ei], b, (uint32_t)(e - first), src_idx, run, w0, w1);
    } else {
      unpad_locate<ND>(p, b, (uint64_t)(e - first), src_idx, run, w0, w1);
    }
    if (run < VE) {  // also covers the ragged tail: run >= VE implies e + VE <= total
      boundary |= 1u << u;
      continue;
    }
    ready |= 1u << u;
    const E* sp = src + src_idx;
    if ((reinterpret_cast<uintptr_t>(sp) & 15) == 0) {
      val[u].v = ld_global_16_stream(sp);
    } else {
#pragma unroll
      for (int k = 0; k < VE; ++k) val[u].e[k] = sp[k];
    }
  }
  // pass 1b: store
#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    if (ready & (1u << u)) st_global_16_stream(dst + tile_e0 + (int64_t)(u * kThreads + threadIdx.x) * VE, val[u].v);
  }

#pragma unroll 1
  while (boundary != 0) {
    const int u = __ffs(boundary) - 1;
    boundary &= boundary - 1;
    const int64_t e = tile_e0 + (int64_t)(u * kThreads + threadIdx.x) * VE;
    int64_t first;
    int64_t b = entry_of(e, first);
    int64_t si, left;
    uint64_t w0, w1;
    unpad_locate<ND>(p, b, (uint64_t)(e - first), si, left, w0, w1);
    Vec out;
#pragma unroll
    for (int k = 0; k < VE; ++k) {
      if (e + k < p.total) {
        if (left == 0) {
          const int64_t* sn = p.sizes + b * p.size_stride;
          bool next_entry = false;
          if (ND == 1) {
            next_entry = true;
          } else if (ND == 2) {
            if (++w0 == (uint64_t)sn[0]) next_entry = true;
          } else {
            if (++w1 == (uint64_t)sn[1]) {
              w1 = 0;
              if (++w0 == (uint64_t)sn[0]) next_entry = true;
            }
          }
          if (next_entry) {
            w0 = w1 = 0;
            do {
              ++b;
            } while (p.offsets[b + 1] == p.offsets[b]);  // skip empty entries; e + k < total bounds b
            sn = p.sizes + b * p.size_stride;
          }
          left = sn[ND - 1] * p.inner;
          si = b * (int64_t)p.P + (ND == 1 ? 0 : (ND == 2 ? (int64_t)(w0 * p.m[1]) : (int64_t)((w0 * p.m[1] + w1) * p.m[2])));
        }
        out.e[k] = src[si];
        ++si;
        --left;
      } else {
        out.e[k] = (E)0;
      }
    }
    if (e + VE <= p.total) {
      st_global_16_stream(dst + e, out.v);
    } else {
#pragma unroll
      for (int k = 0; k < VE; ++k)
        if (e + k < p.total) dst[e + k] = out.e[k];
    }
  }
}

// ------------------------------------------------------------------ row walks (2-3 ragged dims, long rows)
// With two or three ragged dimensions the vector walks above locate every 16-byte vector on its own (three
// multiply-shift divisions, the sizes of its entry, a validity test) and are bound by that arithmetic, not by DRAM,
// when the innermost rows are long (images: 3-4 KB rows).  Here a WARP takes one innermost row of the padded tensor:
// the row is located once (entry, plane, row index, valid length, source row) and its vectors then cost a compare, an
// address step, a load and a store each.  The destination row is walked in 16-byte-aligned vectors with an
// element-wise head and tail; the source row has one phase for the whole row, so its loads are either all aligned
// 16-byte loads or all element-wise.  Used for rows of a few KB and more (row_kernel_min_bytes below).
struct RowParams {
  const void* src;
  void* dst;
  uint8_t* mask;            // pad FUSE: one byte per output element
  const int64_t* offsets;
  const int64_t* sizes;
  int64_t size_stride;
  int64_t batch;
  uint64_t rows_per_entry;  // padded rows per entry: m0 (ND == 2) or m0 * m1 (ND == 3)
  uint64_t m0, m1;          // padded outer extents
  uint64_t m_last;          // padded row length in elements (innermost extent times inner)
  int64_t inner;
  uint64_t pad_bits;
  uint64_t blocks_per_entry;  // unpad: CTAs of kRowWarps rows per entry
};
constexpr int kRowWarps = 8;
constexpr int kRowUnroll = 8;  // vectors per lane in flight: one trip covers a row of 4 KB

template <int ES, int ND, bool FUSE>
__global__ void __launch_bounds__(kRowWarps * 32) pad_rows_kernel(const RowParams p) {
  using E = typename ElemBits<ES>::T;
  constexpr int VE = 16 / ES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t row = (uint64_t)blockIdx.x * kRowWarps + warp;
  if (row >= (uint64_t)p.batch * p.rows_per_entry) return;
  uint64_t b, rr;
  divmod_u64(row, p.rows_per_entry, b, rr);
  const int64_t* s = p.sizes + (int64_t)b * p.size_stride;
  int64_t nv, src_row;  // valid elements at the start of the row, source element index of the row
  if (ND == 2) {
    nv = (int64_t)rr < s[0] ? s[1] * p.inner : 0;
    src_row = p.offsets[b] + (int64_t)rr * (s[1] * p.inner);
  } else {
    uint64_t i0, i1;
    divmod_u64(rr, p.m1, i0, i1);
    const int64_t s1 = s[1], s_last = s[2] * p.inner;
    nv = ((int64_t)i0 < s[0] && (int64_t)i1 < s1) ? s_last : 0;
    src_row = p.offsets[b] + ((int64_t)i0 * s1 + (int64_t)i1) * s_last;
  }
  const E padv = (E)p.pad_bits;
  const int64_t m_last = (int64_t)p.m_last;
  E* __restrict__ drow = reinterpret_cast<E*>(p.dst) + row * p.m_last;
  const E* __restrict__ srow = reinterpret_cast<const E*>(p.src) + src_row;
  uint8_t* mrow = FUSE ? p.mask + row * p.m_last : nullptr;
  int64_t head = (int64_t)(((16 - (reinterpret_cast<uintptr_t>(drow) & 15)) & 15) / ES);
  head = head < m_last ? head : m_last;
  const int64_t nvec = (m_last - head) / VE;
  const int64_t tail0 = head + nvec * VE;
  if (lane < head) {
    drow[lane] = lane < nv ? srow[lane] : padv;
    if (FUSE) mrow[lane] = lane < nv ? 1 : 0;
  }
  if (tail0 + lane < m_last) {
    const int64_t e = tail0 + lane;
    drow[e] = e < nv ? srow[e] : padv;
    if (FUSE) mrow[e] = e < nv ? 1 : 0;
  }
  const bool src_aligned = nv > 0 && ((reinterpret_cast<uintptr_t>(srow + head) & 15) == 0);
  union Vec {
    uint4 v;
    E e[VE];
  };
  Vec padvec;
#pragma unroll
  for (int k = 0; k < VE; ++k) padvec.e[k] = padv;
  constexpr int U = kRowUnroll;
  for (int64_t j0 = lane; j0 < nvec; j0 += 32 * U) {
    Vec val[U];
    int n[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t j = j0 + 32 * u;
      n[u] = -1;
      if (j >= nvec) continue;
      const int64_t e0 = head + j * VE;
      int64_t nn = nv - e0;
      nn = nn < 0 ? 0 : (nn > VE ? VE : nn);
      n[u] = (int)nn;
      if (nn == VE) {
        if (src_aligned) {
          val[u].v = ld_global_16_stream(srow + e0);
        } else {  // (the realigning word loads of the flat pad kernels measured slower here: 4.0 against 4.8 TB/s, bf16)
#pragma unroll
          for (int k = 0; k < VE; ++k) val[u].e[k] = srow[e0 + k];
        }
      } else if (nn == 0) {
        val[u].v = padvec.v;
      } else {
#pragma unroll
        for (int k = 0; k < VE; ++k) val[u].e[k] = k < nn ? srow[e0 + k] : padv;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (n[u] < 0) continue;
      const int64_t e0 = head + (j0 + 32 * u) * VE;
      st_global_16_stream(drow + e0, val[u].v);
      if (FUSE) store_mask_vec<VE>(mrow + e0, ones_bytes(n[u]), VE == 16 ? ones_bytes(n[u] - 8 > 0 ? n[u] - 8 : 0) : 0ull);
    }
  }
}

// The inverse: a warp takes one innermost row of one constituent (source: the padded row, destination: the row in the
// ragged buffer, which starts at any element phase).  CTA c of entry b = blockIdx.x / blocks_per_entry holds rows
// c * kRowWarps ... of that entry; CTAs past the entry's last row exit.
template <int ES, int ND>
__global__ void __launch_bounds__(kRowWarps * 32) unpad_rows_kernel(const RowParams p) {
  using E = typename ElemBits<ES>::T;
  constexpr int VE = 16 / ES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint64_t b, c;
  divmod_u64((uint64_t)blockIdx.x, p.blocks_per_entry, b, c);
  const int64_t* s = p.sizes + (int64_t)b * p.size_stride;
  const int64_t rows_b = ND == 2 ? s[0] : s[0] * s[1];
  const int64_t rr = (int64_t)c * kRowWarps + warp;
  if (rr >= rows_b) return;
  const int64_t s_last64 = s[ND - 1] * p.inner;
  if (s_last64 <= 0) return;
  const uint32_t s_last = (uint32_t)s_last64;  // (a row of the padded tensor has fewer than 2^31 elements)
  int64_t src_row;                             // row index in the padded tensor
  if (ND == 2) {
    src_row = (int64_t)b * (int64_t)p.m0 + rr;
  } else {
    uint64_t i0, i1;
    divmod_u64((uint64_t)rr, (uint64_t)s[1], i0, i1);
    src_row = ((int64_t)b * (int64_t)p.m0 + (int64_t)i0) * (int64_t)p.m1 + (int64_t)i1;
  }
  const E* __restrict__ srow = reinterpret_cast<const E*>(p.src) + src_row * (int64_t)p.m_last;
  E* __restrict__ drow = reinterpret_cast<E*>(p.dst) + p.offsets[b] + rr * s_last64;
  uint32_t head = (uint32_t)(((16 - (reinterpret_cast<uintptr_t>(drow) & 15)) & 15) / ES);
  head = head < s_last ? head : s_last;
  const uint32_t nvec = (s_last - head) / VE;
  const uint32_t tail0 = head + nvec * VE;
  if ((uint32_t)lane < head) drow[lane] = srow[lane];
  if (tail0 + lane < s_last) drow[tail0 + lane] = srow[tail0 + lane];
  const E* __restrict__ sb = srow + head;  // the vector body of the row: source and destination
  uint4* __restrict__ db = reinterpret_cast<uint4*>(drow + head);
  union Vec {
    uint4 v;
    E e[VE];
  };
  constexpr int U = kRowUnroll;
  if ((reinterpret_cast<uintptr_t>(sb) & 15) == 0) {
    const uint4* __restrict__ sv = reinterpret_cast<const uint4*>(sb);
    for (uint32_t j0 = lane; j0 < nvec; j0 += 32 * U) {
      uint4 val[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (j0 + 32 * u < nvec) val[u] = ld_global_16_stream(sv + j0 + 32 * u);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (j0 + 32 * u < nvec) st_global_16_stream(db + j0 + 32 * u, val[u]);
    }
  } else {
    for (uint32_t j0 = lane; j0 < nvec; j0 += 32 * U) {
      Vec val[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t j = j0 + 32 * u;
        if (j < nvec) {
#pragma unroll
          for (int k = 0; k < VE; ++k) val[u].e[k] = sb[j * VE + k];
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (j0 + 32 * u < nvec) st_global_16_stream(db + j0 + 32 * u, val[u].v);
    }
  }
}

// ------------------------------------------------------------- sizes from padded / mask
struct ScanParams {
  const void* src;
  unsigned long long* out_sizes;   // [batch, ND]
  unsigned long long* out_counts;  // [batch]
  int64_t batch;
  int64_t total;
  uint64_t P;
  uint64_t m[3];
  FastDiv divP, div1, div2;
  uint64_t pad_bits;
};

// CMP: 0 bit pattern, 1 IEEE float of the element width, 2 bfloat16
template <int ES, int CMP>
struct NotPad {
  using E = typename ElemBits<ES>::T;
  E pad;
  __device__ explicit NotPad(uint64_t bits) : pad((E)bits) {}
  __device__ __forceinline__ bool operator()(E x) const { return x != pad; }
};
__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
  // exact widening of IEEE binary16
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t ex = (h >> 10) & 0x1fu;
  const uint32_t man = h & 0x3ffu;
  if (ex == 0x1f) return __uint_as_float(sign | 0x7f800000u | (man << 13));
  if (ex == 0) {
    const float f = (float)man * 5.9604644775390625e-8f;  // man * 2^-24
    return sign ? -f : f;
  }
  return __uint_as_float(sign | ((ex + 112u) << 23) | (man << 13));
}
template <>
struct NotPad<2, 1> {
  float pad;
  __device__ explicit NotPad(uint64_t bits) { pad = half_bits_to_float((uint16_t)bits); }
  __device__ __forceinline__ bool operator()(uint16_t x) const { return half_bits_to_float(x) != pad; }
};
template <>
struct NotPad<2, 2> {
  float pad;
  __device__ explicit NotPad(uint64_t bits) { pad = __uint_as_float((uint32_t)(bits & 0xffffu) << 16); }
  __device__ __forceinline__ bool operator()(uint16_t x) const { return __uint_as_float((uint32_t)x << 16) != pad; }
};
template <>
struct NotPad<4, 1> {
  float pad;
  __device__ explicit NotPad(uint64_t bits) { pad = __uint_as_float((uint32_t)bits); }
  __device__ __forceinline__ bool operator()(uint32_t x) const { return __uint_as_float(x) != pad; }
};
template <>
struct NotPad<8, 1> {
  double pad;
  __device__ explicit NotPad(uint64_t bits) { pad = __longlong_as_double((long long)bits); }
  __device__ __forceinline__ bool operator()(uint64_t x) const { return __longlong_as_double((long long)x) != pad; }
};

// Whole-vector form of the same test: true iff all 16 bytes are padding under NotPad<ES, CMP>, in about five
// logic instructions instead of 16 / ES compares (most vectors of a padded batch are padding).  For the float
// comparisons an element equals a non-zero, non-NaN padding value iff its bits are identical, equals +-0 iff
// all bits but the sign are clear, and never equals NaN.
template <int ES, int CMP>
struct VecAllPad {
  uint32_t pl, ph, ml, mh;
  bool never;
  __host__ __device__ explicit VecAllPad(uint64_t bits) {
    const uint64_t emask = ES == 8 ? ~0ull : ((1ull << (8 * (ES & 7))) - 1);
    uint64_t rep = bits & emask, srep = 1ull << (8 * ES - 1), mask = ~0ull;
#pragma unroll
    for (int w = ES; w < 8; w *= 2) {
      rep |= rep << (8 * w);
      srep |= srep << (8 * w);
    }
    never = false;
    if (CMP != 0) {
      const uint64_t v = bits & emask & ~(1ull << (8 * ES - 1));  // magnitude bits of the padding value
      const uint64_t inf = CMP == 2 ? 0x7f80ull : (ES == 2 ? 0x7c00ull : (ES == 4 ? 0x7f800000ull : 0x7ff0000000000000ull));
      if (v > inf) {
        never = true;  // NaN
      } else if (v == 0) {
        rep = 0;
        mask = ~srep;
      }
    }
    pl = (uint32_t)rep, ph = (uint32_t)(rep >> 32), ml = (uint32_t)mask, mh = (uint32_t)(mask >> 32);
  }
  __device__ __forceinline__ bool operator()(const uint4& v) const {
    return !never && ((((v.x ^ pl) & ml) | ((v.y ^ ph) & mh) | ((v.z ^ pl) & ml) | ((v.w ^ ph) & mh)) == 0);
  }
};

// Class of one 16-byte vector under the same test (for a padding value that is not NaN), in integer arithmetic and
// without a branch: any_valid = some element differs from the padding value, all_valid = every element does.  Inside
// a constituent nearly every vector is all_valid and outside it none is, so the per-element compare is needed on the
// boundary vectors only.
template <int ES, int CMP>
__device__ __forceinline__ void vec_class(const VecAllPad<ES, CMP>& t, const uint4& v, bool& any_valid, bool& all_valid) {
  const uint32_t y0 = (v.x ^ t.pl) & t.ml, y1 = (v.y ^ t.ph) & t.mh, y2 = (v.z ^ t.pl) & t.ml, y3 = (v.w ^ t.ph) & t.mh;
  any_valid = (y0 | y1 | y2 | y3) != 0;
  if (ES == 8) {
    all_valid = ((y0 | y1) != 0) & ((y2 | y3) != 0);
  } else if (ES == 4) {
    all_valid = (y0 != 0) & (y1 != 0) & (y2 != 0) & (y3 != 0);
  } else {  // a zero byte / half-word inside a word: (y - 0x01..) & ~y & 0x80..
    constexpr uint32_t lo = ES == 2 ? 0x00010001u : 0x01010101u, hi = ES == 2 ? 0x80008000u : 0x80808080u;
    const uint32_t z = ((y0 - lo) & ~y0) | ((y1 - lo) & ~y1) | ((y2 - lo) & ~y2) | ((y3 - lo) & ~y3);
    all_valid = (z & hi) == 0;
  }
}

template <int ND, bool BIG>
__device__ __forceinline__ void decompose(const ScanParams& p, uint64_t r, uint64_t idx[3]) {
  using IP = IdxPolicy<BIG>;
  using I = typename IP::T;
  if (ND == 1) {
    idx[0] = r;
  } else if (ND == 2) {
    I i0 = IP::div((I)r, p.div1, p.m[1]);
    idx[0] = i0;
    idx[1] = (I)r - i0 * (I)p.m[1];
  } else {
    const uint64_t m12 = p.m[1] * p.m[2];
    I i0 = IP::div((I)r, p.div1, m12);
    I rem = (I)r - i0 * (I)m12;
    I i1 = IP::div(rem, p.div2, p.m[2]);
    idx[0] = i0;
    idx[1] = i1;
    idx[2] = rem - i1 * (I)p.m[2];
  }
}

template <int ND>
__device__ __forceinline__ void scan_flush(const ScanParams& p, int64_t b, unsigned long long cnt,
                                           const unsigned long long mx[3]) {
  if (cnt == 0) return;
  atomicAdd(p.out_counts + b, cnt);
#pragma unroll
  for (int j = 0; j < ND; ++j) atomicMax(p.out_sizes + b * ND + j, mx[j]);
}

constexpr int kScanSlots = 32;  // entries after a tile's first one that are accumulated in shared memory

template <int ES, int ND, int CMP, bool BIG>
__global__ void __launch_bounds__(kThreads) sizes_scan_kernel(const ScanParams p) {
  using E = typename ElemBits<ES>::T;
  using IP = IdxPolicy<BIG>;
  using I = typename IP::T;
  constexpr int VE = 16 / ES;
  constexpr uint32_t kTileElems = kThreads * kVecPerThread * VE;
  const NotPad<ES, CMP> notpad(p.pad_bits);
  const VecAllPad<ES, CMP> all_pad(p.pad_bits);

  const int64_t tile_e0 = (int64_t)blockIdx.x * kTileElems;
  const uint64_t b0 = (uint64_t)tile_e0 / p.P;
  const I r0 = (I)((uint64_t)tile_e0 - b0 * p.P);
  const E* __restrict__ src = reinterpret_cast<const E*>(p.src);

  // accumulators for the tile's first entry in registers (reduced over the block at the end), for the next
  // kScanSlots entries in shared memory (small entries: several per tile; an entry that ends inside a tile), and
  // global atomics only beyond those (entries of less than a thirty-second of a tile)
  // (32-bit while a padded entry has fewer than 2^30 elements: half the instructions of the bookkeeping)
  using A = typename IP::T;
  A cnt0 = 0, mx0[3] = {0, 0, 0};
  __shared__ unsigned long long s_slot[kScanSlots][4];  // count, extents
  if (threadIdx.x < kScanSlots * 4) (&s_slot[0][0])[threadIdx.x] = 0ull;
  __syncthreads();
  // one non-padding run inside one innermost row of entry b0 + q: count c, extents mx
  auto account = [&](uint64_t q, unsigned long long c, const unsigned long long (&mx)[3]) {
    if (q - 1 < (uint64_t)kScanSlots) {
      atomicAdd(&s_slot[q - 1][0], c);
#pragma unroll
      for (int j = 0; j < ND; ++j) atomicMax(&s_slot[q - 1][1 + j], mx[j]);
    } else {
      scan_flush<ND>(p, (int64_t)(b0 + q), c, mx);
    }
  };

  // all loads of the tile first (read-only kernel: memory-level parallelism is everything), then the
  // bookkeeping
  union Vec {
    uint4 v;
    E e[VE];
  };
  Vec inv[kVecPerThread];
#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    const int64_t e = tile_e0 + (uint32_t)(u * kThreads + threadIdx.x) * VE;
    if (e + VE <= p.total) {
      inv[u].v = ld_global_16_stream(src + e);
    } else {
#pragma unroll
      for (int k = 0; k < VE; ++k) inv[u].e[k] = (e + k < p.total) ? src[e + k] : (E)p.pad_bits;
    }
  }

#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    const uint32_t rel = (uint32_t)(u * kThreads + threadIdx.x) * VE;
    const int64_t e = tile_e0 + rel;
    if (e >= p.total) break;
    const Vec& in = inv[u];
    if (all_pad(in.v)) continue;  // (a partial last vector was filled up with the padding value when loaded)
    uint32_t bits = 0;
    bool any_valid = true, all_valid = false;
    if (!all_pad.never && e + VE <= p.total) vec_class(all_pad, in.v, any_valid, all_valid);
    if (all_valid) {
      bits = (1u << VE) - 1u;
    } else {
#pragma unroll
      for (int k = 0; k < VE; ++k)
        if (e + k < p.total && notpad(in.e[k])) bits |= 1u << k;
    }
    if (bits == 0) continue;
    const I t = r0 + (I)rel;
    const I qb = IP::div(t, p.divP, p.P);
    const I r = t - qb * (I)p.P;
    const int64_t b = (int64_t)b0 + (int64_t)qb;

    uint64_t idx[3];
    decompose<ND, BIG>(p, (uint64_t)r, idx);
    const uint64_t row_len = (ND == 1) ? p.P : p.m[ND - 1];
    if (idx[ND - 1] + VE <= row_len) {
      A mx[3];
#pragma unroll
      for (int j = 0; j < ND - 1; ++j) mx[j] = (A)idx[j] + 1;
      mx[ND - 1] = (A)idx[ND - 1] + (A)(32 - __clz(bits));
      const A c = (A)__popc(bits);
      if (qb == 0) {
        cnt0 += c;
#pragma unroll
        for (int j = 0; j < ND; ++j) mx0[j] = mx0[j] > mx[j] ? mx0[j] : mx[j];
      } else {
        unsigned long long mx64[3] = {0, 0, 0};
#pragma unroll
        for (int j = 0; j < ND; ++j) mx64[j] = mx[j];
        account((uint64_t)qb, (unsigned long long)c, mx64);
      }
    } else {
      // the vector crosses the end of an innermost row (row length not a multiple of the vector): element by element
#pragma unroll
      for (int k = 0; k < VE; ++k) {
        if (!(bits & (1u << k))) continue;
        uint64_t rk = (uint64_t)r + k;
        uint64_t qk = (uint64_t)qb;
        while (rk >= p.P) {
          rk -= p.P;
          ++qk;
        }
        uint64_t ik[3];
        decompose<ND, BIG>(p, rk, ik);
        if (qk == 0) {
          cnt0 += 1;
#pragma unroll
          for (int j = 0; j < ND; ++j) mx0[j] = mx0[j] > (A)(ik[j] + 1) ? mx0[j] : (A)(ik[j] + 1);
        } else {
          unsigned long long mx[3] = {0, 0, 0};
#pragma unroll
          for (int j = 0; j < ND; ++j) mx[j] = ik[j] + 1;
          account(qk, 1ull, mx);
        }
      }
    }
  }

  // block reduction of the first-entry accumulators
  __shared__ unsigned long long s_red[kThreads / 32][4];
  const unsigned full = 0xffffffffu;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    cnt0 += __shfl_xor_sync(full, cnt0, o);
#pragma unroll
    for (int j = 0; j < ND; ++j) {
      const A other = __shfl_xor_sync(full, mx0[j], o);
      mx0[j] = mx0[j] > other ? mx0[j] : other;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    s_red[warp][0] = cnt0;
#pragma unroll
    for (int j = 0; j < ND; ++j) s_red[warp][1 + j] = mx0[j];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long c = 0, mx[3] = {0, 0, 0};
    for (int w = 0; w < kThreads / 32; ++w) {
      c += s_red[w][0];
      for (int j = 0; j < ND; ++j) mx[j] = mx[j] > s_red[w][1 + j] ? mx[j] : s_red[w][1 + j];
    }
    if ((int64_t)b0 < p.batch) scan_flush<ND>(p, (int64_t)b0, c, mx);
  }
  if (threadIdx.x >= 32 && threadIdx.x < 32 + kScanSlots) {  // (the barrier above also orders the shared-memory atomics)
    const int q = threadIdx.x - 32;
    const unsigned long long mx[3] = {s_slot[q][1], s_slot[q][2], s_slot[q][3]};
    if (s_slot[q][0] != 0) scan_flush<ND>(p, (int64_t)b0 + 1 + q, s_slot[q][0], mx);
  }
}

// The same scan with the bookkeeping aggregated per WARP (entries of fewer than 2^30 padded elements): the 32 vectors
// of one warp-wide load are 512 contiguous bytes and nearly always belong to one entry, so their counts and extents
// are folded with one warp reduction each and lane 0 carries a running (entry, count, extents) record that is written
// to a shared-memory slot only when the entry changes; the slots go to global memory once per tile.  Rows whose
// length is not a multiple of the vector are handled per vector, not per element: a vector crosses at most one row
// end (rows of at least one vector), and only the maxima over rows matter.  The per-vector atomics of the kernel above
// (every vector of a tile's second entry, every element of a row-crossing vector) made it 10-100 times slower on
// small entries and odd row lengths.
template <int ES, int ND, int CMP>
__global__ void __launch_bounds__(kThreads) sizes_scan_warp_kernel(const ScanParams p) {
  using E = typename ElemBits<ES>::T;
  constexpr int VE = 16 / ES;
  constexpr uint32_t kTileElems = kThreads * kVecPerThread * VE;
  constexpr uint32_t kNone = 0xffffffffu;
  const NotPad<ES, CMP> notpad(p.pad_bits);
  const VecAllPad<ES, CMP> all_pad(p.pad_bits);
  const int lane = threadIdx.x & 31;
  const int64_t tile_e0 = (int64_t)blockIdx.x * kTileElems;
  const uint64_t b0 = (uint64_t)tile_e0 / p.P;
  const uint32_t r0 = (uint32_t)((uint64_t)tile_e0 - b0 * p.P);
  const uint32_t P = (uint32_t)p.P, row_len = (uint32_t)(ND == 1 ? p.P : p.m[ND - 1]);
  const E* __restrict__ src = reinterpret_cast<const E*>(p.src);

  __shared__ unsigned int s_slot[kScanSlots + 1][4];  // per entry b0 + q: count, extents
  for (int i = threadIdx.x; i < (kScanSlots + 1) * 4; i += kThreads) (&s_slot[0][0])[i] = 0u;
  __syncthreads();
  auto account = [&](uint32_t q, uint32_t c, const uint32_t (&mx)[3]) {
    if (q <= (uint32_t)kScanSlots) {
      atomicAdd(&s_slot[q][0], c);
#pragma unroll
      for (int j = 0; j < ND; ++j) atomicMax(&s_slot[q][1 + j], mx[j]);
    } else {
      const unsigned long long m64[3] = {mx[0], mx[1], mx[2]};
      scan_flush<ND>(p, (int64_t)(b0 + q), (unsigned long long)c, m64);
    }
  };

  union Vec {
    uint4 v;
    E e[VE];
  };
  Vec inv[kVecPerThread];
#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    const int64_t e = tile_e0 + (uint32_t)(u * kThreads + threadIdx.x) * VE;
    if (e + VE <= p.total) {
      inv[u].v = ld_global_16_stream(src + e);
    } else {
#pragma unroll
      for (int k = 0; k < VE; ++k) inv[u].e[k] = (e + k < p.total) ? src[e + k] : (E)p.pad_bits;
    }
  }

  uint32_t cur_q = kNone, cur_c = 0, cur_mx[3] = {0, 0, 0};  // lane 0: the entry being accumulated
#pragma unroll
  for (int u = 0; u < kVecPerThread; ++u) {
    const uint32_t rel = (uint32_t)(u * kThreads + threadIdx.x) * VE;
    uint32_t bits = 0;
    if (tile_e0 + rel < p.total && !all_pad(inv[u].v)) {
      bool any_valid = true, all_valid = false;
      if (!all_pad.never) vec_class(all_pad, inv[u].v, any_valid, all_valid);
      if (all_valid) {
        bits = (1u << VE) - 1u;
      } else {
#pragma unroll
        for (int k = 0; k < VE; ++k)
          if (notpad(inv[u].e[k])) bits |= 1u << k;
      }
      // the filler of a partial last vector is the padding value, which a NaN padding value does not equal either
      const int64_t beyond = tile_e0 + rel + VE - p.total;
      if (beyond > 0) bits &= (1u << (VE - (int)beyond)) - 1u;
    }
    if (!__any_sync(0xffffffffu, bits != 0)) continue;  // the whole 512 bytes are padding
    uint32_t q = kNone, c = 0, mx[3] = {0, 0, 0};
    bool simple = true;  // false: the vector reaches into another entry or crosses more than one row end
    if (bits != 0) {
      const uint32_t t = r0 + rel;
      q = fastdiv(t, p.divP);
      const uint32_t r = t - q * P;
      uint64_t idx[3] = {0, 0, 0};
      decompose<ND, false>(p, (uint64_t)r, idx);
      const uint32_t col = (uint32_t)idx[ND - 1], left = row_len - col;  // elements left in this innermost row
      c = (uint32_t)__popc(bits);
      if (left >= (uint32_t)VE) {
#pragma unroll
        for (int j = 0; j < ND - 1; ++j) mx[j] = (uint32_t)idx[j] + 1;
        mx[ND - 1] = col + (uint32_t)(32 - __clz(bits));
      } else {
        const uint32_t lo = bits & ((1u << left) - 1u), hi = bits >> left;  // this row / the next one
        bool next_in_entry = row_len >= (uint32_t)VE && r + left < P;
        uint32_t n0 = (uint32_t)idx[0], n1 = (uint32_t)idx[1];  // outer indices of the next row
        if (ND == 2) {
          n0 += 1;
        } else if (ND == 3) {
          if (++n1 == (uint32_t)p.m[1]) {
            n1 = 0;
            n0 += 1;
          }
        } else {
          next_in_entry = false;  // one dimension: the next "row" is the next entry
        }
        if (hi != 0 && !next_in_entry) {
          simple = false;
        } else {
          const uint32_t end_lo = lo ? col + (uint32_t)(32 - __clz(lo)) : 0u, end_hi = hi ? (uint32_t)(32 - __clz(hi)) : 0u;
          mx[ND - 1] = end_lo > end_hi ? end_lo : end_hi;
          if (ND >= 2) {
            const uint32_t a0 = lo ? (uint32_t)idx[0] + 1 : 0u, b0n = hi ? n0 + 1 : 0u;
            mx[0] = a0 > b0n ? a0 : b0n;
          }
          if (ND == 3) {
            const uint32_t a1 = lo ? (uint32_t)idx[1] + 1 : 0u, b1n = hi ? n1 + 1 : 0u;
            mx[1] = a1 > b1n ? a1 : b1n;
          }
        }
      }
      if (!simple) {  // rare: element by element, straight to the slots
        q = kNone;
#pragma unroll
        for (int k = 0; k < VE; ++k) {
          if (!(bits & (1u << k))) continue;
          uint32_t rk = r + k, qk = fastdiv(t, p.divP);
          while (rk >= P) {
            rk -= P;
            ++qk;
          }
          uint64_t ik[3] = {0, 0, 0};
          decompose<ND, false>(p, (uint64_t)rk, ik);
          const uint32_t m1[3] = {(uint32_t)ik[0] + 1, (uint32_t)ik[1] + 1, (uint32_t)ik[2] + 1};
          account(qk, 1u, m1);
        }
      }
    }
    const uint32_t q_min = __reduce_min_sync(0xffffffffu, q);
    if (q_min == kNone) continue;
    if (__all_sync(0xffffffffu, q == kNone || q == q_min)) {
      const uint32_t C = __reduce_add_sync(0xffffffffu, q == kNone ? 0u : c);
      uint32_t M[3] = {0, 0, 0};
#pragma unroll
      for (int j = 0; j < ND; ++j) M[j] = __reduce_max_sync(0xffffffffu, q == kNone ? 0u : mx[j]);
      if (lane == 0) {
        if (q_min != cur_q) {
          if (cur_q != kNone) account(cur_q, cur_c, cur_mx);
          cur_q = q_min;
          cur_c = 0;
          cur_mx[0] = cur_mx[1] = cur_mx[2] = 0;
        }
        cur_c += C;
#pragma unroll
        for (int j = 0; j < ND; ++j) cur_mx[j] = cur_mx[j] > M[j] ? cur_mx[j] : M[j];
      }
    } else if (q != kNone) {  // the warp's 512 bytes span an entry boundary
      account(q, c, mx);
    }
  }
  if (lane == 0 && cur_q != kNone) account(cur_q, cur_c, cur_mx);
  __syncthreads();
  if (threadIdx.x <= kScanSlots && s_slot[threadIdx.x][0] != 0) {
    const unsigned long long m64[3] = {s_slot[threadIdx.x][1], s_slot[threadIdx.x][2], s_slot[threadIdx.x][3]};
    scan_flush<ND>(p, (int64_t)b0 + threadIdx.x, (unsigned long long)s_slot[threadIdx.x][0], m64);
  }
}

// ------------------------------------------------------------------- offsets (scan)
constexpr int kScanThreads = 1024;

__device__ __forceinline__ int64_t entry_numel(const int64_t* sizes, int64_t stride, int nd, int64_t inner, int64_t b) {
  int64_t n = inner;
  for (int j = 0; j < nd; ++j) n *= sizes[b * stride + j];
  return n;
}

// block-wide exclusive scan of one value per thread; returns the exclusive prefix and
// leaves the block total in *total (valid for all threads after the call)
__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t* total) {
  __shared__ int64_t s_warp[kScanThreads / 32];
  __shared__ int64_t s_total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int64_t n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int64_t w = (lane < kScanThreads / 32) ? s_warp[lane] : 0;
    int64_t wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int64_t n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += n;
    }
    if (lane < kScanThreads / 32) s_warp[lane] = wi - w;  // exclusive prefix of warp sums
    if (lane == 31) s_total = wi;
  }
  __syncthreads();
  const int64_t r = incl - v + s_warp[warp];
  *total = s_total;
  __syncthreads();  // the shared arrays may be reused by the caller's next scan
  return r;
}

// phase 1: per-block exclusive scan of entry sizes; block totals to block_sums (or, for a
// single block, the grand total straight to offsets[batch])
__global__ void __launch_bounds__(kScanThreads) offsets_phase1(const int64_t* sizes, int64_t stride, int nd,
                                                                int64_t inner, int64_t batch, int64_t* offsets,
                                                                int64_t* block_sums) {
  const int64_t b = (int64_t)blockIdx.x * kScanThreads + threadIdx.x;
  const int64_t v = b < batch ? entry_numel(sizes, stride, nd, inner, b) : 0;
  int64_t total;
  const int64_t ex = block_exclusive_scan(v, &total);
  if (b < batch) offsets[b] = ex;
  if (threadIdx.x == 0) {
    if (gridDim.x == 1) offsets[batch] = total;
    else block_sums[blockIdx.x] = total;
  }
}

// phase 2: one block turns block_sums[0..n) into its exclusive scan and writes the grand total
__global__ void __launch_bounds__(kScanThreads) offsets_phase2(int64_t* block_sums, int64_t n, int64_t* grand_total) {
  int64_t carry = 0;
  for (int64_t base = 0; base < n; base += kScanThreads) {
    const int64_t i = base + threadIdx.x;
    const int64_t v = i < n ? block_sums[i] : 0;
    int64_t total;
    const int64_t ex = block_exclusive_scan(v, &total);
    if (i < n) block_sums[i] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0) *grand_total = carry;
}

// phase 3: add each block's base
__global__ void __launch_bounds__(kScanThreads) offsets_phase3(int64_t* offsets, const int64_t* block_sums, int64_t batch) {
  const int64_t b = (int64_t)blockIdx.x * kScanThreads + threadIdx.x;
  if (b < batch) offsets[b] += block_sums[blockIdx.x];
}

// ---------------------------------------------------- built-in scratch for the no-allocation variant
// Block sums for ntb200_offsets_from_sizes_static live here instead of in a caller-provided workspace.
// 4096 entries of 8 bytes = 32 KB, held by every GPU that loads the library until the process exits.
constexpr int64_t kStaticScanBlocks = 4096;
constexpr int64_t kStaticScanMaxBatch = kStaticScanBlocks * kScanThreads;  // 4 194 304 constituents
static __device__ __align__(256) int64_t g_static_block_sums[kStaticScanBlocks];

// In host code `g_static_block_sums` is only a handle for the runtime, not a device address, so the
// address the kernels receive is looked up once per device with cudaGetSymbolAddress.
int64_t* g_static_block_sums_addr[kMaxDevices] = {};

int static_block_sums_for_current_device(int64_t** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return NTB200_LAUNCH_FAILED;
  int64_t* p = __atomic_load_n(&g_static_block_sums_addr[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_static_block_sums) != cudaSuccess || sym == nullptr) return NTB200_LAUNCH_FAILED;
    p = static_cast<int64_t*>(sym);
    __atomic_store_n(&g_static_block_sums_addr[dev], p, __ATOMIC_RELEASE);  // same value from any thread
  }
  *out = p;
  return NTB200_OK;
}

// ---------------------------------------------------------------------- token index
__global__ void __launch_bounds__(kThreads) token_index_kernel(const int64_t* __restrict__ offsets, int64_t batch,
                                                                int64_t total, int32_t* __restrict__ batch_idx,
                                                                int32_t* __restrict__ word_idx) {
  const int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (t >= total) return;
  const int64_t b = find_entry(offsets, 0, batch - 1, t);
  batch_idx[t] = (int32_t)b;
  word_idx[t] = (int32_t)(t - offsets[b]);
}

// ------------------------------------------------------------------------ host side
struct Geometry {
  uint64_t P;
  uint64_t m[3];
  bool big;
};

int make_geometry(int nd, const int64_t* h_max_sizes, int64_t inner, Geometry* g) {
  if (nd < 1 || nd > 3 || h_max_sizes == nullptr || inner < 1) return NTB200_INVALID_ARG;
  g->P = 1;
  g->m[0] = g->m[1] = g->m[2] = 1;
  for (int j = 0; j < nd; ++j) {
    if (h_max_sizes[j] < 0) return NTB200_INVALID_ARG;
    g->m[j] = (uint64_t)h_max_sizes[j];
    if (j == nd - 1) {
      if (g->m[j] != 0 && (uint64_t)inner > (uint64_t)INT64_MAX / g->m[j]) return NTB200_INVALID_ARG;
      g->m[j] *= (uint64_t)inner;
    }
    // overflow-safe product
    if (g->m[j] != 0 && g->P > (uint64_t)INT64_MAX / g->m[j]) return NTB200_INVALID_ARG;
    g->P *= g->m[j];
  }
  g->big = g->P > (1ull << 30);
  return NTB200_OK;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

template <int ES, int ND, bool MASK, bool FUSE>
int launch_pad_es_nd(const PadParams& p, bool big, cudaStream_t st) {
  constexpr int VE = 16 / ES;
  const int64_t tile = (int64_t)kThreads * kVecPerThread * VE;
  const int64_t blocks = ceil_div(p.total, tile);
  if (blocks > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  if (ND == 1) {
    if (big) pad1_kernel<ES, MASK, true, FUSE><<<(unsigned)blocks, kThreads, 0, st>>>(p);
    else pad1_kernel<ES, MASK, false, FUSE><<<(unsigned)blocks, kThreads, 0, st>>>(p);
  } else {
    if (big) pad_kernel<ES, ND, MASK, true, FUSE><<<(unsigned)blocks, kThreads, 0, st>>>(p);
    else pad_kernel<ES, ND, MASK, false, FUSE><<<(unsigned)blocks, kThreads, 0, st>>>(p);
  }
  return status_from_cuda(cudaGetLastError());
}

template <int ES, bool MASK, bool FUSE = false>
int launch_pad_es(const PadParams& p, int nd, bool big, cudaStream_t st) {
  switch (nd) {
    case 1: return launch_pad_es_nd<ES, 1, MASK, FUSE>(p, big, st);
    case 2: return launch_pad_es_nd<ES, 2, MASK, FUSE>(p, big, st);
    case 3: return launch_pad_es_nd<ES, 3, MASK, FUSE>(p, big, st);
  }
  return NTB200_INVALID_ARG;
}

// Where the warp-per-row kernels take over from the vector walks (2-3 ragged dims), by the bytes of an innermost
// padded row.  Measured on B200 with batches of about 400 MB (fp32 and bf16, 2 and 3 ragged dims, rows of 0.5-8 KB):
// at 512-byte rows the row kernels run at 0.25-0.45 of the vector walks' rate (a warp's trip is mostly empty and the
// per-row set-up dominates), they draw level between 2 and 3 KB and win by 10-40 % from there on.
enum RowOp { kRowPad = 0, kRowUnpad = 1, kRowScan = 2 };
inline uint64_t row_kernel_min_bytes(RowOp op, int elem_size) {
  if (op == kRowScan) return 3072;
  return elem_size <= 2 ? 2048 : 2560;
}
inline bool long_rows(int nd, const Geometry& g, int elem_size, RowOp op) {
  return nd >= 2 && g.m[nd - 1] * (uint64_t)elem_size >= row_kernel_min_bytes(op, elem_size) && g.m[nd - 1] < (1ull << 31);
}

template <int ES>
int launch_pad_rows(const RowParams& p, int nd, bool fuse, cudaStream_t st) {
  const uint64_t rows = (uint64_t)p.batch * p.rows_per_entry;
  const uint64_t blocks = (rows + kRowWarps - 1) / kRowWarps;
  if (blocks > 0x7fffffffull) return NTB200_UNSUPPORTED_SHAPE;
  if (nd == 2) {
    if (fuse) pad_rows_kernel<ES, 2, true><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(p);
    else pad_rows_kernel<ES, 2, false><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(p);
  } else {
    if (fuse) pad_rows_kernel<ES, 3, true><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(p);
    else pad_rows_kernel<ES, 3, false><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(p);
  }
  return status_from_cuda(cudaGetLastError());
}

template <int ES>
int launch_unpad_rows(RowParams p, int nd, cudaStream_t st) {
  p.blocks_per_entry = (p.rows_per_entry + kRowWarps - 1) / kRowWarps;
  const uint64_t blocks = (uint64_t)p.batch * p.blocks_per_entry;
  if (blocks > 0x7fffffffull) return NTB200_UNSUPPORTED_SHAPE;
  if (nd == 2) unpad_rows_kernel<ES, 2><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(p);
  else unpad_rows_kernel<ES, 3><<<(unsigned)blocks, kRowWarps * 32, 0, st>>>(p);
  return status_from_cuda(cudaGetLastError());
}

void fill_divs(int nd, const Geometry& g, FastDiv* divP, FastDiv* div1, FastDiv* div2) {
  *divP = make_fastdiv(g.big ? 1 : g.P);
  *div1 = make_fastdiv(1);
  *div2 = make_fastdiv(1);
  if (!g.big) {
    if (nd == 2) *div1 = make_fastdiv(g.m[1]);
    if (nd == 3) {
      *div1 = make_fastdiv(g.m[1] * g.m[2]);
      *div2 = make_fastdiv(g.m[2]);
    }
  }
}

template <int ES, int ND>
int launch_unpad_es_nd(const UnpadParams& p, cudaStream_t st) {
  constexpr int VE = 16 / ES;
  const int64_t tile = (int64_t)kThreads * kVecPerThread * VE;
  const int64_t blocks = ceil_div(p.total, tile);
  if (blocks > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  unpad_kernel<ES, ND><<<(unsigned)blocks, kThreads, 0, st>>>(p);
  return status_from_cuda(cudaGetLastError());
}

template <int ES>
int launch_unpad_es(const UnpadParams& p, int nd, cudaStream_t st) {
  switch (nd) {
    case 1: return launch_unpad_es_nd<ES, 1>(p, st);
    case 2: return launch_unpad_es_nd<ES, 2>(p, st);
    case 3: return launch_unpad_es_nd<ES, 3>(p, st);
  }
  return NTB200_INVALID_ARG;
}

// Row walk of the same scan (2-3 dims, rows of 3 KB and more): a warp reads one innermost row and keeps the
// count of non-padding elements and the end of the last one; thread 0 folds the CTA's eight consecutive rows per
// entry (coordinates by increments, one division per CTA) before the atomics, which are the expensive part: with
// one set of atomics per row instead of per CTA the kernel took 2.5 times as long.  The vector test is vec_class
// (integer, branch-free on the all-valid and all-padding vectors; the caller keeps a NaN padding value away).
// ALIGNED: every row is a whole number of 16-byte vectors (no element-wise head or tail).
template <int ES, int ND, int CMP, bool ALIGNED>
__global__ void __launch_bounds__(kRowWarps * 32) scan_rows_kernel(const ScanParams p) {
  using E = typename ElemBits<ES>::T;
  constexpr int VE = 16 / ES;
  constexpr int U = kRowUnroll;
  const NotPad<ES, CMP> notpad(p.pad_bits);
  const VecAllPad<ES, CMP> t(p.pad_bits);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t rows_per_entry = ND == 2 ? p.m[0] : p.m[0] * p.m[1];
  const uint64_t n_rows = (uint64_t)p.batch * rows_per_entry;
  const uint64_t cta_row0 = (uint64_t)blockIdx.x * kRowWarps;
  const uint64_t row = cta_row0 + warp;
  const uint32_t m_last = (uint32_t)p.m[ND - 1];
  __shared__ uint32_t s_cnt[kRowWarps], s_last[kRowWarps];
  uint32_t cnt = 0, last = 0;
  if (row < n_rows) {
    const E* __restrict__ srow = reinterpret_cast<const E*>(p.src) + row * (uint64_t)m_last;
    uint32_t head = ALIGNED ? 0 : (uint32_t)(((16 - (reinterpret_cast<uintptr_t>(srow) & 15)) & 15) / ES);
    head = head < m_last ? head : m_last;
    const uint32_t nvec = (m_last - head) / VE;
    const uint32_t tail0 = head + nvec * VE;
    if (!ALIGNED && lane < head && notpad(srow[lane])) {
      cnt = 1;
      last = (uint32_t)lane + 1;
    }
    union Vec {
      uint4 v;
      E e[VE];
    };
    const uint4* __restrict__ vrow = reinterpret_cast<const uint4*>(srow + head);
    for (uint32_t j0 = lane; j0 < nvec; j0 += 32 * U) {
      Vec val[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        val[u].v = make_uint4(t.pl, t.ph, t.pl, t.ph);  // past the row: padding
        if (j0 + 32 * u < nvec) val[u].v = ld_global_16_stream(vrow + j0 + 32 * u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        bool any_valid, all_valid;
        vec_class(t, val[u].v, any_valid, all_valid);
        const uint32_t end = head + (j0 + 32 * u + 1) * VE;
        cnt += all_valid ? VE : 0;
        last = all_valid ? end : last;  // j0 and u only grow
        if (any_valid && !all_valid) {
          uint32_t bits = 0;
#pragma unroll
          for (int k = 0; k < VE; ++k)
            if (notpad(val[u].e[k])) bits |= 1u << k;
          cnt += (uint32_t)__popc(bits);
          if (bits != 0) last = end - VE + (uint32_t)(32 - __clz(bits));
        }
      }
    }
    if (!ALIGNED && tail0 + lane < m_last && notpad(srow[tail0 + lane])) {
      cnt += 1;
      last = tail0 + (uint32_t)lane + 1;
    }
  }
  cnt = __reduce_add_sync(0xffffffffu, cnt);
  last = __reduce_max_sync(0xffffffffu, last);
  if (lane == 0) {
    s_cnt[warp] = cnt;
    s_last[warp] = last;
  }
  __syncthreads();
  if (threadIdx.x != 0 || cta_row0 >= n_rows) return;
  uint64_t b, rr, i0 = 0, i1 = 0;
  divmod_u64(cta_row0, rows_per_entry, b, rr);
  if (ND == 2) i0 = rr;
  else divmod_u64(rr, p.m[1], i0, i1);
  unsigned long long c = 0, mx[3] = {0, 0, 0};
  const int n_here = (int)(n_rows - cta_row0 < (uint64_t)kRowWarps ? n_rows - cta_row0 : (uint64_t)kRowWarps);
  for (int w = 0; w < n_here; ++w) {
    const uint32_t cw = s_cnt[w];
    if (cw != 0) {
      c += cw;
      const unsigned long long l = s_last[w];
      mx[ND - 1] = mx[ND - 1] > l ? mx[ND - 1] : l;
      mx[0] = mx[0] > i0 + 1 ? mx[0] : i0 + 1;
      if (ND == 3) mx[1] = mx[1] > i1 + 1 ? mx[1] : i1 + 1;
    }
    bool next_entry;
    if (ND == 2) {
      next_entry = ++i0 == p.m[0];
    } else {
      next_entry = false;
      if (++i1 == p.m[1]) {
        i1 = 0;
        next_entry = ++i0 == p.m[0];
      }
    }
    if (next_entry) {
      scan_flush<ND>(p, (int64_t)b, c, mx);
      c = 0;
      mx[0] = mx[1] = mx[2] = 0;
      i0 = 0;
      ++b;
    }
  }
  scan_flush<ND>(p, (int64_t)b, c, mx);
}

template <int ES, int ND, int CMP>
int launch_scan_es_nd(const ScanParams& p, bool big, cudaStream_t st) {
  constexpr int VE = 16 / ES;
  const int64_t tile = (int64_t)kThreads * kVecPerThread * VE;
  const int64_t blocks = ceil_div(p.total, tile);
  if (blocks > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  // (a NaN padding value equals no element: the row kernel's vector classes assume a value that can match)
  if (ND >= 2 && p.m[ND - 1] * (uint64_t)ES >= row_kernel_min_bytes(kRowScan, ES) && p.m[ND - 1] < (1ull << 31) &&
      !VecAllPad<ES, CMP>(p.pad_bits).never) {
    const uint64_t rows = (uint64_t)p.batch * (ND == 2 ? p.m[0] : p.m[0] * p.m[1]);
    const uint64_t row_blocks = (rows + kRowWarps - 1) / kRowWarps;
    if (row_blocks > 0x7fffffffull) return NTB200_UNSUPPORTED_SHAPE;
    if ((p.m[ND - 1] * (uint64_t)ES) % 16 == 0)  // (the base is 16-byte aligned)
      scan_rows_kernel<ES, (ND >= 2 ? ND : 2), CMP, true><<<(unsigned)row_blocks, kRowWarps * 32, 0, st>>>(p);
    else
      scan_rows_kernel<ES, (ND >= 2 ? ND : 2), CMP, false><<<(unsigned)row_blocks, kRowWarps * 32, 0, st>>>(p);
    return status_from_cuda(cudaGetLastError());
  }
  // Entries that are whole tiles of whole-vector rows keep the kernel with per-thread registers for the tile's one
  // entry (8 % fewer instructions at the 4096 x 1024 x 1024 bf16 batch); every other shape takes the warp-aggregated
  // kernel, whose cost does not depend on where entries and rows end.
  const uint64_t row_len = ND == 1 ? p.P : p.m[ND - 1];
  if (big) sizes_scan_kernel<ES, ND, CMP, true><<<(unsigned)blocks, kThreads, 0, st>>>(p);
  else if (p.P % (uint64_t)tile == 0 && row_len % VE == 0) sizes_scan_kernel<ES, ND, CMP, false><<<(unsigned)blocks, kThreads, 0, st>>>(p);
  else sizes_scan_warp_kernel<ES, ND, CMP><<<(unsigned)blocks, kThreads, 0, st>>>(p);
  return status_from_cuda(cudaGetLastError());
}

template <int ES, int CMP>
int launch_scan_es(const ScanParams& p, int nd, bool big, cudaStream_t st) {
  switch (nd) {
    case 1: return launch_scan_es_nd<ES, 1, CMP>(p, big, st);
    case 2: return launch_scan_es_nd<ES, 2, CMP>(p, big, st);
    case 3: return launch_scan_es_nd<ES, 3, CMP>(p, big, st);
  }
  return NTB200_INVALID_ARG;
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace
}  // namespace ntb200

using namespace ntb200;

extern "C" {

const char* ntb200_status_string(int status) {
  switch (status) {
    case NTB200_OK: return "ok";
    case NTB200_INVALID_ARG: return "invalid argument";
    case NTB200_UNSUPPORTED_DTYPE: return "unsupported dtype";
    case NTB200_MISALIGNED: return "misaligned pointer";
    case NTB200_LAUNCH_FAILED: return "kernel launch failed";
    case NTB200_DEVICE_TIMEOUT: return "device-side wait timed out";
    case NTB200_WORKSPACE_TOO_SMALL: return "workspace too small";
    case NTB200_UNSUPPORTED_SHAPE: return "unsupported shape";
    case NTB200_STATIC_SCRATCH_EXCEEDED: return "size exceeds the built-in scratch of the no-allocation entry point";
  }
  return "unknown status";
}

int ntb200_version(void) { return 1000; }

// to_padded_tensor, optionally with the validity mask of the same shape written in the same pass (fused_mask != NULL)
static int pad_common(const void* ragged, void* padded, uint8_t* fused_mask, const int64_t* offsets, const int64_t* sizes,
                      int64_t size_stride, int nd, int64_t inner, int64_t batch, const int64_t* h_max_sizes,
                      int elem_size, uint64_t pad_bits, void* stream) {
  Geometry g;
  int rc = make_geometry(nd, h_max_sizes, inner, &g);
  if (rc != NTB200_OK) return rc;
  if (batch < 0 || size_stride < nd) return NTB200_INVALID_ARG;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return NTB200_UNSUPPORTED_DTYPE;
  if (batch == 0 || g.P == 0) return NTB200_OK;
  if (g.P > (uint64_t)INT64_MAX / (uint64_t)batch) return NTB200_INVALID_ARG;
  if (padded == nullptr || offsets == nullptr || sizes == nullptr) return NTB200_INVALID_ARG;
  if (!aligned_to(padded, 16)) return NTB200_MISALIGNED;
  if (ragged != nullptr && !aligned_to(ragged, (size_t)elem_size)) return NTB200_MISALIGNED;

  PadParams p;
  p.src = ragged;
  p.dst = padded;
  p.offsets = offsets;
  p.sizes = sizes;
  p.size_stride = size_stride;
  p.batch = batch;
  p.P = g.P;
  p.total = batch * (int64_t)g.P;
  for (int j = 0; j < 3; ++j) p.m[j] = g.m[j];
  fill_divs(nd, g, &p.divP, &p.div1, &p.div2);
  p.pad_bits = pad_bits;
  p.inner = inner;
  p.mask = fused_mask;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (fused_mask != nullptr && !aligned_to(fused_mask, 16)) return NTB200_MISALIGNED;
  if (long_rows(nd, g, elem_size, kRowPad) && ragged != nullptr) {
    RowParams rp;
    rp.src = ragged;
    rp.dst = padded;
    rp.mask = fused_mask;
    rp.offsets = offsets;
    rp.sizes = sizes;
    rp.size_stride = size_stride;
    rp.batch = batch;
    rp.m0 = g.m[0];
    rp.m1 = nd == 3 ? g.m[1] : 1;
    rp.rows_per_entry = nd == 3 ? g.m[0] * g.m[1] : g.m[0];
    rp.m_last = g.m[nd - 1];
    rp.inner = inner;
    rp.pad_bits = pad_bits;
    rp.blocks_per_entry = 0;
    switch (elem_size) {
      case 1: return launch_pad_rows<1>(rp, nd, fused_mask != nullptr, st);
      case 2: return launch_pad_rows<2>(rp, nd, fused_mask != nullptr, st);
      case 4: return launch_pad_rows<4>(rp, nd, fused_mask != nullptr, st);
      case 8: return launch_pad_rows<8>(rp, nd, fused_mask != nullptr, st);
    }
    return NTB200_UNSUPPORTED_DTYPE;
  }
  if (fused_mask != nullptr) {
    switch (elem_size) {
      case 1: return launch_pad_es<1, false, true>(p, nd, g.big, st);
      case 2: return launch_pad_es<2, false, true>(p, nd, g.big, st);
      case 4: return launch_pad_es<4, false, true>(p, nd, g.big, st);
      case 8: return launch_pad_es<8, false, true>(p, nd, g.big, st);
    }
    return NTB200_UNSUPPORTED_DTYPE;
  }
  switch (elem_size) {
    case 1: return launch_pad_es<1, false>(p, nd, g.big, st);
    case 2: return launch_pad_es<2, false>(p, nd, g.big, st);
    case 4: return launch_pad_es<4, false>(p, nd, g.big, st);
    case 8: return launch_pad_es<8, false>(p, nd, g.big, st);
  }
  return NTB200_UNSUPPORTED_DTYPE;
}

int ntb200_pad_nd(const void* ragged, void* padded, const int64_t* offsets, const int64_t* sizes,
                  int64_t size_stride, int nd, int64_t inner, int64_t batch, const int64_t* h_max_sizes,
                  int elem_size, uint64_t pad_bits, void* stream) {
  return pad_common(ragged, padded, nullptr, offsets, sizes, size_stride, nd, inner, batch, h_max_sizes, elem_size, pad_bits,
                    stream);
}

int ntb200_mask_from_sizes(uint8_t* mask, const int64_t* sizes, int64_t size_stride, int nd, int64_t batch,
                           const int64_t* h_max_sizes, void* stream) {
  Geometry g;
  int rc = make_geometry(nd, h_max_sizes, 1, &g);
  if (rc != NTB200_OK) return rc;
  if (batch < 0 || size_stride < nd) return NTB200_INVALID_ARG;
  if (batch == 0 || g.P == 0) return NTB200_OK;
  if (g.P > (uint64_t)INT64_MAX / (uint64_t)batch) return NTB200_INVALID_ARG;
  if (mask == nullptr || sizes == nullptr) return NTB200_INVALID_ARG;
  if (!aligned_to(mask, 16)) return NTB200_MISALIGNED;
  PadParams p;
  p.src = nullptr;
  p.dst = mask;
  p.offsets = nullptr;
  p.sizes = sizes;
  p.size_stride = size_stride;
  p.batch = batch;
  p.P = g.P;
  p.total = batch * (int64_t)g.P;
  for (int j = 0; j < 3; ++j) p.m[j] = g.m[j];
  fill_divs(nd, g, &p.divP, &p.div1, &p.div2);
  p.pad_bits = 0;
  p.inner = 1;
  p.mask = nullptr;
  return launch_pad_es<1, true>(p, nd, g.big, static_cast<cudaStream_t>(stream));
}

int ntb200_pad_with_mask(const void* ragged, void* padded, uint8_t* mask, const int64_t* offsets,
                         const int64_t* sizes, int64_t size_stride, int nd, int64_t inner, int64_t batch,
                         const int64_t* h_max_sizes, int elem_size, const int64_t* mask_sizes,
                         int64_t mask_size_stride, int mask_nd, const int64_t* mask_h_max_sizes, void* stream) {
  // When the mask has the shape of the dense tensor (one byte per output element: images, pad_nt) both are written
  // by ONE kernel in one walk over the output.  A coarser mask (one byte per row of `inner` elements, e.g.
  // (B, max L) beside (B, max L, D) data) is `inner` times smaller than the data and is written by its own launch.
  if (mask == nullptr || mask_nd < 1 || mask_nd > 3 || mask_h_max_sizes == nullptr || h_max_sizes == nullptr || nd < 1 || nd > 3)
    return NTB200_INVALID_ARG;
  bool same_shape = mask_sizes == sizes && mask_size_stride == size_stride;
  if (same_shape) {
    // the mask's dims are the leading tensor dims; it is element-wise when they cover all of them, i.e. when the two
    // padded entry sizes agree and the leading extents coincide
    uint64_t pd = (uint64_t)(inner > 0 ? inner : 0), pm = 1;
    for (int j = 0; j < nd; ++j) pd *= (uint64_t)(h_max_sizes[j] > 0 ? h_max_sizes[j] : 0);
    for (int j = 0; j < mask_nd; ++j) pm *= (uint64_t)(mask_h_max_sizes[j] > 0 ? mask_h_max_sizes[j] : 0);
    same_shape = pd == pm && (inner == 1 ? mask_nd == nd : mask_nd > nd);
    for (int j = 0; same_shape && j < nd && j < mask_nd; ++j) same_shape = mask_h_max_sizes[j] == h_max_sizes[j];
  }
  if (same_shape)
    return pad_common(ragged, padded, mask, offsets, sizes, size_stride, nd, inner, batch, h_max_sizes, elem_size, 0, stream);
  int rc = ntb200_pad_nd(ragged, padded, offsets, sizes, size_stride, nd, inner, batch, h_max_sizes, elem_size, 0,
                         stream);
  if (rc != NTB200_OK) return rc;
  return ntb200_mask_from_sizes(mask, mask_sizes, mask_size_stride, mask_nd, batch, mask_h_max_sizes, stream);
}

int ntb200_unpad_nd(const void* padded, void* ragged, const int64_t* offsets, const int64_t* sizes,
                    int64_t size_stride, int nd, int64_t inner, int64_t batch, const int64_t* h_max_sizes,
                    int64_t total_elems, int elem_size, void* stream) {
  Geometry g;
  int rc = make_geometry(nd, h_max_sizes, inner, &g);
  if (rc != NTB200_OK) return rc;
  if (batch < 0 || size_stride < nd || total_elems < 0) return NTB200_INVALID_ARG;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return NTB200_UNSUPPORTED_DTYPE;
  if (batch == 0 || total_elems == 0) return NTB200_OK;
  if (g.P > (uint64_t)INT64_MAX / (uint64_t)batch) return NTB200_INVALID_ARG;
  if ((uint64_t)total_elems > g.P * (uint64_t)batch) return NTB200_INVALID_ARG;
  if (padded == nullptr || ragged == nullptr || offsets == nullptr || sizes == nullptr) return NTB200_INVALID_ARG;
  if (!aligned_to(ragged, 16)) return NTB200_MISALIGNED;
  if (!aligned_to(padded, (size_t)elem_size)) return NTB200_MISALIGNED;
  UnpadParams p;
  p.src = padded;
  p.dst = ragged;
  p.offsets = offsets;
  p.sizes = sizes;
  p.size_stride = size_stride;
  p.batch = batch;
  p.total = total_elems;
  p.P = g.P;
  for (int j = 0; j < 3; ++j) p.m[j] = g.m[j];
  p.inner = inner;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (long_rows(nd, g, elem_size, kRowUnpad)) {
    RowParams rp;
    rp.src = padded;
    rp.dst = ragged;
    rp.mask = nullptr;
    rp.offsets = offsets;
    rp.sizes = sizes;
    rp.size_stride = size_stride;
    rp.batch = batch;
    rp.m0 = g.m[0];
    rp.m1 = nd == 3 ? g.m[1] : 1;
    rp.rows_per_entry = nd == 3 ? g.m[0] * g.m[1] : g.m[0];
    rp.m_last = g.m[nd - 1];
    rp.inner = inner;
    rp.pad_bits = 0;
    rp.blocks_per_entry = 0;
    switch (elem_size) {
      case 1: return launch_unpad_rows<1>(rp, nd, st);
      case 2: return launch_unpad_rows<2>(rp, nd, st);
      case 4: return launch_unpad_rows<4>(rp, nd, st);
      case 8: return launch_unpad_rows<8>(rp, nd, st);
    }
    return NTB200_UNSUPPORTED_DTYPE;
  }
  switch (elem_size) {
    case 1: return launch_unpad_es<1>(p, nd, st);
    case 2: return launch_unpad_es<2>(p, nd, st);
    case 4: return launch_unpad_es<4>(p, nd, st);
    case 8: return launch_unpad_es<8>(p, nd, st);
  }
  return NTB200_UNSUPPORTED_DTYPE;
}

static int sizes_scan_common(const void* src, int64_t* out_sizes, int64_t* out_counts, int nd, int64_t batch,
                             const int64_t* h_dims, int elem_size, int cmp_kind, uint64_t pad_bits, void* stream) {
  Geometry g;
  int rc = make_geometry(nd, h_dims, 1, &g);
  if (rc != NTB200_OK) return rc;
  if (batch < 0) return NTB200_INVALID_ARG;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return NTB200_UNSUPPORTED_DTYPE;
  if (cmp_kind < 0 || cmp_kind > 2) return NTB200_UNSUPPORTED_DTYPE;
  if (cmp_kind == 2 && elem_size != 2) return NTB200_UNSUPPORTED_DTYPE;
  if (cmp_kind == 1 && elem_size == 1) return NTB200_UNSUPPORTED_DTYPE;
  if (batch == 0) return NTB200_OK;
  if (out_sizes == nullptr || out_counts == nullptr) return NTB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // one clearing launch when the counts follow the sizes in memory (as the operator layer allocates them)
  const bool adjacent = out_counts == out_sizes + batch * nd;
  cudaError_t ce = cudaMemsetAsync(out_sizes, 0, sizeof(int64_t) * (size_t)batch * (adjacent ? nd + 1 : nd), st);
  if (ce != cudaSuccess) return NTB200_LAUNCH_FAILED;
  if (!adjacent) ce = cudaMemsetAsync(out_counts, 0, sizeof(int64_t) * (size_t)batch, st);
  if (ce != cudaSuccess) return NTB200_LAUNCH_FAILED;
  if (g.P == 0) return NTB200_OK;
  if (g.P > (uint64_t)INT64_MAX / (uint64_t)batch) return NTB200_INVALID_ARG;
  if (src == nullptr) return NTB200_INVALID_ARG;
  if (!aligned_to(src, 16)) return NTB200_MISALIGNED;
  ScanParams p;
  p.src = src;
  p.out_sizes = reinterpret_cast<unsigned long long*>(out_sizes);
  p.out_counts = reinterpret_cast<unsigned long long*>(out_counts);
  p.batch = batch;
  p.P = g.P;
  p.total = batch * (int64_t)g.P;
  for (int j = 0; j < 3; ++j) p.m[j] = g.m[j];
  fill_divs(nd, g, &p.divP, &p.div1, &p.div2);
  p.pad_bits = pad_bits;
  if (cmp_kind == 0) {
    switch (elem_size) {
      case 1: return launch_scan_es<1, 0>(p, nd, g.big, st);
      case 2: return launch_scan_es<2, 0>(p, nd, g.big, st);
      case 4: return launch_scan_es<4, 0>(p, nd, g.big, st);
      case 8: return launch_scan_es<8, 0>(p, nd, g.big, st);
    }
  } else if (cmp_kind == 1) {
    switch (elem_size) {
      case 2: return launch_scan_es<2, 1>(p, nd, g.big, st);
      case 4: return launch_scan_es<4, 1>(p, nd, g.big, st);
      case 8: return launch_scan_es<8, 1>(p, nd, g.big, st);
    }
  } else {
    return launch_scan_es<2, 2>(p, nd, g.big, st);
  }
  return NTB200_UNSUPPORTED_DTYPE;
}

int ntb200_sizes_from_padded(const void* padded, int64_t* out_sizes, int64_t* out_counts, int nd, int64_t batch,
                             const int64_t* h_dims, int elem_size, int cmp_kind, uint64_t pad_bits, void* stream) {
  return sizes_scan_common(padded, out_sizes, out_counts, nd, batch, h_dims, elem_size, cmp_kind, pad_bits, stream);
}

int ntb200_sizes_from_mask(const uint8_t* mask, int64_t* out_sizes, int64_t* out_counts, int nd, int64_t batch,
                           const int64_t* h_dims, void* stream) {
  return sizes_scan_common(mask, out_sizes, out_counts, nd, batch, h_dims, 1, 0, 0, stream);
}

size_t ntb200_offsets_workspace_bytes(int64_t batch) {
  if (batch <= kScanThreads) return 0;
  return sizeof(int64_t) * (size_t)ceil_div(batch, kScanThreads);
}

int ntb200_offsets_from_sizes(const int64_t* sizes, int64_t size_stride, int nd, int64_t inner, int64_t batch,
                              int64_t* offsets, void* workspace, size_t workspace_bytes, void* stream) {
  if (batch < 0 || nd < 0 || nd > 8 || size_stride < nd || inner < 0) return NTB200_INVALID_ARG;
  if (offsets == nullptr) return NTB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (batch == 0) {
    return status_from_cuda(cudaMemsetAsync(offsets, 0, sizeof(int64_t), st));
  }
  if (sizes == nullptr && nd > 0) return NTB200_INVALID_ARG;
  const int64_t nblk = ceil_div(batch, kScanThreads);
  if (nblk > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  const size_t need = ntb200_offsets_workspace_bytes(batch);
  if (need > 0) {
    if (workspace == nullptr || workspace_bytes < need) return NTB200_WORKSPACE_TOO_SMALL;
    if (!aligned_to(workspace, 8)) return NTB200_MISALIGNED;
  }
  int64_t* block_sums = static_cast<int64_t*>(workspace);
  offsets_phase1<<<(unsigned)nblk, kScanThreads, 0, st>>>(sizes, size_stride, nd, inner, batch, offsets, block_sums);
  if (nblk > 1) {
    offsets_phase2<<<1, kScanThreads, 0, st>>>(block_sums, nblk, offsets + batch);
    offsets_phase3<<<(unsigned)nblk, kScanThreads, 0, st>>>(offsets, block_sums, batch);
  }
  return status_from_cuda(cudaGetLastError());
}

int64_t ntb200_offsets_static_max_batch(void) { return kStaticScanMaxBatch; }

int ntb200_offsets_from_sizes_static(const int64_t* sizes, int64_t size_stride, int nd, int64_t inner, int64_t batch,
                                     int64_t* offsets, void* stream) {
  if (batch < 0 || nd < 0 || nd > 8 || size_stride < nd || inner < 0) return NTB200_INVALID_ARG;
  if (batch > kStaticScanMaxBatch) return NTB200_STATIC_SCRATCH_EXCEEDED;
  if (offsets == nullptr) return NTB200_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (batch == 0) return status_from_cuda(cudaMemsetAsync(offsets, 0, sizeof(int64_t), st));
  if (sizes == nullptr && nd > 0) return NTB200_INVALID_ARG;
  int64_t* block_sums = nullptr;
  const int rc = static_block_sums_for_current_device(&block_sums);
  if (rc != NTB200_OK) return rc;
  const int64_t nblk = ceil_div(batch, kScanThreads);
  // Every block sum that phase 2 and 3 read is written by phase 1 of this same call, so nothing
  // left in the array by an earlier call can leak into the result and no clearing is needed.
  offsets_phase1<<<(unsigned)nblk, kScanThreads, 0, st>>>(sizes, size_stride, nd, inner, batch, offsets, block_sums);
  if (nblk > 1) {
    offsets_phase2<<<1, kScanThreads, 0, st>>>(block_sums, nblk, offsets + batch);
    offsets_phase3<<<(unsigned)nblk, kScanThreads, 0, st>>>(offsets, block_sums, batch);
  }
  return status_from_cuda(cudaGetLastError());
}

int ntb200_token_index(const int64_t* token_offsets, int64_t batch, int64_t total_tokens, int32_t* batch_idx,
                       int32_t* word_idx, void* stream) {
  if (batch < 0 || total_tokens < 0) return NTB200_INVALID_ARG;
  if (total_tokens == 0) return NTB200_OK;
  if (batch == 0 || token_offsets == nullptr || batch_idx == nullptr || word_idx == nullptr) return NTB200_INVALID_ARG;
  const int64_t blocks = ceil_div(total_tokens, kThreads);
  if (blocks > 0x7fffffffll) return NTB200_UNSUPPORTED_SHAPE;
  token_index_kernel<<<(unsigned)blocks, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      token_offsets, batch, total_tokens, batch_idx, word_idx);
  return status_from_cuda(cudaGetLastError());
}

}  // extern "C"

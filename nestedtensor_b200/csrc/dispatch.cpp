// Torch operator layer of nestedtensor_b200: the `nestedtensor::*` operators of the reference
// (nestedtensor/csrc/masking.cpp:652-675, nestedtensor/csrc/cuda/mha.cpp:109-113) re-implemented
// over a plain record instead of a TensorImpl subclass:
//
//     buffer  1-D CUDA tensor, the constituents concatenated row-major
//     sizes   CPU int64 [B, tensor_dim], one row of extents per constituent
//     meta    CUDA int64 [(B+1) + B*tensor_dim] = element offsets followed by a copy of `sizes`
//
// Every operator validates on the host, allocates its outputs through torch's caching
// allocator and enqueues the sm_100a kernels of libntb200 (C ABI, include/ntb200.h) on the
// CURRENT stream.  There is no CPU implementation: a non-CUDA buffer is an error.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <tuple>
#include <vector>

#include "ntb200.h"

namespace {

using at::Tensor;

void check_rc(int rc, const char* fn) {
  TORCH_CHECK(rc == NTB200_OK, "nestedtensor_b200: ", fn, " failed: ", ntb200_status_string(rc), " (", rc, ")");
}

// NTB200_CHECK_DEVICE_ERRORS=1: after every operator that runs a tcgen05 kernel, wait for the device and raise if one of
// its bounded waits ran out (the affected output tiles would otherwise be returned unwritten).  Off by default: the
// check synchronises.  Callers that leave it off poll nestedtensor_b200.device_error_flags() where it suits them.
void maybe_check_device_errors(const char* op) {
  static const bool enabled = [] {
    const char* v = std::getenv("NTB200_CHECK_DEVICE_ERRORS");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  if (!enabled) return;
  const int flags = ntb200_device_error_flags();
  TORCH_CHECK(flags == 0, "nestedtensor_b200: ", op, ": device error flags 0x", std::hex, flags,
              " (bits 0-2 projection, 8-10 attention: a bounded device-side wait ran out; bit 16: embedding index out of range)");
}

void* cur_stream() { return static_cast<void*>(at::cuda::getCurrentCUDAStream().stream()); }

struct Record {
  int64_t B;
  int64_t tdim;
  const int64_t* sz;  // host sizes, row stride tdim
  const int64_t* d_offsets;
  const int64_t* d_sizes;
  std::vector<int64_t> max_sizes;  // per tensor dim
  std::vector<bool> regular;       // per tensor dim: same extent in every constituent
  bool any_empty;
  int64_t numel;
};

Record make_record(const Tensor& sizes, const Tensor& meta) {
  TORCH_CHECK(sizes.device().is_cpu() && sizes.scalar_type() == at::kLong && sizes.dim() == 2 && sizes.is_contiguous(),
              "nestedtensor_b200: sizes must be a contiguous CPU int64 [B, tensor_dim] tensor");
  Record r;
  r.B = sizes.size(0);
  r.tdim = sizes.size(1);
  r.sz = sizes.data_ptr<int64_t>();
  TORCH_CHECK(meta.is_cuda(),
              "nestedtensor_b200: this operator needs a CUDA nested tensor (this build has no CPU implementation)");
  TORCH_CHECK(meta.scalar_type() == at::kLong && meta.is_contiguous() && meta.numel() == (r.B + 1) + r.B * r.tdim,
              "nestedtensor_b200: meta must be a CUDA int64 tensor of (B+1) + B*tensor_dim entries");
  r.d_offsets = meta.data_ptr<int64_t>();
  r.d_sizes = r.d_offsets + (r.B + 1);
  // One pass over the host sizes per operator call: kept branch-light (batches of 10^5 short sequences make this
  // loop, not the kernel, the cost of a call).
  constexpr int kMaxDims = 8;
  TORCH_CHECK(r.tdim <= kMaxDims, "nestedtensor_b200: at most ", kMaxDims, " tensor dimensions");
  int64_t mx[kMaxDims] = {0}, differs[kMaxDims] = {0}, min_seen = 0, numel = 0, empties = 0;
  const int64_t td = r.tdim;
  const int64_t* __restrict__ sz = r.sz;
  for (int64_t b = 0; b < r.B; ++b) {
    int64_t n = 1;
    for (int64_t j = 0; j < td; ++j) {
      const int64_t v = sz[b * td + j];
      min_seen = v < min_seen ? v : min_seen;
      n *= v;
      mx[j] = v > mx[j] ? v : mx[j];
      differs[j] |= v ^ sz[j];
    }
    empties += n == 0;
    numel += n;
  }
  TORCH_CHECK(min_seen >= 0, "nestedtensor_b200: negative size");
  r.max_sizes.assign(mx, mx + td);
  r.regular.resize(td);
  for (int64_t j = 0; j < td; ++j) r.regular[j] = differs[j] == 0;
  r.any_empty = empties != 0;
  r.numel = numel;
  return r;
}

// Fold trailing regular dims: the kernels see `nd` leading dims and `inner` contiguous elements per
// innermost index.  `dense_dims` (optional) are the dense tensor's trailing extents; a regular
// dim can only be folded when the dense extent equals the common size.
void fold_dims(const Record& r, const int64_t* dense_dims, int* nd, int64_t* inner) {
  int64_t k = r.tdim;
  int64_t in = 1;
  while (k > 1) {
    const int64_t j = k - 1;
    const bool foldable = r.regular[j] && (dense_dims == nullptr || dense_dims[j] == r.max_sizes[j]) && r.max_sizes[j] > 0;
    if (!foldable) break;
    in *= r.max_sizes[j];
    --k;
  }
  TORCH_CHECK(k >= 1 && k <= 3, "nestedtensor_b200: at most 3 leading ragged dimensions are supported, got ", k);
  *nd = (int)k;
  *inner = in;
}

uint64_t scalar_bits(const at::Scalar& value, at::ScalarType dtype, int64_t elem_size) {
  Tensor t = at::full({1}, value, at::TensorOptions().dtype(dtype).device(at::kCPU));
  uint64_t bits = 0;
  std::memcpy(&bits, t.data_ptr(), (size_t)elem_size);
  return bits;
}

void check_buffer(const Tensor& buffer, const Record& r, const char* op) {
  TORCH_CHECK(buffer.is_cuda(), "nestedtensor_b200: ", op,
              " needs a CUDA nested tensor (this build has no CPU implementation)");
  TORCH_CHECK(buffer.dim() == 1 && buffer.is_contiguous() && buffer.numel() == r.numel,
              "nestedtensor_b200: buffer must be 1-D contiguous with sum(numel) elements");
  const int64_t es = buffer.element_size();
  TORCH_CHECK(es == 1 || es == 2 || es == 4 || es == 8, "Input datatype ", buffer.dtype(), " is not supported.");
}

std::vector<int64_t> dense_shape(const Record& r) {
  std::vector<int64_t> shape;
  shape.push_back(r.B);
  for (auto m : r.max_sizes) shape.push_back(m);
  return shape;
}

// ------------------------------------------------------------------ to_padded_tensor
// nestedtensor/csrc/masking.cpp:558-650
Tensor to_padded_tensor(const Tensor& buffer, const Tensor& sizes, const Tensor& meta, double padding) {
  Record r = make_record(sizes, meta);
  if (r.B == 0) return at::scalar_tensor(padding, at::TensorOptions().dtype(at::kDouble)).reshape({1});
  check_buffer(buffer, r, "to_padded_tensor");
  c10::cuda::CUDAGuard guard(buffer.device());
  if (r.tdim == 0) return buffer.clone();  // constituents are scalars: already dense
  Tensor out = at::empty(dense_shape(r), buffer.options());
  if (out.numel() == 0) return out;
  int nd;
  int64_t inner;
  fold_dims(r, nullptr, &nd, &inner);
  const int64_t es = buffer.element_size();
  const uint64_t bits = scalar_bits(at::Scalar(padding), buffer.scalar_type(), es);
  check_rc(ntb200_pad_nd(buffer.data_ptr(), out.data_ptr(), r.d_offsets, r.d_sizes, r.tdim, nd, inner, r.B,
                         r.max_sizes.data(), (int)es, bits, cur_stream()),
           "ntb200_pad_nd");
  return out;
}

// Same operator writing into a caller-provided dense tensor whose extents may exceed the batch maxima
// (slices of one large padded tensor filled batch range by batch range, e.g. by the host-buffer pipeline).
// No counterpart in the reference, whose to_padded_tensor always allocates (masking.cpp:558-650).
Tensor& to_padded_tensor_out(const Tensor& buffer, const Tensor& sizes, const Tensor& meta, double padding, Tensor& out) {
  Record r = make_record(sizes, meta);
  check_buffer(buffer, r, "to_padded_tensor_out");
  TORCH_CHECK(r.B > 0 && r.tdim >= 1, "nestedtensor_b200: to_padded_tensor_out needs a non-empty batch of tensors");
  TORCH_CHECK(out.is_cuda() && out.device() == buffer.device() && out.scalar_type() == buffer.scalar_type() &&
                  out.is_contiguous(),
              "nestedtensor_b200: out must be a contiguous tensor on the input's device and of its dtype");
  TORCH_CHECK(out.dim() == r.tdim + 1 && out.size(0) == r.B, "nestedtensor_b200: out must have shape (batch, extents...)");
  std::vector<int64_t> dense(r.tdim);
  for (int64_t d = 0; d < r.tdim; ++d) {
    dense[d] = out.size(d + 1);
    TORCH_CHECK(dense[d] >= r.max_sizes[d], "nestedtensor_b200: out extent ", dense[d], " of dim ", d + 1,
                " is smaller than the largest constituent (", r.max_sizes[d], ")");
  }
  if (out.numel() == 0) return out;
  c10::cuda::CUDAGuard guard(buffer.device());
  int nd;
  int64_t inner;
  fold_dims(r, dense.data(), &nd, &inner);
  const int64_t es = buffer.element_size();
  const uint64_t bits = scalar_bits(at::Scalar(padding), buffer.scalar_type(), es);
  check_rc(ntb200_pad_nd(buffer.data_ptr(), out.data_ptr(), r.d_offsets, r.d_sizes, r.tdim, nd, inner, r.B, dense.data(),
                         (int)es, bits, cur_stream()),
           "ntb200_pad_nd");
  return out;
}

// Number of mask dims left after the reference's collapse rule (merge_tensor_mask,
// nestedtensor/csrc/masking.cpp:12-43), derived from the sizes alone: a trailing mask dim can be
// dropped iff that tensor dim is regular (every slice is then all-1 or all-0); the batch dim can
// be dropped because no constituent is empty.  Sets *collapsed when at least one dim was dropped.
int64_t resolve_mask_dim(const Record& r, c10::optional<int64_t> mask_dim, bool* collapsed) {
  int64_t md = r.tdim + 1;
  *collapsed = false;
  while (true) {
    if (mask_dim && md == *mask_dim) break;
    if (md == 0) break;
    const bool can = (md == 1) ? true : r.regular[md - 2];
    if (can) {
      --md;
      *collapsed = true;
      continue;
    }
    if (mask_dim && *mask_dim != md) {
      TORCH_CHECK(false, "Mask dimension is too small to represent data tensor.");
    }
    break;
  }
  return md;
}

Tensor alloc_mask(const Record& r, int64_t md, bool as_bool, const at::Device& dev) {
  std::vector<int64_t> shape;
  if (md >= 1) shape.push_back(r.B);
  for (int64_t j = 0; j + 1 < md; ++j) shape.push_back(r.max_sizes[j]);
  return at::empty(shape, at::TensorOptions().dtype(as_bool ? at::kBool : at::kByte).device(dev));
}

void check_mask_dim_arg(c10::optional<int64_t> mask_dim, int64_t dim) {
  TORCH_CHECK(!mask_dim || *mask_dim <= dim, "Requested mask dimension ", *mask_dim, " is bigger than dimension ", dim,
              " of given NestedTensor.");
}

// ------------------------------------------------------------------ to_tensor_mask
// nestedtensor/csrc/masking.cpp:251-320
std::tuple<Tensor, Tensor> to_tensor_mask(const Tensor& buffer, const Tensor& sizes, const Tensor& meta,
                                          c10::optional<int64_t> mask_dim) {
  Record r = make_record(sizes, meta);
  check_mask_dim_arg(mask_dim, r.tdim + 1);
  if (r.B == 0) {
    // masking.cpp:152-155 then the collapse of a one-element all-false mask
    Tensor t = at::zeros({1}, at::TensorOptions().dtype(at::kLong));
    if (mask_dim && *mask_dim == 1) return std::make_tuple(t, at::zeros({1}, at::TensorOptions().dtype(at::kByte)));
    return std::make_tuple(t, at::zeros({}, at::TensorOptions().dtype(at::kBool)));
  }
  check_buffer(buffer, r, "to_tensor_mask");
  c10::cuda::CUDAGuard guard(buffer.device());
  if (r.tdim == 0 && r.B == 1) {
    // masking.cpp:305-313
    Tensor m = (!mask_dim || *mask_dim == 0) ? at::ones({}, at::TensorOptions().dtype(at::kBool))
                                             : at::ones({1}, at::TensorOptions().dtype(at::kBool));
    return std::make_tuple(buffer.reshape({-1}), m);
  }
  TORCH_CHECK(!r.any_empty, "Empty tensors are not yet supported.");
  bool collapsed;
  const int64_t md = resolve_mask_dim(r, mask_dim, &collapsed);
  const bool as_bool = collapsed || r.tdim == 0;
  Tensor mask = alloc_mask(r, md, as_bool, buffer.device());
  if (r.tdim == 0) {
    mask.fill_(true);
    return std::make_tuple(buffer.clone(), mask);
  }
  Tensor out = at::empty(dense_shape(r), buffer.options());
  int nd;
  int64_t inner;
  fold_dims(r, nullptr, &nd, &inner);
  const int64_t es = buffer.element_size();
  if (md >= 2) {
    const int mask_nd = (int)(md - 1);
    TORCH_CHECK(mask_nd <= 3, "nestedtensor_b200: masks over more than 3 ragged dimensions are not supported");
    check_rc(ntb200_pad_with_mask(buffer.data_ptr(), out.data_ptr(), static_cast<uint8_t*>(mask.data_ptr()),
                                  r.d_offsets, r.d_sizes, r.tdim, nd, inner, r.B, r.max_sizes.data(), (int)es,
                                  r.d_sizes, r.tdim, mask_nd, r.max_sizes.data(), cur_stream()),
             "ntb200_pad_with_mask");
  } else {
    check_rc(ntb200_pad_nd(buffer.data_ptr(), out.data_ptr(), r.d_offsets, r.d_sizes, r.tdim, nd, inner, r.B,
                           r.max_sizes.data(), (int)es, 0, cur_stream()),
             "ntb200_pad_nd");
    mask.fill_(true);  // (B,) or scalar: every constituent is non-empty
  }
  return std::make_tuple(out, mask);
}

// ------------------------------------------------------------------ get_max_size / pad_nt
// nestedtensor/csrc/masking.cpp:83-108: per-dimension maximum of the constituent sizes
std::vector<int64_t> get_max_size(const Tensor& sizes) {
  TORCH_CHECK(sizes.device().is_cpu() && sizes.scalar_type() == at::kLong && sizes.dim() == 2 && sizes.is_contiguous(),
              "nestedtensor_b200: sizes must be a contiguous CPU int64 [B, tensor_dim] tensor");
  std::vector<int64_t> mx(sizes.size(1), 0);
  const int64_t* p = sizes.data_ptr<int64_t>();
  for (int64_t b = 0; b < sizes.size(0); ++b)
    for (int64_t j = 0; j < sizes.size(1); ++j) mx[j] = std::max(mx[j], p[b * sizes.size(1) + j]);
  return mx;
}

// nestedtensor/csrc/masking.cpp:138-179: every constituent zero-padded to `shape` and stacked, with the uint8
// mask of the same shape (1 inside a constituent).  One kernel writes data and mask in a single pass over the output
// (ntb200_pad_with_mask, same-shape case) instead of a pad + stack per constituent.
std::tuple<Tensor, Tensor> pad_nt(const Tensor& buffer, const Tensor& sizes, const Tensor& meta, at::IntArrayRef shape) {
  Record r = make_record(sizes, meta);
  if (r.B == 0)  // masking.cpp:164-166
    return std::make_tuple(at::zeros({1}, at::TensorOptions().dtype(at::kLong)), at::zeros({1}, at::TensorOptions().dtype(at::kByte)));
  check_buffer(buffer, r, "pad_nt");
  TORCH_CHECK(!r.any_empty, "Empty tensors are not yet supported.");
  TORCH_CHECK((int64_t)shape.size() == r.tdim, "nestedtensor_b200: pad_nt needs one extent per tensor dimension");
  TORCH_CHECK(r.tdim >= 1 && r.tdim <= 3, "nestedtensor_b200: pad_nt supports 1 to 3 tensor dimensions");
  std::vector<int64_t> dense(shape.begin(), shape.end()), full{r.B};
  for (int64_t d = 0; d < r.tdim; ++d) {
    TORCH_CHECK(dense[d] >= r.max_sizes[d], "nestedtensor_b200: pad_nt shape ", dense[d], " of dim ", d,
                " is smaller than the largest constituent (", r.max_sizes[d], ")");
    full.push_back(dense[d]);
  }
  c10::cuda::CUDAGuard guard(buffer.device());
  Tensor out = at::empty(full, buffer.options());
  Tensor mask = at::empty(full, buffer.options().dtype(at::kByte));
  if (out.numel() == 0) return std::make_tuple(out, mask);
  int nd;
  int64_t inner;
  fold_dims(r, dense.data(), &nd, &inner);
  check_rc(ntb200_pad_with_mask(buffer.data_ptr(), out.data_ptr(), static_cast<uint8_t*>(mask.data_ptr()), r.d_offsets,
                                r.d_sizes, r.tdim, nd, inner, r.B, dense.data(), (int)buffer.element_size(), r.d_sizes,
                                r.tdim, (int)r.tdim, dense.data(), cur_stream()),
           "ntb200_pad_with_mask");
  return std::make_tuple(out, mask);
}

// ------------------------------------------------------------------ to_mask
// nestedtensor/csrc/masking.cpp:408-457.  The reference builds this mask on the host; here it is
// written on the device that holds the nested tensor.
Tensor to_mask(const Tensor& sizes, const Tensor& meta, c10::optional<int64_t> mask_dim) {
  Record r = make_record(sizes, meta);
  const int64_t dim = r.tdim + 1;
  check_mask_dim_arg(mask_dim, dim);
  c10::cuda::CUDAGuard guard(meta.device());
  if (r.tdim == 0 && r.B == 1) {
    return (!mask_dim || *mask_dim == 0) ? at::ones({}, at::TensorOptions().dtype(at::kBool))
                                         : at::ones({1}, at::TensorOptions().dtype(at::kBool));
  }
  if (dim > 1 && mask_dim && *mask_dim > 1) {
    // leading (mask_dim-1) tensor dims, no collapse (masking.cpp:426-453)
    const int mask_nd = (int)(*mask_dim - 1);
    if (!(*mask_dim == 2 && dim == 3)) {
      for (int64_t b = 0; b < r.B; ++b) {
        int64_t n = 1;
        for (int j = 0; j < mask_nd; ++j) n *= r.sz[b * r.tdim + j];
        TORCH_CHECK(n > 0, "Empty tensors are not yet supported.");
      }
    }
    TORCH_CHECK(mask_nd <= 3, "nestedtensor_b200: masks over more than 3 ragged dimensions are not supported");
    Tensor mask = alloc_mask(r, *mask_dim, false, meta.device());
    if (mask.numel() > 0)
      check_rc(ntb200_mask_from_sizes(static_cast<uint8_t*>(mask.data_ptr()), r.d_sizes, r.tdim, mask_nd, r.B,
                                      r.max_sizes.data(), cur_stream()),
               "ntb200_mask_from_sizes");
    return mask;
  }
  if (r.B == 0) {
    if (mask_dim && *mask_dim == 1) return at::zeros({1}, at::TensorOptions().dtype(at::kByte));
    return at::zeros({}, at::TensorOptions().dtype(at::kBool));
  }
  TORCH_CHECK(!r.any_empty, "Empty tensors are not yet supported.");
  bool collapsed;
  const int64_t md = resolve_mask_dim(r, mask_dim, &collapsed);
  Tensor mask = alloc_mask(r, md, collapsed || r.tdim == 0, meta.device());
  if (md >= 2) {
    TORCH_CHECK(md - 1 <= 3, "nestedtensor_b200: masks over more than 3 ragged dimensions are not supported");
    check_rc(ntb200_mask_from_sizes(static_cast<uint8_t*>(mask.data_ptr()), r.d_sizes, r.tdim, (int)(md - 1), r.B,
                                    r.max_sizes.data(), cur_stream()),
             "ntb200_mask_from_sizes");
  } else {
    mask.fill_(true);
  }
  return mask;
}

// ------------------------------------------------------------------ from_padded_tensor
// nestedtensor/csrc/masking.cpp:459-533 — returns the ragged buffer for the given target sizes.
Tensor from_padded_tensor(const Tensor& padded_, const Tensor& sizes, const Tensor& meta) {
  Record r = make_record(sizes, meta);
  TORCH_CHECK(padded_.dim() == r.tdim + 1, "Target size has different dimension as input padded Tensor.");
  TORCH_CHECK(padded_.is_cuda(), "nestedtensor_b200: from_padded_tensor needs a CUDA tensor (this build has no CPU implementation)");
  TORCH_CHECK(padded_.size(0) == r.B, "nestedtensor_b200: padded.size(0) differs from the number of target sizes");
  c10::cuda::CUDAGuard guard(padded_.device());
  Tensor padded = padded_.contiguous();
  const int64_t es = padded.element_size();
  TORCH_CHECK(es == 1 || es == 2 || es == 4 || es == 8, "Input datatype ", padded.dtype(), " is not supported.");
  Tensor out = at::empty({r.numel}, padded.options());
  if (r.numel == 0) return out;
  if (r.tdim == 0) {
    out.copy_(padded.reshape({-1}));
    return out;
  }
  std::vector<int64_t> dims(padded.sizes().begin() + 1, padded.sizes().end());
  for (int64_t j = 0; j < r.tdim; ++j)
    TORCH_CHECK(r.max_sizes[j] <= dims[j], "nestedtensor_b200: target size exceeds the padded tensor along dim ", j + 1);
  int nd;
  int64_t inner;
  fold_dims(r, dims.data(), &nd, &inner);
  check_rc(ntb200_unpad_nd(padded.data_ptr(), out.data_ptr(), r.d_offsets, r.d_sizes, r.tdim, nd, inner, r.B,
                           dims.data(), r.numel, (int)es, cur_stream()),
           "ntb200_unpad_nd");
  return out;
}

// ------------------------------------------------------------------ sizes from dense data
int cmp_kind_of(at::ScalarType t) {
  switch (t) {
    case at::kHalf: return 1;
    case at::kFloat: return 1;
    case at::kDouble: return 1;
    case at::kBFloat16: return 2;
    default: return 0;
  }
}

// (sizes [B, nd], counts [B]) on the device for `tensor != padding`
// (nestedtensor/nested/masking.py:12-14 without materialising the mask).
std::tuple<Tensor, Tensor> sizes_from_padded(const Tensor& tensor_, const at::Scalar& padding) {
  TORCH_CHECK(tensor_.is_cuda(), "nestedtensor_b200: sizes_from_padded needs a CUDA tensor (this build has no CPU implementation)");
  TORCH_CHECK(tensor_.dim() >= 2 && tensor_.dim() <= 4, "nestedtensor_b200: sizes_from_padded supports 2 to 4 dimensional tensors");
  c10::cuda::CUDAGuard guard(tensor_.device());
  Tensor tensor = tensor_.contiguous();
  const int64_t B = tensor.size(0);
  const int nd = (int)tensor.dim() - 1;
  const int64_t es = tensor.element_size();
  TORCH_CHECK(es == 1 || es == 2 || es == 4 || es == 8, "Input datatype ", tensor.dtype(), " is not supported.");
  std::vector<int64_t> dims(tensor.sizes().begin() + 1, tensor.sizes().end());
  auto opt = at::TensorOptions().dtype(at::kLong).device(tensor.device());
  Tensor scan_out = at::empty({B * (nd + 1)}, opt);  // sizes, then counts: the library clears both with one launch
  Tensor out_sizes = scan_out.narrow(0, 0, B * nd).view({B, nd});
  Tensor out_counts = scan_out.narrow(0, B * nd, B);
  // A padding value the dtype cannot hold exactly equals no element: everything is valid.
  const int kind = cmp_kind_of(tensor.scalar_type());
  bool representable = true;
  if (kind == 0) {
    if (padding.isFloatingPoint()) {
      const double v = padding.toDouble();
      representable = (v == (double)(int64_t)v);
    }
    if (representable) {
      Tensor probe = at::full({1}, padding, at::TensorOptions().dtype(tensor.scalar_type()));
      representable = probe.to(at::kDouble).item<double>() == padding.toDouble();
    }
  }
  if (!representable) {
    Tensor full = at::tensor(dims, at::TensorOptions().dtype(at::kLong)).to(tensor.device());
    out_sizes.copy_(full.unsqueeze(0).expand({B, nd}));
    int64_t P = 1;
    for (auto d : dims) P *= d;
    out_counts.fill_(P);
    return std::make_tuple(out_sizes, out_counts);
  }
  const uint64_t bits = scalar_bits(padding, tensor.scalar_type(), es);
  check_rc(ntb200_sizes_from_padded(tensor.data_ptr(), out_sizes.data_ptr<int64_t>(), out_counts.data_ptr<int64_t>(),
                                    nd, B, dims.data(), (int)es, kind, bits, cur_stream()),
           "ntb200_sizes_from_padded");
  return std::make_tuple(out_sizes, out_counts);
}

std::tuple<Tensor, Tensor> sizes_from_mask(const Tensor& mask_) {
  TORCH_CHECK(mask_.is_cuda(), "nestedtensor_b200: sizes_from_mask needs a CUDA tensor (this build has no CPU implementation)");
  TORCH_CHECK(mask_.dim() >= 2 && mask_.dim() <= 4, "nestedtensor_b200: sizes_from_mask supports 2 to 4 dimensional masks");
  TORCH_CHECK(mask_.scalar_type() == at::kBool || mask_.scalar_type() == at::kByte,
              "nestedtensor_b200: mask must be bool or uint8");
  c10::cuda::CUDAGuard guard(mask_.device());
  Tensor mask = mask_.contiguous();
  const int64_t B = mask.size(0);
  const int nd = (int)mask.dim() - 1;
  std::vector<int64_t> dims(mask.sizes().begin() + 1, mask.sizes().end());
  auto opt = at::TensorOptions().dtype(at::kLong).device(mask.device());
  Tensor scan_out = at::empty({B * (nd + 1)}, opt);  // sizes, then counts: the library clears both with one launch
  Tensor out_sizes = scan_out.narrow(0, 0, B * nd).view({B, nd});
  Tensor out_counts = scan_out.narrow(0, B * nd, B);
  check_rc(ntb200_sizes_from_mask(static_cast<const uint8_t*>(mask.data_ptr()), out_sizes.data_ptr<int64_t>(),
                                  out_counts.data_ptr<int64_t>(), nd, B, dims.data(), cur_stream()),
           "ntb200_sizes_from_mask");
  return std::make_tuple(out_sizes, out_counts);
}

// ------------------------------------------------------------------ merge_tensor_mask
// nestedtensor/csrc/masking.cpp:12-43: trailing mask dimensions whose slices are all-0 or all-1 are dropped until
// `mask_dim` is reached (or, with no `mask_dim`, as far as possible).  A plain-tensor operator on either device; one
// host read per level instead of the reference's two.
std::tuple<Tensor, Tensor> merge_tensor_mask(const Tensor& tensor, const Tensor& mask_, c10::optional<int64_t> mask_dim) {
  Tensor mask = mask_;
  while (true) {
    if (mask_dim && mask.dim() == *mask_dim) return std::make_tuple(tensor, mask);
    if (mask.dim() == 0) return std::make_tuple(tensor, mask);
    const int64_t last = mask.size(-1);
    Tensor collapsed = mask.sum(-1);
    const bool uniform = at::logical_or(collapsed == last, collapsed == 0).all().item<bool>();
    if (!uniform) break;
    mask = collapsed.to(at::kBool);
  }
  TORCH_CHECK(!(mask_dim && *mask_dim != mask.dim()), "Mask dimension is too small to represent data tensor.");
  return std::make_tuple(tensor.contiguous(), mask.contiguous());
}

// ------------------------------------------------------------------ nt_from_tensor_mask
// nestedtensor/csrc/masking.cpp:181-249 for nested_dim 1.  The reference walks the mask on the host with one .item()
// per element and returns a NestedTensor; here one kernel recovers every entry's extents from the mask, the host checks
// that they describe a padding mask (every entry keeps a leading box), the unpad kernel gathers the data, and the
// result is the record (buffer, sizes, meta) that the Python class wraps.
std::tuple<Tensor, Tensor, Tensor> record_from_extents(const Tensor& tensor, const Tensor& sizes_dev, const Tensor& counts_dev,
                                                       int64_t lead_dims);

std::tuple<Tensor, Tensor, Tensor> whole_entries(const Tensor& src) {
  const int64_t B = src.size(0), tdim = src.dim() - 1;
  Tensor sizes = at::empty({B, tdim}, at::TensorOptions().dtype(at::kLong));
  int64_t* p = sizes.data_ptr<int64_t>();
  for (int64_t b = 0; b < B; ++b)
    for (int64_t j = 0; j < tdim; ++j) p[b * tdim + j] = src.size(j + 1);
  int64_t per = 1;
  for (int64_t j = 0; j < tdim; ++j) per *= src.size(j + 1);
  Tensor meta_h = at::empty({(B + 1) + B * tdim}, at::TensorOptions().dtype(at::kLong));
  int64_t* m = meta_h.data_ptr<int64_t>();
  for (int64_t b = 0; b <= B; ++b) m[b] = b * per;
  for (int64_t i = 0; i < B * tdim; ++i) m[B + 1 + i] = p[i];
  return std::make_tuple(src.reshape({-1}).clone(), sizes, meta_h.to(src.device()));
}

std::tuple<Tensor, Tensor, Tensor> nt_from_tensor_mask(const Tensor& tensor, const Tensor& mask_, int64_t nested_dim) {
  TORCH_CHECK(nested_dim == 1, "Only nested_dim of 1 is currently supported.");
  TORCH_CHECK(tensor.dim() >= 1, "Can't construct nested tensor from a scalar.");
  if (tensor.numel() == 0) {
    if (tensor.dim() > 1) return whole_entries(tensor);
    return std::make_tuple(tensor.reshape({-1}).clone(), at::zeros({0, 0}, at::TensorOptions().dtype(at::kLong)),
                           at::zeros({1}, at::TensorOptions().dtype(at::kLong).device(tensor.device())));
  }
  TORCH_CHECK(tensor.is_cuda(), "nestedtensor_b200: nested_tensor_from_tensor_mask needs a CUDA tensor (this build has no CPU implementation)");
  c10::cuda::CUDAGuard guard(tensor.device());
  if (mask_.numel() == 1) {
    if (mask_.reshape({-1}).to(at::kBool).item<bool>()) return whole_entries(tensor);
    return std::make_tuple(at::empty({0}, tensor.options()), at::zeros({0, 0}, at::TensorOptions().dtype(at::kLong)),
                           at::zeros({1}, at::TensorOptions().dtype(at::kLong).device(tensor.device())));
  }
  bool prefix = mask_.dim() <= tensor.dim();
  for (int64_t j = 0; prefix && j < mask_.dim(); ++j) prefix = mask_.size(j) == tensor.size(j);
  TORCH_CHECK(prefix, "nestedtensor_b200: mask shape ", mask_.sizes(), " must equal the leading dimensions of the tensor shape ",
              tensor.sizes());
  Tensor mask = mask_.to(tensor.device());
  if (mask.scalar_type() != at::kBool && mask.scalar_type() != at::kByte) mask = mask != 0;
  if (mask.dim() == 1)  // one flag per entry: entries are kept or dropped whole (masking.cpp:185-201)
    return whole_entries(tensor.index({mask.to(at::kBool)}));
  auto ext = sizes_from_mask(mask);
  return record_from_extents(tensor, std::get<0>(ext), std::get<1>(ext), mask.dim() - 1);
}

// Host validation of device-computed extents, then the gather: an entry must keep exactly its leading box.
std::tuple<Tensor, Tensor, Tensor> record_from_extents(const Tensor& tensor, const Tensor& sizes_dev, const Tensor& counts_dev,
                                                       int64_t lead_dims) {
  const int64_t B = tensor.size(0);
  Tensor both = at::cat({sizes_dev, counts_dev.unsqueeze(1)}, 1).cpu();  // the one synchronising copy
  const int64_t* q = both.data_ptr<int64_t>();
  const int64_t trail = tensor.dim() - 1 - lead_dims, tdim = lead_dims + trail;
  Tensor sizes = at::empty({B, tdim}, at::TensorOptions().dtype(at::kLong));
  int64_t* p = sizes.data_ptr<int64_t>();
  for (int64_t b = 0; b < B; ++b) {
    int64_t box = 1;
    for (int64_t j = 0; j < lead_dims; ++j) box *= q[b * (lead_dims + 1) + j];
    const int64_t count = q[b * (lead_dims + 1) + lead_dims];
    TORCH_CHECK(count == box, "nestedtensor_b200: entry ", b, " of the mask is not a padding mask (", count,
                " valid elements do not fill its leading box); only masks that keep a leading box of every entry are supported");
    for (int64_t j = 0; j < lead_dims; ++j) p[b * tdim + j] = q[b * (lead_dims + 1) + j];
    for (int64_t j = 0; j < trail; ++j) p[b * tdim + lead_dims + j] = tensor.size(1 + lead_dims + j);
    if (count == 0) {
      // an all-false entry keeps its outer extents and gets an empty innermost one (masking.cpp:203-216)
      for (int64_t j = 0; j + 1 < lead_dims; ++j) p[b * tdim + j] = tensor.size(1 + j);
      p[b * tdim + lead_dims - 1] = 0;
    }
  }
  Tensor meta_h = at::empty({(B + 1) + B * tdim}, at::TensorOptions().dtype(at::kLong).pinned_memory(true));
  int64_t* m = meta_h.data_ptr<int64_t>();
  m[0] = 0;
  for (int64_t b = 0; b < B; ++b) {
    int64_t n = 1;
    for (int64_t j = 0; j < tdim; ++j) n *= p[b * tdim + j];
    m[b + 1] = m[b] + n;
  }
  for (int64_t i = 0; i < B * tdim; ++i) m[B + 1 + i] = p[i];
  Tensor meta = meta_h.to(tensor.device(), /*non_blocking=*/true);
  Tensor buffer = from_padded_tensor(tensor, sizes, meta);
  return std::make_tuple(buffer, sizes, meta);
}

// ------------------------------------------------------------------ metadata on the device
// meta = [offsets (B+1) | sizes (B*tdim)] from device-resident sizes
// (device-side batch_offsets_from_efficient_size, nestedtensor/csrc/masking.cpp:110-125).
Tensor meta_from_device_sizes(const Tensor& d_sizes) {
  TORCH_CHECK(d_sizes.is_cuda() && d_sizes.scalar_type() == at::kLong && d_sizes.dim() == 2 && d_sizes.is_contiguous(),
              "nestedtensor_b200: device sizes must be a contiguous CUDA int64 [B, tensor_dim] tensor");
  c10::cuda::CUDAGuard guard(d_sizes.device());
  const int64_t B = d_sizes.size(0), tdim = d_sizes.size(1);
  Tensor meta = at::empty({(B + 1) + B * tdim}, d_sizes.options());
  const size_t ws_bytes = ntb200_offsets_workspace_bytes(B);
  Tensor ws = at::empty({(int64_t)((ws_bytes + 7) / 8)}, d_sizes.options());
  check_rc(ntb200_offsets_from_sizes(d_sizes.data_ptr<int64_t>(), tdim, (int)tdim, 1, B, meta.data_ptr<int64_t>(),
                                     ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, cur_stream()),
           "ntb200_offsets_from_sizes");
  if (B * tdim > 0) meta.narrow(0, B + 1, B * tdim).copy_(d_sizes.reshape({-1}));
  return meta;
}

// batch_idx / word_idx of every token (compress_bert_input, nestedtensor/csrc/cuda/cuda_kernels.cu:171-223)
std::tuple<Tensor, Tensor> token_index(const Tensor& token_offsets, int64_t total_tokens) {
  TORCH_CHECK(token_offsets.is_cuda() && token_offsets.scalar_type() == at::kLong && token_offsets.is_contiguous() &&
                  token_offsets.dim() == 1 && token_offsets.numel() >= 1,
              "nestedtensor_b200: token_offsets must be a contiguous CUDA int64 [B+1] tensor");
  c10::cuda::CUDAGuard guard(token_offsets.device());
  auto opt = at::TensorOptions().dtype(at::kInt).device(token_offsets.device());
  Tensor bi = at::empty({total_tokens}, opt), wi = at::empty({total_tokens}, opt);
  check_rc(ntb200_token_index(token_offsets.data_ptr<int64_t>(), token_offsets.numel() - 1, total_tokens,
                              bi.data_ptr<int32_t>(), wi.data_ptr<int32_t>(), cur_stream()),
           "ntb200_token_index");
  return std::make_tuple(bi, wi);
}

// ------------------------------------------------------------------ self-attention
int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return NTB200_F32;
    case at::kHalf: return NTB200_F16;
    case at::kBFloat16: return NTB200_BF16;
    default: TORCH_CHECK(false, "nestedtensor_b200: this operator supports float32, float16 and bfloat16, got ", t);
  }
}

// bt_min_mha (nestedtensor/csrc/cuda/mha.cpp:22-107) on the packed token buffer:
//   qkv = x W_in^T + b_in   ->  varlen softmax(scaling * q k^T) v per sequence and head  ->  out W_out^T + b_out
// Dropout arguments are accepted and ignored exactly as in the reference (inference path).  Unlike the
// reference (mha.cpp:106) the output projection bias IS added, as in min_mha (nestedtensor/csrc/mha.cpp:66-67).
// QKV projection and the varlen attention core: returns the [T, E] context (before the output projection).
Tensor bt_min_mha_core(int64_t num_heads, int64_t head_dim, const Tensor& buffer, const Tensor& sizes, const Tensor& meta,
                       const Tensor& attr_kernel, const Tensor& attr_bias, double scaling) {
  Record r = make_record(sizes, meta);
  TORCH_CHECK(r.tdim == 2, "query needs to be 3 dim.");
  check_buffer(buffer, r, "bt_min_mha");
  const int64_t E = num_heads * head_dim;
  TORCH_CHECK(r.B == 0 || (r.regular[1] && r.max_sizes[1] == E), "query's third dimension must be regular.");
  TORCH_CHECK(num_heads >= 1 && head_dim >= 1 && head_dim <= 256, "nestedtensor_b200: head_dim must be in [1, 256]");
  const int dt = dtype_code(buffer.scalar_type());
  auto same = [&](const Tensor& w, const char* name) {
    TORCH_CHECK(w.is_cuda() && w.device() == buffer.device() && w.scalar_type() == buffer.scalar_type(),
                "nestedtensor_b200: ", name, " must be on the input's device and of its dtype");
  };
  same(attr_kernel, "in_proj_weight");
  same(attr_bias, "in_proj_bias");
  TORCH_CHECK(attr_kernel.dim() == 2 && attr_kernel.size(0) == 3 * E && attr_kernel.size(1) == E, "in_proj_weight must be [3E, E]");
  TORCH_CHECK(attr_bias.numel() == 3 * E, "in_proj_bias must have 3E entries");
  c10::cuda::CUDAGuard guard(buffer.device());
  const int64_t T = r.numel / (E > 0 ? E : 1);
  Tensor attn = at::empty({T, E}, buffer.options());
  if (T == 0) return attn;
  Tensor w_in = attr_kernel.contiguous(), b_in = attr_bias.contiguous();
  Tensor qkv = at::empty({T, 3 * E}, buffer.options());
  void* st = cur_stream();
  check_rc(ntb200_gemm_bias(buffer.data_ptr(), w_in.data_ptr(), b_in.data_ptr(), qkv.data_ptr(), T, 3 * E, E, dt, 0, st),
           "ntb200_gemm_bias");
  const size_t ws_bytes = ntb200_varlen_attention_workspace_bytes(r.B, T, (int)num_heads, (int)head_dim, dt);
  Tensor ws;
  if (ws_bytes > 0) ws = at::empty({(int64_t)ws_bytes}, buffer.options().dtype(at::kByte));
  check_rc(ntb200_varlen_attention(qkv.data_ptr(), attn.data_ptr(), r.d_offsets, r.B, T, (int)num_heads, (int)head_dim,
                                   r.max_sizes[0], (float)scaling, dt, 0, ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, st),
           "ntb200_varlen_attention");
  return attn;
}

Tensor bt_min_mha(int64_t num_heads, int64_t head_dim, double /*dropout_p*/, bool /*training*/, const Tensor& buffer,
                  const Tensor& sizes, const Tensor& meta, const Tensor& attr_kernel, const Tensor& attr_bias,
                  double scaling, const Tensor& out_proj_weight, const c10::optional<Tensor>& out_proj_bias) {
  const int64_t E = num_heads * head_dim;
  TORCH_CHECK(out_proj_weight.is_cuda() && out_proj_weight.device() == buffer.device() &&
                  out_proj_weight.scalar_type() == buffer.scalar_type(),
              "nestedtensor_b200: out_proj_weight must be on the input's device and of its dtype");
  TORCH_CHECK(out_proj_weight.dim() == 2 && out_proj_weight.size(0) == E && out_proj_weight.size(1) == E, "out_proj_weight must be [E, E]");
  Tensor attn = bt_min_mha_core(num_heads, head_dim, buffer, sizes, meta, attr_kernel, attr_bias, scaling);
  const int64_t T = attn.size(0);
  c10::cuda::CUDAGuard guard(buffer.device());
  Tensor out = at::empty({T * E}, buffer.options());
  if (T == 0) return out;
  Tensor w_out = out_proj_weight.contiguous();
  const void* b_out = nullptr;
  Tensor b_out_t;
  if (out_proj_bias && out_proj_bias->defined()) {
    TORCH_CHECK(out_proj_bias->is_cuda() && out_proj_bias->device() == buffer.device() &&
                    out_proj_bias->scalar_type() == buffer.scalar_type(),
                "nestedtensor_b200: out_proj_bias must be on the input's device and of its dtype");
    TORCH_CHECK(out_proj_bias->numel() == E, "out_proj_bias must have E entries");
    b_out_t = out_proj_bias->contiguous();
    b_out = b_out_t.data_ptr();
  }
  check_rc(ntb200_gemm_bias(attn.data_ptr(), w_out.data_ptr(), b_out, out.data_ptr(), T, E, E, dtype_code(buffer.scalar_type()), 0,
                            cur_stream()),
           "ntb200_gemm_bias");
  maybe_check_device_errors("bt_min_mha");
  return out;
}

// min_mha (nestedtensor/csrc/mha.cpp:18-69) for query != key: q, k and v are projected from three nested
// tensors with the three thirds of in_proj (k and v in one GEMM when key and value are the same tensor), the
// queries of sequence b attend over the keys of sequence b, then the output projection.
Tensor min_mha_cross(int64_t num_heads, int64_t head_dim, const Tensor& q_buffer, const Tensor& q_sizes, const Tensor& q_meta,
                     const Tensor& k_buffer, const Tensor& k_sizes, const Tensor& k_meta, const Tensor& v_buffer,
                     const Tensor& attr_kernel, const Tensor& attr_bias, double scaling, const Tensor& out_proj_weight,
                     const c10::optional<Tensor>& out_proj_bias) {
  Record rq = make_record(q_sizes, q_meta), rk = make_record(k_sizes, k_meta);
  TORCH_CHECK(rq.tdim == 2, "query needs to be 3 dim.");
  TORCH_CHECK(rk.tdim == 2, "key needs to be 3 dim.");
  TORCH_CHECK(rq.B == rk.B, "nestedtensor_b200: query and key must hold the same number of sequences");
  check_buffer(q_buffer, rq, "min_mha");
  check_buffer(k_buffer, rk, "min_mha");
  check_buffer(v_buffer, rk, "min_mha");
  const int64_t E = num_heads * head_dim;
  TORCH_CHECK(rq.B == 0 || (rq.regular[1] && rq.max_sizes[1] == E), "query's third dimension must be regular.");
  TORCH_CHECK(rk.B == 0 || (rk.regular[1] && rk.max_sizes[1] == E), "key's third dimension must be regular.");
  TORCH_CHECK(num_heads >= 1 && head_dim >= 1 && head_dim <= 256, "nestedtensor_b200: head_dim must be in [1, 256]");
  const int dt = dtype_code(q_buffer.scalar_type());
  auto same = [&](const Tensor& w, const char* name) {
    TORCH_CHECK(w.is_cuda() && w.device() == q_buffer.device() && w.scalar_type() == q_buffer.scalar_type(),
                "nestedtensor_b200: ", name, " must be on the query's device and of its dtype");
  };
  same(k_buffer, "key");
  same(v_buffer, "value");
  same(attr_kernel, "in_proj_weight");
  same(attr_bias, "in_proj_bias");
  same(out_proj_weight, "out_proj_weight");
  TORCH_CHECK(attr_kernel.dim() == 2 && attr_kernel.size(0) == 3 * E && attr_kernel.size(1) == E, "in_proj_weight must be [3E, E]");
  TORCH_CHECK(attr_bias.numel() == 3 * E, "in_proj_bias must have 3E entries");
  TORCH_CHECK(out_proj_weight.dim() == 2 && out_proj_weight.size(0) == E && out_proj_weight.size(1) == E, "out_proj_weight must be [E, E]");
  c10::cuda::CUDAGuard guard(q_buffer.device());
  const int64_t Tq = rq.numel / (E > 0 ? E : 1), Tk = rk.numel / (E > 0 ? E : 1);
  Tensor out = at::empty({Tq * E}, q_buffer.options());
  if (Tq == 0) return out;
  Tensor w = attr_kernel.contiguous(), b = attr_bias.contiguous().view({3 * E}), w_out = out_proj_weight.contiguous();
  const int64_t es = q_buffer.element_size();
  const char* wp = static_cast<const char*>(w.data_ptr());
  const char* bp = static_cast<const char*>(b.data_ptr());
  void* st = cur_stream();
  Tensor q = at::empty({Tq, E}, q_buffer.options());
  check_rc(ntb200_gemm_bias(q_buffer.data_ptr(), wp, bp, q.data_ptr(), Tq, E, E, dt, 0, st), "ntb200_gemm_bias");
  Tensor kv;
  const void *kptr, *vptr;
  int64_t ldkv;
  if (v_buffer.data_ptr() == k_buffer.data_ptr()) {  // key is value: one [Tk, 2E] projection
    kv = at::empty({std::max<int64_t>(Tk, 1), 2 * E}, q_buffer.options());
    check_rc(ntb200_gemm_bias(k_buffer.data_ptr(), wp + E * E * es, bp + E * es, kv.data_ptr(), Tk, 2 * E, E, dt, 0, st),
             "ntb200_gemm_bias");
    kptr = kv.data_ptr();
    vptr = static_cast<const char*>(kv.data_ptr()) + E * es;
    ldkv = 2 * E;
  } else {
    kv = at::empty({2, std::max<int64_t>(Tk, 1), E}, q_buffer.options());
    check_rc(ntb200_gemm_bias(k_buffer.data_ptr(), wp + E * E * es, bp + E * es, kv[0].data_ptr(), Tk, E, E, dt, 0, st),
             "ntb200_gemm_bias");
    check_rc(ntb200_gemm_bias(v_buffer.data_ptr(), wp + 2 * E * E * es, bp + 2 * E * es, kv[1].data_ptr(), Tk, E, E, dt, 0, st),
             "ntb200_gemm_bias");
    kptr = kv[0].data_ptr();
    vptr = kv[1].data_ptr();
    ldkv = E;
  }
  Tensor attn = at::empty({Tq, E}, q_buffer.options());
  // head_dim 64 in fp16 / bf16 runs on the tcgen05 kernel (three tensor maps, device-built work list in `ws`)
  const size_t ws_bytes = ntb200_varlen_cross_attention_workspace_bytes(rq.B, Tq, (int)num_heads, (int)head_dim, dt);
  Tensor ws = at::empty({(int64_t)std::max<size_t>(ws_bytes, 16)}, q_buffer.options().dtype(at::kByte));
  check_rc(ntb200_varlen_cross_attention_ws(q.data_ptr(), E, kptr, ldkv, vptr, ldkv, attn.data_ptr(), rq.d_offsets, rk.d_offsets, rq.B,
                                            Tq, Tk, (int)num_heads, (int)head_dim, rq.max_sizes[0], (float)scaling, dt, 0,
                                            ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, st),
           "ntb200_varlen_cross_attention_ws");
  const void* b_out = nullptr;
  Tensor b_out_t;
  if (out_proj_bias && out_proj_bias->defined()) {
    same(*out_proj_bias, "out_proj_bias");
    TORCH_CHECK(out_proj_bias->numel() == E, "out_proj_bias must have E entries");
    b_out_t = out_proj_bias->contiguous();
    b_out = b_out_t.data_ptr();
  }
  check_rc(ntb200_gemm_bias(attn.data_ptr(), w_out.data_ptr(), b_out, out.data_ptr(), Tq, E, E, dt, 0, st), "ntb200_gemm_bias");
  maybe_check_device_errors("min_mha");
  return out;
}

// Attention probabilities for need_weights=True: q and k are projected (two GEMMs with the first two thirds of in_proj), a
// separate kernel writes softmax(scaling q k^T) per sequence.  Returns (weights buffer, sizes [B, 2 or 3]): one
// (Lq_b x Lk_b) matrix per sequence averaged over the heads, or (H x Lq_b x Lk_b) with average = false.  The
// reference returns None for the weights (nestedtensor/nn/mha.py:57-83).
std::tuple<Tensor, Tensor> attention_weights(int64_t num_heads, int64_t head_dim, const Tensor& q_buffer, const Tensor& q_sizes,
                                             const Tensor& q_meta, const Tensor& k_buffer, const Tensor& k_sizes, const Tensor& k_meta,
                                             const Tensor& attr_kernel, const Tensor& attr_bias, double scaling, bool average) {
  Record rq = make_record(q_sizes, q_meta), rk = make_record(k_sizes, k_meta);
  TORCH_CHECK(rq.tdim == 2, "query needs to be 3 dim.");
  TORCH_CHECK(rk.tdim == 2, "key needs to be 3 dim.");
  TORCH_CHECK(rq.B == rk.B, "nestedtensor_b200: query and key must hold the same number of sequences");
  check_buffer(q_buffer, rq, "attention_weights");
  check_buffer(k_buffer, rk, "attention_weights");
  const int64_t E = num_heads * head_dim;
  TORCH_CHECK(rq.B == 0 || (rq.regular[1] && rq.max_sizes[1] == E), "query's third dimension must be regular.");
  TORCH_CHECK(rk.B == 0 || (rk.regular[1] && rk.max_sizes[1] == E), "key's third dimension must be regular.");
  TORCH_CHECK(num_heads >= 1 && head_dim >= 1 && head_dim <= 256, "nestedtensor_b200: head_dim must be in [1, 256]");
  const int dt = dtype_code(q_buffer.scalar_type());
  TORCH_CHECK(k_buffer.is_cuda() && k_buffer.device() == q_buffer.device() && k_buffer.scalar_type() == q_buffer.scalar_type() &&
                  attr_kernel.is_cuda() && attr_kernel.device() == q_buffer.device() && attr_kernel.scalar_type() == q_buffer.scalar_type() &&
                  attr_bias.is_cuda() && attr_bias.device() == q_buffer.device() && attr_bias.scalar_type() == q_buffer.scalar_type(),
              "nestedtensor_b200: key and the projection parameters must be on the query's device and of its dtype");
  TORCH_CHECK(attr_kernel.dim() == 2 && attr_kernel.size(0) == 3 * E && attr_kernel.size(1) == E, "in_proj_weight must be [3E, E]");
  TORCH_CHECK(attr_bias.numel() == 3 * E, "in_proj_bias must have 3E entries");
  c10::cuda::CUDAGuard guard(q_buffer.device());
  const int64_t B = rq.B, Tq = rq.numel / (E > 0 ? E : 1), Tk = rk.numel / (E > 0 ? E : 1);
  const int64_t wd = average ? 2 : 3;
  Tensor w_sizes = at::empty({B, wd}, at::TensorOptions().dtype(at::kLong));
  Tensor w_off_h = at::empty({B + 1}, at::TensorOptions().dtype(at::kLong).pinned_memory(B > 0));
  int64_t* ws = w_sizes.data_ptr<int64_t>();
  int64_t* wo = w_off_h.data_ptr<int64_t>();
  wo[0] = 0;
  for (int64_t b = 0; b < B; ++b) {
    const int64_t lq = rq.sz[b * 2], lk = rk.sz[b * 2];
    if (average) {
      ws[b * 2] = lq;
      ws[b * 2 + 1] = lk;
    } else {
      ws[b * 3] = num_heads;
      ws[b * 3 + 1] = lq;
      ws[b * 3 + 2] = lk;
    }
    wo[b + 1] = wo[b] + (average ? 1 : num_heads) * lq * lk;
  }
  Tensor weights = at::zeros({wo[B]}, q_buffer.options());
  if (wo[B] == 0) return std::make_tuple(weights, w_sizes);
  Tensor w_off = w_off_h.to(q_buffer.device(), /*non_blocking=*/true);
  Tensor w = attr_kernel.contiguous(), bias = attr_bias.contiguous().view({3 * E});
  const int64_t es = q_buffer.element_size();
  const char* wp = static_cast<const char*>(w.data_ptr());
  const char* bp = static_cast<const char*>(bias.data_ptr());
  void* st = cur_stream();
  Tensor q = at::empty({Tq, E}, q_buffer.options()), k = at::empty({Tk, E}, q_buffer.options());
  check_rc(ntb200_gemm_bias(q_buffer.data_ptr(), wp, bp, q.data_ptr(), Tq, E, E, dt, 0, st), "ntb200_gemm_bias");
  check_rc(ntb200_gemm_bias(k_buffer.data_ptr(), wp + E * E * es, bp + E * es, k.data_ptr(), Tk, E, E, dt, 0, st), "ntb200_gemm_bias");
  check_rc(ntb200_varlen_attention_weights(q.data_ptr(), E, k.data_ptr(), E, weights.data_ptr(), rq.d_offsets, rk.d_offsets,
                                           w_off.data_ptr<int64_t>(), B, Tq, (int)num_heads, (int)head_dim, rk.max_sizes[0],
                                           (float)scaling, dt, average ? 1 : 0, st),
           "ntb200_varlen_attention_weights");
  return std::make_tuple(weights, w_sizes);
}

// ------------------------------------------------------------------ packed row operators and projections
// Dense CUDA [T, cols] views of a packed buffer go straight to the C ABI.
void check_rows(const Tensor& x, const char* op) {
  TORCH_CHECK(x.is_cuda(), "nestedtensor_b200: ", op, " needs CUDA tensors (this build has no CPU implementation)");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous(), "nestedtensor_b200: ", op, " expects a contiguous [tokens, features] tensor");
  dtype_code(x.scalar_type());
}

const void* opt_vec(const c10::optional<Tensor>& t, const Tensor& like, int64_t n, const char* name, Tensor* keep) {
  if (!t || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->device() == like.device() && t->scalar_type() == like.scalar_type(), "nestedtensor_b200: ",
              name, " must be on the input's device and of its dtype");
  TORCH_CHECK(t->numel() == n, "nestedtensor_b200: ", name, " must have ", n, " entries");
  *keep = t->contiguous();
  return keep->data_ptr();
}

// out = LayerNorm(x + residual + bias) * weight + beta over the last dim of the packed [T, E] matrix
Tensor add_bias_residual_layer_norm(const Tensor& x, const c10::optional<Tensor>& residual, const c10::optional<Tensor>& bias,
                                    const c10::optional<Tensor>& weight, const c10::optional<Tensor>& beta, double eps) {
  check_rows(x, "add_bias_residual_layer_norm");
  const int64_t T = x.size(0), E = x.size(1);
  TORCH_CHECK((weight && weight->defined()) == (beta && beta->defined()), "Either both weight and bias are used or not.");
  Tensor keep_r, keep_b, keep_g, keep_be;
  const void* r = opt_vec(residual, x, T * E, "residual", &keep_r);
  const void* b = opt_vec(bias, x, E, "bias", &keep_b);
  const void* g = opt_vec(weight, x, E, "weight", &keep_g);
  const void* be = opt_vec(beta, x, E, "beta", &keep_be);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = at::empty_like(x);
  check_rc(ntb200_add_bias_residual_layer_norm(x.data_ptr(), r, b, g, be, (float)eps, out.data_ptr(), T, E,
                                               dtype_code(x.scalar_type()), cur_stream()),
           "ntb200_add_bias_residual_layer_norm");
  return out;
}

// nestedtensor/csrc/functions.cpp:65-110 + nestedtensor/csrc/cuda/layernorm.cpp:14-76, on the record
Tensor layer_norm(const Tensor& buffer, const Tensor& sizes, const Tensor& meta, at::IntArrayRef normalized_shape,
                  const c10::optional<Tensor>& weight, const c10::optional<Tensor>& bias, double eps) {
  Record r = make_record(sizes, meta);
  TORCH_CHECK(normalized_shape.size() == 1, "Currently only singleton tuples of integers supported for layer_norm.");
  TORCH_CHECK(r.tdim >= 1, "Cannot normalize across irregular dimension ", r.tdim);
  TORCH_CHECK(r.B == 0 || r.regular[r.tdim - 1], "Cannot normalize across irregular dimension ", r.tdim);
  const int64_t E = r.B > 0 ? r.max_sizes[r.tdim - 1] : normalized_shape[0];
  TORCH_CHECK(E == normalized_shape[0], "Normalized shape [", normalized_shape[0],
              "] does not match the size of the last dimension (", E, ") of input.");
  const bool has_w = weight && weight->defined(), has_b = bias && bias->defined();
  TORCH_CHECK(has_w == has_b, "Either both weight and bias are used or not.");
  check_buffer(buffer, r, "layer_norm");
  if (buffer.numel() == 0) return buffer.clone();
  TORCH_CHECK(E > 0, "nestedtensor_b200: layer_norm over an empty dimension");
  return add_bias_residual_layer_norm(buffer.view({buffer.numel() / E, E}), c10::nullopt, c10::nullopt, weight, bias, eps)
      .view({buffer.numel()});
}

// C = act(x W^T + bias) + residual on the packed [T, K] matrix (act: 0 identity, 1 GELU tanh form, 2 ReLU)
Tensor packed_linear(const Tensor& x, const Tensor& weight, const c10::optional<Tensor>& bias, int64_t act,
                     const c10::optional<Tensor>& residual) {
  check_rows(x, "packed_linear");
  TORCH_CHECK(weight.is_cuda() && weight.device() == x.device() && weight.scalar_type() == x.scalar_type() && weight.dim() == 2 &&
                  weight.size(1) == x.size(1),
              "nestedtensor_b200: weight must be [out_features, in_features] on the input's device and of its dtype");
  const int64_t T = x.size(0), K = x.size(1), N = weight.size(0);
  Tensor w = weight.contiguous(), keep_b, keep_r;
  const void* b = opt_vec(bias, x, N, "bias", &keep_b);
  const void* r = opt_vec(residual, x, T * N, "residual", &keep_r);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = at::empty({T, N}, x.options());
  check_rc(ntb200_gemm_bias_act(x.data_ptr(), w.data_ptr(), b, r, out.data_ptr(), T, N, K, dtype_code(x.scalar_type()), (int)act,
                                0, cur_stream()),
           "ntb200_gemm_bias_act");
  maybe_check_device_errors("packed_linear");
  return out;
}

Tensor add_bias_gelu(const Tensor& x, const c10::optional<Tensor>& bias) {
  check_rows(x, "add_bias_gelu");
  Tensor keep_b;
  const void* b = opt_vec(bias, x, x.size(1), "bias", &keep_b);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = at::empty_like(x);
  check_rc(ntb200_add_bias_gelu(x.data_ptr(), b, out.data_ptr(), x.size(0), x.size(1), dtype_code(x.scalar_type()), cur_stream()),
           "ntb200_add_bias_gelu");
  return out;
}

// ------------------------------------------------------------------ construction
// nested_tensor(list of CUDA tensors): one pointer-array gather instead of one copy per constituent
// (nestedtensor/csrc/storage/Packed.h:75-98).  Returns (buffer, sizes on the host, meta); the pointer table,
// the offsets and the sizes travel to the device in one pinned asynchronous copy, and meta is a view of it.
std::tuple<Tensor, Tensor, Tensor> pack_list(at::TensorList tensors) {
  const int64_t B = (int64_t)tensors.size();
  TORCH_CHECK(B > 0, "nestedtensor_b200: pack_list needs at least one tensor");
  const Tensor& first = tensors[0];
  TORCH_CHECK(first.is_cuda(), "nestedtensor_b200: pack_list needs CUDA tensors (this build has no CPU implementation)");
  const int64_t tdim = first.dim();
  const int64_t es = first.element_size();
  TORCH_CHECK(es == 1 || es == 2 || es == 4 || es == 8, "Input datatype ", first.dtype(), " is not supported.");
  std::vector<Tensor> keep;
  keep.reserve(B);
  Tensor host = at::empty({B + (B + 1) + B * tdim}, at::TensorOptions().dtype(at::kLong).pinned_memory(true));
  int64_t* h = host.data_ptr<int64_t>();
  Tensor sizes = at::empty({B, tdim}, at::TensorOptions().dtype(at::kLong));
  int64_t* hs = sizes.data_ptr<int64_t>();
  int64_t total = 0;
  for (int64_t b = 0; b < B; ++b) {
    const Tensor& t = tensors[b];
    TORCH_CHECK(t.is_cuda() && t.device() == first.device() && t.scalar_type() == first.scalar_type() && t.dim() == tdim,
                "nestedtensor_b200: pack_list needs tensors of one device, dtype and dimension");
    keep.push_back(t.contiguous());
    h[b] = reinterpret_cast<int64_t>(keep.back().data_ptr());
    h[B + b] = total;
    total += t.numel();
    for (int64_t j = 0; j < tdim; ++j) hs[b * tdim + j] = h[B + (B + 1) + b * tdim + j] = t.size(j);
  }
  h[B + B] = total;
  c10::cuda::CUDAGuard guard(first.device());
  Tensor dev = host.to(first.device(), /*non_blocking=*/true);
  Tensor buffer = at::empty({total}, first.options());
  check_rc(ntb200_pack_pointers(reinterpret_cast<const void* const*>(dev.data_ptr<int64_t>()), dev.data_ptr<int64_t>() + B, B,
                                buffer.data_ptr(), total, (int)es, cur_stream()),
           "ntb200_pack_pointers");
  // `keep` (contiguous copies, if any were needed) is released here: the caching allocator orders reuse of that
  // memory after this stream's work, which includes the gather
  return std::make_tuple(buffer, sizes, dev.slice(0, B));
}

// nestedtensor/csrc/functions.cpp:29-56: embedding of a nested tensor of 1-D index sequences = one gather on
// its packed index buffer; the result has sizes (L_i, embedding_dim).
Tensor embedding(const Tensor& weight, const Tensor& index_buffer, const Tensor& sizes, const Tensor& meta) {
  Record r = make_record(sizes, meta);
  TORCH_CHECK(r.tdim == 1, "nestedtensor_b200: embedding expects a nested tensor of 1-D index sequences");
  TORCH_CHECK(weight.is_cuda() && weight.dim() == 2, "nestedtensor_b200: embedding needs a 2-D CUDA weight");
  TORCH_CHECK(index_buffer.is_cuda() && index_buffer.device() == weight.device() && index_buffer.dim() == 1 &&
                  index_buffer.is_contiguous() && index_buffer.numel() == r.numel,
              "nestedtensor_b200: the index buffer must be 1-D contiguous on the weight's device");
  TORCH_CHECK(index_buffer.scalar_type() == at::kLong || index_buffer.scalar_type() == at::kInt,
              "Expected tensor for argument #1 'indices' to have one of the following scalar types: Long, Int");
  const int64_t es = weight.element_size();
  TORCH_CHECK(es == 1 || es == 2 || es == 4 || es == 8, "Input datatype ", weight.dtype(), " is not supported.");
  Tensor w = weight.contiguous();
  c10::cuda::CUDAGuard guard(weight.device());
  Tensor out = at::empty({r.numel * w.size(1)}, w.options());
  check_rc(ntb200_embedding(w.data_ptr(), index_buffer.data_ptr(), (int)index_buffer.element_size(), out.data_ptr(), r.numel,
                            w.size(0), w.size(1), (int)es, cur_stream()),
           "ntb200_embedding");
  return out;
}

// ------------------------------------------------------------------ ragged NCHW <-> NHWC
// nestedtensor/csrc/transpose.cpp:124-150 and :186-202 on the record: (C, H_i, W_i) -> (H_i, W_i, C) and back.
Tensor transpose_images(const Tensor& buffer, const Tensor& sizes, const Tensor& meta, bool to_nhwc) {
  Record r = make_record(sizes, meta);
  const char* name = to_nhwc ? "transpose_nchw_nhwc" : "transpose_nhwc_nchw";
  TORCH_CHECK(r.tdim == 3, name, " needs 4d input.");
  const int64_t cdim = to_nhwc ? 0 : 2;
  TORCH_CHECK(r.B == 0 || r.regular[cdim], to_nhwc ? "Expected first dimension to be regular." : "Expected last dimension to be regular.");
  check_buffer(buffer, r, name);
  Tensor out = at::empty_like(buffer);
  if (buffer.numel() == 0) return out;
  const int64_t C = r.max_sizes[cdim];
  int64_t max_pixels = 0;
  for (int64_t b = 0; b < r.B; ++b) {
    const int64_t* s = r.sz + b * 3;
    const int64_t px = to_nhwc ? s[1] * s[2] : s[0] * s[1];
    max_pixels = std::max(max_pixels, px);
  }
  c10::cuda::CUDAGuard guard(buffer.device());
  check_rc(ntb200_transpose_ragged(buffer.data_ptr(), out.data_ptr(), r.d_offsets, r.B, C, to_nhwc ? 1 : 0, max_pixels,
                                   (int)buffer.element_size(), cur_stream()),
           "ntb200_transpose_ragged");
  return out;
}
Tensor transpose_nchw_nhwc(const Tensor& buffer, const Tensor& sizes, const Tensor& meta) {
  return transpose_images(buffer, sizes, meta, true);
}
Tensor transpose_nhwc_nchw(const Tensor& buffer, const Tensor& sizes, const Tensor& meta) {
  return transpose_images(buffer, sizes, meta, false);
}

}  // namespace

// The operator names follow the reference's `nestedtensor` namespace
// (nestedtensor/csrc/masking.cpp:652-675); the nested tensor argument is spelled out as its
// record (buffer, sizes, meta) and the Python wrapper's __torch_function__ does the spelling.
TORCH_LIBRARY(nestedtensor, m) {
  m.def("to_padded_tensor(Tensor buffer, Tensor sizes, Tensor meta, float padding) -> Tensor", &to_padded_tensor);
  m.def("to_padded_tensor_out(Tensor buffer, Tensor sizes, Tensor meta, float padding, Tensor(a!) out) -> Tensor(a!)",
        &to_padded_tensor_out);
  m.def("to_tensor_mask(Tensor buffer, Tensor sizes, Tensor meta, int? mask_dim) -> (Tensor, Tensor)", &to_tensor_mask);
  m.def("to_mask(Tensor sizes, Tensor meta, int? mask_dim) -> Tensor", &to_mask);
  m.def("get_max_size(Tensor sizes) -> int[]", &get_max_size);
  m.def("pad_nt(Tensor buffer, Tensor sizes, Tensor meta, int[] shape) -> (Tensor, Tensor)", &pad_nt);
  m.def("merge_tensor_mask(Tensor tensor, Tensor mask, int? mask_dim=None) -> (Tensor, Tensor)", &merge_tensor_mask);
  m.def("nt_from_tensor_mask(Tensor tensor, Tensor mask, int nested_dim) -> (Tensor, Tensor, Tensor)", &nt_from_tensor_mask);
  m.def("from_padded_tensor(Tensor padded, Tensor sizes, Tensor meta) -> Tensor", &from_padded_tensor);
  m.def("sizes_from_padded(Tensor tensor, Scalar padding) -> (Tensor, Tensor)", &sizes_from_padded);
  m.def("sizes_from_mask(Tensor mask) -> (Tensor, Tensor)", &sizes_from_mask);
  m.def("meta_from_device_sizes(Tensor sizes) -> Tensor", &meta_from_device_sizes);
  m.def("token_index(Tensor token_offsets, int total_tokens) -> (Tensor, Tensor)", &token_index);
  m.def(
      "bt_min_mha(int num_heads, int head_dim, float dropout_p, bool training, Tensor buffer, Tensor sizes, Tensor meta, "
      "Tensor attr_kernel, Tensor attr_bias, float scaling, Tensor out_proj_weight, Tensor? out_proj_bias) -> Tensor",
      &bt_min_mha);
  m.def(
      "min_mha(int num_heads, int head_dim, float dropout_p, bool training, Tensor buffer, Tensor sizes, Tensor meta, "
      "Tensor attr_kernel, Tensor attr_bias, float scaling, Tensor out_proj_weight, Tensor? out_proj_bias) -> Tensor",
      &bt_min_mha);
  m.def(
      "bt_min_mha_core(int num_heads, int head_dim, Tensor buffer, Tensor sizes, Tensor meta, Tensor attr_kernel, "
      "Tensor attr_bias, float scaling) -> Tensor",
      &bt_min_mha_core);
  m.def(
      "min_mha_cross(int num_heads, int head_dim, Tensor q_buffer, Tensor q_sizes, Tensor q_meta, Tensor k_buffer, "
      "Tensor k_sizes, Tensor k_meta, Tensor v_buffer, Tensor attr_kernel, Tensor attr_bias, float scaling, "
      "Tensor out_proj_weight, Tensor? out_proj_bias) -> Tensor",
      &min_mha_cross);
  m.def(
      "attention_weights(int num_heads, int head_dim, Tensor q_buffer, Tensor q_sizes, Tensor q_meta, Tensor k_buffer, Tensor k_sizes, "
      "Tensor k_meta, Tensor attr_kernel, Tensor attr_bias, float scaling, bool average) -> (Tensor, Tensor)",
      &attention_weights);
  m.def("layer_norm(Tensor buffer, Tensor sizes, Tensor meta, int[] normalized_shape, Tensor? weight, Tensor? bias, float eps) -> Tensor",
        &layer_norm);
  m.def("add_bias_residual_layer_norm(Tensor x, Tensor? residual, Tensor? bias, Tensor? weight, Tensor? beta, float eps) -> Tensor",
        &add_bias_residual_layer_norm);
  m.def("packed_linear(Tensor x, Tensor weight, Tensor? bias, int act, Tensor? residual) -> Tensor", &packed_linear);
  m.def("add_bias_gelu(Tensor x, Tensor? bias) -> Tensor", &add_bias_gelu);
  m.def("transpose_nchw_nhwc(Tensor buffer, Tensor sizes, Tensor meta) -> Tensor", &transpose_nchw_nhwc);
  m.def("transpose_nhwc_nchw(Tensor buffer, Tensor sizes, Tensor meta) -> Tensor", &transpose_nhwc_nchw);
  m.def("pack_list(Tensor[] tensors) -> (Tensor, Tensor, Tensor)", &pack_list);
  m.def("embedding(Tensor weight, Tensor index_buffer, Tensor sizes, Tensor meta) -> Tensor", &embedding);
}

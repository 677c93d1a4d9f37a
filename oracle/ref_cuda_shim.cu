// C entry points around the REFERENCE's own CUDA padding launchers and its attention helper launchers
// (nestedtensor/csrc/cuda/attention.h:25-52), for cross-checks and as a secondary timing comparator.  TEST INFRASTRUCTURE: nothing in the product links or loads this; only tests and bench.py do.
//
// The launchers (add_padding_kernelLauncher / remove_padding_kernelLauncher, nestedtensor/csrc/cuda/padding.h:12-45)
// are compiled from the reference's source file where it lies (oracle/build_ref.py passes
// nestedtensor/csrc/cuda/padding.cu to nvcc for sm_100a, unmodified); this file only gives them C names.  Argument
// meaning is the reference's (nestedtensor/csrc/masking.cpp:578-616 and :463-507): int32 element offsets per entry,
// int32 sizes [batch, dim], padded extents including the batch dimension.  The reference indexes with `int`: callers
// keep batch * padded-entry elements below 2^31, and never use the one-dimensional remove_padding case
// (output_dim == 1 takes the three-dimensional kernel, padding.cu:375-393, which then reads sizes it was not given).
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include <c10/util/Half.h>
#include <nestedtensor/csrc/cuda/attention.h>
#include <nestedtensor/csrc/cuda/padding.h>

extern "C" {

// dtype: 0 = float, 1 = half.  output_sizes: input_dim + 1 extents (batch first).  Returns the CUDA error code.
int ntref_add_padding(const void* input, void* output, float padding, const int* offsets, const int* input_sizes, int input_dim,
                      const int64_t* output_sizes, int batch, int dtype, void* stream) {
  if (input_dim < 1 || input_dim > 3 || batch < 1) return -1;
  std::vector<int64_t> out(output_sizes, output_sizes + input_dim + 1);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    nested_tensor::cuda::add_padding_kernelLauncher<float>(static_cast<float*>(const_cast<void*>(input)), static_cast<float*>(output),
                                                           padding, offsets, input_sizes, input_dim, out, batch, st);
  else if (dtype == 1)
    nested_tensor::cuda::add_padding_kernelLauncher<c10::Half>(static_cast<c10::Half*>(const_cast<void*>(input)),
                                                               static_cast<c10::Half*>(output), (c10::Half)padding, offsets,
                                                               input_sizes, input_dim, out, batch, st);
  else
    return -2;
  return (int)cudaGetLastError();
}

// padded_sizes: output_dim + 1 int32 extents of the dense tensor on the DEVICE (batch first); target_sizes: int32
// [batch, output_dim] on the device.  output_dim must be 2 or 3.
int ntref_remove_padding(const void* input, void* output, const int* offsets, const int* padded_sizes, const int* target_sizes,
                         int output_dim, int batch, int dtype, void* stream) {
  if (output_dim < 2 || output_dim > 3 || batch < 1) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    nested_tensor::cuda::remove_padding_kernelLauncher<float>(static_cast<const float*>(input), static_cast<float*>(output), offsets,
                                                              padded_sizes, target_sizes, output_dim, batch, st);
  else if (dtype == 1)
    nested_tensor::cuda::remove_padding_kernelLauncher<c10::Half>(static_cast<const c10::Half*>(input), static_cast<c10::Half*>(output),
                                                                  offsets, padded_sizes, target_sizes, output_dim, batch, st);
  else
    return -2;
  return (int)cudaGetLastError();
}

// The reference's fused data + mask kernel for (L_i, inner) sequences (padding.cu:217-284: one THREAD per sequence):
// output [batch, max_len * inner] (left untouched past each sequence, the caller zero-fills), mask int32 [batch, max_len].
// offsets: batch + 1 int32 row offsets.  dtype: 0 = float, 1 = half.
int ntref_add_padding_mask(const void* input, void* output, int* mask, const int* offsets, int batch, int max_len, int inner, int dtype,
                           void* stream) {
  if (batch < 1 || max_len < 1 || inner < 1) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    nested_tensor::cuda::add_padding_mask_kernelLauncher<float>(static_cast<float*>(const_cast<void*>(input)), static_cast<float*>(output),
                                                                mask, offsets, batch, max_len, max_len * inner, inner, st);
  else if (dtype == 1)
    nested_tensor::cuda::add_padding_mask_kernelLauncher<c10::Half>(static_cast<c10::Half*>(const_cast<void*>(input)),
                                                                    static_cast<c10::Half*>(output), mask, offsets, batch, max_len,
                                                                    max_len * inner, inner, st);
  else
    return -2;
  return (int)cudaGetLastError();
}

// In-place softmax of scores [batch, heads, seq_len, seq_len] under a mask [batch, seq_len, seq_len] of the same dtype
// (1 = attend), the reference's arithmetic: scores * scaling + (1 - mask) * -10000, row sum + 1e-6
// (attention.cu:182-482; seq_len <= 1024).  dtype: 0 = float, 1 = half.
int ntref_softmax(void* scores, const void* mask, int batch, int heads, int seq_len, float scaling, int dtype, void* stream) {
  if (batch < 1 || heads < 1 || seq_len < 1 || seq_len > 1024) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    nteffectivetransformer::cuda::softmax_kernel_kernelLauncher<float>(static_cast<float*>(scores), static_cast<const float*>(mask), batch,
                                                                       heads, seq_len, scaling, st);
  else if (dtype == 1)
    nteffectivetransformer::cuda::softmax_kernel_kernelLauncher<c10::Half>(static_cast<c10::Half*>(scores),
                                                                           static_cast<const c10::Half*>(mask), batch, heads, seq_len,
                                                                           (c10::Half)scaling, st);
  else
    return -2;
  return (int)cudaGetLastError();
}

// fp32 only (the reference instantiates nothing else): q/k/v_buf[b, h, l, :] = Q/K/V[t, h*d + :] + bias for the valid
// tokens t = (batch_idx[t], word_idx[t]) (attention.cu:107-174); heads * head_dim <= 1024.
int ntref_add_qkv_bias_padding(void* q, const void* bias_q, void* k, const void* bias_k, void* v, const void* bias_v, void* q_buf,
                               void* k_buf, void* v_buf, int valid_tokens, int batch, int seq_len, int heads, int head_dim,
                               const int* batch_idx, const int* word_idx, void* stream) {
  if (valid_tokens < 1 || heads * head_dim > 1024) return -1;
  nteffectivetransformer::cuda::add_QKV_bias_padding_kernelLauncher<float>(
      static_cast<float*>(q), static_cast<const float*>(bias_q), static_cast<float*>(k), static_cast<const float*>(bias_k),
      static_cast<float*>(v), static_cast<const float*>(bias_v), static_cast<float*>(q_buf), static_cast<float*>(k_buf),
      static_cast<float*>(v_buf), valid_tokens, batch, seq_len, heads, head_dim, batch_idx, word_idx, static_cast<cudaStream_t>(stream));
  return (int)cudaGetLastError();
}

// fp32 only: dst[t, h*d + :] = src[b, h, l, :] for the valid tokens (attention.cu:488-538).
int ntref_transpose_rm_padding(void* src, void* dst, int valid_tokens, int batch, int seq_len, int heads, int head_dim,
                               const int* batch_idx, const int* word_idx, void* stream) {
  if (valid_tokens < 1 || heads * head_dim > 1024) return -1;
  nteffectivetransformer::cuda::transpose_rm_padding_kernelLauncher<float>(static_cast<float*>(src), static_cast<float*>(dst), valid_tokens,
                                                                           batch, seq_len, heads, head_dim, batch_idx, word_idx,
                                                                           static_cast<cudaStream_t>(stream));
  return (int)cudaGetLastError();
}

}  // extern "C"

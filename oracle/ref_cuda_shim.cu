// C entry points around the REFERENCE's own CUDA padding launchers, for cross-checks and as a secondary timing
// comparator.  TEST INFRASTRUCTURE: nothing in the product links or loads this; only tests and bench.py do.
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

}  // extern "C"

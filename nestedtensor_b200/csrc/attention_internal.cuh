// Internal interface between the attention entry point (attention.cu) and the tcgen05 kernel
// (attention_tcgen05.cu), and between the error-flag query (gemm_bias.cu) and both.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace ntb200 {

int64_t attn_tcgen05_item_capacity(int64_t batch, int64_t total_tokens);
size_t attn_tcgen05_workspace_bytes(int64_t batch, int64_t total_tokens);
bool attn_tcgen05_supported(int64_t batch, int64_t total_tokens, int num_heads, int head_dim, int dtype);
int attn_tcgen05_launch(const void* qkv, void* out, const int64_t* offsets, int64_t batch, int64_t total_tokens, int H,
                        float scaling, int dtype, void* workspace, cudaStream_t st);
int attn_tcgen05_error_flags_read_and_clear();
int construct_error_flags_read_and_clear();  // construct.cu: bit 0 = embedding index out of range

}  // namespace ntb200

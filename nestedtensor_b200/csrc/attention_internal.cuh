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
// skip_short > 0 (then it must be 32): sequences of at most that many tokens get no work item; single warps of the
// launch that builds the work list compute them
int attn_tcgen05_launch(const void* qkv, void* out, const int64_t* offsets, int64_t batch, int64_t total_tokens, int H,
                        float scaling, int dtype, void* workspace, cudaStream_t st, int skip_short);
// queries of sequence b over the keys / values of sequence b of other matrices (row strides in elements, multiples of 8;
// k_tokens = rows of the key / value matrices); workspace as for the self-attention launch with (batch, q_tokens)
int attn_tcgen05_cross_launch(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, void* out,
                              const int64_t* offsets_q, const int64_t* offsets_k, int64_t batch, int64_t q_tokens, int64_t k_tokens,
                              int H, float scaling, int dtype, void* workspace, cudaStream_t st);
int attn_tcgen05_error_flags_read_and_clear();
int construct_error_flags_read_and_clear();  // construct.cu: bit 0 = embedding index out of range

}  // namespace ntb200

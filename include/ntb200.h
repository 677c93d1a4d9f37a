/*
 * ntb200 — C ABI of the B200 (sm_100a) kernels behind nestedtensor's ragged<->dense,
 * mask and varlen multi-head-attention path.
 *
 * Conventions for every entry point
 *   - plain pointers and sizes only; all data pointers are DEVICE pointers unless the
 *     parameter name starts with `h_` (host);
 *   - returns NTB200_OK (0) or a negative ntb200_status; never throws, never allocates
 *     (scratch memory, where a kernel needs it, is passed in by the caller and sized by the
 *     matching *_workspace_bytes function), and never synchronises - with two exceptions
 *     stated at their declarations: ntb200_device_error_flags() waits for the device, and
 *     ntb200_offsets_from_sizes_static keeps its scratch inside the library;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = default stream);
 *   - re-entrant and thread-safe, except ntb200_offsets_from_sizes_static, whose calls share
 *     one scratch array per GPU (see its comment); arguments are validated on the host
 *     before any launch, so an invalid call launches nothing;
 *   - "ragged buffer" = the constituents of a nested tensor concatenated row-major in
 *     one 1-D buffer; `offsets[b]` = element offset of constituent b in that buffer
 *     (B+1 entries, int64, offsets[0] = 0); `sizes[b*size_stride + j]` = extent of
 *     constituent b along its j-th irregular dimension (int64).
 *
 * The reference (pytorch/nestedtensor) has no C ABI: it exposes C++ template launchers
 * that return void and never check launch errors.  Each function below cites the
 * reference interface it replaces as  path:line  inside that project.
 */
#ifndef NTB200_H_
#define NTB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ntb200_status {
  NTB200_OK = 0,
  NTB200_INVALID_ARG = -1,
  NTB200_UNSUPPORTED_DTYPE = -2,
  NTB200_MISALIGNED = -3,
  NTB200_LAUNCH_FAILED = -4,
  NTB200_DEVICE_TIMEOUT = -5,
  NTB200_WORKSPACE_TOO_SMALL = -6,
  NTB200_UNSUPPORTED_SHAPE = -7,
  NTB200_STATIC_SCRATCH_EXCEEDED = -8
} ntb200_status;

/* element types of the MHA entry points (copies take an element size instead) */
typedef enum ntb200_dtype {
  NTB200_F32 = 0,
  NTB200_F16 = 1,
  NTB200_BF16 = 2
} ntb200_dtype;

/* Human-readable name of a status code (static storage). */
const char* ntb200_status_string(int status);

/* ABI version of the loaded library: major*1000 + minor. */
int ntb200_version(void);

/* ------------------------------------------------------------------ ragged -> dense
 * out[b, i_0..i_{nd-1}] = (i_j < sizes[b][j] for all j) ? ragged[offsets[b] + lin_b(i)] : pad
 * with lin_b the row-major index inside constituent b and the dense output shaped
 * (B, h_max_sizes[0..nd-2], h_max_sizes[nd-1]*inner).  `inner` (>= 1) is the number of
 * contiguous elements per innermost index, i.e. the product of the trailing regular
 * dimensions: a (L_i, D) constituent is nd = 1, sizes[b] = L_i, inner = D.
 *   elem_size  1, 2, 4 or 8 bytes; the copy is bit-exact for any dtype of that width
 *   pad_bits   the padding value's bit pattern in the low elem_size bytes
 *   padded     must be 16-byte aligned; ragged must be elem_size aligned
 * Replaces add_padding_kernelLauncher<T> + add_padding_{1,2,3}
 * (nestedtensor/csrc/cuda/padding.cu:10-215, declared nestedtensor/csrc/cuda/padding.h:12-22),
 * called from to_padded_tensor (nestedtensor/csrc/masking.cpp:591-616).
 */
int ntb200_pad_nd(const void* ragged, void* padded, const int64_t* offsets, const int64_t* sizes,
                  int64_t size_stride, int nd, int64_t inner, int64_t batch,
                  const int64_t* h_max_sizes, int elem_size, uint64_t pad_bits, void* stream);

/* ------------------------------------------------------------------ dense -> ragged
 * ragged[offsets[b] + lin_b(i)] = padded[b, i] for every i inside sizes[b].
 *   total_elems = offsets[batch] (the caller knows it on the host)
 *   ragged must be 16-byte aligned; padded must be elem_size aligned
 * Replaces remove_padding_kernelLauncher<T> + remove_padding_2 / remove_padding
 * (nestedtensor/csrc/cuda/padding.cu:286-414, padding.h:36-45), called from
 * from_padded_tensor (nestedtensor/csrc/masking.cpp:459-509).
 */
int ntb200_unpad_nd(const void* padded, void* ragged, const int64_t* offsets, const int64_t* sizes,
                    int64_t size_stride, int nd, int64_t inner, int64_t batch,
                    const int64_t* h_max_sizes, int64_t total_elems, int elem_size, void* stream);

/* ------------------------------------------------------------------ validity mask
 * mask[b, i_0..i_{nd-1}] = (i_j < sizes[b][j] for all j) ? 1 : 0, one byte per entry,
 * shape (B, h_max_sizes[0..nd-1]); `mask` must be 16-byte aligned.
 * Replaces the host double loop of to_mask (nestedtensor/csrc/masking.cpp:436-451), the
 * per-constituent pad of a ones tensor in pad_nt/_create_nt_mask (masking.cpp:138-179,353-406)
 * and the mask half of add_padding_mask (nestedtensor/csrc/cuda/padding.cu:217-236).
 */
int ntb200_mask_from_sizes(uint8_t* mask, const int64_t* sizes, int64_t size_stride, int nd,
                           int64_t batch, const int64_t* h_max_sizes, void* stream);

/* ------------------------------------------------------------------ data + mask in one call
 * Zero-padded data and the validity mask over the leading mask_nd tensor dimensions
 * (mask_h_max_sizes), on `stream`.  When the mask has the shape of the dense tensor (one byte
 * per output element: mask_sizes == sizes, the same stride and the same padded extents) ONE
 * kernel writes both in a single walk over the output; a coarser mask (one byte per row of
 * `inner` elements) is written by a second, `inner` times smaller launch.
 * Replaces add_padding_mask_kernelLauncher<T> (nestedtensor/csrc/cuda/padding.cu:217-284,
 * padding.h:24-34) called from to_tensor_mask (nestedtensor/csrc/masking.cpp:254-296),
 * without its pre-zeroing passes and int32 -> bool cast.
 */
int ntb200_pad_with_mask(const void* ragged, void* padded, uint8_t* mask, const int64_t* offsets,
                         const int64_t* sizes, int64_t size_stride, int nd, int64_t inner,
                         int64_t batch, const int64_t* h_max_sizes, int elem_size,
                         const int64_t* mask_sizes, int64_t mask_size_stride, int mask_nd,
                         const int64_t* mask_h_max_sizes, void* stream);

/* ------------------------------------------------------------------ sizes from a padded tensor
 * For a dense (B, h_dims[0..nd-1]) tensor: out_sizes[b][j] = 1 + the largest index along
 * dimension j of an element of entry b that differs from the padding value (0 if none),
 * out_counts[b] = number of such elements.  An entry is a well-formed padded constituent
 * iff out_counts[b] == prod_j out_sizes[b][j].  Comparison follows the dtype's `!=`
 * (IEEE for floating point: -0.0 == 0.0, NaN != anything).
 *   cmp_kind  0 = compare bit patterns (integers, bool), 1 = IEEE float of that width
 *             (elem_size 2: f16), 2 = bfloat16 (elem_size 2)
 * out_sizes (B*nd int64) and out_counts (B int64) are cleared by this call (with one launch
 * instead of two when out_counts == out_sizes + B*nd, i.e. one allocation holds both).
 * Replaces `tensor != padding` (nestedtensor/nested/masking.py:12-14) plus the per-element
 * host recursion of nt_from_tensor_mask (nestedtensor/csrc/masking.cpp:181-249).
 */
int ntb200_sizes_from_padded(const void* padded, int64_t* out_sizes, int64_t* out_counts, int nd,
                             int64_t batch, const int64_t* h_dims, int elem_size, int cmp_kind,
                             uint64_t pad_bits, void* stream);

/* Same, for an explicit byte mask (non-zero = valid) of shape (B, h_dims[0..nd-1]):
 * the sizes a prefix mask describes.  Replaces the mask walk of nt_from_tensor_mask
 * (nestedtensor/csrc/masking.cpp:181-249). */
int ntb200_sizes_from_mask(const uint8_t* mask, int64_t* out_sizes, int64_t* out_counts, int nd,
                           int64_t batch, const int64_t* h_dims, void* stream);

/* ------------------------------------------------------------------ offsets (exclusive scan)
 * offsets[0] = 0, offsets[b+1] = offsets[b] + inner * prod_j sizes[b*size_stride + j], j < nd.
 * Device-side replacement of the host loop batch_offsets_from_efficient_size
 * (nestedtensor/csrc/masking.cpp:110-125) and of exclusiveScan_kernelLauncher
 * (nestedtensor/csrc/cuda/cuda_kernels.cu:282-517).
 * `workspace` must hold ntb200_offsets_workspace_bytes(batch) bytes (8-byte aligned).
 */
size_t ntb200_offsets_workspace_bytes(int64_t batch);
int ntb200_offsets_from_sizes(const int64_t* sizes, int64_t size_stride, int nd, int64_t inner,
                              int64_t batch, int64_t* offsets, void* workspace,
                              size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ offsets, no allocation anywhere
 * Same result as ntb200_offsets_from_sizes, for hosts that cannot hand the library a workspace:
 * runtimes that carve one fixed device arena at start-up and forbid any later cudaMalloc (a
 * database or inference server with a hard memory budget, an embedded control loop), and foreign
 * language bindings that have no device allocator to call at all.  The block sums that the
 * multi-block scan needs are kept in a 32 KB array compiled into the library (one copy on every
 * GPU that loads it, for the life of the process), so this call takes no workspace and performs
 * no cudaMalloc / cudaFree / allocating library call.
 *   limit        batch <= ntb200_offsets_static_max_batch() (4 194 304); larger batches return
 *                NTB200_STATIC_SCRATCH_EXCEEDED and launch nothing - use ntb200_offsets_from_sizes
 *   first call   on each device looks up the array's device address once (cudaGetSymbolAddress, with
 *                that device current); make that first call before starting any stream capture
 *   sharing      every call on a device uses the same array: two calls whose kernels can overlap
 *                on the GPU (different streams, no dependency between them) race and may both
 *                return wrong offsets; calls on one stream are safe.  Nothing needs clearing
 *                between calls: each call overwrites every entry it later reads.
 *   reset        the looked-up address belongs to the device's primary context: a host that destroys
 *                that context (cudaDeviceReset) and goes on using the library in the same process
 *                must not call this entry point again on that device.
 * This entry point has no counterpart in the reference.
 */
int64_t ntb200_offsets_static_max_batch(void);
int ntb200_offsets_from_sizes_static(const int64_t* sizes, int64_t size_stride, int nd, int64_t inner,
                                     int64_t batch, int64_t* offsets, void* stream);

/* ------------------------------------------------------------------ token index
 * For token t in [0, total_tokens): batch_idx[t] = b and word_idx[t] = t - token_offsets[b]
 * with token_offsets[b] <= t < token_offsets[b+1] (int32 outputs).
 * Replaces compress_bert_input (nestedtensor/csrc/cuda/cuda_kernels.cu:171-223).
 */
int ntb200_token_index(const int64_t* token_offsets, int64_t batch, int64_t total_tokens,
                       int32_t* batch_idx, int32_t* word_idx, void* stream);


/* ------------------------------------------------------------------ packed projection
 * C[M,N] = A[M,K] * W[N,K]^T + bias[N] (bias may be NULL); all row-major, element type `dtype`,
 * fp32 accumulation.  A is the packed token buffer [sum(L_i), K] of a nested tensor, so the
 * grouped variable-length projection is a single GEMM.  fp16/bf16 with K % 8 == 0, N % 8 == 0 and
 * 16-byte aligned pointers run on tcgen05/TMEM fed by TMA; other cases on a SIMT kernel.
 *   force_simt  0 = best available (M > 128: pairs of CTAs on 256x256 tiles with cta_group::2 MMAs,
 *               else one CTA per 128x256 tile);  1 = SIMT kernel;  2 = single-CTA tcgen05 kernel;
 *               3 = CTA-pair tcgen05 kernel (1-3 for cross-checks)
 * Replaces NestedTensor_matmul's packed path (nestedtensor/csrc/matmul.cpp:12-45) and the bias add of
 * NestedTensor_add_Tensor (nestedtensor/csrc/BinaryOps.cpp:97-107), i.e. steps 1 and 9 of bt_min_mha
 * (nestedtensor/csrc/cuda/mha.cpp:57,106).
 */
int ntb200_gemm_bias(const void* A, const void* W, const void* bias, void* C, int64_t M, int64_t N,
                     int64_t K, int dtype, int force_simt, void* stream);

/* The same projection with the rest of a transformer layer's epilogue fused into the store:
 *   C = act(A W^T + bias) + residual      act: 0 = identity, 1 = GELU (tanh form), 2 = ReLU; residual [M,N] or NULL
 * so the feed-forward up-projection (bias + GELU) and the two down-projections (bias + residual) make no
 * separate pass over their [sum(L_i), N] outputs.  Replaces add_bias_act_kernelLauncher
 * (nestedtensor/csrc/cuda/cuda_kernels.cu:73-104) and add_bias_input_kernelLauncher
 * (nestedtensor/csrc/cuda/transformer_kernels.cu:235-258) run after a cuBLAS GEMM.
 * With a residual, K < 2048 and the CTA-pair kernel, the residual tile is staged in shared memory by TMA;
 *   force_simt  as above, and 4 = CTA-pair kernel that reads the residual rows per thread whatever K is
 *               (the form used from K = 2048 on; for comparisons).
 */
int ntb200_gemm_bias_act(const void* A, const void* W, const void* bias, const void* residual, void* C,
                         int64_t M, int64_t N, int64_t K, int dtype, int act, int force_simt, void* stream);

/* Bit mask of device-side conditions recorded since the last call (0 = none): bounded waits of the tcgen05
 * kernels that ran out (projection GEMM: bit 0 TMA producer, bit 1 MMA issuer, bit 2 epilogue; attention:
 * the same roles in bits 8-10) and bit 16 = ntb200_embedding met an index outside [0, vocab) (that row
 * was zero-filled); synchronises the device; negative on a CUDA error.  No counterpart in the reference. */
int ntb200_device_error_flags(void);

/* ------------------------------------------------------------------ varlen self-attention
 * out[t, h*d:(h+1)*d] = softmax(scaling * Q_b,h K_b,h^T) V_b,h for token t of sequence b, reading
 * q|k|v of token t from row t of the packed qkv buffer [total_tokens, 3*H*d] and attending only
 * to the tokens of the same sequence; `offsets` are the ELEMENT offsets of the sequences in the
 * [total_tokens, H*d] input (B+1 entries, multiples of H*d), max_len the longest sequence.
 * Padded tokens are never materialised.
 *   path       0 = best available: when max_len <= 32 (fp16/bf16, head_dim 32 / 64 / 128) one warp per
 *              (sequence, head) on mma.sync, so that batches of very short sequences cost by the token
 *              and not by the sequence; else head_dim 64 in fp16/bf16 runs on tcgen05/TMEM fed by TMA when a
 *              workspace is supplied (its sequences of at most 32 tokens still on single warps, inside the
 *              launch that builds the work list: which kernel computes a sequence depends on its own
 *              length only, so shards of a batch reproduce the one-call result bit for bit), on an mma.sync
 *              flash kernel when it is not (as do head_dim 32 and 128), everything else on a SIMT kernel;
 *              1 = SIMT;  2 = mma.sync kernel;  3 = tcgen05 kernel for every sequence;
 *              4 = the warp-per-(sequence, head) kernel (1-4: for cross-checks, NTB200_UNSUPPORTED_SHAPE when
 *              the shape does not fit).  Sequences longer than max_len are not computed by paths 0, 2 and 4.
 *   workspace  device scratch of ntb200_varlen_attention_workspace_bytes(...) bytes, 16-byte aligned
 *              (holds the device-built list of (sequence, query tile) work items); may be NULL
 * Replaces steps 2-8 of bt_min_mha (nestedtensor/csrc/cuda/mha.cpp:59-105) including
 * softmax_kernel_kernelLauncher (nestedtensor/csrc/cuda/attention.h:25-33).
 */
size_t ntb200_varlen_attention_workspace_bytes(int64_t batch, int64_t total_tokens, int num_heads,
                                               int head_dim, int dtype);
int ntb200_varlen_attention(const void* qkv, void* out, const int64_t* offsets, int64_t batch,
                            int64_t total_tokens, int num_heads, int head_dim, int64_t max_len,
                            float scaling, int dtype, int path, void* workspace,
                            size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ packed row operators
 * Rows are the tokens of the packed [rows = sum(L_i), cols] matrix of a nested tensor; arithmetic in fp32,
 * one read and one write per element; `out` may be `x` (in place).
 *
 * out = (x - mean(x)) * rsqrt(var(x) + eps) * gamma + beta per row (gamma and beta both NULL: no affine).
 * Replaces fastertransformer::layer_norm (nestedtensor/csrc/cuda/transformer_kernels.cu:260-335) behind
 * cuda::NestedTensor_layer_norm (nestedtensor/csrc/cuda/layernorm.cpp:14-76).
 */
int ntb200_layer_norm(const void* x, const void* gamma, const void* beta, float eps, void* out,
                      int64_t rows, int64_t cols, int dtype, void* stream);
/* The same on x + residual + bias (residual [rows,cols] and bias [cols], either may be NULL).
 * Replaces add_bias_input_layernorm_kernelLauncher (nestedtensor/csrc/cuda/transformer_kernels.cu:64-156,
 * nestedtensor/csrc/cuda/cuda_kernels.cu:114-159), whose eps is fixed at 1e-6. */
int ntb200_add_bias_residual_layer_norm(const void* x, const void* residual, const void* bias,
                                        const void* gamma, const void* beta, float eps, void* out,
                                        int64_t rows, int64_t cols, int dtype, void* stream);
/* out = gelu_tanh(x + bias) (bias [cols] or NULL).  Replaces add_bias_act_kernelLauncher
 * (nestedtensor/csrc/cuda/cuda_kernels.cu:73-104) and add_bias_gelu
 * (nestedtensor/csrc/cuda/transformer_kernels.cu:52-62). */
int ntb200_add_bias_gelu(const void* x, const void* bias, void* out, int64_t rows, int64_t cols,
                         int dtype, void* stream);

/* ------------------------------------------------------------------ construction
 * out[offsets[b] + i] = srcs[b][i] for i < offsets[b+1] - offsets[b]: packs `batch` separately allocated
 * device tensors into the one buffer of a nested tensor with a single launch.  `srcs` is a DEVICE array of
 * `batch` device pointers (element-aligned), `offsets` the B+1 element offsets, `out` 16-byte aligned.
 * Replaces the per-constituent copy loop of the packed storage constructor
 * (nestedtensor/csrc/storage/Packed.h:75-98, nestedtensor/csrc/creation.cpp:191-222).
 */
int ntb200_pack_pointers(const void* const* srcs, const int64_t* offsets, int64_t batch, void* out,
                         int64_t total_elems, int elem_size, void* stream);
/* out[t, :] = weight[index[t], :] for the `tokens` entries of the packed index buffer of a nested tensor of
 * 1-D index sequences (index_bytes 4 or 8).  An index outside [0, vocab) zero-fills its row and sets bit 16
 * of ntb200_device_error_flags (the reference's at::embedding would trip a device assert).
 * Replaces the packed fast path of NestedTensor_embedding (nestedtensor/csrc/functions.cpp:29-56).
 */
int ntb200_embedding(const void* weight, const void* index, int index_bytes, void* out, int64_t tokens,
                     int64_t vocab, int64_t embed_dim, int elem_size, void* stream);

/* Attention of the queries of sequence b over the keys / values of sequence b of ANOTHER nested tensor
 * (cross-attention, or self-attention with separately stored q / k / v):
 *   out[tq, h*d:(h+1)*d] = softmax(scaling * q_b,h k_b,h^T) v_b,h
 * q / k / v point at head 0 of token 0 of their matrices, ldq / ldk / ldv are the row strides in elements
 * (>= H*d; k and v may be the two halves of one [Tk, 2*H*d] projection output); offsets_q / offsets_k are the
 * B+1 ELEMENT offsets of the sequences in the [tokens, H*d] query and key inputs; out is [q_tokens, H*d].
 * A query whose key sequence is empty gets zeros.  path: 0 = mma.sync flash kernel for head_dim 32 / 64 / 128
 * in fp16/bf16 with 16-byte aligned rows, else SIMT;  1 = SIMT;  2 = flash kernel (error if unsupported).
 * Replaces the generic per-sequence attention of min_mha (nestedtensor/csrc/mha.cpp:18-69) for query != key,
 * which the reference's CUDA path does not accelerate (nestedtensor/nn/mha.py:57).
 */
int ntb200_varlen_cross_attention(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v,
                                  int64_t ldv, void* out, const int64_t* offsets_q,
                                  const int64_t* offsets_k, int64_t batch, int64_t q_tokens, int num_heads,
                                  int head_dim, int64_t max_len_q, float scaling, int dtype, int path,
                                  void* stream);

/* The same with a workspace, which opens the tcgen05 kernel to cross-attention (head_dim 64, fp16/bf16, q / k / v and out
 * 16-byte aligned, row strides multiples of 8 elements): Q, K and V tiles are fetched through three tensor maps over
 * the query, key and value projections (k_tokens = rows of the key / value matrices), the work list is built on the
 * device from both offset arrays.  path: 0 = tcgen05 when the shape allows it and a workspace is given, else as
 * ntb200_varlen_cross_attention;  1 = SIMT;  2 = mma.sync kernel;  3 = tcgen05 (error if unsupported).
 * `workspace`: ntb200_varlen_cross_attention_workspace_bytes(...) bytes, 16-byte aligned, or NULL.
 * Replaces the per-sequence attention of min_mha (nestedtensor/csrc/mha.cpp:18-69) for query != key.
 */
size_t ntb200_varlen_cross_attention_workspace_bytes(int64_t batch, int64_t q_tokens, int num_heads, int head_dim,
                                                     int dtype);
int ntb200_varlen_cross_attention_ws(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v,
                                     int64_t ldv, void* out, const int64_t* offsets_q, const int64_t* offsets_k,
                                     int64_t batch, int64_t q_tokens, int64_t k_tokens, int num_heads,
                                     int head_dim, int64_t max_len_q, float scaling, int dtype, int path,
                                     void* workspace, size_t workspace_bytes, void* stream);

/* The attention probabilities themselves (torch.nn.MultiheadAttention(need_weights=True)):
 *   average != 0   weights[weight_offsets[b] + i*Lk_b + j]            = mean over heads of softmax_j(scaling q_b,h,i . k_b,h,j)
 *   average == 0   weights[weight_offsets[b] + (h*Lq_b + i)*Lk_b + j] = softmax_j(scaling q_b,h,i . k_b,h,j)
 * q / k, ldq / ldk, offsets_q / offsets_k as in ntb200_varlen_cross_attention; weight_offsets holds the B element
 * offsets of the per-sequence matrices; max_len_k sizes the shared-memory row (about 25 000 keys at most).  Rows of
 * sequences without keys are left untouched.  A separate, slower kernel: the attention kernels above never
 * materialise the probabilities.  The reference returns None for the weights on both of its paths
 * (nestedtensor/nn/mha.py:57-83); this entry point has no counterpart there.
 */
int ntb200_varlen_attention_weights(const void* q, int64_t ldq, const void* k, int64_t ldk, void* weights,
                                    const int64_t* offsets_q, const int64_t* offsets_k,
                                    const int64_t* weight_offsets, int64_t batch, int64_t q_tokens, int num_heads,
                                    int head_dim, int64_t max_len_k, float scaling, int dtype, int average,
                                    void* stream);

/* ------------------------------------------------------------------ ragged NCHW <-> NHWC
 * Constituent b (at element offset offsets[b]) is a row-major matrix with one regular extent `regular`
 * (channels) and one ragged extent n_b = (offsets[b+1] - offsets[b]) / regular (pixels); `out` receives its
 * transpose at the same offset.  regular_is_rows = 1: [regular x n_b] -> [n_b x regular] (NCHW -> NHWC);
 * 0: [n_b x regular] -> [regular x n_b] (NHWC -> NCHW).  max_ragged = max n_b (sizes the grid).  in != out.
 * Replaces transpose_nchw_nhwc_kernelLauncher / transpose_nhwc_nchw_kernelLauncher
 * (nestedtensor/csrc/cuda/transpose.cu:10-238) and their host-built block tables
 * (nestedtensor/csrc/transpose.cpp:16-85).
 */
int ntb200_transpose_ragged(const void* in, void* out, const int64_t* offsets, int64_t batch, int64_t regular,
                            int regular_is_rows, int64_t max_ragged, int elem_size, void* stream);

/* ------------------------------------------------------------------ reference-shaped helpers
 * q/k/v_buf[b, h, l, :] = qkv[tok(b,l), {0,E,2E} + h*d + :] + bias  for valid tokens (padded
 * positions are left untouched): bias add fused with packed -> padded head-major scatter.
 * Replaces add_QKV_bias_padding_kernelLauncher (nestedtensor/csrc/cuda/attention.cu:107-174,
 * attention.h:35-44).
 */
int ntb200_add_qkv_bias_pad(const void* qkv, const void* bias, void* q_buf, void* k_buf, void* v_buf,
                            const int64_t* offsets, int64_t batch, int64_t total_tokens,
                            int num_heads, int head_dim, int64_t max_len, int dtype, void* stream);

/* dst[t, h*d + :] = src[b, h, l, :]: padded head-major -> packed token-major.
 * Replaces transpose_rm_padding_kernelLauncher (nestedtensor/csrc/cuda/attention.cu:488-538,
 * attention.h:46-52). */
int ntb200_transpose_rm_padding(const void* src, void* dst, const int64_t* offsets, int64_t batch,
                                int64_t total_tokens, int num_heads, int head_dim, int64_t max_len,
                                int dtype, void* stream);

/* In-place masked softmax over the last dim of padded scores [B, H, len_q, len_k] with the reference's
 * arithmetic: logits*scaling + (1-mask)*-10000, row sum + 1e-6; mask[b,i,j] = i < len_b && j < len_b
 * with len_b = (offsets[b+1]-offsets[b]) / row_elems.
 * Replaces softmax_kernel_kernelLauncher (nestedtensor/csrc/cuda/attention.cu:182-482). */
int ntb200_softmax_masked(void* scores, const int64_t* offsets, int64_t row_elems, int64_t batch,
                          int num_heads, int64_t len_q, int64_t len_k, float scaling, int dtype,
                          void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NTB200_H_ */

/*
 * brk.h -- C ABI of libbrk.so, the sm_100a kernel library behind BlackRiver's device tensor.
 *
 * Every entry point takes raw DEVICE pointers, sizes and a CUDA stream (passed as void*, a
 * cudaStream_t), launches asynchronously on that stream, never allocates, never synchronises
 * and never throws.  The return value is 0 (BRK_OK) or a negative code whose first four
 * values are the reference's br::ComputingReturn (blackriver/operators.hpp:12-18), so the
 * device-tensor shim can hand it straight back through the operator interface.
 *
 * `dtype` selects the storage type of activations / weights: BRK_F32 or BRK_F16.  All
 * arithmetic accumulates in fp32.  Statistics (LayerNorm mean/var, per-row losses) are fp32
 * regardless of dtype.
 *
 * Each declaration cites the reference interface it replaces (file:line inside the
 * reference project).
 */
#ifndef BRK_H_
#define BRK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported symbol marker: the library is built with hidden visibility by default. */
#define BRK_API __attribute__((visibility("default")))

#define BRK_OK 0
#define BRK_TODO_ERROR (-1)   /* br::OP_TODO_ERROR   */
#define BRK_INPUT_ERROR (-2)  /* br::OP_INPUT_ERROR  */
#define BRK_OUTPUT_ERROR (-3) /* br::OP_OUTPUT_ERROR */
#define BRK_ATTR_ERROR (-4)   /* br::OP_ATTR_ERROR   */
#define BRK_CUDA_ERROR (-5)   /* a CUDA launch/runtime call failed; see brk_last_cuda_error() */

#define BRK_F32 0
#define BRK_F16 1

/* Library / device introspection. */
BRK_API int brk_version(void);
BRK_API const char* brk_last_cuda_error(void);
BRK_API int brk_sm_count(void);

/* ---- LayerNorm -------------------------------------------------------------------------
 * Replaces CUDATensor::op_layernorm (blackriver/cuda_tensor.cpp:236-255) and
 * kernels::launch_layer_norm_float (blackriver/kernels/normalize_kernels.cu:87-102).
 * y = (x-mean)*rsqrt(var)*gamma+beta per row; mean[row], var[row] = biased variance + eps
 * (fp32, may be NULL).  x,y [rows,hidden]; gamma,beta [hidden] in `dtype`. y may alias x. */
BRK_API int brk_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* var,
                      int64_t rows, int64_t hidden, float eps, int dtype, void* stream);

/* Replaces CUDATensor::op_layernorm_backward (blackriver/cuda_tensor.cpp:700-727) and
 * kernels::launch_ln_bw_float (blackriver/kernels/normalize_kernels.cu:361-383).
 * Inputs: dy, the LayerNorm OUTPUT y (not x), gamma, beta, var (= sigma^2+eps from the forward).
 * Outputs: dx [rows,hidden]; dgamma, dbeta [hidden] in `dtype`, overwritten, or added to when
 * `accumulate` != 0.  dx may alias dy or y.  `workspace` holds per-CTA partial column sums;
 * its size must be at least brk_layernorm_bwd_workspace_bytes(rows, hidden). */
BRK_API size_t brk_layernorm_bwd_workspace_bytes(int64_t rows, int64_t hidden);
BRK_API int brk_layernorm_bwd(const void* dy, const void* gamma, const void* beta, const float* var, const void* y,
                      void* dgamma, void* dbeta, void* dx, int64_t rows, int64_t hidden, float eps,
                      void* workspace, size_t workspace_bytes, int accumulate, int dtype, void* stream);

/* The same with the residual branch of the block folded in: dx = residual + (LayerNorm input gradient), what the
 * reference's backward kernel takes as its residual_grad input (blackriver/kernels/normalize_kernels.cu:134-221) and
 * the words otherwise compute with a separate op_add.  residual [rows,hidden] in `dtype`, NULL = none (then identical
 * to brk_layernorm_bwd); it may alias dx.  The sum is formed in fp32 and rounded once. */
BRK_API int brk_layernorm_bwd_residual(const void* dy, const void* gamma, const void* beta, const float* var, const void* y,
                      const void* residual, void* dgamma, void* dbeta, void* dx, int64_t rows, int64_t hidden, float eps,
                      void* workspace, size_t workspace_bytes, int accumulate, int dtype, void* stream);

/* Kernel selection of the LayerNorm kernels, for measurements (no counterpart in the reference).
 * Mode 0 (default): rows of 2 KiB and more are prefetched through shared memory with asynchronous
 * copies, several rows ahead; mode 1 keeps to the register-resident kernels. */
BRK_API int brk_layernorm_set_mode(int mode);

/* LayerNorm backward for callers that cannot hand over a workspace.  It has no counterpart in the
 * reference.  Same arguments and results as brk_layernorm_bwd, but the partial column sums go to
 * an array built into the library (brk_layernorm_bwd_static_capacity() bytes, 16 MiB, reserved on
 * every GPU that loads the library for the life of the process), so the call performs no device
 * or host allocation of any kind.  Meant for plugins living inside an engine that owns all device
 * memory, for processes under a fixed GPU memory quota, and for code reached during stream capture,
 * where allocation calls are not allowed.
 *  - Problem sizes whose brk_layernorm_bwd_workspace_bytes(rows, hidden) exceeds the capacity are
 *    refused with BRK_ATTR_ERROR and an explanatory brk_last_cuda_error() message.
 *  - The first call on each device looks up the array's device address (once, cached); make that
 *    first call before any stream capture begins.
 *  - All calls share the one array.  Each call fully rewrites the part it uses, so no clearing is
 *    needed, but calls that may execute concurrently on the GPU (two streams, unordered threads)
 *    corrupt each other: serialise them. */
BRK_API size_t brk_layernorm_bwd_static_capacity(void);
BRK_API int brk_layernorm_bwd_static(const void* dy, const void* gamma, const void* beta, const float* var, const void* y,
                             void* dgamma, void* dbeta, void* dx, int64_t rows, int64_t hidden, float eps,
                             int accumulate, int dtype, void* stream);

/* ---- bloom GELU ------------------------------------------------------------------------
 * Replaces CUDATensor::op_gelu / op_gelu_backward (blackriver/cuda_tensor.cpp:401-412,
 * 815-828) and kernels::gelu_forward / gelu_backward (blackriver/kernels/gelu.cu:46-85).
 * y = 0.5x(1+tanh(0.79788456x(1+0.044715x^2))).  Outputs may alias inputs. */
BRK_API int brk_gelu_fwd(const void* x, void* y, int64_t n, int dtype, void* stream);
BRK_API int brk_gelu_bwd(const void* dy, const void* x, void* dx, int64_t n, int dtype, void* stream);

/* ---- vocabulary log-softmax + NLL --------------------------------------------------------
 * Replaces the cudnnSoftmaxForward(LOG) + kernels::nllloss_forward + cudnnSoftmaxBackward
 * sequence of CUDATensor::op_loss_backward (blackriver/cuda_tensor.cpp:535-553, 642-671;
 * blackriver/kernels/nll_loss.cu:10-58) with one kernel over materialised logits
 * [rows,vocab].  target[row] outside [0,vocab) (e.g. -100) marks an ignored row: loss 0,
 * gradient 0.  row_loss[row] = logsumexp - logit[target] (fp32).  row_lse may be NULL.
 * The fwd_bwd form also writes dlogits = (softmax - onehot) * grad_scale in `dtype`;
 * dlogits may alias logits. */
BRK_API int brk_logsoftmax_nll_fwd(const void* logits, const int32_t* target, float* row_loss, float* row_lse,
                           int64_t rows, int64_t vocab, int dtype, void* stream);
BRK_API int brk_logsoftmax_nll_fwd_bwd(const void* logits, const int32_t* target, float* row_loss, void* dlogits,
                               int64_t rows, int64_t vocab, float grad_scale, int dtype, void* stream);

/* Same kernel with the gradient factor formed on the device: grad_scale = scale_numerator / max(count[0], 1),
 * count = the number of counted positions written by brk_loss_targets.  Replaces the stream synchronisation
 * with which the reference fetches that count before scaling (blackriver/cuda_tensor.cpp:569-577), so the
 * loss step can be queued without a host round trip. */
BRK_API int brk_logsoftmax_nll_fwd_bwd_counted(const void* logits, const int32_t* target, float* row_loss, void* dlogits,
                                       int64_t rows, int64_t vocab, float scale_numerator, const int32_t* count,
                                       int dtype, void* stream);

/* Deterministic sum of n fp32 values into out[0] (single CTA, fixed order); the loss total. */
BRK_API int brk_sum_f32(const float* x, float* out, int64_t n, void* stream);
/* out[0] = sum(x[0..n)) / max(count[0], 1): the mean loss over counted positions (the division the reference
 * does on the host, blackriver/cuda_tensor.cpp:691), kept on the device. */
BRK_API int brk_sum_div_f32(const float* x, const int32_t* count, float* out, int64_t n, void* stream);
/* flag[0] = value, written by the device in stream order after everything queued before it, with a system-wide
 * fence first; `flag` may live in a peer GPU's memory.  It has no counterpart in the reference: it is the
 * arrival / release signal of the one-sided stage hand-offs that replace io_nccl_send / io_nccl_recv
 * (blackriver/cuda_tensor.cpp:75-96) in the overlapped pipeline. */
BRK_API int brk_signal_u32(uint32_t* flag, uint32_t value, void* stream);

/* Loss targets on the device, bit-exact restatement of the host loops at
 * blackriver/cuda_tensor.cpp:555-568 and 597-625: target[b,t] = ids[b,t+1] when t < T-1 and
 * mask[b,t] != 0 and mask[b,t+1] != 0, else -100.  count[0] receives the number of counted
 * positions (int32, overwritten). */
BRK_API int brk_loss_targets(const int32_t* ids, const int32_t* mask, int32_t* target, int32_t* count,
                     int batch, int tokens, void* stream);

/* ---- elementwise / data movement ---------------------------------------------------------
 * brk_add_bcast replaces CUDATensor::op_add (blackriver/cuda_tensor.cpp:207-232): c = a + b,
 * 4-D, dims of b that are 1 broadcast; c may alias a or b. */
BRK_API int brk_add_bcast(const void* a, const void* b, void* c, const int64_t adims[4], const int64_t bdims[4],
                  int dtype, void* stream);
/* Replaces CUDATensor::op_fill / op_zero (blackriver/cuda_tensor.cpp:100-125). */
BRK_API int brk_fill(void* x, float value, int64_t n, int dtype, void* stream);
/* fp32 <-> fp16 conversion (new: the reference has no fp16 path). */
BRK_API int brk_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, void* stream);
/* Replaces CUDATensor::op_transpos_0213 (blackriver/cuda_tensor.cpp:258-275) and
 * kernels::launch_transform_0213 (blackriver/kernels/transform_kernels.cu:40-87):
 * x [a,b,c,d] -> y [a,c,b,d]. */
BRK_API int brk_transpose_0213(const void* x, void* y, int64_t a, int64_t b, int64_t c, int64_t d, int dtype, void* stream);
/* Column sums, out[j] = sum_i x[i,j] (overwrite or accumulate): the bias gradient that the
 * reference takes with cudnnReduceTensor (blackriver/cuda_tensor.cpp:738-761). */
BRK_API int brk_colsum(const void* x, void* out, int64_t rows, int64_t cols, int accumulate, int dtype, void* stream);
/* Same result through a two-stage reduction that streams at HBM speed; `workspace` holds fp32 partial
 * sums (brk_colsum_workspace_bytes).  Falls back to brk_colsum for small or unaligned inputs. */
BRK_API size_t brk_colsum_workspace_bytes(int64_t rows, int64_t cols);
BRK_API int brk_colsum_ws(const void* x, void* out, int64_t rows, int64_t cols, int accumulate, int dtype, void* workspace,
                  size_t workspace_bytes, void* stream);
/* Row softmax and its backward on [rows,cols]: CUDATensor::op_softmax / op_softmax_backward
 * (blackriver/cuda_tensor.cpp:333-356, 891-918).  In-place allowed. */
BRK_API int brk_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, int dtype, void* stream);
BRK_API int brk_softmax_bwd(const void* dy, const void* out, void* dx, int64_t rows, int64_t cols, int dtype, void* stream);
/* Embedding gather, x[i,:] = table[ids[i],:]: the host memcpy loop of BloomInput::fetch_data
 * (blackriver/train_bloom.cpp:50-56), bit-exact.  ids outside [0,vocab) give a zero row. */
BRK_API int brk_embedding_gather(const void* table, const int32_t* ids, void* out, int64_t n, int64_t hidden, int64_t vocab,
                         int dtype, void* stream);
/* ALiBi [heads,tokens] and additive mask [batch,tokens,tokens] in fp32, bit-exact restatement
 * of BloomInput::fetch_data (blackriver/train_bloom.cpp:58-90).  slopes are computed on the
 * host in double by brk_alibi_slopes and passed in. */
BRK_API void brk_alibi_slopes(int heads, double* slopes_out);
BRK_API int brk_alibi_build(const double* slopes_dev, float* alibi, int heads, int tokens, void* stream);
BRK_API int brk_xmask_build(const int32_t* mask, float* xmask, int batch, int tokens, void* stream);

/* ---- parameter-side kernels (new: the reference has no optimizer, no embedding gradient and
 * loads pretrained weights; kernels.h:147 only declares a parameter update) ------------------------
 * Adam with torch.optim.Adam semantics on fp32 master weights and moments; `grad` is fp16 or fp32 and
 * is multiplied by grad_scale first (un-scaling of loss-scaled gradients); w16 (may be NULL) receives
 * the fp16 working copy.  step counts from 1.  Pointers 16-byte aligned. */
BRK_API int brk_adam_step(void* master_w, void* m, void* v, const void* grad, int grad_dtype, void* w16, int64_t n, float lr,
                  float beta1, float beta2, float eps, int step, float grad_scale, void* stream);
/* Elements whose scaled gradient is not finite (an fp16 gradient that overflowed under the loss scale) are skipped by
 * brk_adam_step -- weight and moments keep their values -- and remembered: brk_adam_status() (synchronous) returns 1
 * if that happened since the last query, so that a driver can lower its loss scale. */
BRK_API int brk_adam_status(void);
/* table_g[ids[r], :] += dx[r, :]: gradient of brk_embedding_gather (atomic adds). */
BRK_API int brk_embedding_scatter_add(const void* dx, const int32_t* ids, void* table_g, int64_t n, int64_t hidden, int64_t vocab,
                              int dtype, void* stream);
/* x[i] ~ N(mean, std), a pure function of (seed, i): seeded random initialisation on the device. */
BRK_API int brk_init_normal(void* x, int64_t n, float mean, float std, uint64_t seed, int dtype, void* stream);

/* ---- GEMM (fp32 SIMT parity path) ----------------------------------------------------------
 * C[b] = alpha * op(A[b]) * op(B[b]) + beta * C[b], row-major, op = transpose when the flag is
 * non-zero; op(A) is [m,k], op(B) is [k,n]; lda/ldb/ldc are row strides of the stored
 * matrices; `batch` problems at element strides sa/sb/sc.  Stands in for kernels::LtSgemm
 * (blackriver/kernels/LtSgemm.cu:55-126) on the fp32 path (fp16 storage is accepted too). */
BRK_API int brk_gemm(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
             int64_t lda, int64_t ldb, int64_t ldc, int64_t batch, int64_t sa, int64_t sb, int64_t sc,
             float alpha, float beta, const void* bias, int dtype, void* stream);

/* ---- GEMM, fp16 on the tcgen05 tensor cores ------------------------------------------------------
 * Same row-major convention as brk_gemm (op(A) [m,k], op(B) [k,n]; trans flag = stored transposed),
 * fp16 operands and output, fp32 accumulation in tensor memory.  This is the throughput path that
 * stands in for kernels::LtSgemm (blackriver/kernels/LtSgemm.cu:55-126) and for the bias pass that
 * follows it (cudnnAddTensor, blackriver/cuda_tensor.cpp:180-188), with the epilogue
 *     out = acc (+ bias[n]) (+ residual[m,n]) (+ C[m,n] when accumulate != 0);  C = fp16(out);
 *     gelu_out = fp16(bloom_gelu(out)) when gelu_out != NULL.
 * Requirements: lda, ldb multiples of 8 elements and a, b 16-byte aligned (TMA); any m, n, k.  bias,
 * residual, gelu_out and c may have any alignment (16-byte aligned pointers with row strides that are
 * multiples of 8 take the 128-bit paths, anything else a scalar epilogue).
 * brk_gemm_f16_supported() answers whether a problem meets them (callers fall back to brk_gemm).
 * The kernels bound every internal wait; brk_gemm_f16_status() (synchronous) returns non-zero if
 * one of them gave up since the last query. */
BRK_API int brk_gemm_f16_supported(int64_t m, int64_t n, int64_t k, int trans_a, int trans_b, int64_t lda, int64_t ldb,
                           const void* a, const void* b);
BRK_API int brk_gemm_f16(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                 int64_t lda, int64_t ldb, int64_t ldc, const void* bias, const void* residual, int64_t ldr,
                 void* gelu_out, int64_t ldg, int accumulate, void* stream);
BRK_API int brk_gemm_f16_status(void);
/* Kernel selection for measurements: 0 = by shape (default), 1 = single-CTA tiles only, 2 = CTA-pair
 * (cta_group::2, 256 x 256 tiles) whenever m, n > 128. */
BRK_API void brk_gemm_f16_set_mode(int mode);
/* Epilogue selection of the CTA-pair kernel, for measurements: 0 (default) = outputs without residual or
 * GELU side output whose C is 16-byte aligned with ldc a multiple of 8 leave through shared memory as TMA
 * tiled stores (TMA tiled reductions when accumulate != 0, so C is never read by the SMs: the sum
 * C + fp16(acc) is then rounded to fp16 at the memory side); 1 = always the register epilogue. */
BRK_API void brk_gemm_f16_set_epilogue(int mode);
/* Split-k of the CTA-pair kernel, for measurements: 0 (default) = where the pair tiles do not fill the last wave
 * of CTA pairs (e.g. 128 tiles on 74 pairs) and k is long, each tile's k range is cut into 2..4 work items that add
 * their partial products into C through the TMA reduction (C is cleared first unless accumulate != 0; partial
 * products are rounded to fp16 before they are added); 1 = never. */
BRK_API void brk_gemm_f16_set_split_k(int mode);
/* The rule behind it, as a pure function (no device needed): work items per tile for `tiles` pair tiles on `pairs`
 * CTA pairs with `kblocks` 64-wide k-blocks per tile. */
BRK_API int brk_gemm_f16_split_items(int tiles, int pairs, int kblocks);

/* ---- fused attention (fp16, tcgen05) ------------------------------------------------------------
 * Replaces the op_qk -> op_add(alibi) -> op_add(xmask) -> op_softmax -> op_attn chain of layer_forward
 * (bloomz-7b/train.words:147-166; blackriver/cuda_tensor.cpp:207-232, 278-398) and the four
 * op_transpos_0213 calls around it, plus the host-built ALiBi and additive mask tensors
 * (blackriver/train_bloom.cpp:58-90), with one kernel:
 *     P = softmax(Q K^T / sqrt(d) + slopes[h] * key_index) over keys with key <= query and key < lens[b]
 *     out = P V
 * q, k, v: token-major fp16, head h at columns h*head_dim.., common row stride ld_qkv (so the three
 * thirds of a fused QKV projection [batch*tokens, 3*heads*head_dim] can be passed as q, q+H, q+2H).
 * out: token-major [batch*tokens, ld_out].  lse: [batch, heads, tokens] fp32 (may be NULL when no
 * backward follows).  lens: [batch] int32 valid lengths (right padding, the assumption the
 * reference mask builder makes) or NULL for full length; slopes: [heads] fp32 or NULL.
 * head_dim 64 or 128; ld_qkv a multiple of 8; pointers 16-byte aligned. */
BRK_API int brk_flash_attn_fwd(const void* q, const void* k, const void* v, int64_t ld_qkv, void* out, int64_t ld_out,
                       float* lse, const int32_t* lens, const float* slopes, int batch, int tokens, int heads,
                       int head_dim, void* stream);
/* Backward of brk_flash_attn_fwd; replaces op_softmax_attn_backward + op_qk_backward and the four
 * transposes of layer_backward (bloomz-7b/train.words:215-227; blackriver/cuda_tensor.cpp:921-1063).
 * Inputs: q, k, v as in the forward, the forward's out and lse, the upstream gradient d_out
 * (token-major, row stride ld_out like out).  Outputs dq, dk, dv: token-major with row stride ld_g
 * (e.g. the three thirds of one [batch*tokens, 3H] buffer), overwritten.  workspace: at least
 * brk_flash_attn_bwd_workspace_bytes() bytes of device scratch (row sums of d_out * out). */
BRK_API size_t brk_flash_attn_bwd_workspace_bytes(int batch, int tokens, int heads);
BRK_API int brk_flash_attn_bwd(const void* q, const void* k, const void* v, int64_t ld_qkv, const void* out, const void* d_out,
                       int64_t ld_out, const float* lse, void* dq, void* dk, void* dv, int64_t ld_g,
                       const int32_t* lens, const float* slopes, int batch, int tokens, int heads, int head_dim,
                       void* workspace, size_t workspace_bytes, void* stream);
BRK_API int brk_flash_attn_status(void);

#ifdef __cplusplus
}
#endif
#endif /* BRK_H_ */

/*
 * qb200.h -- C ABI of libqb200: MLX-format affine group-quantized inference
 * operators for NVIDIA B200 (sm_100a).
 *
 * Every operator mirrors, argument for argument, the mlx-c entry point that
 * mlx-serve binds in src/mlx.zig, so the Zig host code can call it in place of
 * mlx-c for this path.  Differences that follow from leaving MLX's lazy graph:
 *   - tensors are plain descriptors (device pointer, dtype, shape, element
 *     strides) instead of refcounted mlx_array handles;
 *   - results are caller-allocated: `res` must describe a buffer of the
 *     operator's output shape and dtype (the `*_shape` helpers compute it);
 *   - work is enqueued on the given cudaStream_t and is complete when the
 *     stream is synchronised (MLX: when the graph is evaluated);
 *   - status codes: 0 on success like mlx-c (src/mlx.zig:547-550), a
 *     qb200_status value otherwise; the message goes to the error handler
 *     (src/mlx.zig:396-397) and to qb200_last_error().
 * Nothing here allocates or frees device memory.  No operator launches on
 * invalid input, and none aborts the process.
 *
 * Packed layout (src/kv_quant.zig:102-106, tests/dsv4_imatrix.py:107-163):
 *   value i of a row is in uint32 word i/(32/bits) at bit (i%(32/bits))*bits;
 *   w = q*scale + bias, one bf16 (scale, bias) per group_size consecutive
 *   values along the last axis.  W [..., rows, in*bits/32] uint32,
 *   scales/biases [..., rows, in/group_size].
 */
#ifndef QB200_H
#define QB200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define QB200_API
#else
#define QB200_API __attribute__((visibility("default")))
#endif

#define QB200_MAX_DIMS 8

/* Same numeric values as mlx_dtype (src/mlx.zig:20-35). */
typedef enum qb200_dtype {
  QB200_BOOL = 0,
  QB200_UINT8 = 1,
  QB200_UINT16 = 2,
  QB200_UINT32 = 3,
  QB200_UINT64 = 4,
  QB200_INT8 = 5,
  QB200_INT16 = 6,
  QB200_INT32 = 7,
  QB200_INT64 = 8,
  QB200_FLOAT16 = 9,
  QB200_FLOAT32 = 10,
  QB200_FLOAT64 = 11,
  QB200_BFLOAT16 = 12
} qb200_dtype;

typedef enum qb200_status {
  QB200_OK = 0,
  QB200_ERR_UNSUPPORTED = 1, /* valid request this library declines (caller falls through) */
  QB200_ERR_BAD_SHAPE = 2,
  QB200_ERR_BAD_STRIDE = 3,
  QB200_ERR_BAD_DTYPE = 4,
  QB200_ERR_BAD_ARG = 5,
  QB200_ERR_CUDA = 6,
  QB200_ERR_WORKSPACE = 7,
  QB200_ERR_TIMEOUT = 8
} qb200_status;

/* Tensor descriptor.  `stride` is in ELEMENTS.  A tensor with data == NULL and
 * ndim == 0 stands for mlx-c's empty handle (`mlx_array{ .ctx = null }`). */
typedef struct qb200_tensor {
  void* data;
  int32_t dtype; /* qb200_dtype */
  int32_t ndim;
  int64_t shape[QB200_MAX_DIMS];
  int64_t stride[QB200_MAX_DIMS];
} qb200_tensor;

/* mlx_optional_int / mlx_optional_dtype (src/mlx.zig:40-62, :313-316). */
typedef struct qb200_optional_int {
  int value;
  bool has_value;
} qb200_optional_int;
typedef struct qb200_optional_dtype {
  int value; /* qb200_dtype */
  bool has_value;
} qb200_optional_dtype;
typedef struct qb200_optional_float {
  float value;
  bool has_value;
} qb200_optional_float;

typedef void* qb200_stream; /* cudaStream_t */

/* ---- error reporting (replaces mlx_set_error_handler, src/mlx.zig:396-397) ---- */
typedef void (*qb200_error_handler_func)(const char* msg, void* data);
QB200_API void qb200_set_error_handler(qb200_error_handler_func handler, void* data, void (*dtor)(void*));
QB200_API const char* qb200_last_error(void); /* thread-local; "" when none */
QB200_API const char* qb200_version(void);
/* Diagnostic without a reference counterpart: 0, or the code of the bounded barrier wait that
 * expired inside the tensor-core prefill kernel (synchronises the device). */
QB200_API int qb200_debug_tc_status(void);
/* Clears that code (it is sticky: once set it stays until cleared).  A host should read the status once per step
 * after its stream synchronisation -- a non-zero code means a result of that step is incomplete -- and clear it. */
QB200_API void qb200_debug_tc_reset(void);

/* ---- mlx_quantized_matmul (src/mlx.zig:262) ----
 * transpose_w = true : y[..., m, n] = sum_k x[..., m, k] * What[..., n, k]
 *                      (w [..., N, K*bits/32], scales/biases [..., N, K/gs]);
 * transpose_w = false: y[..., m, n] = sum_k x[..., m, k] * What[..., k, n]
 *                      (w [..., K, N*bits/32], groups run along n;
 *                      src/kv_quant.zig:657-660, :1038-1094).
 * Leading dims of x and of (w, scales, biases) broadcast (src/kv_quant.zig:968-975).
 * fp32 accumulate, res dtype == x dtype (bf16 or f32).  group_size defaults to
 * 64 and bits to 4 when not given, as in MLX.  mode must be "affine". */
QB200_API int qb200_quantized_matmul(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* w,
                                     const qb200_tensor* scales, const qb200_tensor* biases, bool transpose_w,
                                     qb200_optional_int group_size, qb200_optional_int bits, const char* mode,
                                     qb200_stream s);
/* Several weight matrices applied to the SAME activations in one call: res[i] = x . What_i^T.
 * Same result as `count` calls of qb200_quantized_matmul; at decode widths the matrices share one
 * kernel launch and one staging of x.  It serves the call sites where the reference issues
 * back-to-back mlx_quantized_matmul calls on one input: q, k, v (src/transformer.zig:9202-9207,
 * :9658, :9688) and gate, up (src/transformer.zig:9452-9454, :9852-9858); MLX's lazy graph leaves
 * their scheduling to the runtime, an eager ABI has to be told. */
QB200_API int qb200_quantized_matmul_batch(qb200_tensor* const* res, const qb200_tensor* x,
                                           const qb200_tensor* const* w, const qb200_tensor* const* scales,
                                           const qb200_tensor* const* biases, int count, bool transpose_w,
                                           qb200_optional_int group_size, qb200_optional_int bits, const char* mode,
                                           qb200_stream s);
/* Output shape of qb200_quantized_matmul: fills out_shape[0..*out_ndim). */
QB200_API int qb200_quantized_matmul_shape(const qb200_tensor* x, const qb200_tensor* w, const qb200_tensor* scales,
                                           bool transpose_w, qb200_optional_int group_size, qb200_optional_int bits,
                                           int64_t* out_shape, int32_t* out_ndim);

/* ---- mlx_gather_qmm (src/mlx.zig:265; caller src/transformer.zig:20763-20784) ----
 * w [E, N, K*bits/32], scales/biases [E, N, K/gs]; x [*xb, M, K]; rhs_indices
 * any int32/uint32/int64 tensor of shape I; lhs_indices empty or of shape I.
 * res [*I, M, N]: res[i] = x[lhs(i)] . What[rhs[i]]^T, where lhs(i) is
 * lhs_indices[i] into x's flattened batch dims, or, when lhs_indices is empty,
 * the position obtained by broadcasting x's batch dims against I.
 * sorted_indices is a performance hint and never changes values
 * (src/transformer.zig:20772-20774).  transpose_w must be true (the only form
 * the reference uses). */
QB200_API int qb200_gather_qmm(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* w,
                               const qb200_tensor* scales, const qb200_tensor* biases,
                               const qb200_tensor* lhs_indices, const qb200_tensor* rhs_indices, bool transpose_w,
                               qb200_optional_int group_size, qb200_optional_int bits, const char* mode,
                               bool sorted_indices, qb200_stream s);

/* ---- fused gate/up projection + SwiGLU of the routed-expert block ----
 * res[i] = silu(x[lhs(i)] . Wgate[rhs[i]]^T) * (x[lhs(i)] . Wup[rhs[i]]^T), both banks of one shape, read once,
 * with the activations staged once.  Replaces two gatherExpertMm calls and fusedSwiGLU in moeMLP2
 * (src/transformer.zig:15007-15035, :19925-19931) and the single-token gatherQmvGateUp kernel
 * (src/transformer.zig:20303-20396, :20145-20203).  Rounding points of the bf16 form are the reference's
 * (src/transformer.zig:19842-19851): both projections rounded to bf16, the sigmoid of the rounded gate read from
 * a table over all bf16 patterns, g*sig rounded, then *up rounded; fp32 inputs compute (g*sigmoid(g))*u in fp32.
 * Served by the streaming kernel's shapes (at most 2048 index entries, K <= 4096 and a multiple of 256);
 * anything else returns QB200_ERR_UNSUPPORTED and the caller keeps the unfused chain.  The first call on a
 * device uploads the 128 KiB sigmoid table with a synchronous copy, so it must not happen while the stream is
 * being captured into a CUDA graph (it fails with a CUDA error then; call once before capturing). */
QB200_API int qb200_gather_qmm_swiglu(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* w_gate,
                                      const qb200_tensor* scales_gate, const qb200_tensor* biases_gate,
                                      const qb200_tensor* w_up, const qb200_tensor* scales_up,
                                      const qb200_tensor* biases_up, const qb200_tensor* lhs_indices,
                                      const qb200_tensor* rhs_indices, qb200_optional_int group_size,
                                      qb200_optional_int bits, const char* mode, bool sorted_indices, qb200_stream s);

/* ---- down projection + router weighting + sum over top-k in one launch, for the single-token decode step ----
 * res[t, n] = sum_j round(round(act[t, j, :] . Wdown[inds[t, j]][n, :]) * scores[t, j]), ascending j, every step
 * rounded to the activation dtype.  Replaces gatherQmvDownReduce (src/transformer.zig:20559-20623, :20675-20761)
 * with its rounding points: the per-slot dot product as the unfused gather_qmm would store it, the rounded product
 * with the score, the ascending accumulate in the input dtype.  act [T, k, K] (or [T, k, 1, K]), w [E, N, K*bits/32]
 * with scales/biases [E, N, K/gs], inds [T, k] int32/int64, scores [T, k] and res [T, N] of act's dtype (bf16/f32).
 * Served for at most 4 tokens and 16 slots, K a multiple of 256; anything else returns QB200_ERR_UNSUPPORTED and the
 * caller keeps qb200_gather_qmm + qb200_moe_weighted_sum (same values). */
QB200_API int qb200_moe_down_reduce(qb200_tensor* res, const qb200_tensor* act, const qb200_tensor* w,
                                    const qb200_tensor* scales, const qb200_tensor* biases, const qb200_tensor* inds,
                                    const qb200_tensor* scores, qb200_optional_int group_size, qb200_optional_int bits,
                                    const char* mode, qb200_stream s);

/* ---- the router of the routed-expert block (moeRoutingChain, src/transformer.zig:17022-17063) ----
 * logits [..., T, E] (bf16 or f32, E <= 1024) -> inds [..., T, k] int32: the k largest logits of each row, larger
 * first, equal logits by lower index -- the order of the reference's one-kernel router (src/transformer.zig:17485-17500;
 * the unfused chain takes the set from mlx_argpartition, which leaves the order open); norm_scores [..., T, k] of the
 * logits' dtype: softmax over the row in fp32 rounded to that dtype, the k entries divided by their sum, the sum
 * accumulated in that dtype in selection order (:17530-17534), the quotient rounded to it. */
QB200_API int qb200_moe_route(qb200_tensor* inds, qb200_tensor* norm_scores, const qb200_tensor* logits, int k,
                              qb200_stream s);

/* ---- sort of the routed-expert block's index list by expert (moeMLP2, src/transformer.zig:14961-15006) ----
 * inds [..., T, k] (int32/uint32/int64, flattened to n = T*k entries) -> all int32 [n], each optional (pass an
 * empty tensor to skip it):
 *   order        = argsort(flat_inds), stable: equal experts keep their original order (mlx_argsort_axis, :14972);
 *   inv_order    = argsort(order) (:14975), the row of entry i after sorting;
 *   sorted_inds  = flat_inds[order] (:14980), the rhs_indices of the three gather_qmm calls;
 *   token_rows   = order / k (:14983-14987), the lhs_indices that stand for the x_rep gather (:14995-15005);
 *   expert_offsets [num_experts + 1]: rows of expert e are [offsets[e], offsets[e+1]) (no counterpart in the
 *                  reference; the expert-parallel exchange cuts the sorted list by it).
 * A counting sort: one launch up to 2048 entries, two above (count per slice, then place; the per-slice counts live
 * in a small array inside the library, so calls that overlap on the GPU from different streams must be serialised).
 * Index values outside [0, num_experts) sort behind every expert; num_experts <= 1024. */
QB200_API int qb200_moe_sort_by_expert(qb200_tensor* order, qb200_tensor* inv_order, qb200_tensor* sorted_inds,
                                       qb200_tensor* token_rows, qb200_tensor* expert_offsets, const qb200_tensor* inds,
                                       int num_experts, qb200_stream s);

/* ---- the tail of the routed-expert block: rows back to token order, times the scores, summed over top-k ----
 * res[t, h] = sum_j round(y[inv_order[t*k + j], h] * scores[t, j]).  Replaces mlx_take_axis(inv_order) +
 * mlx_multiply(norm_scores) + mlx_sum_axis(-2) of moeMLP2 (src/transformer.zig:15036-15042, :15127-15140).
 * y [T*k, H] or [T*k, 1, H] in the order its rows were computed (sorted by expert), scores [.., T, k] and res
 * [.., T, H] of y's dtype (bf16 or f32), inv_order [T*k] int32/int64 or empty (rows already in token order).  With
 * inv_order y may hold any number of rows (entries outside [0, rows) contribute nothing: the expert-parallel block
 * picks its rows out of the returned exchange buffer this way).
 * bf16: each product is rounded to bf16, as the reference's multiply in the activation dtype is, and the sum over k
 * is an ascending accumulate in bf16, rounded after every add: the reference's fused down+reduce kernel documents
 * that as MLX's behaviour and replicates it (src/transformer.zig:20566-20571).  f32: plain fp32 sum. */
QB200_API int qb200_moe_weighted_sum(qb200_tensor* res, const qb200_tensor* y, const qb200_tensor* scores,
                                     const qb200_tensor* inv_order, qb200_stream s);

/* ---- mlx_dequantize (src/mlx.zig:271; caller src/kv_quant.zig:407-430) ----
 * res [..., in] = q*scale + bias, computed as a rounded fp32 product plus a
 * rounded fp32 add, then cast to `dtype` (default: the dtype of scales).
 * global_scale must be NULL/empty (non-affine modes are out of scope). */
QB200_API int qb200_dequantize(qb200_tensor* res, const qb200_tensor* w, const qb200_tensor* scales,
                               const qb200_tensor* biases, qb200_optional_int group_size, qb200_optional_int bits,
                               const char* mode, const qb200_tensor* global_scale, qb200_optional_dtype dtype,
                               qb200_stream s);

/* ---- mlx_quantize (src/mlx.zig:275; caller src/kv_quant.zig:126-162) ----
 * mlx-c returns the vector [q, scales, biases]; here the three results are
 * separate caller-allocated tensors in that order.  w is bf16 or f32
 * [..., D] with D % group_size == 0; scales/biases take w's dtype when w is
 * bf16 and bf16 otherwise. */
QB200_API int qb200_quantize(qb200_tensor* res_q, qb200_tensor* res_scales, qb200_tensor* res_biases,
                             const qb200_tensor* w, qb200_optional_int group_size, qb200_optional_int bits,
                             const char* mode, const qb200_tensor* global_scale, qb200_stream s);

/* ---- decode attention read directly from the packed KV cache ----
 * Replaces kv_quant.quantAttention (src/kv_quant.zig:478-488) and the packed
 * decode kernel + merge (src/transformer.zig:5063-5070, :5204-5246) for
 * T_q == 1, and extends them to a batch of sequences with per-sequence
 * lengths, which the reference serves by dequantising, padding and masking
 * (src/transformer.zig:9758-9792, :10216-10249).  The verify widths T_q = 2..8 of
 * qkvAttnVerifyKernel (src/transformer.zig:5464-5588) are served with mask_mode "causal":
 * query position tq sees the first T - T_q + 1 + tq cache positions (src/transformer.zig:5314-5318);
 * one launch pair per sequence, workspace sized with T_q in place of B.
 *   q            [B, Hq, T_q, D]  bf16 or f32
 *   k_q/k_s/k_b  [B, Hkv, T, D*bits/32 | D/gs | D/gs]  strided cache views
 *   v_q/v_s/v_b  [B, Hkv, T, Dv*bits/32 | Dv/gs | Dv/gs]
 *   mask_mode    "" | "causal" (a no-op at T_q == 1) | "array"
 *   mask_arr     additive row broadcastable to [B, 1, 1, T] in q's dtype or f32
 *                ("array" only; empty otherwise)
 *   kv_lens      empty, or int32 [B] on the device: positions >= kv_lens[b] are masked
 *   res          [B, Hq, T_q, Dv] in q's dtype
 *   workspace    device scratch of at least qb200_kv_decode_attention_workspace_size bytes
 */
QB200_API int qb200_kv_decode_attention(qb200_tensor* res, const qb200_tensor* q, const qb200_tensor* k_q,
                                        const qb200_tensor* k_scales, const qb200_tensor* k_biases,
                                        const qb200_tensor* v_q, const qb200_tensor* v_scales,
                                        const qb200_tensor* v_biases, int bits, int group_size, float scale,
                                        const char* mask_mode, const qb200_tensor* mask_arr,
                                        const qb200_tensor* kv_lens, void* workspace, size_t workspace_bytes,
                                        qb200_stream s);
QB200_API size_t qb200_kv_decode_attention_workspace_size(int64_t B, int64_t Hq, int64_t Hkv, int64_t T,
                                                          int64_t Dv);

/* ---- the same attention over a batch whose sequences own separate caches ----
 * The reference's slots each hold a B = 1 cache with its own capacity and length (src/scheduler.zig:463-480); its
 * batched decode dequantises every slot's cache, pads to the longest and concatenates before one attention call
 * (forwardBatchedDecode, src/transformer.zig:9742-9792; padAndStackBatchedKV, :10165-10211; buildBatchedDecodeMask,
 * :10216-10249).  Here the packed views are read in place: k_q[b] ... v_biases[b] are the six views of sequence b,
 * each [1, Hkv, T_b, last] with its own strides and its own length T_b; q is [num_seqs, Hq, 1, D], res
 * [num_seqs, Hq, 1, Dv].  mask_arr (mode "array") broadcasts to [num_seqs, 1, 1, T_max] with T_max the longest
 * view; kv_lens, when given, further limits sequence b to its first kv_lens[b] positions.  The descriptors are read
 * on the host during the call (they need not outlive it).  Workspace: qb200_kv_decode_attention_ptrs_workspace_size. */
QB200_API int qb200_kv_decode_attention_ptrs(qb200_tensor* res, const qb200_tensor* q, const qb200_tensor* const* k_q,
                                             const qb200_tensor* const* k_scales, const qb200_tensor* const* k_biases,
                                             const qb200_tensor* const* v_q, const qb200_tensor* const* v_scales,
                                             const qb200_tensor* const* v_biases, int num_seqs, int bits, int group_size,
                                             float scale, const char* mask_mode, const qb200_tensor* mask_arr,
                                             const qb200_tensor* kv_lens, void* workspace, size_t workspace_bytes,
                                             qb200_stream s);
QB200_API size_t qb200_kv_decode_attention_ptrs_workspace_size(int64_t num_seqs, int64_t Hq, int64_t Hkv, int64_t T_max,
                                                               int64_t Dv);

/* ---- the same attention for callers that cannot allocate device memory ----
 * No counterpart in the reference (MLX allocates its own temporaries).  Identical arguments and
 * results to qb200_kv_decode_attention minus the workspace: the split-KV partials go to an 8 MiB
 * array built into the library (qb200_kv_decode_attention_noalloc_max_scratch() bytes, held on
 * every GPU that loads the library until the process exits).  Shapes whose partials do not fit are
 * rejected with QB200_ERR_WORKSPACE before anything is launched.  The call itself allocates and
 * frees nothing.  The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress); make that first call outside any stream capture.  All calls on a device
 * share the one array and its contents are whatever the last call left there (each call overwrites
 * every entry it later reads, so nothing needs clearing); two calls whose kernels overlap on the
 * GPU -- different streams, or one stream per thread -- race on it and must be serialised by the
 * caller. */
QB200_API int qb200_kv_decode_attention_noalloc(qb200_tensor* res, const qb200_tensor* q, const qb200_tensor* k_q,
                                                const qb200_tensor* k_scales, const qb200_tensor* k_biases,
                                                const qb200_tensor* v_q, const qb200_tensor* v_scales,
                                                const qb200_tensor* v_biases, int bits, int group_size, float scale,
                                                const char* mask_mode, const qb200_tensor* mask_arr,
                                                const qb200_tensor* kv_lens, qb200_stream s);
QB200_API size_t qb200_kv_decode_attention_noalloc_max_scratch(void);

/* ---- quantise new K/V rows into the cache in place ----
 * Steps 2 and 5 of KVCache.updateAffine (src/transformer.zig:3224-3337):
 * quantise dense [B, Hkv, S, D] and write the triple at token `offset` of the
 * capacity buffers cache_q/cache_s/cache_b [B, Hkv, cap, *]. */
QB200_API int qb200_kv_append(qb200_tensor* cache_q, qb200_tensor* cache_scales, qb200_tensor* cache_biases,
                              const qb200_tensor* dense, int64_t offset, int bits, int group_size, qb200_stream s);

/* ==== the small operators of the batched decode step around the path (forwardBatchedDecode,
 * src/transformer.zig:9562-9924); bf16 activations, one launch each ==== */

/* mlx_fast_rms_norm (src/mlx.zig:319; rmsNorm / rmsNormEps, src/transformer.zig:7770-7779):
 * res[..., i] = round(weight[i] * round(x[..., i] * rsqrt(mean(x^2) + eps))), mean and first product in fp32. */
QB200_API int qb200_rms_norm(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* weight, float eps, qb200_stream s);
/* mlx_add followed by rmsNorm, as the decode step does after the attention and MLP projections
 * (src/transformer.zig:9836-9843, :9856-9859): sum_res = round(a + b), norm_res = rms_norm(sum_res).  Either result
 * may be empty (sum only at the end of the last layer; with b empty this is qb200_rms_norm). */
QB200_API int qb200_add_rms_norm(qb200_tensor* sum_res, qb200_tensor* norm_res, const qb200_tensor* a, const qb200_tensor* b,
                                 const qb200_tensor* weight, float eps, qb200_stream s);
/* mlx_fast_rope_dynamic (src/mlx.zig:324; callers src/transformer.zig:9678, :9735): x [N, heads, 1, D], one position
 * offsets[n] (int32, on the device) per sequence; element i of the first dims/2 pairs with i + dims/2, angle
 * scale * offset * base^(-2i/dims); elements beyond dims pass through.  res may be x.  traditional must be false and
 * freqs empty (a frequency table and the interleaved pairing are declined). */
QB200_API int qb200_rope(qb200_tensor* res, const qb200_tensor* x, int dims, bool traditional, qb200_optional_float base,
                         float scale, const qb200_tensor* offsets, const qb200_tensor* freqs, qb200_stream s);
/* fusedSwiGLU of the dense MLP (computeGeglu, src/transformer.zig:8220-8243): silu(gate) * up with the rounding points
 * of the reference's kernel (src/transformer.zig:19842-19851).  The first call on a device uploads the 128 KiB sigmoid
 * table (call once before capturing a graph). */
QB200_API int qb200_swiglu(qb200_tensor* res, const qb200_tensor* gate, const qb200_tensor* up, qb200_stream s);
/* The rotation of the TurboQuant cache schemes (src/kv_quant.zig:164-403; quantizeTurbo = rotate then mlx_quantize,
 * dequantizeTurbo = mlx_dequantize then rotate): res = x @ R along the last axis, R = diag(sg) H diag(sg) / sqrt(D) with H
 * the Sylvester Hadamard matrix and sg the +-1 vector of the reference's generator seeded with `seed` (TurboState uses
 * 0x9E37 ^ layer for K and 0x85EB ^ layer for V).  R is symmetric and orthogonal, so the same call rotates back.
 * bf16, D a power of two in [32, 1024] (the reference refuses other head dims); res may be x.  Computed as a fast
 * Walsh-Hadamard transform in fp32, scaled by bf16(1 / sqrt(D)) -- the magnitude of every entry of the reference's bf16
 * matrix -- and rounded once; the reference's mlx_matmul sums the same products in another order. */
QB200_API int qb200_turbo_rotate(qb200_tensor* res, const qb200_tensor* x, uint64_t seed, qb200_stream s);
/* The sign vector itself (bit e set = -1), for hosts that build R as a matrix. */
QB200_API int qb200_turbo_signs(uint64_t seed, int n, uint32_t* bits);
/* One new token per sequence into per-sequence packed caches: the per-slot KVCache.update loop of the batched decode
 * (src/transformer.zig:9738-9756; updateAffine, :3224-3337) as one launch for K and V of every sequence.
 * k_q[n] ... v_biases[n]: the capacity buffers [1, Hkv, cap_n, last] of sequence n; dense_k / dense_v
 * [num_seqs, Hkv, 1, D]; offsets[n] (host array) = the token position to write in sequence n. */
QB200_API int qb200_kv_append_seqs(qb200_tensor* const* k_q, qb200_tensor* const* k_scales, qb200_tensor* const* k_biases,
                                   qb200_tensor* const* v_q, qb200_tensor* const* v_scales, qb200_tensor* const* v_biases,
                                   const qb200_tensor* dense_k, const qb200_tensor* dense_v, const int64_t* offsets, int num_seqs,
                                   int bits, int group_size, qb200_stream s);
/* The two steps before the attention of a batched decode tick as one launch: mlx_fast_rope_dynamic on the queries and
 * on the new keys (src/transformer.zig:9678, :9735; non-traditional pairing, position offsets[n] for sequence n), then
 * the cache update above with the rotated keys.  q [num_seqs, Hq, 1, D] is rotated in place; dense_k is read only (its
 * rotated values go to the cache, rounded to bf16 first, so the cache holds exactly what qb200_rope followed by
 * qb200_kv_append_seqs would have written).  dims / 2 must be a multiple of the values per packed word. */
QB200_API int qb200_rope_kv_append_seqs(qb200_tensor* q, int dims, float base, float scale, qb200_tensor* const* k_q,
                                        qb200_tensor* const* k_scales, qb200_tensor* const* k_biases, qb200_tensor* const* v_q,
                                        qb200_tensor* const* v_scales, qb200_tensor* const* v_biases, const qb200_tensor* dense_k,
                                        const qb200_tensor* dense_v, const int64_t* offsets, int num_seqs, int bits, int group_size,
                                        qb200_stream s);

/* ==== checkpoint -> device loader: MLX-format quantized safetensors (host side; the device layout is the file's) ==== */

/* One opened .safetensors file (memory-mapped).  Quantized linears are stored as <name>.weight (uint32 packed codes),
 * <name>.scales and <name>.biases, exactly the triples the operators above take. */
typedef struct qb200_checkpoint qb200_checkpoint;
QB200_API int qb200_checkpoint_open(qb200_checkpoint** out, const char* path);
QB200_API void qb200_checkpoint_close(qb200_checkpoint* ck);
QB200_API int qb200_checkpoint_num_tensors(const qb200_checkpoint* ck);
QB200_API const char* qb200_checkpoint_tensor_name(const qb200_checkpoint* ck, int i);
/* Shape and dtype as loaded (desc->data stays NULL; strides are contiguous); *nbytes = bytes to allocate. */
QB200_API int qb200_checkpoint_tensor_info(const qb200_checkpoint* ck, const char* name, qb200_tensor* desc, size_t* nbytes);
/* Copies the tensor into caller-allocated device memory, synchronously.  An f16 tensor the narrowing rule covers
 * arrives as bf16 (f16 -> f32 exactly, then round to nearest even). */
QB200_API int qb200_checkpoint_load_tensor(const qb200_checkpoint* ck, const char* name, void* device_dst, size_t dst_bytes);
/* The same bytes into host memory (for hosts that stage their own uploads). */
QB200_API int qb200_checkpoint_read_tensor(const qb200_checkpoint* ck, const char* name, void* host_dst, size_t cap, size_t* nbytes);
/* narrowsLoadedF16 (src/model.zig:3030-3061): an f16 tensor named *.scales / *.biases, or any 1-D f16 tensor, is
 * narrowed to bf16 at load time so that it does not promote bf16 activations. */
QB200_API bool qb200_narrows_loaded_f16(const char* name, int ndim, int dtype);
/* affineParamsFromGeometry (src/transformer.zig:16763-16790): bits = w_cols * 32 / in_dim, group = in_dim / s_cols. */
QB200_API int qb200_affine_params_from_geometry(int64_t w_cols, int64_t s_cols, int64_t in_dim, int* bits, int* group_size);
/* config.json's top-level "quantization" object (src/model.zig:1480-1505): bits, group_size, mode ("affine" when absent);
 * QB200_ERR_UNSUPPORTED for a file without one, or for an affine width MLX has no kernels for. */
QB200_API int qb200_config_quantization(const char* json_text, int* bits, int* group_size, char* mode, size_t mode_cap);

/* ==== Chunked persistence of the quantized KV cache: the chunk files of mlx-serve's SSD tier for its prefix cache
 * (src/kv_disk_cache.zig:1-48).  One safetensors file per position range, holding for every layer with a cache the
 * token slice of its six capacity buffers under "l{i}.k", "l{i}.v", "l{i}.ks", "l{i}.kb", "l{i}.vs", "l{i}.vb"
 * (:1062-1074), each [1, Hkv, positions, cols].  The index around the chunks (meta.json, tokens.bin, prefix lookup,
 * eviction) stays with the host. ==== */
/* One layer's capacity buffers [1, Hkv, cap, cols] as qb200_kv_append takes them; k_q.data == NULL: the layer keeps no
 * KV cache (it is left out of a chunk, and skipped when one is restored). */
typedef struct qb200_kv_layer {
  qb200_tensor k_q, k_scales, k_biases, v_q, v_scales, v_biases;
} qb200_kv_layer;
/* Writes positions [pos0, pos1) of every layer to `path` (under a temporary name, then renamed).  Synchronous:
 * returns after the copies on `s` and the write are done. */
QB200_API int qb200_kv_chunk_save(const char* path, const qb200_kv_layer* layers, int n_layers, int64_t pos0, int64_t pos1,
                                  qb200_stream s);
/* restoreKvInto for one chunk (src/kv_disk_cache.zig:320-440): the first `need` stored positions of every layer in
 * the file go to positions [pos0, pos0 + need) of the cache's buffers.  A chunk holding more positions than `need` is
 * sliced down; fewer positions, a missing key of a present layer, another rank, geometry or dtype: QB200_ERR_BAD_SHAPE
 * (a corrupt chunk -- nothing of the file is trusted then; the caller resets the cache and prefills).  Synchronous. */
QB200_API int qb200_kv_chunk_restore(const char* path, const qb200_kv_layer* layers, int n_layers, int64_t pos0, int64_t need,
                                     qb200_stream s);

#ifdef __cplusplus
}
#endif
#endif /* QB200_H */

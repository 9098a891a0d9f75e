// Internal launch interface between the C ABI (api.cu) and the kernels.
// Every launcher returns a cudaError_t and never allocates.
#pragma once
#include <mutex>

#include "common.cuh"

namespace qb {

// Plain launch through cudaLaunchKernelEx (kernel parameters by value, no launch attributes).  Programmatic dependent
// launch was measured for the chain of small kernels of a decode tick (norm, rope, append, attention, merge, SwiGLU)
// and not kept: with it the 13-launch layer tick took 100 / 148 / 164 us at 8 / 16 / 32 sequences against 98 / 133 /
// 148 us without, on the same GPU -- the early-scheduled grids only wait, on SMs the weight-streaming kernels want.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

int report_error(int status, const char* msg);  // api.cu: last-error string + handler
int sm_count();                                 // device.cu: SMs of the current device
std::mutex& setup_mutex();                      // device.cu: guards every first-use-per-device set-up

// ---- elementwise.cu ----
struct DequantArgs {
  const uint32_t* w; const void* s; const void* b; void* out;
  RowMap wmap, sbmap, omap;   // row -> element offset for w, scales/biases, out
  int64_t rows; int64_t d;    // logical row length (values)
  int gs, bits;
  int sb_dtype, out_dtype;    // qb200_dtype
};
cudaError_t launch_dequantize(const DequantArgs& a, cudaStream_t st);

// Score-weighted sum over the top-k axis of the routed-expert block, with the rows taken back from expert order:
// out[t, h] = sum_j round(y[inv[t*k + j], h] * scores[t, j]).
struct MoeSumArgs {
  const void* y; const void* scores; const void* inv; void* out;
  int inv_i64;            // inv may be null: row t*k + j
  int64_t T, topk, H;
  int64_t R;              // rows of y (T * topk unless inv picks rows out of a larger buffer)
  int dtype;              // QB200_BFLOAT16 or QB200_FLOAT32 (y, scores and out)
};
cudaError_t launch_moe_weighted_sum(const MoeSumArgs& a, cudaStream_t st);

// Router of the routed-expert block: the k largest logits of every row, softmax over the row, the k probabilities
// renormalised to sum to one.
struct MoeRouteArgs {
  const void* logits; int* inds; void* scores;
  int64_t T; int E, topk;
  int dtype;              // QB200_BFLOAT16 or QB200_FLOAT32 (logits and scores)
};
cudaError_t launch_moe_route(const MoeRouteArgs& a, cudaStream_t st);

// Stable sort of the flattened top-k index list by expert (moe_sort.cu).  Every output may be null.
struct MoeSortArgs {
  const void* inds; int inds_i64;
  int* order;        // [n]: order[p] = position in inds of the p-th entry in expert order
  int* inv_order;    // [n]: inv_order[order[p]] = p
  int* sorted_inds;  // [n]: inds[order[p]]
  int* token_rows;   // [n]: order[p] / topk (the token a sorted row belongs to)
  int* offsets;      // [E + 1]: rows of expert e are [offsets[e], offsets[e + 1])
  int64_t n; int E; int topk;
};
cudaError_t launch_moe_sort(const MoeSortArgs& a, cudaStream_t st);

// ---- moe_down_reduce.cu: down projection + router weighting + sum over top-k for a few tokens ----
struct MoeDownReduceArgs {
  const void* act; const uint32_t* w; const void* s; const void* b; void* y;
  const void* inds; const void* scores;
  int inds_i64;
  int64_t T, N, K, E, wes, ses;
  int topk, gs, bits, dtype;
};
bool moe_down_reduce_supported(const MoeDownReduceArgs& a);
cudaError_t launch_moe_down_reduce(const MoeDownReduceArgs& a, cudaStream_t st);

struct QuantArgs {
  const void* x; uint32_t* q; void* s; void* b;
  RowMap xmap, qmap, sbmap;
  int64_t rows; int64_t d;
  int gs, bits;
  int x_dtype, sb_dtype;
};
cudaError_t launch_quantize(const QuantArgs& a, cudaStream_t st);

// ---- qmm_generic.cu : any shape, CUDA cores (safety net + transpose=false) ----
struct QmmArgs {
  const void* x; const uint32_t* w; const void* s; const void* b; void* y;
  int x_dtype;                 // bf16 / f32 / f16 (y has the same dtype)
  int64_t M, N, K;
  int64_t ldx, ldw, lds, ldy;  // row pitches in elements
  int gs, bits;
  bool transpose;
  int64_t nbatch;
  BatchMap xb, wb, sb, yb;
};
cudaError_t launch_qmm_generic(const QmmArgs& a, cudaStream_t st);

// ---- qmv_rows.cu : transpose=false at attention widths (attn @ V over the packed value cache), one pass over W ----
bool qmv_rows_supported(const QmmArgs& a);
cudaError_t launch_qmv_rows(const QmmArgs& a, cudaStream_t st);

// ---- qmv_shortk.cu : batched transpose=true with a short contraction (q @ K^T over the packed key cache) ----
bool qmv_shortk_supported(const QmmArgs& a);
cudaError_t launch_qmv_shortk(const QmmArgs& a, cudaStream_t st);

// ---- qmv_mma.cu : small-M weight-streaming kernels (tensor-core dots, HBM-bound) ----
bool qmv_mma_supported(const QmmArgs& a);
cudaError_t launch_qmv_mma(const QmmArgs& a, cudaStream_t st);

// ---- qmv_stream.cu : persistent cp.async-ring weight-streaming kernel (decode widths) ----
bool qmv_stream_supported(const QmmArgs& a);
cudaError_t launch_qmv_stream(const QmmArgs& a, cudaStream_t st);
cudaError_t launch_qmv_stream_multi(const QmmArgs* a, int count, cudaStream_t st);  // same x, <= 4 matrices

// ---- qmv_wide.cu : 9..32 tokens per pass, every packed word read once (stream-K over a persistent grid) ----
bool qmv_wide_supported(const QmmArgs& a);
cudaError_t launch_qmv_wide(const QmmArgs& a, cudaStream_t st);
cudaError_t launch_qmv_wide_multi(const QmmArgs* a, int count, cudaStream_t st);   // same x, <= 4 matrices
int qmv_wide_error_code();    // 0, or the code of a bounded wait that expired
void qmv_wide_error_reset();

// ---- qmm_tc.cu : prefill widths on tcgen05 (dequantise into the swizzled smem operand, TMEM accumulate) ----
bool qmm_tc_supported(const QmmArgs& a);
cudaError_t launch_qmm_tc(const QmmArgs& a, cudaStream_t st);
bool qmm_tc_multi_supported(const QmmArgs* a, int count);   // several matrices, same activations, one launch (<= 256 tokens)
cudaError_t launch_qmm_tc_multi(const QmmArgs* a, int count, cudaStream_t st);
void qmm_tc_error_reset();
int qmm_tc_error_code();  // 0, or the code of a bounded wait that expired in the last failing launch
struct GatherArgs;
bool gather_tc_supported(const GatherArgs& a);   // rows sorted by expert, many rows: grouped GEMM on the same kernel
cudaError_t launch_gather_tc(const GatherArgs& a, cudaStream_t st);

struct GatherArgs {
  const void* x; const uint32_t* w; const void* s; const void* b; void* y;
  int x_dtype;
  int64_t I;                   // number of output batch elements
  int64_t M, N, K;
  int64_t x_batch_stride;      // elements between consecutive x batch entries ([XB, M, K] contiguous)
  int64_t XB;                  // number of x batch entries
  int64_t w_expert_stride, s_expert_stride;  // elements per expert
  int64_t E;
  const void* lhs; int lhs_dtype;   // may be null: lhs(i) = broadcast position
  const void* rhs; int rhs_dtype;
  // broadcast of x batch dims against the index shape when lhs == null:
  BatchMap xbcast;             // index-space position -> x batch entry (stride in batch entries)
  int gs, bits;
  bool sorted;
  // fused gate/up form (gather_stream only): a second bank of the same geometry, y = silu(x . w^T) * (x . w2^T)
  const uint32_t* w2 = nullptr; const void* s2 = nullptr; const void* b2 = nullptr;
};
bool gather_mma_supported(const GatherArgs& a);
cudaError_t launch_gather_mma(const GatherArgs& a, cudaStream_t st);
cudaError_t launch_gather_generic(const GatherArgs& a, cudaStream_t st);
// sigmoid of every bf16 bit pattern as bf16 (device table, uploaded on first use; null + *err when that fails)
const uint16_t* sigmoid_table(cudaStream_t st, cudaError_t* err);
// few rows, each with its own expert (single-token decode): a CTA per (row, 16 output rows), moe_down_reduce.cu
bool gather_small_supported(const GatherArgs& a);
cudaError_t launch_gather_small(const GatherArgs& a, cudaStream_t st);
bool gather_stream_supported(const GatherArgs& a);   // qmv_stream.cu: persistent streaming kernel, gather form
cudaError_t launch_gather_stream(const GatherArgs& a, cudaStream_t st);

// ---- decode_step.cu: the small operators of the batched decode step (bf16) ----
cudaError_t launch_rms_norm(const uint16_t* a, const uint16_t* b, const uint16_t* w, uint16_t* sum_out, uint16_t* norm_out,
                            int64_t rows, int d, int64_t lda, int64_t ldb, int64_t lds, int64_t ldn, float eps, cudaStream_t st);
cudaError_t launch_rope(const uint16_t* x, uint16_t* out, const int32_t* offsets, int64_t n, int heads, int d, int dims, float base,
                        float scale, int64_t xsn, int64_t xsh, int64_t osn, int64_t osh, cudaStream_t st);
cudaError_t launch_turbo_rotate(const uint16_t* x, uint16_t* out, int64_t rows, int d, int64_t ldx, int64_t ldo, const uint32_t* signs,
                                cudaStream_t st);
cudaError_t launch_swiglu(const uint16_t* gate, const uint16_t* up, uint16_t* out, int64_t rows, int d, int64_t ldg, int64_t ldu,
                          int64_t ldo, cudaStream_t st);
struct KvAppendSeqsArgs {     // host side: [K, V] lists over the sequences, token rows already resolved
  uint32_t* const* q[2]; uint16_t* const* s[2]; uint16_t* const* b[2];
  const int64_t* q_head[2]; const int64_t* sb_head[2];
  const uint16_t* dense[2]; int64_t dsn[2], dsh[2];
  int n, heads, d[2], gs, bits;
  // rope form (rope_dims > 0): K is rotated on its way into the cache and the queries rq [n, q_heads, 1, d[0]] in place,
  // each sequence at position pos[i]
  const int* pos = nullptr;
  uint16_t* rq = nullptr; int64_t qsn = 0, qsh = 0; int q_heads = 0;
  int rope_dims = 0; float rope_base = 0.f, rope_scale = 1.f;
};
cudaError_t launch_kv_append_seqs(const KvAppendSeqsArgs& a, cudaStream_t st);

// ---- kv_attn.cu ----
struct KvAttnArgs {
  const void* q; void* out; int q_dtype;
  const uint32_t* kq; const void* ks; const void* kb;
  const uint32_t* vq; const void* vs; const void* vb;
  int64_t B, Hq, Hkv, T, D, Dv;
  int64_t q_str[2], o_str[2];          // (batch, head) strides in elements; last dim contiguous
  int64_t kq_str[3], ksb_str[3];       // (batch, head, token)
  int64_t vq_str[3], vsb_str[3];
  int gs, bits;
  float scale;
  const int32_t* kv_lens;              // device, may be null
  const void* mask; int mask_dtype; int64_t mask_bstride;  // additive row [B?, T], may be null
  void* workspace; size_t workspace_bytes;
};
// Per-sequence cache views for a batch whose sequences own separate caches (the reference's slots each hold a
// B = 1 cache with its own capacity, src/scheduler.zig:463-480): base pointers, (head, token) strides in
// elements and the view's length.  The table travels as a kernel parameter.
constexpr int kMaxSeqPtrs = 32;   // sequences per launch (the reference batches at most 32 slots, src/scheduler.zig:5147)
struct KvSeq {
  const uint32_t* kq; const void* ks; const void* kb;
  const uint32_t* vq; const void* vs; const void* vb;
  int64_t kq_str[2], ksb_str[2], vq_str[2], vsb_str[2];
  int64_t T;
};
struct KvSeqTable { KvSeq s[kMaxSeqPtrs]; };
struct KvNoTable {};
size_t kv_attn_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t T, int64_t Dv);
bool kv_attn_supported(const KvAttnArgs& a);
bool kv_fast_supported(const KvAttnArgs& a, const KvSeqTable* seqs = nullptr);
cudaError_t launch_kv_attn(const KvAttnArgs& a, cudaStream_t st, const KvSeqTable* seqs = nullptr);  // seqs: a.B <= kMaxSeqPtrs views, a.T their longest

}  // namespace qb

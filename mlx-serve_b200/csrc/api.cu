// C ABI of libqb200: argument validation, shape inference and kernel dispatch.
// Every entry point mirrors the mlx-c operator mlx-serve binds in src/mlx.zig
// (see include/qb200.h for the line references).  Validation happens entirely
// on the host before any CUDA call, so bad input never reaches a kernel.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "kernels.h"

using namespace qb;

namespace {

thread_local std::string g_last_error;
std::mutex g_handler_mu;
qb200_error_handler_func g_handler = nullptr;
void* g_handler_data = nullptr;
void (*g_handler_dtor)(void*) = nullptr;

int fail(int status, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  qb200_error_handler_func h;
  void* d;
  {
    std::lock_guard<std::mutex> lk(g_handler_mu);
    h = g_handler;
    d = g_handler_data;
  }
  if (h) h(buf, d);
  return status;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(QB200_ERR_CUDA, "%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
}

bool is_empty(const qb200_tensor* t) { return t == nullptr || (t->data == nullptr && t->ndim == 0); }

int dtype_size(int dt) {
  switch (dt) {
    case QB200_BOOL: case QB200_UINT8: case QB200_INT8: return 1;
    case QB200_UINT16: case QB200_INT16: case QB200_FLOAT16: case QB200_BFLOAT16: return 2;
    case QB200_UINT32: case QB200_INT32: case QB200_FLOAT32: return 4;
    case QB200_UINT64: case QB200_INT64: case QB200_FLOAT64: return 8;
    default: return 0;
  }
}
bool is_float_dtype(int dt) { return dt == QB200_BFLOAT16 || dt == QB200_FLOAT32 || dt == QB200_FLOAT16; }
bool is_index_dtype(int dt) { return dt == QB200_INT32 || dt == QB200_UINT32 || dt == QB200_INT64; }

// Basic descriptor sanity.  Returns 0 or a status (after recording the message).
int check_tensor(const qb200_tensor* t, const char* name, int min_ndim) {
  if (t == nullptr) return fail(QB200_ERR_BAD_ARG, "%s: null tensor", name);
  if (t->ndim < min_ndim || t->ndim > QB200_MAX_DIMS)
    return fail(QB200_ERR_BAD_SHAPE, "%s: ndim %d outside [%d, %d]", name, t->ndim, min_ndim, QB200_MAX_DIMS);
  if (dtype_size(t->dtype) == 0) return fail(QB200_ERR_BAD_DTYPE, "%s: unknown dtype %d", name, t->dtype);
  int64_t n = 1;
  for (int d = 0; d < t->ndim; ++d) {
    if (t->shape[d] < 0) return fail(QB200_ERR_BAD_SHAPE, "%s: negative extent in dim %d", name, d);
    if (t->stride[d] < 0) return fail(QB200_ERR_BAD_STRIDE, "%s: negative stride in dim %d", name, d);
    n *= t->shape[d];
  }
  if (n > 0 && t->data == nullptr) return fail(QB200_ERR_BAD_ARG, "%s: null data pointer", name);
  if (t->ndim > 0 && t->shape[t->ndim - 1] > 1 && t->stride[t->ndim - 1] != 1)
    return fail(QB200_ERR_BAD_STRIDE, "%s: last axis must be contiguous (stride %lld)", name,
                (long long)t->stride[t->ndim - 1]);
  return 0;
}

int64_t numel(const qb200_tensor* t) {
  int64_t n = 1;
  for (int d = 0; d < t->ndim; ++d) n *= t->shape[d];
  return n;
}

bool fully_contiguous(const qb200_tensor* t) {
  int64_t expect = 1;
  for (int d = t->ndim - 1; d >= 0; --d) {
    if (t->shape[d] != 1 && t->stride[d] != expect) return false;
    expect *= t->shape[d];
  }
  return true;
}

int resolve_mode(const char* mode, qb200_optional_int group_size, qb200_optional_int bits, int* gs, int* nb) {
  if (mode == nullptr || std::strcmp(mode, "affine") != 0)
    return fail(QB200_ERR_UNSUPPORTED, "quantization mode '%s' is not served (only \"affine\")", mode ? mode : "(null)");
  *gs = group_size.has_value ? group_size.value : 64;
  *nb = bits.has_value ? bits.value : 4;
  if (*nb != 2 && *nb != 4 && *nb != 8) return fail(QB200_ERR_UNSUPPORTED, "bits=%d is not served (2, 4, 8)", *nb);
  if (*gs != 32 && *gs != 64 && *gs != 128)
    return fail(QB200_ERR_UNSUPPORTED, "group_size=%d is not served (32, 64, 128)", *gs);
  return 0;
}

// Rows of a tensor = all dims but the last.
RowMap make_rowmap(const qb200_tensor* t) {
  RowMap m;
  m.nd = t->ndim - 1;
  bool contig = true;
  int64_t expect = t->ndim >= 2 ? t->stride[t->ndim - 2] : t->shape[t->ndim - 1];
  m.row_pitch = expect;
  for (int d = t->ndim - 2; d >= 0; --d) {
    m.shape[d] = t->shape[d];
    m.stride[d] = t->stride[d];
    if (t->shape[d] != 1 && t->stride[d] != expect) contig = false;
    expect *= t->shape[d];
  }
  for (int d = m.nd; d < kMaxLead; ++d) { m.shape[d] = 1; m.stride[d] = 0; }
  if (m.nd == 0) m.row_pitch = 0;
  m.contiguous = contig ? 1 : 0;
  return m;
}

int64_t rows_of(const qb200_tensor* t) {
  int64_t n = 1;
  for (int d = 0; d < t->ndim - 1; ++d) n *= t->shape[d];
  return n;
}

bool same_leading(const qb200_tensor* a, const qb200_tensor* b) {
  if (a->ndim != b->ndim) return false;
  for (int d = 0; d < a->ndim - 1; ++d)
    if (a->shape[d] != b->shape[d]) return false;
  return true;
}
bool same_strides(const qb200_tensor* a, const qb200_tensor* b) {
  if (a->ndim != b->ndim) return false;
  for (int d = 0; d < a->ndim; ++d)
    if (a->shape[d] != 1 && a->stride[d] != b->stride[d]) return false;
  return true;
}

struct QmmPlan {
  int64_t M, N, K;
  int nb;                     // batch dims
  int64_t bshape[kMaxLead];
  bool x_was_1d;
};

int plan_qmm(const qb200_tensor* x, const qb200_tensor* w, const qb200_tensor* scales, bool transpose, int gs,
             int bits, QmmPlan* p) {
  const int vpw = 32 / bits;
  p->x_was_1d = x->ndim == 1;
  const int xnd = x->ndim;
  p->K = x->shape[xnd - 1];
  p->M = p->x_was_1d ? 1 : x->shape[xnd - 2];
  const int64_t wrows = w->shape[w->ndim - 2], wcols = w->shape[w->ndim - 1];
  if (transpose) {
    p->N = wrows;
    if (wcols * vpw != p->K)
      return fail(QB200_ERR_BAD_SHAPE, "quantized_matmul: x inner dim %lld != w cols %lld * %d", (long long)p->K,
                  (long long)wcols, vpw);
    if (p->K % gs != 0 || scales->shape[scales->ndim - 1] != p->K / gs)
      return fail(QB200_ERR_BAD_SHAPE, "quantized_matmul: scales last dim %lld != K/group_size = %lld",
                  (long long)scales->shape[scales->ndim - 1], (long long)(p->K / gs));
  } else {
    p->N = wcols * vpw;
    if (wrows != p->K)
      return fail(QB200_ERR_BAD_SHAPE, "quantized_matmul: x inner dim %lld != w rows %lld (transpose_w=false)",
                  (long long)p->K, (long long)wrows);
    if (p->N % gs != 0 || scales->shape[scales->ndim - 1] != p->N / gs)
      return fail(QB200_ERR_BAD_SHAPE, "quantized_matmul: scales last dim %lld != N/group_size = %lld",
                  (long long)scales->shape[scales->ndim - 1], (long long)(p->N / gs));
  }
  if (scales->shape[scales->ndim - 2] != wrows)
    return fail(QB200_ERR_BAD_SHAPE, "quantized_matmul: scales rows %lld != w rows %lld",
                (long long)scales->shape[scales->ndim - 2], (long long)wrows);
  const int xb = p->x_was_1d ? 0 : xnd - 2, wb = w->ndim - 2;
  p->nb = xb > wb ? xb : wb;
  for (int d = 0; d < p->nb; ++d) {
    const int xd = d - (p->nb - xb), wd = d - (p->nb - wb);
    const int64_t xs = xd >= 0 ? x->shape[xd] : 1, ws = wd >= 0 ? w->shape[wd] : 1;
    if (xs != ws && xs != 1 && ws != 1)
      return fail(QB200_ERR_BAD_SHAPE, "quantized_matmul: batch dims do not broadcast (%lld vs %lld)", (long long)xs,
                  (long long)ws);
    p->bshape[d] = xs == 1 ? ws : xs;
  }
  return 0;
}

// Broadcast batch map of an operand whose last `inner` dims are the matrix.
BatchMap make_batchmap(const qb200_tensor* t, int inner, const QmmPlan& p) {
  BatchMap m;
  m.nd = p.nb;
  const int tb = t->ndim - inner;
  for (int d = 0; d < kMaxLead; ++d) { m.shape[d] = 1; m.stride[d] = 0; }
  for (int d = 0; d < p.nb; ++d) {
    m.shape[d] = p.bshape[d];
    const int td = d - (p.nb - tb);
    m.stride[d] = (td >= 0 && t->shape[td] != 1) ? t->stride[td] : 0;
  }
  return m;
}

}  // namespace

namespace qb {
// Records an error message and notifies the handler, for entry points that live in other files.
int report_error(int status, const char* msg) { return fail(status, "%s", msg); }
}  // namespace qb

extern "C" {

QB200_API void qb200_set_error_handler(qb200_error_handler_func handler, void* data, void (*dtor)(void*)) {
  std::lock_guard<std::mutex> lk(g_handler_mu);
  if (g_handler_dtor && g_handler_data) g_handler_dtor(g_handler_data);
  g_handler = handler;
  g_handler_data = data;
  g_handler_dtor = dtor;
}

QB200_API const char* qb200_last_error(void) { return g_last_error.c_str(); }
QB200_API const char* qb200_version(void) { return "qb200 0.1 (sm_100a)"; }
QB200_API int qb200_debug_tc_status(void) {
  const int tc = qmm_tc_error_code();
  return tc ? tc : qmv_wide_error_code();
}
QB200_API void qb200_debug_tc_reset(void) {
  qmm_tc_error_reset();
  qmv_wide_error_reset();
}

QB200_API int qb200_quantized_matmul_shape(const qb200_tensor* x, const qb200_tensor* w, const qb200_tensor* scales,
                                           bool transpose_w, qb200_optional_int group_size, qb200_optional_int bits,
                                           int64_t* out_shape, int32_t* out_ndim) {
  int gs, nb, st;
  if ((st = resolve_mode("affine", group_size, bits, &gs, &nb))) return st;
  if ((st = check_tensor(x, "x", 1)) || (st = check_tensor(w, "w", 2)) || (st = check_tensor(scales, "scales", 2)))
    return st;
  if (out_shape == nullptr || out_ndim == nullptr) return fail(QB200_ERR_BAD_ARG, "null output shape");
  QmmPlan p;
  if ((st = plan_qmm(x, w, scales, transpose_w, gs, nb, &p))) return st;
  int n = 0;
  for (int d = 0; d < p.nb; ++d) out_shape[n++] = p.bshape[d];
  if (!p.x_was_1d) out_shape[n++] = p.M;
  out_shape[n++] = p.N;
  *out_ndim = n;
  return QB200_OK;
}

// Validates one quantized_matmul request and fills the kernel arguments.  *empty is set when the
// result has no elements (nothing to launch).
static int prepare_qmm(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* w, const qb200_tensor* scales,
                       const qb200_tensor* biases, bool transpose_w, qb200_optional_int group_size,
                       qb200_optional_int bits, const char* mode, QmmArgs* out, bool* empty) {
  int gs, nb, st;
  if ((st = resolve_mode(mode, group_size, bits, &gs, &nb))) return st;
  if (is_empty(biases)) return fail(QB200_ERR_UNSUPPORTED, "quantized_matmul: biases are required (affine mode)");
  if ((st = check_tensor(res, "res", 1)) || (st = check_tensor(x, "x", 1)) || (st = check_tensor(w, "w", 2)) ||
      (st = check_tensor(scales, "scales", 2)) || (st = check_tensor(biases, "biases", 2)))
    return st;
  if (w->dtype != QB200_UINT32) return fail(QB200_ERR_BAD_DTYPE, "quantized_matmul: w must be uint32");
  if (!is_float_dtype(x->dtype)) return fail(QB200_ERR_BAD_DTYPE, "quantized_matmul: x must be bf16, f16 or f32");
  if (scales->dtype != QB200_BFLOAT16 || biases->dtype != QB200_BFLOAT16)
    return fail(QB200_ERR_UNSUPPORTED, "quantized_matmul: scales and biases must be bf16");
  if (res->dtype != x->dtype) return fail(QB200_ERR_BAD_DTYPE, "quantized_matmul: res dtype must equal x dtype");
  if (scales->ndim != w->ndim || !same_leading(scales, w) || !same_leading(biases, scales) ||
      biases->shape[biases->ndim - 1] != scales->shape[scales->ndim - 1])
    return fail(QB200_ERR_BAD_SHAPE, "quantized_matmul: w, scales and biases must share their leading shape");
  if (!same_strides(scales, biases))
    return fail(QB200_ERR_BAD_STRIDE, "quantized_matmul: scales and biases must have identical strides");
  QmmPlan p;
  if ((st = plan_qmm(x, w, scales, transpose_w, gs, nb, &p))) return st;
  // expected result shape
  int64_t eshape[QB200_MAX_DIMS];
  int en = 0;
  for (int d = 0; d < p.nb; ++d) eshape[en++] = p.bshape[d];
  if (!p.x_was_1d) eshape[en++] = p.M;
  eshape[en++] = p.N;
  if (res->ndim != en) return fail(QB200_ERR_BAD_SHAPE, "quantized_matmul: res ndim %d, expected %d", res->ndim, en);
  for (int d = 0; d < en; ++d)
    if (res->shape[d] != eshape[d])
      return fail(QB200_ERR_BAD_SHAPE, "quantized_matmul: res dim %d is %lld, expected %lld", d,
                  (long long)res->shape[d], (long long)eshape[d]);

  QmmArgs& a = *out;
  a.x = x->data; a.w = (const uint32_t*)w->data; a.s = scales->data; a.b = biases->data; a.y = res->data;
  a.x_dtype = x->dtype;
  a.M = p.M; a.N = p.N; a.K = p.K;
  a.ldx = p.x_was_1d ? p.K : x->stride[x->ndim - 2];
  a.ldw = w->stride[w->ndim - 2];
  a.lds = scales->stride[scales->ndim - 2];
  a.ldy = p.x_was_1d ? p.N : res->stride[res->ndim - 2];
  a.gs = gs; a.bits = nb; a.transpose = transpose_w;
  a.nbatch = 1;
  for (int d = 0; d < p.nb; ++d) a.nbatch *= p.bshape[d];
  a.xb = make_batchmap(x, p.x_was_1d ? 1 : 2, p);
  a.wb = make_batchmap(w, 2, p);
  a.sb = make_batchmap(scales, 2, p);
  a.yb = make_batchmap(res, p.x_was_1d ? 1 : 2, p);
  *empty = (a.M == 0 || a.N == 0 || a.nbatch == 0);
  if (!*empty && a.K == 0) return fail(QB200_ERR_BAD_SHAPE, "quantized_matmul: empty contraction axis");
  return QB200_OK;
}

// Routing by token count.  Up to 8 tokens: the narrow streaming kernel (one launch).  9 .. 32 (bf16 activations): the
// wide streaming kernel, which reads every packed word once for up to 64 tokens per pass.  Above that the
// tensor-core kernel, whose time does not depend on the token count up to 128 (measured on the C2 layer through the
// batch entry: 110 us at 32 tokens and 170 us at 64 on the wide kernel, 140 / 143 / 149 us at 32 / 64 / 128 on the
// tensor-core kernel).  QB200_WIDE_MAX_TOKENS in the environment moves the upper limit (0 turns the wide kernel off,
// 64 is the most it serves; a diagnostic for measuring the crossover, read once).
static int64_t wide_max_tokens() {
  static const int64_t v = [] {
    const char* e = getenv("QB200_WIDE_MAX_TOKENS");
    return e ? (int64_t)atoll(e) : (int64_t)32;
  }();
  return v;
}
static bool takes_wide(const QmmArgs& a) { return a.M > 8 && a.M <= wide_max_tokens() && qmv_wide_supported(a); }

static cudaError_t dispatch_qmm(const QmmArgs& a, cudaStream_t s) {
  if (!a.transpose) return qmv_rows_supported(a) ? launch_qmv_rows(a, s) : launch_qmm_generic(a, s);
  if (a.nbatch > 1 && qmv_shortk_supported(a)) return launch_qmv_shortk(a, s);   // one W per batch element, short K: q @ K^T
  if (takes_wide(a)) return launch_qmv_wide(a, s);
  if (a.M > wide_max_tokens() && a.M > 8 && qmm_tc_supported(a)) return launch_qmm_tc(a, s);
  if (a.M > 8 && !qmv_stream_supported(a) && qmm_tc_supported(a)) return launch_qmm_tc(a, s);
  if (qmv_stream_supported(a)) return launch_qmv_stream(a, s);
  if (qmv_mma_supported(a)) return launch_qmv_mma(a, s);
  return launch_qmm_generic(a, s);
}

QB200_API int qb200_quantized_matmul(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* w,
                                     const qb200_tensor* scales, const qb200_tensor* biases, bool transpose_w,
                                     qb200_optional_int group_size, qb200_optional_int bits, const char* mode,
                                     qb200_stream s) {
  QmmArgs a;
  bool empty = false;
  int st = prepare_qmm(res, x, w, scales, biases, transpose_w, group_size, bits, mode, &a, &empty);
  if (st) return st;
  if (empty) return QB200_OK;
  cudaError_t e = dispatch_qmm(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "quantized_matmul");
  return QB200_OK;
}

QB200_API int qb200_quantized_matmul_batch(qb200_tensor* const* res, const qb200_tensor* x,
                                           const qb200_tensor* const* w, const qb200_tensor* const* scales,
                                           const qb200_tensor* const* biases, int count, bool transpose_w,
                                           qb200_optional_int group_size, qb200_optional_int bits, const char* mode,
                                           qb200_stream s) {
  if (count < 0 || (count > 0 && (!res || !w || !scales || !biases)))
    return fail(QB200_ERR_BAD_ARG, "quantized_matmul_batch: null operand list");
  constexpr int kChunk = 4;
  for (int i0 = 0; i0 < count; i0 += kChunk) {
    const int n = count - i0 < kChunk ? count - i0 : kChunk;
    QmmArgs a[kChunk];
    bool empty[kChunk];
    bool fuse = n > 1, wide = n > 1;
    for (int i = 0; i < n; ++i) {
      int st = prepare_qmm(res[i0 + i], x, w[i0 + i], scales[i0 + i], biases[i0 + i], transpose_w, group_size, bits,
                           mode, &a[i], &empty[i]);
      if (st) return st;
      // the matrices share a launch where the single call would take a streaming kernel (same rule as dispatch_qmm)
      wide = wide && !empty[i] && takes_wide(a[i]) && a[i].K == a[0].K;
      fuse = fuse && !empty[i] && a[i].M <= 8 && qmv_stream_supported(a[i]) && a[i].K == a[0].K;
    }
    // beyond the streaming kernels' widths, up to 256 tokens: one launch of the tensor-core kernel over all matrices
    bool tc = n > 1 && !wide && !fuse;
    for (int i = 0; i < n && tc; ++i) tc = !empty[i] && a[i].M > wide_max_tokens() && a[i].M > 8;
    tc = tc && qmm_tc_multi_supported(a, n);
    cudaError_t e = cudaSuccess;
    if (wide) {
      e = launch_qmv_wide_multi(a, n, (cudaStream_t)s);
    } else if (tc) {
      e = launch_qmm_tc_multi(a, n, (cudaStream_t)s);
    } else if (fuse) {
      e = launch_qmv_stream_multi(a, n, (cudaStream_t)s);
    } else {
      for (int i = 0; i < n && e == cudaSuccess; ++i)
        if (!empty[i]) e = dispatch_qmm(a[i], (cudaStream_t)s);
    }
    if (e != cudaSuccess) return cuda_fail(e, "quantized_matmul_batch");
  }
  return QB200_OK;
}

// Validation and geometry of one gather_qmm call; *skip is set when there is nothing to compute.
static int prepare_gather(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* w,
                          const qb200_tensor* scales, const qb200_tensor* biases,
                          const qb200_tensor* lhs_indices, const qb200_tensor* rhs_indices, bool transpose_w,
                          qb200_optional_int group_size, qb200_optional_int bits, const char* mode,
                          bool sorted_indices, GatherArgs* out, bool* skip) {
  *skip = false;
  int gs, nb, st;
  if ((st = resolve_mode(mode, group_size, bits, &gs, &nb))) return st;
  if (!transpose_w) return fail(QB200_ERR_UNSUPPORTED, "gather_qmm: only transpose_w=true is served");
  if (is_empty(biases)) return fail(QB200_ERR_UNSUPPORTED, "gather_qmm: biases are required (affine mode)");
  if (is_empty(rhs_indices)) return fail(QB200_ERR_UNSUPPORTED, "gather_qmm: rhs_indices are required");
  if ((st = check_tensor(res, "res", 2)) || (st = check_tensor(x, "x", 2)) || (st = check_tensor(w, "w", 3)) ||
      (st = check_tensor(scales, "scales", 3)) || (st = check_tensor(biases, "biases", 3)) ||
      (st = check_tensor(rhs_indices, "rhs_indices", 0)))
    return st;
  if (w->ndim != 3 || scales->ndim != 3 || biases->ndim != 3)
    return fail(QB200_ERR_UNSUPPORTED, "gather_qmm: w, scales, biases must be [E, N, *]");
  if (w->dtype != QB200_UINT32) return fail(QB200_ERR_BAD_DTYPE, "gather_qmm: w must be uint32");
  if (!is_float_dtype(x->dtype)) return fail(QB200_ERR_BAD_DTYPE, "gather_qmm: x must be bf16, f16 or f32");
  if (scales->dtype != QB200_BFLOAT16 || biases->dtype != QB200_BFLOAT16)
    return fail(QB200_ERR_UNSUPPORTED, "gather_qmm: scales and biases must be bf16");
  if (res->dtype != x->dtype) return fail(QB200_ERR_BAD_DTYPE, "gather_qmm: res dtype must equal x dtype");
  if (!is_index_dtype(rhs_indices->dtype)) return fail(QB200_ERR_BAD_DTYPE, "gather_qmm: rhs_indices must be int32/uint32/int64");
  // Operands reaching gather_qmm must be row-contiguous (mlx-serve docs/gotchas/engine-mlx.md:16-20);
  // non-contiguous ones are rejected instead of being read wrongly.
  if (!fully_contiguous(w) || !fully_contiguous(scales) || !fully_contiguous(biases))
    return fail(QB200_ERR_BAD_STRIDE, "gather_qmm: w, scales and biases must be contiguous");
  if (!fully_contiguous(x) || !fully_contiguous(res) || !fully_contiguous(rhs_indices))
    return fail(QB200_ERR_BAD_STRIDE, "gather_qmm: x, res and indices must be contiguous");
  const int vpw = 32 / nb;
  const int64_t E = w->shape[0], N = w->shape[1], K = w->shape[2] * vpw;
  const int64_t M = x->shape[x->ndim - 2];
  if (x->shape[x->ndim - 1] != K)
    return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: x inner dim %lld != w cols %lld * %d",
                (long long)x->shape[x->ndim - 1], (long long)w->shape[2], vpw);
  if (K % gs != 0 || scales->shape[0] != E || scales->shape[1] != N || scales->shape[2] != K / gs ||
      biases->shape[0] != E || biases->shape[1] != N || biases->shape[2] != K / gs)
    return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: scales/biases must be [E, N, K/group_size]");
  const int ind = rhs_indices->ndim;
  if (ind + 2 > QB200_MAX_DIMS) return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: too many index dims");
  if (res->ndim != ind + 2) return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: res ndim %d, expected %d", res->ndim, ind + 2);
  for (int d = 0; d < ind; ++d)
    if (res->shape[d] != rhs_indices->shape[d])
      return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: res dim %d != index dim", d);
  if (res->shape[ind] != M || res->shape[ind + 1] != N)
    return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: res inner dims must be [M=%lld, N=%lld]", (long long)M, (long long)N);

  GatherArgs a;
  a.x = x->data; a.w = (const uint32_t*)w->data; a.s = scales->data; a.b = biases->data; a.y = res->data;
  a.x_dtype = x->dtype;
  a.I = numel(rhs_indices);
  a.M = M; a.N = N; a.K = K;
  a.x_batch_stride = M * K;
  a.XB = 1;
  for (int d = 0; d < x->ndim - 2; ++d) a.XB *= x->shape[d];
  a.w_expert_stride = N * w->shape[2];
  a.s_expert_stride = N * (K / gs);
  a.E = E;
  a.rhs = rhs_indices->data; a.rhs_dtype = rhs_indices->dtype;
  a.lhs = nullptr; a.lhs_dtype = QB200_INT32;
  a.xbcast.nd = ind;
  for (int d = 0; d < kMaxLead; ++d) { a.xbcast.shape[d] = 1; a.xbcast.stride[d] = 0; }
  if (!is_empty(lhs_indices)) {
    if ((st = check_tensor(lhs_indices, "lhs_indices", 0))) return st;
    if (!is_index_dtype(lhs_indices->dtype)) return fail(QB200_ERR_BAD_DTYPE, "gather_qmm: lhs_indices must be int32/uint32/int64");
    if (lhs_indices->ndim != ind || !fully_contiguous(lhs_indices))
      return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: lhs_indices must match rhs_indices and be contiguous");
    for (int d = 0; d < ind; ++d)
      if (lhs_indices->shape[d] != rhs_indices->shape[d])
        return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: lhs_indices shape != rhs_indices shape");
    a.lhs = lhs_indices->data; a.lhs_dtype = lhs_indices->dtype;
  } else {
    // broadcast x's batch dims against the index shape
    const int xbn = x->ndim - 2;
    if (xbn > ind) return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: x has more batch dims than the indices");
    int64_t run = 1;
    for (int d = ind - 1; d >= 0; --d) {
      const int xd = d - (ind - xbn);
      const int64_t xs = xd >= 0 ? x->shape[xd] : 1;
      a.xbcast.shape[d] = rhs_indices->shape[d];
      if (xs == 1) a.xbcast.stride[d] = 0;
      else if (xs == rhs_indices->shape[d]) { a.xbcast.stride[d] = run; }
      else return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: x batch dim %lld does not broadcast against index dim %lld",
                       (long long)xs, (long long)rhs_indices->shape[d]);
      run *= xs;
    }
  }
  a.gs = gs; a.bits = nb; a.sorted = sorted_indices;
  *out = a;
  if (a.I == 0 || M == 0 || N == 0) { *skip = true; return QB200_OK; }
  if (K == 0) return fail(QB200_ERR_BAD_SHAPE, "gather_qmm: empty contraction axis");
  return QB200_OK;
}

QB200_API int qb200_gather_qmm(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* w,
                               const qb200_tensor* scales, const qb200_tensor* biases,
                               const qb200_tensor* lhs_indices, const qb200_tensor* rhs_indices, bool transpose_w,
                               qb200_optional_int group_size, qb200_optional_int bits, const char* mode,
                               bool sorted_indices, qb200_stream s) {
  GatherArgs a;
  bool skip = false;
  const int st = prepare_gather(res, x, w, scales, biases, lhs_indices, rhs_indices, transpose_w, group_size, bits, mode,
                                sorted_indices, &a, &skip);
  if (st || skip) return st;
  cudaError_t e;
  // Few rows per expert: stream every hit expert once.  Many sorted rows (MoE prefill): grouped GEMM on the
  // tensor-core kernel, from 32 rows per expert on average.
  const bool many = a.I >= 32 * a.E && a.I >= 1024;
  // Up to 16 rows (single-token decode: every row its own expert): a CTA per (row, 16 output rows).
  if (gather_small_supported(a)) e = launch_gather_small(a, (cudaStream_t)s);
  else if (many && gather_tc_supported(a)) e = launch_gather_tc(a, (cudaStream_t)s);
  else if (gather_stream_supported(a)) e = launch_gather_stream(a, (cudaStream_t)s);
  else if (gather_tc_supported(a) && a.I >= 1024) e = launch_gather_tc(a, (cudaStream_t)s);
  else if (gather_mma_supported(a)) e = launch_gather_mma(a, (cudaStream_t)s);
  else e = launch_gather_generic(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "gather_qmm");
  return QB200_OK;
}

QB200_API int qb200_gather_qmm_swiglu(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* w_gate,
                                      const qb200_tensor* scales_gate, const qb200_tensor* biases_gate,
                                      const qb200_tensor* w_up, const qb200_tensor* scales_up,
                                      const qb200_tensor* biases_up, const qb200_tensor* lhs_indices,
                                      const qb200_tensor* rhs_indices, qb200_optional_int group_size,
                                      qb200_optional_int bits, const char* mode, bool sorted_indices, qb200_stream s) {
  GatherArgs a;
  bool skip = false;
  int st = prepare_gather(res, x, w_gate, scales_gate, biases_gate, lhs_indices, rhs_indices, true, group_size, bits, mode,
                          sorted_indices, &a, &skip);
  if (st) return st;
  if ((st = check_tensor(w_up, "w_up", 3)) || (st = check_tensor(scales_up, "scales_up", 3)) ||
      (st = check_tensor(biases_up, "biases_up", 3)))
    return st;
  if (w_up->dtype != QB200_UINT32 || scales_up->dtype != QB200_BFLOAT16 || biases_up->dtype != QB200_BFLOAT16)
    return fail(QB200_ERR_BAD_DTYPE, "gather_qmm_swiglu: the up bank must be uint32 codes with bf16 scales and biases");
  if (w_up->ndim != 3 || scales_up->ndim != 3 || biases_up->ndim != 3)
    return fail(QB200_ERR_BAD_SHAPE, "gather_qmm_swiglu: the up bank must be [E, N, *]");
  for (int d = 0; d < 3; ++d)
    if (w_up->shape[d] != w_gate->shape[d] || scales_up->shape[d] != scales_gate->shape[d] ||
        biases_up->shape[d] != biases_gate->shape[d])
      return fail(QB200_ERR_BAD_SHAPE, "gather_qmm_swiglu: gate and up banks must have the same shape");
  if (!fully_contiguous(w_up) || !fully_contiguous(scales_up) || !fully_contiguous(biases_up))
    return fail(QB200_ERR_BAD_STRIDE, "gather_qmm_swiglu: w, scales and biases must be contiguous");
  if (skip) return QB200_OK;
  if (x->dtype != QB200_BFLOAT16 && x->dtype != QB200_FLOAT32)
    return fail(QB200_ERR_UNSUPPORTED, "gather_qmm_swiglu: x must be bf16 or f32");
  a.w2 = (const uint32_t*)w_up->data; a.s2 = scales_up->data; a.b2 = biases_up->data;
  // Declined shapes leave the caller on the unfused chain (two gather_qmm calls and its own SwiGLU), as the
  // reference's fused path does (src/transformer.zig:19925-19931).
  const bool small = gather_small_supported(a);
  if (!small && (!gather_stream_supported(a) || (((uintptr_t)a.w2) & 15) != 0 || (((uintptr_t)a.s2) & 7) != 0 || (((uintptr_t)a.b2) & 7) != 0))
    return fail(QB200_ERR_UNSUPPORTED, "gather_qmm_swiglu: shape not served by the fused streaming kernel");
  const cudaError_t e = small ? launch_gather_small(a, (cudaStream_t)s) : launch_gather_stream(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "gather_qmm_swiglu");
  return QB200_OK;
}

QB200_API int qb200_moe_down_reduce(qb200_tensor* res, const qb200_tensor* act, const qb200_tensor* w,
                                    const qb200_tensor* scales, const qb200_tensor* biases, const qb200_tensor* inds,
                                    const qb200_tensor* scores, qb200_optional_int group_size, qb200_optional_int bits,
                                    const char* mode, qb200_stream s) {
  int gs, nb, st;
  if ((st = resolve_mode(mode, group_size, bits, &gs, &nb))) return st;
  if ((st = check_tensor(res, "res", 1)) || (st = check_tensor(act, "act", 2)) || (st = check_tensor(w, "w", 3)) ||
      (st = check_tensor(scales, "scales", 3)) || (st = check_tensor(biases, "biases", 3)) ||
      (st = check_tensor(inds, "inds", 1)) || (st = check_tensor(scores, "scores", 1)))
    return st;
  if (w->ndim != 3 || scales->ndim != 3 || biases->ndim != 3)
    return fail(QB200_ERR_UNSUPPORTED, "moe_down_reduce: w, scales, biases must be [E, N, *]");
  if (w->dtype != QB200_UINT32 || scales->dtype != QB200_BFLOAT16 || biases->dtype != QB200_BFLOAT16)
    return fail(QB200_ERR_BAD_DTYPE, "moe_down_reduce: w must be uint32 with bf16 scales and biases");
  if (act->dtype != QB200_BFLOAT16 && act->dtype != QB200_FLOAT32)
    return fail(QB200_ERR_UNSUPPORTED, "moe_down_reduce: act must be bf16 or f32");
  if (res->dtype != act->dtype || scores->dtype != act->dtype)
    return fail(QB200_ERR_BAD_DTYPE, "moe_down_reduce: act, scores and res must share a dtype");
  if (!is_index_dtype(inds->dtype)) return fail(QB200_ERR_BAD_DTYPE, "moe_down_reduce: inds must be int32/uint32/int64");
  if (!fully_contiguous(w) || !fully_contiguous(scales) || !fully_contiguous(biases) || !fully_contiguous(act) ||
      !fully_contiguous(res) || !fully_contiguous(inds) || !fully_contiguous(scores))
    return fail(QB200_ERR_BAD_STRIDE, "moe_down_reduce: tensors must be contiguous");
  const int vpw = 32 / nb;
  const int64_t E = w->shape[0], N = w->shape[1], K = w->shape[2] * vpw;
  const int64_t topk = scores->shape[scores->ndim - 1];
  const int64_t T = topk > 0 ? numel(scores) / topk : 0;
  if (act->shape[act->ndim - 1] != K || numel(act) != T * topk * K)
    return fail(QB200_ERR_BAD_SHAPE, "moe_down_reduce: act must be [T, k, K] (or [T, k, 1, K]) for scores [T, k]");
  if (numel(inds) != T * topk) return fail(QB200_ERR_BAD_SHAPE, "moe_down_reduce: inds must be [T, k]");
  if (K % gs != 0 || scales->shape[0] != E || scales->shape[1] != N || scales->shape[2] != K / gs ||
      biases->shape[0] != E || biases->shape[1] != N || biases->shape[2] != K / gs)
    return fail(QB200_ERR_BAD_SHAPE, "moe_down_reduce: scales/biases must be [E, N, K/group_size]");
  if (res->shape[res->ndim - 1] != N || numel(res) != T * N)
    return fail(QB200_ERR_BAD_SHAPE, "moe_down_reduce: res must be [T, N]");
  if (T == 0 || N == 0) return QB200_OK;
  MoeDownReduceArgs a;
  a.act = act->data; a.w = (const uint32_t*)w->data; a.s = scales->data; a.b = biases->data; a.y = res->data;
  a.inds = inds->data; a.scores = scores->data; a.inds_i64 = inds->dtype == QB200_INT64;
  a.T = T; a.N = N; a.K = K; a.E = E; a.wes = N * w->shape[2]; a.ses = N * (K / gs);
  a.topk = (int)topk; a.gs = gs; a.bits = nb; a.dtype = act->dtype;
  // Every token streams its own k experts: meant for the single-token decode step (a few tokens at most); wider
  // batches are declined and keep gather_qmm + moe_weighted_sum, which read each expert once for all its rows.
  if (T > 4 || topk > 16 || !moe_down_reduce_supported(a))
    return fail(QB200_ERR_UNSUPPORTED, "moe_down_reduce: shape not served by the fused kernel");
  const cudaError_t e = launch_moe_down_reduce(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "moe_down_reduce");
  return QB200_OK;
}

QB200_API int qb200_moe_route(qb200_tensor* inds, qb200_tensor* norm_scores, const qb200_tensor* logits, int k,
                              qb200_stream s) {
  int st;
  if ((st = check_tensor(inds, "inds", 1)) || (st = check_tensor(norm_scores, "norm_scores", 1)) ||
      (st = check_tensor(logits, "logits", 1)))
    return st;
  if (logits->dtype != QB200_BFLOAT16 && logits->dtype != QB200_FLOAT32)
    return fail(QB200_ERR_UNSUPPORTED, "moe_route: logits must be bf16 or f32");
  if (norm_scores->dtype != logits->dtype) return fail(QB200_ERR_BAD_DTYPE, "moe_route: norm_scores must have the logits' dtype");
  if (inds->dtype != QB200_INT32 && inds->dtype != QB200_UINT32) return fail(QB200_ERR_BAD_DTYPE, "moe_route: inds must be int32/uint32");
  if (!fully_contiguous(inds) || !fully_contiguous(norm_scores) || !fully_contiguous(logits))
    return fail(QB200_ERR_BAD_STRIDE, "moe_route: tensors must be contiguous");
  const int64_t E = logits->shape[logits->ndim - 1];
  const int64_t T = E > 0 ? numel(logits) / E : 0;
  if (k < 1 || k > 32 || k > E) return fail(QB200_ERR_UNSUPPORTED, "moe_route: k must be in 1..min(32, E)");
  if (E > 1024) return fail(QB200_ERR_UNSUPPORTED, "moe_route: at most 1024 experts");
  if (inds->shape[inds->ndim - 1] != k || norm_scores->shape[norm_scores->ndim - 1] != k || numel(inds) != T * k ||
      numel(norm_scores) != T * k)
    return fail(QB200_ERR_BAD_SHAPE, "moe_route: inds and norm_scores must be [..., T, k] for logits [..., T, E]");
  MoeRouteArgs a;
  a.logits = logits->data; a.inds = (int*)inds->data; a.scores = norm_scores->data;
  a.T = T; a.E = (int)E; a.topk = k; a.dtype = logits->dtype;
  if (T == 0) return QB200_OK;
  const cudaError_t e = launch_moe_route(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "moe_route");
  return QB200_OK;
}

QB200_API int qb200_moe_sort_by_expert(qb200_tensor* order, qb200_tensor* inv_order, qb200_tensor* sorted_inds,
                                       qb200_tensor* token_rows, qb200_tensor* expert_offsets, const qb200_tensor* inds,
                                       int num_experts, qb200_stream s) {
  int st;
  if ((st = check_tensor(inds, "inds", 1))) return st;
  if (!is_index_dtype(inds->dtype)) return fail(QB200_ERR_BAD_DTYPE, "moe_sort_by_expert: inds must be int32/uint32/int64");
  if (!fully_contiguous(inds)) return fail(QB200_ERR_BAD_STRIDE, "moe_sort_by_expert: inds must be contiguous");
  if (num_experts < 1 || num_experts > 1024) return fail(QB200_ERR_UNSUPPORTED, "moe_sort_by_expert: 1..1024 experts are served");
  const int64_t n = numel(inds), topk = inds->shape[inds->ndim - 1];
  if (n >= (int64_t)1 << 24) return fail(QB200_ERR_UNSUPPORTED, "moe_sort_by_expert: at most 2^24 - 1 index entries");
  MoeSortArgs a;
  std::memset(&a, 0, sizeof(a));
  a.inds = inds->data; a.inds_i64 = inds->dtype == QB200_INT64; a.n = n; a.E = num_experts; a.topk = (int)(topk > 0 ? topk : 1);
  qb200_tensor* outs[4] = {order, inv_order, sorted_inds, token_rows};
  const char* names[4] = {"order", "inv_order", "sorted_inds", "token_rows"};
  int** dst[4] = {&a.order, &a.inv_order, &a.sorted_inds, &a.token_rows};
  for (int i = 0; i < 4; ++i) {
    if (is_empty(outs[i])) continue;
    if ((st = check_tensor(outs[i], names[i], 1))) return st;
    if (outs[i]->dtype != QB200_INT32 && outs[i]->dtype != QB200_UINT32)
      return fail(QB200_ERR_BAD_DTYPE, "moe_sort_by_expert: %s must be int32/uint32", names[i]);
    if (numel(outs[i]) != n || !fully_contiguous(outs[i]))
      return fail(QB200_ERR_BAD_SHAPE, "moe_sort_by_expert: %s must hold one contiguous entry per index", names[i]);
    *dst[i] = (int*)outs[i]->data;
  }
  if (!is_empty(expert_offsets)) {
    if ((st = check_tensor(expert_offsets, "expert_offsets", 1))) return st;
    if (expert_offsets->dtype != QB200_INT32 && expert_offsets->dtype != QB200_UINT32)
      return fail(QB200_ERR_BAD_DTYPE, "moe_sort_by_expert: expert_offsets must be int32/uint32");
    if (numel(expert_offsets) != (int64_t)num_experts + 1 || !fully_contiguous(expert_offsets))
      return fail(QB200_ERR_BAD_SHAPE, "moe_sort_by_expert: expert_offsets must be [num_experts + 1]");
    a.offsets = (int*)expert_offsets->data;
  }
  const cudaError_t e = launch_moe_sort(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "moe_sort_by_expert");
  return QB200_OK;
}

QB200_API int qb200_moe_weighted_sum(qb200_tensor* res, const qb200_tensor* y, const qb200_tensor* scores,
                                     const qb200_tensor* inv_order, qb200_stream s) {
  int st;
  if ((st = check_tensor(res, "res", 1)) || (st = check_tensor(y, "y", 1)) || (st = check_tensor(scores, "scores", 1))) return st;
  if (y->dtype != QB200_BFLOAT16 && y->dtype != QB200_FLOAT32)
    return fail(QB200_ERR_UNSUPPORTED, "moe_weighted_sum: y must be bf16 or f32");
  if (scores->dtype != y->dtype || res->dtype != y->dtype)
    return fail(QB200_ERR_BAD_DTYPE, "moe_weighted_sum: y, scores and res must share a dtype");
  if (!fully_contiguous(y) || !fully_contiguous(scores) || !fully_contiguous(res))
    return fail(QB200_ERR_BAD_STRIDE, "moe_weighted_sum: y, scores and res must be contiguous");
  const int64_t H = y->shape[y->ndim - 1], topk = scores->shape[scores->ndim - 1];
  const int64_t R = H > 0 ? numel(y) / H : 0, T = topk > 0 ? numel(scores) / topk : 0;
  if (res->shape[res->ndim - 1] != H || numel(res) != T * H || (is_empty(inv_order) && R != T * topk))
    return fail(QB200_ERR_BAD_SHAPE, "moe_weighted_sum: y [T*k rows, H], scores [T, k], res [T, H] expected");
  if (H % 8 != 0) return fail(QB200_ERR_UNSUPPORTED, "moe_weighted_sum: H must be a multiple of 8");
  const int esz = y->dtype == QB200_FLOAT32 ? 4 : 2;
  if ((((uintptr_t)y->data) | ((uintptr_t)res->data)) & 15 || (H * esz) % 16 != 0)
    return fail(QB200_ERR_UNSUPPORTED, "moe_weighted_sum: rows must be 16-byte aligned");
  MoeSumArgs a;
  a.y = y->data; a.scores = scores->data; a.out = res->data; a.inv = nullptr; a.inv_i64 = 0;
  a.T = T; a.topk = topk; a.H = H; a.R = R; a.dtype = y->dtype;
  if (!is_empty(inv_order)) {
    if ((st = check_tensor(inv_order, "inv_order", 0))) return st;
    if (inv_order->dtype != QB200_INT32 && inv_order->dtype != QB200_UINT32 && inv_order->dtype != QB200_INT64)
      return fail(QB200_ERR_BAD_DTYPE, "moe_weighted_sum: inv_order must be int32/uint32/int64");
    if (numel(inv_order) != T * topk || !fully_contiguous(inv_order))
      return fail(QB200_ERR_BAD_SHAPE, "moe_weighted_sum: inv_order must hold one contiguous entry per (token, slot)");
    a.inv = inv_order->data; a.inv_i64 = inv_order->dtype == QB200_INT64;
  }
  if (T == 0 || H == 0) return QB200_OK;
  const cudaError_t e = launch_moe_weighted_sum(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "moe_weighted_sum");
  return QB200_OK;
}

QB200_API int qb200_dequantize(qb200_tensor* res, const qb200_tensor* w, const qb200_tensor* scales,
                               const qb200_tensor* biases, qb200_optional_int group_size, qb200_optional_int bits,
                               const char* mode, const qb200_tensor* global_scale, qb200_optional_dtype dtype,
                               qb200_stream s) {
  int gs, nb, st;
  if ((st = resolve_mode(mode, group_size, bits, &gs, &nb))) return st;
  if (!is_empty(global_scale)) return fail(QB200_ERR_UNSUPPORTED, "dequantize: global_scale belongs to non-affine modes");
  if (is_empty(biases)) return fail(QB200_ERR_UNSUPPORTED, "dequantize: biases are required (affine mode)");
  if ((st = check_tensor(res, "res", 1)) || (st = check_tensor(w, "w", 1)) || (st = check_tensor(scales, "scales", 1)) ||
      (st = check_tensor(biases, "biases", 1)))
    return st;
  if (w->dtype != QB200_UINT32) return fail(QB200_ERR_BAD_DTYPE, "dequantize: w must be uint32");
  if (!is_float_dtype(scales->dtype) || biases->dtype != scales->dtype)
    return fail(QB200_ERR_BAD_DTYPE, "dequantize: scales/biases must share a float dtype");
  const int out_dt = dtype.has_value ? dtype.value : scales->dtype;
  if (!is_float_dtype(out_dt)) return fail(QB200_ERR_BAD_DTYPE, "dequantize: output dtype %d is not served", out_dt);
  if (res->dtype != out_dt) return fail(QB200_ERR_BAD_DTYPE, "dequantize: res dtype %d != requested %d", res->dtype, out_dt);
  const int64_t d = w->shape[w->ndim - 1] * (32 / nb);
  if (d % gs != 0 || scales->shape[scales->ndim - 1] != d / gs)
    return fail(QB200_ERR_BAD_SHAPE, "dequantize: scales last dim %lld != %lld / group_size",
                (long long)scales->shape[scales->ndim - 1], (long long)d);
  if (!same_leading(w, scales) || !same_leading(scales, biases) || !same_leading(w, res) ||
      biases->shape[biases->ndim - 1] != scales->shape[scales->ndim - 1] || res->shape[res->ndim - 1] != d)
    return fail(QB200_ERR_BAD_SHAPE, "dequantize: w/scales/biases/res shapes disagree");
  if (!same_strides(scales, biases)) return fail(QB200_ERR_BAD_STRIDE, "dequantize: scales and biases must have identical strides");
  DequantArgs a;
  a.w = (const uint32_t*)w->data; a.s = scales->data; a.b = biases->data; a.out = res->data;
  a.wmap = make_rowmap(w); a.sbmap = make_rowmap(scales); a.omap = make_rowmap(res);
  a.rows = rows_of(w); a.d = d; a.gs = gs; a.bits = nb;
  a.sb_dtype = scales->dtype; a.out_dtype = out_dt;
  if (a.rows * d == 0) return QB200_OK;
  cudaError_t e = launch_dequantize(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "dequantize");
  return QB200_OK;
}

static int quantize_impl(qb200_tensor* res_q, qb200_tensor* res_scales, qb200_tensor* res_biases, const qb200_tensor* w,
                         int gs, int nb, qb200_stream s, const char* who) {
  int st;
  if ((st = check_tensor(res_q, "res_q", 1)) || (st = check_tensor(res_scales, "res_scales", 1)) ||
      (st = check_tensor(res_biases, "res_biases", 1)) || (st = check_tensor(w, "w", 1)))
    return st;
  if (!is_float_dtype(w->dtype)) return fail(QB200_ERR_BAD_DTYPE, "%s: input must be bf16, f16 or f32", who);
  if (res_q->dtype != QB200_UINT32) return fail(QB200_ERR_BAD_DTYPE, "%s: packed output must be uint32", who);
  if (!is_float_dtype(res_scales->dtype) || res_biases->dtype != res_scales->dtype)
    return fail(QB200_ERR_BAD_DTYPE, "%s: scales/biases must share a float dtype", who);
  const int64_t d = w->shape[w->ndim - 1];
  if (d % gs != 0) return fail(QB200_ERR_BAD_SHAPE, "%s: last dim %lld is not a multiple of group_size %d", who, (long long)d, gs);
  if (!same_leading(w, res_q) || !same_leading(w, res_scales) || !same_leading(w, res_biases) ||
      res_q->shape[res_q->ndim - 1] != d * nb / 32 || res_scales->shape[res_scales->ndim - 1] != d / gs ||
      res_biases->shape[res_biases->ndim - 1] != d / gs)
    return fail(QB200_ERR_BAD_SHAPE, "%s: outputs must be [..., D*bits/32] and [..., D/group_size]", who);
  if (!same_strides(res_scales, res_biases)) return fail(QB200_ERR_BAD_STRIDE, "%s: scales and biases must have identical strides", who);
  QuantArgs a;
  a.x = w->data; a.q = (uint32_t*)res_q->data; a.s = res_scales->data; a.b = res_biases->data;
  a.xmap = make_rowmap(w); a.qmap = make_rowmap(res_q); a.sbmap = make_rowmap(res_scales);
  a.rows = rows_of(w); a.d = d; a.gs = gs; a.bits = nb;
  a.x_dtype = w->dtype; a.sb_dtype = res_scales->dtype;
  if (a.rows * d == 0) return QB200_OK;
  cudaError_t e = launch_quantize(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, who);
  return QB200_OK;
}

QB200_API int qb200_quantize(qb200_tensor* res_q, qb200_tensor* res_scales, qb200_tensor* res_biases,
                             const qb200_tensor* w, qb200_optional_int group_size, qb200_optional_int bits,
                             const char* mode, const qb200_tensor* global_scale, qb200_stream s) {
  int gs, nb, st;
  if ((st = resolve_mode(mode, group_size, bits, &gs, &nb))) return st;
  if (!is_empty(global_scale)) return fail(QB200_ERR_UNSUPPORTED, "quantize: global_scale belongs to non-affine modes");
  return quantize_impl(res_q, res_scales, res_biases, w, gs, nb, s, "quantize");
}

QB200_API int qb200_kv_append(qb200_tensor* cache_q, qb200_tensor* cache_scales, qb200_tensor* cache_biases,
                              const qb200_tensor* dense, int64_t offset, int bits, int group_size, qb200_stream s) {
  int gs, nb, st;
  qb200_optional_int og = {group_size, true}, ob = {bits, true};
  if ((st = resolve_mode("affine", og, ob, &gs, &nb))) return st;
  if ((st = check_tensor(cache_q, "cache_q", 4)) || (st = check_tensor(cache_scales, "cache_scales", 4)) ||
      (st = check_tensor(cache_biases, "cache_biases", 4)) || (st = check_tensor(dense, "dense", 4)))
    return st;
  if (cache_q->ndim != 4 || cache_scales->ndim != 4 || cache_biases->ndim != 4 || dense->ndim != 4)
    return fail(QB200_ERR_BAD_SHAPE, "kv_append: tensors must be [B, Hkv, tokens, last]");
  const int64_t S = dense->shape[2], cap = cache_q->shape[2];
  if (offset < 0 || offset + S > cap || cache_scales->shape[2] != cap || cache_biases->shape[2] != cap)
    return fail(QB200_ERR_BAD_SHAPE, "kv_append: offset %lld + %lld tokens exceeds capacity %lld", (long long)offset,
                (long long)S, (long long)cap);
  qb200_tensor vq = *cache_q, vs = *cache_scales, vb = *cache_biases;
  vq.shape[2] = vs.shape[2] = vb.shape[2] = S;
  vq.data = (char*)cache_q->data + offset * cache_q->stride[2] * 4;
  vs.data = (char*)cache_scales->data + offset * cache_scales->stride[2] * dtype_size(cache_scales->dtype);
  vb.data = (char*)cache_biases->data + offset * cache_biases->stride[2] * dtype_size(cache_biases->dtype);
  return quantize_impl(&vq, &vs, &vb, dense, gs, nb, s, "kv_append");
}

// Mask mode, additive mask row and per-sequence lengths of the decode attention entries (T = the longest view).
static int parse_kv_mask(KvAttnArgs& a, const qb200_tensor* q, const char* mask_mode, const qb200_tensor* mask_arr,
                         const qb200_tensor* kv_lens, int64_t B, int64_t T) {
  int st;
  const char* mm = mask_mode ? mask_mode : "";
  if (std::strcmp(mm, "array") == 0) {
    if (is_empty(mask_arr)) return fail(QB200_ERR_BAD_ARG, "kv_decode_attention: mask_mode \"array\" needs mask_arr");
    if ((st = check_tensor(mask_arr, "mask_arr", 1))) return st;
    if (mask_arr->dtype != q->dtype && mask_arr->dtype != QB200_FLOAT32)
      return fail(QB200_ERR_BAD_DTYPE, "kv_decode_attention: mask must be q's dtype or f32");
    if (mask_arr->shape[mask_arr->ndim - 1] != T)
      return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: mask last dim %lld != T %lld",
                  (long long)mask_arr->shape[mask_arr->ndim - 1], (long long)T);
    // additive row broadcastable to [B, 1, 1, T]: every dim but the last (and an optional batch dim) is 1
    int64_t bstride = 0;
    for (int d = 0; d < mask_arr->ndim - 1; ++d) {
      if (mask_arr->shape[d] == 1) continue;
      if (d == mask_arr->ndim - 4 && mask_arr->shape[d] == B) { bstride = mask_arr->stride[d]; continue; }
      if (mask_arr->ndim < 4 && d == 0 && mask_arr->shape[d] == B && mask_arr->ndim == 2) { bstride = mask_arr->stride[d]; continue; }
      return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention: mask must broadcast as [B|1, 1, 1, T]");
    }
    a.mask = mask_arr->data; a.mask_dtype = mask_arr->dtype; a.mask_bstride = bstride;
  } else if (std::strcmp(mm, "") != 0 && std::strcmp(mm, "causal") != 0) {
    return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention: mask_mode '%s' is not served", mm);
  }
  if (!is_empty(kv_lens)) {
    if ((st = check_tensor(kv_lens, "kv_lens", 1))) return st;
    if (kv_lens->dtype != QB200_INT32 || kv_lens->ndim != 1 || kv_lens->shape[0] != B)
      return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: kv_lens must be int32 [B]");
    a.kv_lens = (const int32_t*)kv_lens->data;
  }
  return 0;
}

QB200_API size_t qb200_kv_decode_attention_workspace_size(int64_t B, int64_t Hq, int64_t Hkv, int64_t T, int64_t Dv) {
  return kv_attn_workspace_bytes(B, Hq, Hkv, T, Dv);   // for T_q > 1 pass T_q as the batch
}

QB200_API int qb200_kv_decode_attention(qb200_tensor* res, const qb200_tensor* q, const qb200_tensor* k_q,
                                        const qb200_tensor* k_scales, const qb200_tensor* k_biases,
                                        const qb200_tensor* v_q, const qb200_tensor* v_scales,
                                        const qb200_tensor* v_biases, int bits, int group_size, float scale,
                                        const char* mask_mode, const qb200_tensor* mask_arr,
                                        const qb200_tensor* kv_lens, void* workspace, size_t workspace_bytes,
                                        qb200_stream s) {
  int gs, nb, st;
  qb200_optional_int og = {group_size, true}, ob = {bits, true};
  if ((st = resolve_mode("affine", og, ob, &gs, &nb))) return st;
  if (nb == 2) return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention: bits must be 4 or 8");
  const qb200_tensor* ts[8] = {res, q, k_q, k_scales, k_biases, v_q, v_scales, v_biases};
  const char* names[8] = {"res", "q", "k_q", "k_scales", "k_biases", "v_q", "v_scales", "v_biases"};
  for (int i = 0; i < 8; ++i) {
    if ((st = check_tensor(ts[i], names[i], 4))) return st;
    if (ts[i]->ndim != 4) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: %s must be 4-D", names[i]);
  }
  if (q->dtype != QB200_BFLOAT16 && q->dtype != QB200_FLOAT32)
    return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention: q must be bf16 or f32");
  if (res->dtype != q->dtype) return fail(QB200_ERR_BAD_DTYPE, "kv_decode_attention: res dtype must equal q dtype");
  if (k_q->dtype != QB200_UINT32 || v_q->dtype != QB200_UINT32)
    return fail(QB200_ERR_BAD_DTYPE, "kv_decode_attention: packed K/V must be uint32");
  if (k_scales->dtype != QB200_BFLOAT16 || k_biases->dtype != QB200_BFLOAT16 || v_scales->dtype != QB200_BFLOAT16 ||
      v_biases->dtype != QB200_BFLOAT16)
    return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention: scales and biases must be bf16");
  const int64_t B = q->shape[0], Hq = q->shape[1], Tq = q->shape[2], D = q->shape[3];
  const int64_t Hkv = k_q->shape[1], T = k_q->shape[2];
  const int vpw = 32 / nb;
  const int64_t Dk = k_q->shape[3] * vpw, Dv = v_q->shape[3] * vpw;
  // Decode width only, as qkvAttnDecodeKernel (mlx-serve src/transformer.zig:5077); wider queries are declined.
  // Decode width, or the verify widths 2..8 of qkvAttnVerifyKernel (src/transformer.zig:5464-5588), causal only.
  if (Tq < 1 || Tq > 8) return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention: T_q=%lld (1..8 are served)", (long long)Tq);
  if (Tq > 1 && (mask_mode == nullptr || std::strcmp(mask_mode, "causal") != 0 || !is_empty(kv_lens)))
    return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention: T_q > 1 is served with mask_mode \"causal\" and without kv_lens");
  if (Dk != D) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: q head dim %lld != K head dim %lld", (long long)D, (long long)Dk);
  if (Hkv <= 0 || Hq % Hkv != 0) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: Hq %lld not a multiple of Hkv %lld", (long long)Hq, (long long)Hkv);
  if (D % gs != 0 || Dv % gs != 0) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: head dims must be multiples of group_size");
  const int64_t kshape[4] = {B, Hkv, T, 0};
  for (int i = 2; i < 8; ++i)
    for (int d = 0; d < 3; ++d)
      if (ts[i]->shape[d] != kshape[d])
        return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: %s dim %d is %lld, expected %lld", names[i], d,
                    (long long)ts[i]->shape[d], (long long)kshape[d]);
  if (k_scales->shape[3] != D / gs || k_biases->shape[3] != D / gs || v_scales->shape[3] != Dv / gs ||
      v_biases->shape[3] != Dv / gs)
    return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: scales/biases last dim must be D/group_size");
  if (!same_strides(k_scales, k_biases) || !same_strides(v_scales, v_biases))
    return fail(QB200_ERR_BAD_STRIDE, "kv_decode_attention: scales and biases must have identical strides");
  if (res->shape[0] != B || res->shape[1] != Hq || res->shape[2] != Tq || res->shape[3] != Dv)
    return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: res must be [B, Hq, T_q, Dv]");

  KvAttnArgs a;
  std::memset(&a, 0, sizeof(a));
  a.q = q->data; a.out = res->data; a.q_dtype = q->dtype;
  a.kq = (const uint32_t*)k_q->data; a.ks = k_scales->data; a.kb = k_biases->data;
  a.vq = (const uint32_t*)v_q->data; a.vs = v_scales->data; a.vb = v_biases->data;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.T = T; a.D = D; a.Dv = Dv;
  a.q_str[0] = q->stride[0]; a.q_str[1] = q->stride[1];
  a.o_str[0] = res->stride[0]; a.o_str[1] = res->stride[1];
  for (int d = 0; d < 3; ++d) {
    a.kq_str[d] = k_q->stride[d]; a.ksb_str[d] = k_scales->stride[d];
    a.vq_str[d] = v_q->stride[d]; a.vsb_str[d] = v_scales->stride[d];
  }
  a.gs = gs; a.bits = nb; a.scale = scale;
  if ((st = parse_kv_mask(a, q, mask_mode, mask_arr, kv_lens, B, T))) return st;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  if (B == 0 || Hq == 0 || Dv == 0) return QB200_OK;
  // An empty cache view has no softmax to take; it is refused here, before the workspace check and before any
  // launch, so that no kernel is ever planned for zero tokens.
  if (T <= 0) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: the cache view holds no tokens (T = %lld)", (long long)T);
  if (!kv_attn_supported(a))
    return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention: geometry not served (D=%lld Dv=%lld gs=%d gqa=%lld)",
                (long long)D, (long long)Dv, gs, (long long)(Hq / Hkv));
  const size_t need = kv_attn_workspace_bytes(Tq > 1 ? Tq : B, Hq, Hkv, T, Dv);
  if (need == 0 || workspace == nullptr || workspace_bytes < need)
    return fail(QB200_ERR_WORKSPACE, "kv_decode_attention: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  if (Tq > 1) {
    // Verify widths: query position tq of sequence b attends to the first T - T_q + 1 + tq cache positions (the
    // end-aligned causal tail, src/transformer.zig:5314-5318).  Every (b, tq) runs as a sequence of its own over the
    // same cache view, with that length; the cache is read T_q times, the repeats out of L2.
    if (T < Tq) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention: the cache view must hold at least T_q tokens");
    const int esz = dtype_size(q->dtype);
    for (int64_t b = 0; b < B; ++b) {   // one launch per sequence: its T_q query positions as T_q "sequences"
      KvSeqTable tab;
      std::memset(&tab, 0, sizeof(tab));
      for (int64_t tq = 0; tq < Tq; ++tq) {
        KvSeq& e = tab.s[tq];
        e.kq = a.kq + b * a.kq_str[0]; e.vq = a.vq + b * a.vq_str[0];
        e.ks = (const uint16_t*)a.ks + b * a.ksb_str[0]; e.kb = (const uint16_t*)a.kb + b * a.ksb_str[0];
        e.vs = (const uint16_t*)a.vs + b * a.vsb_str[0]; e.vb = (const uint16_t*)a.vb + b * a.vsb_str[0];
        for (int d = 0; d < 2; ++d) {
          e.kq_str[d] = a.kq_str[d + 1]; e.ksb_str[d] = a.ksb_str[d + 1];
          e.vq_str[d] = a.vq_str[d + 1]; e.vsb_str[d] = a.vsb_str[d + 1];
        }
        e.T = T - Tq + 1 + tq;
      }
      KvAttnArgs c = a;
      c.B = Tq;
      c.q = (const char*)q->data + b * q->stride[0] * esz;
      c.out = (char*)res->data + b * res->stride[0] * esz;
      c.q_str[0] = q->stride[2];
      c.o_str[0] = res->stride[2];
      const cudaError_t ev = launch_kv_attn(c, (cudaStream_t)s, &tab);
      if (ev != cudaSuccess) return cuda_fail(ev, "kv_decode_attention");
    }
    return QB200_OK;
  }
  cudaError_t e = launch_kv_attn(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "kv_decode_attention");
  return QB200_OK;
}

QB200_API size_t qb200_kv_decode_attention_ptrs_workspace_size(int64_t num_seqs, int64_t Hq, int64_t Hkv, int64_t T_max,
                                                               int64_t Dv) {
  size_t need = 0;
  for (int64_t b0 = 0; b0 < num_seqs; b0 += kMaxSeqPtrs) {
    const int64_t nb = num_seqs - b0 < kMaxSeqPtrs ? num_seqs - b0 : kMaxSeqPtrs;
    const size_t n = kv_attn_workspace_bytes(nb, Hq, Hkv, T_max, Dv);
    need = n > need ? n : need;
  }
  return need;
}

QB200_API int qb200_kv_decode_attention_ptrs(qb200_tensor* res, const qb200_tensor* q, const qb200_tensor* const* k_q,
                                             const qb200_tensor* const* k_scales, const qb200_tensor* const* k_biases,
                                             const qb200_tensor* const* v_q, const qb200_tensor* const* v_scales,
                                             const qb200_tensor* const* v_biases, int num_seqs, int bits, int group_size,
                                             float scale, const char* mask_mode, const qb200_tensor* mask_arr,
                                             const qb200_tensor* kv_lens, void* workspace, size_t workspace_bytes,
                                             qb200_stream s) {
  int gs, nb, st;
  qb200_optional_int og = {group_size, true}, ob = {bits, true};
  if ((st = resolve_mode("affine", og, ob, &gs, &nb))) return st;
  if (nb == 2) return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention_ptrs: bits must be 4 or 8");
  if ((st = check_tensor(res, "res", 4)) || (st = check_tensor(q, "q", 4))) return st;
  if (res->ndim != 4 || q->ndim != 4) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention_ptrs: q and res must be 4-D");
  if (num_seqs < 0 || (num_seqs > 0 && (!k_q || !k_scales || !k_biases || !v_q || !v_scales || !v_biases)))
    return fail(QB200_ERR_BAD_ARG, "kv_decode_attention_ptrs: null view list");
  if (q->dtype != QB200_BFLOAT16 && q->dtype != QB200_FLOAT32)
    return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention_ptrs: q must be bf16 or f32");
  if (res->dtype != q->dtype) return fail(QB200_ERR_BAD_DTYPE, "kv_decode_attention_ptrs: res dtype must equal q dtype");
  const int64_t B = q->shape[0], Hq = q->shape[1], Tq = q->shape[2], D = q->shape[3];
  if (B != num_seqs) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention_ptrs: q holds %lld sequences, %d views given", (long long)B, num_seqs);
  if (Tq != 1) return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention_ptrs: T_q=%lld (only decode width 1 is served)", (long long)Tq);
  if (B == 0) return QB200_OK;
  const int vpw = 32 / nb;
  int64_t Hkv = 0, Dv = 0, T_max = 0;
  // every sequence: six 4-D views [1, Hkv, T_b, last] of its own capacity buffers
  for (int64_t b = 0; b < B; ++b) {
    const qb200_tensor* ts[6] = {k_q[b], k_scales[b], k_biases[b], v_q[b], v_scales[b], v_biases[b]};
    const char* names[6] = {"k_q", "k_scales", "k_biases", "v_q", "v_scales", "v_biases"};
    for (int i = 0; i < 6; ++i) {
      if ((st = check_tensor(ts[i], names[i], 4))) return st;
      if (ts[i]->ndim != 4 || ts[i]->shape[0] != 1)
        return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention_ptrs: %s of sequence %lld must be [1, Hkv, T, last]", names[i], (long long)b);
      if (ts[i]->dtype != ((i == 0 || i == 3) ? QB200_UINT32 : QB200_BFLOAT16))
        return fail(QB200_ERR_BAD_DTYPE, "kv_decode_attention_ptrs: %s must be %s", names[i], (i == 0 || i == 3) ? "uint32" : "bf16");
    }
    if (b == 0) { Hkv = ts[0]->shape[1]; Dv = ts[3]->shape[3] * vpw; }
    const int64_t T = ts[0]->shape[2];
    for (int i = 0; i < 6; ++i)
      if (ts[i]->shape[1] != Hkv || ts[i]->shape[2] != T)
        return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention_ptrs: the six views of sequence %lld disagree on [Hkv, T]", (long long)b);
    if (ts[0]->shape[3] * vpw != D || ts[3]->shape[3] * vpw != Dv || ts[1]->shape[3] != D / gs || ts[2]->shape[3] != D / gs ||
        ts[4]->shape[3] != Dv / gs || ts[5]->shape[3] != Dv / gs)
      return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention_ptrs: head dims of sequence %lld do not match q / group_size", (long long)b);
    if (!same_strides(ts[1], ts[2]) || !same_strides(ts[4], ts[5]))
      return fail(QB200_ERR_BAD_STRIDE, "kv_decode_attention_ptrs: scales and biases must have identical strides");
    if (T <= 0) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention_ptrs: the cache view of sequence %lld holds no tokens", (long long)b);
    T_max = T > T_max ? T : T_max;
  }
  if (Hkv <= 0 || Hq % Hkv != 0) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention_ptrs: Hq %lld not a multiple of Hkv %lld", (long long)Hq, (long long)Hkv);
  if (D % gs != 0 || Dv % gs != 0) return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention_ptrs: head dims must be multiples of group_size");
  if (res->shape[0] != B || res->shape[1] != Hq || res->shape[2] != 1 || res->shape[3] != Dv)
    return fail(QB200_ERR_BAD_SHAPE, "kv_decode_attention_ptrs: res must be [B, Hq, 1, Dv]");

  KvAttnArgs a;
  std::memset(&a, 0, sizeof(a));
  a.q_dtype = q->dtype;
  a.Hq = Hq; a.Hkv = Hkv; a.T = T_max; a.D = D; a.Dv = Dv;
  a.q_str[0] = q->stride[0]; a.q_str[1] = q->stride[1];
  a.o_str[0] = res->stride[0]; a.o_str[1] = res->stride[1];
  a.gs = gs; a.bits = nb; a.scale = scale;
  if ((st = parse_kv_mask(a, q, mask_mode, mask_arr, kv_lens, B, T_max))) return st;
  a.B = B < kMaxSeqPtrs ? B : kMaxSeqPtrs;
  if (Hq == 0 || Dv == 0) return QB200_OK;
  if (!kv_attn_supported(a))
    return fail(QB200_ERR_UNSUPPORTED, "kv_decode_attention_ptrs: geometry not served (D=%lld Dv=%lld gs=%d gqa=%lld)",
                (long long)D, (long long)Dv, gs, (long long)(Hq / Hkv));
  const size_t need = qb200_kv_decode_attention_ptrs_workspace_size(B, Hq, Hkv, T_max, Dv);
  if (need == 0 || workspace == nullptr || workspace_bytes < need)
    return fail(QB200_ERR_WORKSPACE, "kv_decode_attention_ptrs: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  const int esz = dtype_size(q->dtype);
  const int msz = a.mask ? dtype_size(a.mask_dtype) : 0;
  // at most kMaxSeqPtrs sequences per launch: their views travel as a kernel parameter
  for (int64_t b0 = 0; b0 < B; b0 += kMaxSeqPtrs) {
    KvSeqTable tab;
    std::memset(&tab, 0, sizeof(tab));
    const int64_t nbq = B - b0 < kMaxSeqPtrs ? B - b0 : kMaxSeqPtrs;
    for (int64_t i = 0; i < nbq; ++i) {
      KvSeq& e = tab.s[i];
      const int64_t b = b0 + i;
      e.kq = (const uint32_t*)k_q[b]->data; e.ks = k_scales[b]->data; e.kb = k_biases[b]->data;
      e.vq = (const uint32_t*)v_q[b]->data; e.vs = v_scales[b]->data; e.vb = v_biases[b]->data;
      for (int d = 0; d < 2; ++d) {
        e.kq_str[d] = k_q[b]->stride[d + 1]; e.ksb_str[d] = k_scales[b]->stride[d + 1];
        e.vq_str[d] = v_q[b]->stride[d + 1]; e.vsb_str[d] = v_scales[b]->stride[d + 1];
      }
      e.T = k_q[b]->shape[2];
    }
    KvAttnArgs c = a;
    c.B = nbq;
    c.q = (const char*)q->data + b0 * q->stride[0] * esz;
    c.out = (char*)res->data + b0 * res->stride[0] * esz;
    if (a.kv_lens) c.kv_lens = a.kv_lens + b0;
    if (a.mask) c.mask = (const char*)a.mask + b0 * a.mask_bstride * msz;
    const cudaError_t e = launch_kv_attn(c, (cudaStream_t)s, &tab);
    if (e != cudaSuccess) return cuda_fail(e, "kv_decode_attention_ptrs");
  }
  return QB200_OK;
}

// ---- the small operators of the batched decode step (bf16 activations) ----
static int row_view(const qb200_tensor* t, const char* name, int64_t* rows, int64_t* d, int64_t* pitch) {
  int st;
  if ((st = check_tensor(t, name, 1))) return st;
  if (t->dtype != QB200_BFLOAT16) return fail(QB200_ERR_UNSUPPORTED, "%s: bf16 only", name);
  const RowMap m = make_rowmap(t);
  if (!m.contiguous) return fail(QB200_ERR_BAD_STRIDE, "%s: rows must be evenly spaced", name);
  *rows = rows_of(t); *d = t->shape[t->ndim - 1]; *pitch = t->ndim >= 2 ? m.row_pitch : *d;
  return 0;
}

QB200_API int qb200_add_rms_norm(qb200_tensor* sum_res, qb200_tensor* norm_res, const qb200_tensor* a, const qb200_tensor* b,
                                 const qb200_tensor* weight, float eps, qb200_stream s) {
  int st;
  int64_t rows, d, lda, r2, d2, ldb = 0, lds = 0, ldn = 0;
  if ((st = row_view(a, "a", &rows, &d, &lda))) return st;
  if (d % 2 != 0 || d > 32768) return fail(QB200_ERR_UNSUPPORTED, "rms_norm: row length must be even and at most 32768");
  if ((((uintptr_t)a->data) | (uintptr_t)(lda * 2)) & 3) return fail(QB200_ERR_UNSUPPORTED, "rms_norm: rows must be 4-byte aligned");
  const uint16_t* bp = nullptr; uint16_t* sp = nullptr; uint16_t* np_ = nullptr; const uint16_t* wp = nullptr;
  if (!is_empty(b)) {
    if ((st = row_view(b, "b", &r2, &d2, &ldb))) return st;
    if (r2 != rows || d2 != d || ((((uintptr_t)b->data) | (uintptr_t)(ldb * 2)) & 3)) return fail(QB200_ERR_BAD_SHAPE, "add_rms_norm: a and b must have the same shape");
    bp = (const uint16_t*)b->data;
    if (!is_empty(sum_res)) {
      if ((st = row_view(sum_res, "sum_res", &r2, &d2, &lds))) return st;
      if (r2 != rows || d2 != d || ((((uintptr_t)sum_res->data) | (uintptr_t)(lds * 2)) & 3)) return fail(QB200_ERR_BAD_SHAPE, "add_rms_norm: sum_res must have a's shape");
      sp = (uint16_t*)sum_res->data;
    }
  } else if (!is_empty(sum_res)) {
    return fail(QB200_ERR_BAD_ARG, "add_rms_norm: sum_res without b");
  }
  if (!is_empty(norm_res)) {
    if ((st = row_view(norm_res, "norm_res", &r2, &d2, &ldn))) return st;
    if (r2 != rows || d2 != d || ((((uintptr_t)norm_res->data) | (uintptr_t)(ldn * 2)) & 3)) return fail(QB200_ERR_BAD_SHAPE, "rms_norm: res must have x's shape");
    if ((st = check_tensor(weight, "weight", 1))) return st;
    if (weight->dtype != QB200_BFLOAT16 || weight->ndim != 1 || weight->shape[0] != d || (((uintptr_t)weight->data) & 3))
      return fail(QB200_ERR_BAD_SHAPE, "rms_norm: weight must be bf16 [d]");
    np_ = (uint16_t*)norm_res->data; wp = (const uint16_t*)weight->data;
  }
  if (!sp && !np_) return QB200_OK;
  const cudaError_t e = launch_rms_norm((const uint16_t*)a->data, bp, wp, sp, np_, rows, (int)d, lda, ldb, lds, ldn, eps, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "rms_norm");
  return QB200_OK;
}

QB200_API int qb200_rms_norm(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* weight, float eps, qb200_stream s) {
  return qb200_add_rms_norm(nullptr, res, x, nullptr, weight, eps, s);
}

QB200_API int qb200_rope(qb200_tensor* res, const qb200_tensor* x, int dims, bool traditional, qb200_optional_float base,
                         float scale, const qb200_tensor* offsets, const qb200_tensor* freqs, qb200_stream s) {
  int st;
  if ((st = check_tensor(res, "res", 4)) || (st = check_tensor(x, "x", 4)) || (st = check_tensor(offsets, "offsets", 1))) return st;
  if (traditional) return fail(QB200_ERR_UNSUPPORTED, "rope: the traditional (interleaved) pairing is not served");
  if (!is_empty(freqs) || !base.has_value) return fail(QB200_ERR_UNSUPPORTED, "rope: a frequency table is not served (give a base)");
  if (x->ndim != 4 || res->ndim != 4 || x->dtype != QB200_BFLOAT16 || res->dtype != QB200_BFLOAT16)
    return fail(QB200_ERR_UNSUPPORTED, "rope: x and res must be bf16 [N, heads, 1, D]");
  const int64_t N = x->shape[0], Hh = x->shape[1], D = x->shape[3];
  if (x->shape[2] != 1) return fail(QB200_ERR_UNSUPPORTED, "rope: sequence length 1 only (the decode step)");
  for (int d = 0; d < 4; ++d)
    if (res->shape[d] != x->shape[d]) return fail(QB200_ERR_BAD_SHAPE, "rope: res must have x's shape");
  if (dims <= 0 || dims % 2 != 0 || dims > D || D % 2 != 0) return fail(QB200_ERR_BAD_SHAPE, "rope: dims must be even and at most D");
  if (offsets->dtype != QB200_INT32 || offsets->ndim != 1 || offsets->shape[0] != N || offsets->stride[0] != 1)
    return fail(QB200_ERR_BAD_SHAPE, "rope: offsets must be int32 [N]");
  if (N == 0 || Hh == 0) return QB200_OK;
  const cudaError_t e = launch_rope((const uint16_t*)x->data, (uint16_t*)res->data, (const int32_t*)offsets->data, N, (int)Hh, (int)D,
                                    dims, base.value, scale, x->stride[0], x->stride[1], res->stride[0], res->stride[1], (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "rope");
  return QB200_OK;
}


// The +-1 vector of TurboState's cloneWithSignFlip (src/kv_quant.zig:318-330): a 64-bit LCG stepped once per entry,
// bit 33 of the state picks the sign; bit e of the result set = -1.
static void turbo_sign_bits(uint64_t seed, int n, uint32_t* bits) {
  for (int i = 0; i < (n + 31) / 32; ++i) bits[i] = 0u;
  uint64_t st = seed * 6364136223846793005ull;
  for (int e = 0; e < n; ++e) {
    st = st * 6364136223846793005ull + 1442695040888963407ull;
    if ((st >> 33) & 1ull) bits[e >> 5] |= 1u << (e & 31);
  }
}

QB200_API int qb200_turbo_signs(uint64_t seed, int n, uint32_t* bits) {
  if (!bits || n <= 0 || n > 4096) return fail(QB200_ERR_BAD_ARG, "turbo_signs: 1..4096 entries");
  turbo_sign_bits(seed, n, bits);
  return QB200_OK;
}

QB200_API int qb200_turbo_rotate(qb200_tensor* res, const qb200_tensor* x, uint64_t seed, qb200_stream s) {
  int st;
  int64_t rows, d, ldx, r2, d2, ldo;
  if ((st = row_view(x, "x", &rows, &d, &ldx)) || (st = row_view(res, "res", &r2, &d2, &ldo))) return st;
  if (r2 != rows || d2 != d) return fail(QB200_ERR_BAD_SHAPE, "turbo_rotate: res must have x's shape");
  if (d < 32 || d > 1024 || (d & (d - 1)) != 0)
    return fail(QB200_ERR_UNSUPPORTED, "turbo_rotate: the last axis must be a power of two between 32 and 1024 (the reference refuses other head dims too)");
  if (rows == 0) return QB200_OK;
  uint32_t bits[32];
  turbo_sign_bits(seed, (int)d, bits);
  const cudaError_t e = launch_turbo_rotate((const uint16_t*)x->data, (uint16_t*)res->data, rows, (int)d, ldx, ldo, bits, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "turbo_rotate");
  return QB200_OK;
}

QB200_API int qb200_swiglu(qb200_tensor* res, const qb200_tensor* gate, const qb200_tensor* up, qb200_stream s) {
  int st;
  int64_t rows, d, ldg, r2, d2, ldu, ldo;
  if ((st = row_view(gate, "gate", &rows, &d, &ldg)) || (st = row_view(up, "up", &r2, &d2, &ldu))) return st;
  if (r2 != rows || d2 != d) return fail(QB200_ERR_BAD_SHAPE, "swiglu: gate and up must have the same shape");
  if ((st = row_view(res, "res", &r2, &d2, &ldo))) return st;
  if (r2 != rows || d2 != d) return fail(QB200_ERR_BAD_SHAPE, "swiglu: res must have gate's shape");
  if (d % 2 != 0 || ((((uintptr_t)gate->data) | ((uintptr_t)up->data) | ((uintptr_t)res->data) | (uintptr_t)((ldg | ldu | ldo) * 2)) & 3))
    return fail(QB200_ERR_UNSUPPORTED, "swiglu: rows must be even and 4-byte aligned");
  const cudaError_t e = launch_swiglu((const uint16_t*)gate->data, (const uint16_t*)up->data, (uint16_t*)res->data, rows, (int)d, ldg, ldu,
                                      ldo, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "swiglu");
  return QB200_OK;
}

// q_rope != NULL: the rope form (K rotated on its way into the cache, the queries in place, both at position offsets[n])
static int kv_append_seqs_impl(qb200_tensor* q_rope, int rope_dims, float rope_base, float rope_scale,
                               qb200_tensor* const* k_q, qb200_tensor* const* k_scales, qb200_tensor* const* k_biases,
                               qb200_tensor* const* v_q, qb200_tensor* const* v_scales, qb200_tensor* const* v_biases,
                               const qb200_tensor* dense_k, const qb200_tensor* dense_v, const int64_t* offsets, int num_seqs,
                               int bits, int group_size, qb200_stream s) {
  int gs, nb, st;
  qb200_optional_int og = {group_size, true}, ob = {bits, true};
  if ((st = resolve_mode("affine", og, ob, &gs, &nb))) return st;
  if (nb == 2) return fail(QB200_ERR_UNSUPPORTED, "kv_append_seqs: bits must be 4 or 8");
  if ((st = check_tensor(dense_k, "dense_k", 4)) || (st = check_tensor(dense_v, "dense_v", 4))) return st;
  if (dense_k->ndim != 4 || dense_v->ndim != 4 || dense_k->dtype != QB200_BFLOAT16 || dense_v->dtype != QB200_BFLOAT16)
    return fail(QB200_ERR_UNSUPPORTED, "kv_append_seqs: dense K and V must be bf16 [N, Hkv, 1, D]");
  const int64_t N = dense_k->shape[0], Hkv = dense_k->shape[1];
  if (N != num_seqs || dense_v->shape[0] != N || dense_v->shape[1] != Hkv || dense_k->shape[2] != 1 || dense_v->shape[2] != 1)
    return fail(QB200_ERR_BAD_SHAPE, "kv_append_seqs: one new token per sequence, dense [num_seqs, Hkv, 1, D]");
  if (num_seqs < 0 || (num_seqs > 0 && (!k_q || !k_scales || !k_biases || !v_q || !v_scales || !v_biases || !offsets)))
    return fail(QB200_ERR_BAD_ARG, "kv_append_seqs: null list");
  if (num_seqs == 0) return QB200_OK;
  if (num_seqs > 4096) return fail(QB200_ERR_UNSUPPORTED, "kv_append_seqs: at most 4096 sequences");
  const int vpw = 32 / nb;
  const int64_t D[2] = {dense_k->shape[3], dense_v->shape[3]};
  if (D[0] % gs != 0 || D[1] % gs != 0) return fail(QB200_ERR_BAD_SHAPE, "kv_append_seqs: head dims must be multiples of group_size");
  std::vector<uint32_t*> q[2]; std::vector<uint16_t*> sc[2], bi[2]; std::vector<int64_t> qh[2], sbh[2];
  for (int64_t n = 0; n < N; ++n) {
    qb200_tensor* const ts[2][3] = {{k_q[n], k_scales[n], k_biases[n]}, {v_q[n], v_scales[n], v_biases[n]}};
    for (int kv = 0; kv < 2; ++kv) {
      for (int i = 0; i < 3; ++i) {
        if ((st = check_tensor(ts[kv][i], "cache", 4))) return st;
        if (ts[kv][i]->ndim != 4 || ts[kv][i]->shape[0] != 1 || ts[kv][i]->shape[1] != Hkv)
          return fail(QB200_ERR_BAD_SHAPE, "kv_append_seqs: every cache buffer must be [1, Hkv, cap, last]");
        if (ts[kv][i]->dtype != (i == 0 ? QB200_UINT32 : QB200_BFLOAT16))
          return fail(QB200_ERR_BAD_DTYPE, "kv_append_seqs: codes uint32, scales and biases bf16");
        if (ts[kv][i]->shape[2] != ts[kv][0]->shape[2]) return fail(QB200_ERR_BAD_SHAPE, "kv_append_seqs: the three buffers of a cache disagree on capacity");
      }
      if (ts[kv][0]->shape[3] * vpw != D[kv] || ts[kv][1]->shape[3] != D[kv] / gs || ts[kv][2]->shape[3] != D[kv] / gs)
        return fail(QB200_ERR_BAD_SHAPE, "kv_append_seqs: cache widths do not match the dense rows");
      if (!same_strides(ts[kv][1], ts[kv][2])) return fail(QB200_ERR_BAD_STRIDE, "kv_append_seqs: scales and biases must have identical strides");
      if (offsets[n] < 0 || offsets[n] >= ts[kv][0]->shape[2])
        return fail(QB200_ERR_BAD_SHAPE, "kv_append_seqs: offset %lld outside the capacity %lld of sequence %lld", (long long)offsets[n],
                    (long long)ts[kv][0]->shape[2], (long long)n);
      q[kv].push_back((uint32_t*)ts[kv][0]->data + offsets[n] * ts[kv][0]->stride[2]);
      sc[kv].push_back((uint16_t*)ts[kv][1]->data + offsets[n] * ts[kv][1]->stride[2]);
      bi[kv].push_back((uint16_t*)ts[kv][2]->data + offsets[n] * ts[kv][2]->stride[2]);
      qh[kv].push_back(ts[kv][0]->stride[1]);
      sbh[kv].push_back(ts[kv][1]->stride[1]);
    }
  }
  KvAppendSeqsArgs a;
  const qb200_tensor* dn[2] = {dense_k, dense_v};
  for (int kv = 0; kv < 2; ++kv) {
    a.q[kv] = q[kv].data(); a.s[kv] = sc[kv].data(); a.b[kv] = bi[kv].data();
    a.q_head[kv] = qh[kv].data(); a.sb_head[kv] = sbh[kv].data();
    a.dense[kv] = (const uint16_t*)dn[kv]->data; a.dsn[kv] = dn[kv]->stride[0]; a.dsh[kv] = dn[kv]->stride[1]; a.d[kv] = (int)D[kv];
  }
  a.n = (int)N; a.heads = (int)Hkv; a.gs = gs; a.bits = nb;
  std::vector<int> pos;
  if (q_rope) {
    if ((st = check_tensor(q_rope, "q", 4))) return st;
    if (q_rope->ndim != 4 || q_rope->dtype != QB200_BFLOAT16 || q_rope->shape[0] != N || q_rope->shape[2] != 1 || q_rope->shape[3] != D[0] ||
        q_rope->stride[3] != 1 || dense_k->stride[3] != 1)
      return fail(QB200_ERR_BAD_SHAPE, "rope_kv_append_seqs: q must be bf16 [num_seqs, Hq, 1, D] with K's head dim, rows contiguous");
    if (rope_dims <= 0 || rope_dims % 2 != 0 || rope_dims > D[0] || (rope_dims / 2) % vpw != 0 || !(rope_base > 0.f))
      return fail(QB200_ERR_UNSUPPORTED, "rope_kv_append_seqs: dims must be even, at most D, with dims / 2 a multiple of the values per packed word");
    for (int64_t n = 0; n < N; ++n) {
      if (offsets[n] > 0x7fffffff) return fail(QB200_ERR_BAD_SHAPE, "rope_kv_append_seqs: position out of range");
      pos.push_back((int)offsets[n]);
    }
    a.pos = pos.data();
    a.rq = (uint16_t*)q_rope->data; a.qsn = q_rope->stride[0]; a.qsh = q_rope->stride[1]; a.q_heads = (int)q_rope->shape[1];
    a.rope_dims = rope_dims; a.rope_base = rope_base; a.rope_scale = rope_scale;
  }
  const cudaError_t e = launch_kv_append_seqs(a, (cudaStream_t)s);
  if (e != cudaSuccess) return cuda_fail(e, "kv_append_seqs");
  return QB200_OK;
}

QB200_API int qb200_kv_append_seqs(qb200_tensor* const* k_q, qb200_tensor* const* k_scales, qb200_tensor* const* k_biases,
                                   qb200_tensor* const* v_q, qb200_tensor* const* v_scales, qb200_tensor* const* v_biases,
                                   const qb200_tensor* dense_k, const qb200_tensor* dense_v, const int64_t* offsets, int num_seqs,
                                   int bits, int group_size, qb200_stream s) {
  return kv_append_seqs_impl(nullptr, 0, 0.f, 1.f, k_q, k_scales, k_biases, v_q, v_scales, v_biases, dense_k, dense_v, offsets, num_seqs, bits,
                             group_size, s);
}

QB200_API int qb200_rope_kv_append_seqs(qb200_tensor* q, int dims, float base, float scale, qb200_tensor* const* k_q,
                                        qb200_tensor* const* k_scales, qb200_tensor* const* k_biases, qb200_tensor* const* v_q,
                                        qb200_tensor* const* v_scales, qb200_tensor* const* v_biases, const qb200_tensor* dense_k,
                                        const qb200_tensor* dense_v, const int64_t* offsets, int num_seqs, int bits, int group_size,
                                        qb200_stream s) {
  if (!q) return fail(QB200_ERR_BAD_ARG, "rope_kv_append_seqs: q is required");
  return kv_append_seqs_impl(q, dims, base, scale, k_q, k_scales, k_biases, v_q, v_scales, v_biases, dense_k, dense_v, offsets, num_seqs, bits,
                             group_size, s);
}

}  // extern "C"

// The small operators of the batched decode step around the quantized projections and the packed-cache attention
// (forwardBatchedDecode, mlx-serve src/transformer.zig:9562-9924): RMS norm (alone, or after the residual add that
// precedes it), rotary embedding with one position per sequence, the dense SwiGLU between gate/up and down, and the
// append of one new token per sequence into per-sequence packed caches.  Each is one launch; rounding points are
// the reference graph's: every operator output is rounded to the activation dtype.
#include <cmath>
#include <cstring>

#include "kernels.h"

namespace qb {
namespace {

__device__ __forceinline__ float rbf16(float x) { return __uint_as_float((uint32_t)f32_to_bf16_bits(x) << 16); }

// One CTA per row.  sum_out (optional) = a + b rounded to bf16 (mlx_add, src/transformer.zig:9838-9841), and the
// norm is taken of that sum: y = bf16(w * bf16(x * rsqrt(mean(x^2) + eps))) (mlx_fast_rms_norm).
// VEC: eight values per thread and step through 128-bit loads, the weight row fetched before the reduction (rows of a
// few thousand values are one step for a CTA of up to 1024 threads: every load of the row is in flight at once);
// otherwise two values per step (any alignment of even d).
template <bool VEC>
__global__ void __launch_bounds__(1024) rms_norm_kernel(const uint16_t* a, const uint16_t* b, const uint16_t* w, uint16_t* sum_out,
                                                        uint16_t* norm_out, int64_t lda, int64_t ldb, int64_t lds, int64_t ldn,
                                                        int d, float eps) {
  extern __shared__ float xs[];   // the row in fp32
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const uint16_t* ar = a + row * lda;
  const uint16_t* br = b ? b + row * ldb : nullptr;
  constexpr int V = VEC ? 8 : 2;
  float acc = 0.f;
  uint4 wv0 = make_uint4(0u, 0u, 0u, 0u);   // VEC: the weights of this thread's first step
  if (VEC && norm_out && (int)threadIdx.x * V < d) wv0 = *(const uint4*)(w + threadIdx.x * V);
  for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
    uint32_t av[V / 2], bv[V / 2];
    if constexpr (VEC) {
      const uint4 t = *(const uint4*)(ar + i);
      av[0] = t.x; av[1] = t.y; av[2] = t.z; av[3] = t.w;
      if (br) { const uint4 u = *(const uint4*)(br + i); bv[0] = u.x; bv[1] = u.y; bv[2] = u.z; bv[3] = u.w; }
    } else {
      av[0] = *(const uint32_t*)(ar + i);
      if (br) bv[0] = *(const uint32_t*)(br + i);
    }
    uint32_t sv[V / 2];
#pragma unroll
    for (int j = 0; j < V / 2; ++j) {
      float x0 = bf16lo(av[j]), x1 = bf16hi(av[j]);
      if (br) {
        x0 = rbf16(x0 + bf16lo(bv[j]));
        x1 = rbf16(x1 + bf16hi(bv[j]));
        sv[j] = pack_bf16x2(x0, x1);
      }
      xs[i + 2 * j] = x0; xs[i + 2 * j + 1] = x1;
      acc += x0 * x0 + x1 * x1;
    }
    if (br && sum_out) {
      if constexpr (VEC) *(uint4*)(sum_out + row * lds + i) = make_uint4(sv[0], sv[1], sv[2], sv[3]);
      else *(uint32_t*)(sum_out + row * lds + i) = sv[0];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)d + eps);
  if (!norm_out) return;
  for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
    uint32_t wv[V / 2], ov[V / 2];
    if constexpr (VEC) {
      const uint4 t = i == (int)threadIdx.x * V ? wv0 : *(const uint4*)(w + i);
      wv[0] = t.x; wv[1] = t.y; wv[2] = t.z; wv[3] = t.w;
    } else {
      wv[0] = *(const uint32_t*)(w + i);
    }
#pragma unroll
    for (int j = 0; j < V / 2; ++j)
      ov[j] = pack_bf16x2(bf16lo(wv[j]) * rbf16(xs[i + 2 * j] * inv), bf16hi(wv[j]) * rbf16(xs[i + 2 * j + 1] * inv));
    if constexpr (VEC) *(uint4*)(norm_out + row * ldn + i) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
    else *(uint32_t*)(norm_out + row * ldn + i) = ov[0];
  }
}

// The rotation of one pair: angle = scale * position * base^(-i / half); products and sums as separate fp32 operations
// (no contraction), so that every kernel that rotates gives the same bits.
__device__ __forceinline__ void rope_sincos(int pos, int i, int half, float log2_base, float scale, float* sn, float* c) {
  const float theta = __fmul_rn(__fmul_rn(scale, (float)pos), exp2f(__fmul_rn(-__fdiv_rn((float)i, (float)half), log2_base)));
  sincosf(theta, sn, c);
}
__device__ __forceinline__ float rope_lo(float x1, float x2, float sn, float c) { return __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn)); }
__device__ __forceinline__ float rope_hi(float x1, float x2, float sn, float c) { return __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, c)); }

// Rotary embedding, non-traditional pairing (i, i + dims/2), one position per sequence (mlx_fast_rope_dynamic).
// x [n, heads, 1, d] with strides (sn, sh); in place when out == x.  One thread per pair.
__global__ void __launch_bounds__(256) rope_kernel(const uint16_t* x, uint16_t* out, const int32_t* offsets, int64_t n, int heads,
                                                   int d, int dims, float log2_base, float scale, int64_t xsn, int64_t xsh,
                                                   int64_t osn, int64_t osh) {
  const int half = dims / 2, per_head = d / 2;   // threads per head: the pairs, then the pass-through elements in twos
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * heads * per_head) return;
  const int i = (int)(idx % per_head);
  const int64_t hh = idx / per_head;
  const int h = (int)(hh % heads);
  const int64_t s = hh / heads;
  const uint16_t* xr = x + s * xsn + (int64_t)h * xsh;
  uint16_t* o = out + s * osn + (int64_t)h * osh;
  if (i < half) {
    float sn, c;
    rope_sincos(offsets[s], i, half, log2_base, scale, &sn, &c);
    const float x1 = bf16_bits_to_f32(xr[i]), x2 = bf16_bits_to_f32(xr[i + half]);
    o[i] = f32_to_bf16_bits(rope_lo(x1, x2, sn, c));
    o[i + half] = f32_to_bf16_bits(rope_hi(x1, x2, sn, c));
  } else if (out != x || osn != xsn || osh != xsh) {
    const int e = dims + 2 * (i - half);
    o[e] = xr[e];
    o[e + 1] = xr[e + 1];
  }
}

// silu(gate) * up with the rounding points of the reference's fused kernel (src/transformer.zig:19842-19851): the
// sigmoid of the bf16 gate from a table over all bf16 patterns, g * sig rounded, then * up rounded.
__global__ void __launch_bounds__(256) swiglu_kernel(const uint16_t* gate, const uint16_t* up, uint16_t* out, const uint16_t* sigtab,
                                                     int64_t rows, int d, int64_t ldg, int64_t ldu, int64_t ldo) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = d / 2;
  if (idx >= rows * per_row) return;
  const int64_t r = idx / per_row;
  const int i = (int)(idx - r * per_row) * 2;
  const uint32_t gv = *(const uint32_t*)(gate + r * ldg + i), uv = *(const uint32_t*)(up + r * ldu + i);
  const float g0 = bf16lo(gv), g1 = bf16hi(gv);
  const float s0 = bf16_bits_to_f32(sigtab[gv & 0xFFFFu]), s1 = bf16_bits_to_f32(sigtab[gv >> 16]);
  const float y0 = rbf16(g0 * s0) * bf16lo(uv), y1 = rbf16(g1 * s1) * bf16hi(uv);
  *(uint32_t*)(out + r * ldo + i) = pack_bf16x2(y0, y1);
}

// ---- one new token per sequence into per-sequence packed caches (KVCache.updateAffine per slot,
// src/transformer.zig:9738-9756, :3224-3337): quantise K and V rows and write the triples at each cache's offset ----
struct AppendSeq {
  uint32_t* q[2]; uint16_t* s[2]; uint16_t* b[2];   // [K, V]: the token row of head 0
  int64_t q_head[2], sb_head[2];                    // head strides in elements
  int pos;                                          // position of the new token (the rotary angle's factor)
};
struct AppendTable { AppendSeq s[kMaxSeqPtrs]; };
struct AppendArgs {
  const uint16_t* dense[2];       // K, V rows [n, heads, 1, d]
  int64_t dsn[2], dsh[2];
  int n, heads, d[2], gs;
  // ROPE form: the rotary embedding of K happens on the way into the cache, and the same launch rotates the
  // queries [n, q_heads, 1, d[0]] in place (mlx_fast_rope_dynamic on q and k, then updateAffine: one launch for both)
  uint16_t* rq; int64_t qsn, qsh; int q_heads;
  int dims; float log2_base, scale;
};

template <int BITS, bool ROPE>
__global__ void __launch_bounds__(256) kv_append_seqs_kernel(const __grid_constant__ AppendArgs a, const __grid_constant__ AppendTable tab) {
  constexpr int VPW = 32 / BITS;
  // thread -> (which of K / V, sequence, head, packed word); the threads of a group are adjacent lanes
  const int wpr0 = a.d[0] / VPW, wpr1 = a.d[1] / VPW;
  const int64_t n0 = (int64_t)a.n * a.heads * wpr0, total = n0 + (int64_t)a.n * a.heads * wpr1;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if constexpr (ROPE) {
    // the blocks behind the quantiser's rotate the queries: one thread per pair (whole blocks, so no warp is mixed)
    const int64_t qblk0 = (total + blockDim.x - 1) / blockDim.x;
    if ((int64_t)blockIdx.x >= qblk0) {
      const int half = a.dims / 2, per_head = a.d[0] / 2;
      const int64_t qi = ((int64_t)blockIdx.x - qblk0) * blockDim.x + threadIdx.x;
      if (qi >= (int64_t)a.n * a.q_heads * per_head) return;
      const int i = (int)(qi % per_head);
      const int64_t hh = qi / per_head;
      const int h = (int)(hh % a.q_heads), sq = (int)(hh / a.q_heads);
      if (i >= half) return;   // pass-through elements stay where they are (in place)
      uint16_t* xr = a.rq + (int64_t)sq * a.qsn + (int64_t)h * a.qsh;
      float sn, c;
      rope_sincos(tab.s[sq].pos, i, half, a.log2_base, a.scale, &sn, &c);
      const float x1 = bf16_bits_to_f32(xr[i]), x2 = bf16_bits_to_f32(xr[i + half]);
      xr[i] = f32_to_bf16_bits(rope_lo(x1, x2, sn, c));
      xr[i + half] = f32_to_bf16_bits(rope_hi(x1, x2, sn, c));
      return;
    }
  }
  const bool live = idx < total;
  if (!live) idx = total - 1;   // keep the warp converged for the shuffles
  const int kv = idx >= n0 ? 1 : 0;
  const int64_t li = kv ? idx - n0 : idx;
  const int wpr = kv ? wpr1 : wpr0;
  const int wi = (int)(li % wpr);
  const int64_t rh = li / wpr;
  const int h = (int)(rh % a.heads);
  const int s = (int)(rh / a.heads);
  const uint16_t* xr = a.dense[kv] + (int64_t)s * a.dsn[kv] + (int64_t)h * a.dsh[kv] + wi * VPW;
  float v[VPW];
#pragma unroll
  for (int k = 0; k < VPW; ++k) v[k] = bf16_bits_to_f32(xr[k]);
  if constexpr (ROPE) {
    // K: this word's values rotated with their partners half a rotary width away (a word lies on one side of the
    // pairing: dims / 2 is a multiple of the values per word), rounded to bf16 as the separate rope would store them
    const int e0 = wi * VPW, half = a.dims / 2;
    if (kv == 0 && e0 < a.dims) {
      const bool low = e0 < half;
      const uint16_t* pr = low ? xr + half : xr - half;
#pragma unroll
      for (int k = 0; k < VPW; ++k) {
        const float other = bf16_bits_to_f32(pr[k]);
        float sn, c;
        rope_sincos(tab.s[s].pos, (low ? e0 : e0 - half) + k, half, a.log2_base, a.scale, &sn, &c);
        const float r = low ? rope_lo(v[k], other, sn, c) : rope_hi(other, v[k], sn, c);
        v[k] = bf16_bits_to_f32(f32_to_bf16_bits(r));
      }
    }
  }
  float xmin = v[0], xmax = v[0];
#pragma unroll
  for (int k = 1; k < VPW; ++k) { xmin = fminf(xmin, v[k]); xmax = fmaxf(xmax, v[k]); }
  const int tpg = a.gs / VPW;   // threads per group: a power of two, at most 32
  for (int off = tpg >> 1; off > 0; off >>= 1) {
    xmin = fminf(xmin, __shfl_xor_sync(0xffffffffu, xmin, off));
    xmax = fmaxf(xmax, __shfl_xor_sync(0xffffffffu, xmax, off));
  }
  // the affine rule of mlx_quantize as the reference restates it (tests/dsv4_imatrix.py:169-183, codes :264)
  const float n_bins = (float)((1 << BITS) - 1);
  const bool mask = fabsf(xmin) > fabsf(xmax);
  float scale = fmaxf(__fdiv_rn(__fsub_rn(xmax, xmin), n_bins), 1e-7f);
  scale = mask ? scale : -scale;
  const float edge = mask ? xmin : xmax;
  const float q0 = rintf(__fdiv_rn(edge, scale));
  float bias = 0.0f;
  if (q0 != 0.0f) { scale = __fdiv_rn(edge, q0); bias = edge; }
  uint32_t word = 0;
#pragma unroll
  for (int k = 0; k < VPW; ++k) {
    float c = rintf(__fdiv_rn(__fsub_rn(v[k], bias), scale));
    c = fminf(fmaxf(c, 0.0f), n_bins);
    word |= ((uint32_t)c) << (k * BITS);
  }
  if (!live) return;
  const AppendSeq& e = tab.s[s];
  e.q[kv][(int64_t)h * e.q_head[kv] + wi] = word;
  if ((wi % tpg) == 0) {
    const int64_t o = (int64_t)h * e.sb_head[kv] + (wi * VPW) / a.gs;
    e.s[kv][o] = f32_to_bf16_bits(scale);
    e.b[kv][o] = f32_to_bf16_bits(bias);
  }
}


// ---- the rotation of the TurboQuant cache schemes (src/kv_quant.zig:164-403): out = x @ R along the last axis with
// R = diag(sg) H diag(sg) / sqrt(D), H the Sylvester Hadamard matrix and sg a +-1 vector -- symmetric and orthogonal, so
// the same call rotates back.  The reference multiplies by the [D, D] bf16 matrix; every entry of it is +-r with
// r = bf16(1 / sqrt(D)), so the product is r * sg[e] * sum_j H[e][j] * sg[j] * x[j]: a fast Walsh-Hadamard transform,
// D log2 D additions per row instead of D^2 multiply-adds.  One warp per row, element e = j * 32 + lane: the low five
// bits of e are the lane (shuffles), the rest stay in the lane's registers. ----
struct TurboSigns { uint32_t bits[32]; };   // bit e of the vector: 1 = -1 (D <= 1024)

template <int PER>   // values per lane: D / 32
__global__ void __launch_bounds__(256) turbo_rotate_kernel(const uint16_t* x, uint16_t* out, int64_t rows, int64_t ldx, int64_t ldo,
                                                           float r, const __grid_constant__ TurboSigns sg) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint16_t* xr = x + row * ldx;
  float v[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const float f = bf16_bits_to_f32(xr[j * 32 + lane]);
    v[j] = ((sg.bits[j] >> lane) & 1u) ? -f : f;
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {   // bits of the lane
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
      v[j] = (lane & m) ? __fsub_rn(o, v[j]) : __fadd_rn(v[j], o);
    }
  }
#pragma unroll
  for (int m = 1; m < PER; m <<= 1) {   // bits of the register index
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      if ((j & m) == 0) {
        const float a = v[j], b = v[j | m];
        v[j] = __fadd_rn(a, b);
        v[j | m] = __fsub_rn(a, b);
      }
    }
  }
  uint16_t* orow = out + row * ldo;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const float y = __fmul_rn(v[j], r);
    orow[j * 32 + lane] = f32_to_bf16_bits(((sg.bits[j] >> lane) & 1u) ? -y : y);
  }
}

}  // namespace

cudaError_t launch_rms_norm(const uint16_t* a, const uint16_t* b, const uint16_t* w, uint16_t* sum_out, uint16_t* norm_out,
                            int64_t rows, int d, int64_t lda, int64_t ldb, int64_t lds, int64_t ldn, float eps, cudaStream_t st) {
  if (rows <= 0 || d <= 0) return cudaSuccess;
  // 128-bit form when every row of every operand is 16-byte aligned; a CTA of up to 1024 threads, one step per row
  // where the row is short enough
  auto al16 = [](const void* p, int64_t ld) { return p == nullptr || (((uintptr_t)p & 15) == 0 && (ld * 2) % 16 == 0); };
  const bool vec = d % 8 == 0 && al16(a, lda) && al16(b, ldb) && al16(w, 0) && al16(sum_out, lds) && al16(norm_out, ldn);
  const int per = vec ? 8 : 2;
  int threads = (d + per - 1) / per;
  threads = (threads + 31) / 32 * 32;
  threads = threads > 1024 ? 1024 : (threads < 64 ? 64 : threads);
  if ((size_t)d * sizeof(float) > 48 * 1024) {   // rows beyond 12288 values: the fp32 copy of a row needs the opt-in shared memory
    std::lock_guard<std::mutex> lk(setup_mutex());
    static bool done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !done[dev]) {
      cudaError_t e = cudaFuncSetAttribute(rms_norm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * (int)sizeof(float));
      if (e == cudaSuccess) e = cudaFuncSetAttribute(rms_norm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * (int)sizeof(float));
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  if (vec)
    return launch_kernel(rms_norm_kernel<true>, dim3((unsigned)rows), dim3(threads), (size_t)d * sizeof(float), st, a, b, w, sum_out, norm_out, lda, ldb, lds, ldn, d, eps);
  return launch_kernel(rms_norm_kernel<false>, dim3((unsigned)rows), dim3(threads), (size_t)d * sizeof(float), st, a, b, w, sum_out, norm_out, lda, ldb, lds, ldn, d, eps);
}

cudaError_t launch_rope(const uint16_t* x, uint16_t* out, const int32_t* offsets, int64_t n, int heads, int d, int dims, float base,
                        float scale, int64_t xsn, int64_t xsh, int64_t osn, int64_t osh, cudaStream_t st) {
  const int64_t total = n * heads * (d / 2);
  if (total <= 0) return cudaSuccess;
  return launch_kernel(rope_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, x, out, offsets, n, heads, d, dims, log2f(base), scale, xsn, xsh, osn, osh);
}

cudaError_t launch_swiglu(const uint16_t* gate, const uint16_t* up, uint16_t* out, int64_t rows, int d, int64_t ldg, int64_t ldu,
                          int64_t ldo, cudaStream_t st) {
  const int64_t total = rows * (d / 2);
  if (total <= 0) return cudaSuccess;
  cudaError_t te;
  const uint16_t* tab = sigmoid_table(st, &te);
  if (!tab) return te;
  return launch_kernel(swiglu_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, gate, up, out, tab, rows, d, ldg, ldu, ldo);
}

cudaError_t launch_kv_append_seqs(const KvAppendSeqsArgs& h, cudaStream_t st) {
  for (int s0 = 0; s0 < h.n; s0 += kMaxSeqPtrs) {
    const int nb = h.n - s0 < kMaxSeqPtrs ? h.n - s0 : kMaxSeqPtrs;
    AppendTable tab;
    std::memset(&tab, 0, sizeof(tab));
    for (int i = 0; i < nb; ++i)
      for (int kv = 0; kv < 2; ++kv) {
        tab.s[i].q[kv] = h.q[kv][s0 + i]; tab.s[i].s[kv] = h.s[kv][s0 + i]; tab.s[i].b[kv] = h.b[kv][s0 + i];
        tab.s[i].q_head[kv] = h.q_head[kv][s0 + i]; tab.s[i].sb_head[kv] = h.sb_head[kv][s0 + i];
        tab.s[i].pos = h.pos ? h.pos[s0 + i] : 0;
      }
    AppendArgs a;
    for (int kv = 0; kv < 2; ++kv) {
      a.dense[kv] = h.dense[kv] + (int64_t)s0 * h.dsn[kv];
      a.dsn[kv] = h.dsn[kv]; a.dsh[kv] = h.dsh[kv]; a.d[kv] = h.d[kv];
    }
    a.n = nb; a.heads = h.heads; a.gs = h.gs;
    a.rq = h.rq ? h.rq + (int64_t)s0 * h.qsn : nullptr; a.qsn = h.qsn; a.qsh = h.qsh; a.q_heads = h.q_heads;
    a.dims = h.rope_dims; a.log2_base = h.rope_dims > 0 ? log2f(h.rope_base) : 0.f; a.scale = h.rope_scale;
    const int vpw = 32 / h.bits;
    const int64_t total = (int64_t)nb * h.heads * (h.d[0] / vpw + h.d[1] / vpw);
    unsigned blocks = (unsigned)((total + 255) / 256);
    cudaError_t e;
    if (h.rope_dims > 0) {
      blocks += (unsigned)(((int64_t)nb * h.q_heads * (h.d[0] / 2) + 255) / 256);   // the blocks that rotate the queries
      e = h.bits == 4 ? launch_kernel(kv_append_seqs_kernel<4, true>, dim3(blocks), dim3(256), 0, st, a, tab)
                      : launch_kernel(kv_append_seqs_kernel<8, true>, dim3(blocks), dim3(256), 0, st, a, tab);
    } else {
      e = h.bits == 4 ? launch_kernel(kv_append_seqs_kernel<4, false>, dim3(blocks), dim3(256), 0, st, a, tab)
                      : launch_kernel(kv_append_seqs_kernel<8, false>, dim3(blocks), dim3(256), 0, st, a, tab);
    }
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// signs: bit e set = -1, the vector of TurboState's cloneWithSignFlip (src/kv_quant.zig:318-330)
cudaError_t launch_turbo_rotate(const uint16_t* x, uint16_t* out, int64_t rows, int d, int64_t ldx, int64_t ldo, const uint32_t* signs,
                                cudaStream_t st) {
  if (rows <= 0) return cudaSuccess;
  TurboSigns sg;
  std::memset(&sg, 0, sizeof(sg));
  for (int i = 0; i < d / 32; ++i) sg.bits[i] = signs[i];
  // r = bf16(1 / sqrt(d)): the magnitude of every entry of the reference's bf16 matrix
  float r = 1.0f / std::sqrt((float)d);
  {
    uint32_t u;
    std::memcpy(&u, &r, 4);
    u = (u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u;   // round to nearest even at bf16 precision
    std::memcpy(&r, &u, 4);
  }
  const dim3 grid((unsigned)((rows + 7) / 8)), block(256);
  switch (d / 32) {
    case 1: return launch_kernel(turbo_rotate_kernel<1>, grid, block, 0, st, x, out, rows, ldx, ldo, r, sg);
    case 2: return launch_kernel(turbo_rotate_kernel<2>, grid, block, 0, st, x, out, rows, ldx, ldo, r, sg);
    case 4: return launch_kernel(turbo_rotate_kernel<4>, grid, block, 0, st, x, out, rows, ldx, ldo, r, sg);
    case 8: return launch_kernel(turbo_rotate_kernel<8>, grid, block, 0, st, x, out, rows, ldx, ldo, r, sg);
    case 16: return launch_kernel(turbo_rotate_kernel<16>, grid, block, 0, st, x, out, rows, ldx, ldo, r, sg);
    case 32: return launch_kernel(turbo_rotate_kernel<32>, grid, block, 0, st, x, out, rows, ldx, ldo, r, sg);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace qb

/*
 * qoracle.c -- CPU restatement of the affine group-quantized inference path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is
 * compared against (tests/, the smoke check and the cpu_baseline leg of the
 * benchmark).  Nothing in the shipped library links, loads or calls it.
 *
 * What it restates (paths are relative to the mlx-serve source tree):
 *   - packed layout, unpack, dequantize : tests/dsv4_imatrix.py:107-163
 *     (pack_bits / unpack_bits / dequant_np), cross-checked by the unpack in
 *     src/transformer.zig:20098-20109 and :4931-4937
 *   - bf16 round-to-nearest-even        : tests/convert_dsv4_weights.py:154-162
 *   - quantize (scale/bias selection)   : tests/dsv4_imatrix.py:169-183
 *     (_mlx_minmax_sb) and the code derivation at :264
 *   - quantized_matmul, both transposes : src/kv_quant.zig:968-1094 and the
 *     ground-truth loops in src/transformer.zig:24735-24744
 *   - gather_qmm                        : src/transformer.zig:24735-24744,
 *     :24799-24808, call shapes :15007-15035 and :15091-15119
 *   - decode attention over packed K/V  : src/kv_quant.zig:478-687, kernel
 *     semantics src/transformer.zig:4890-5006, batch length mask :10216-10249
 *
 * The arithmetic itself lives in ml-explore/mlx v0.32.0 (an un-vendored
 * submodule, lib/mlx-src, absent from the checkout).  Parity is therefore
 * pinned to the reference's own Python restatement above: the golden vectors
 * under tests/golden/ were produced by importing tests/dsv4_imatrix.py and this
 * file must reproduce them bit for bit (tests/test_oracle_golden.py).
 *
 * Two definitions no reference test pins, fixed here and mirrored on the GPU:
 *   dequantize: bf16_rne( fmul(float(q), float(scale)) + float(bias) ) with a
 *               separate fp32 multiply and add (build with -ffp-contract=off);
 *   quantize:   codes are derived from the UNROUNDED fp32 (scale, bias); the
 *               stored scale/bias are those values rounded to bf16.
 * Matmul/attention accumulate in fp32 in index order; the weight term is the
 * fp32 value q*s+b (not rounded to bf16).
 *
 * The decode step around the kernels (src/transformer.zig:9562-9924) adds two operators whose arithmetic also lives in
 * MLX (mlx_fast_rms_norm, mlx_fast_rope_dynamic; src/mlx.zig:319-324).  Their restatement here follows MLX's
 * published definition of the fused operators' fallback graphs and is unpinned against MLX itself:
 *   rms_norm: y = bf16( w * bf16( x * rsqrt(mean(x^2) + eps) ) ), the mean and the first product in fp32;
 *   rope (non-traditional): pairs (i, i + dims/2), angle = scale * offset * base^(-2i/dims), rotation in fp32,
 *             one rounding; elements beyond `dims` pass through.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define QO_API __attribute__((visibility("default")))

/* ---- bf16 <-> f32 (tests/convert_dsv4_weights.py:154-162) ---- */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t r = u + 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(r >> 16);
}

QO_API void qo_f32_to_bf16(const float* x, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(x[i]);
}
QO_API void qo_bf16_to_f32(const uint16_t* x, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = bf16_to_f32(x[i]);
}

/* ---- fused SwiGLU of the MoE block: y = silu(gate) * up, elementwise (src/transformer.zig:19842-19851) ----
 * bf16 form: gate and up are first rounded to bf16 (they are the stored outputs of the two projections);
 * sig = bf16(sigmoid(gate)) (the reference reads it from a table of mlx_sigmoid over all bf16 patterns,
 * src/transformer.zig:19853-19885); act = bf16(gate * sig); y = bf16(act * up).
 * Parity unpinned: the last bit of mlx_sigmoid itself is not pinned by any reference test; this restatement uses
 * the two-sided form the reference quotes from MLX's Sigmoid (src/transformer.zig:17566-17570) in fp32. */
static inline float sigmoid_f32(float x) {
  const float sy = 1.0f / (1.0f + expf(fabsf(x)));
  return x < 0.0f ? sy : 1.0f - sy;
}
QO_API void qo_swiglu_bf16(const float* gate, const float* up, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    const float g = bf16_to_f32(f32_to_bf16(gate[i]));
    const float u = bf16_to_f32(f32_to_bf16(up[i]));
    const float sig = bf16_to_f32(f32_to_bf16(sigmoid_f32(g)));
    const float act = bf16_to_f32(f32_to_bf16(g * sig));
    out[i] = f32_to_bf16(act * u);
  }
}
/* ---- router (src/transformer.zig:17022-17063): indices of the k largest logits (larger first, ties by lower
 * index, as the reference's one-kernel router picks them, :17485-17500), softmax over the row in fp32 rounded to the
 * logits' dtype, the k entries renormalised by their sum accumulated in that dtype.
 * logits are fp32 carriers (bf16 values when as_bf16). */
QO_API void qo_moe_route(const float* logits, int64_t T, int64_t E, int64_t k, int as_bf16, int32_t* inds, float* scores) {
  unsigned char* taken = (unsigned char*)malloc((size_t)E);
  for (int64_t t = 0; t < T; ++t) {
    const float* x = logits + t * E;
    float mx = -INFINITY, sum = 0.0f;
    for (int64_t e = 0; e < E; ++e) mx = x[e] > mx ? x[e] : mx;
    for (int64_t e = 0; e < E; ++e) sum += expf(x[e] - mx);
    memset(taken, 0, (size_t)E);
    float wsum = 0.0f;
    for (int64_t j = 0; j < k; ++j) {
      int64_t best = -1;
      for (int64_t e = 0; e < E; ++e)
        if (!taken[e] && (best < 0 || x[e] > x[best])) best = e;
      taken[best] = 1;
      inds[t * k + j] = (int32_t)best;
      float pr = expf(x[best] - mx) / sum;
      if (as_bf16) pr = bf16_to_f32(f32_to_bf16(pr));
      scores[t * k + j] = pr;
      wsum = as_bf16 ? bf16_to_f32(f32_to_bf16(wsum + pr)) : wsum + pr;   /* accumulate in the input dtype (:17530-17534) */
    }
    for (int64_t j = 0; j < k; ++j) {
      const float ns = scores[t * k + j] / wsum;
      scores[t * k + j] = as_bf16 ? bf16_to_f32(f32_to_bf16(ns)) : ns;
    }
  }
  free(taken);
}

/* ---- score-weighted sum over top-k with the rows taken back from expert order
 * (src/transformer.zig:15036-15042, :15127-15140): out[t,h] = sum_j y[inv[t*k+j], h] * scores[t, j].
 * bf16 form (as_bf16 != 0): y and scores are bf16 values, each product is rounded to bf16 and added to a bf16
 * accumulator in ascending j, rounded after every add (src/transformer.zig:20566-20571: "MLX's bf16 sum reduction
 * accumulates in the input dtype").  inv may be NULL (identity). */
QO_API void qo_moe_weighted_sum(const float* y, const float* scores, const int64_t* inv, int64_t T, int64_t k, int64_t H,
                                int as_bf16, float* out) {
  for (int64_t t = 0; t < T; ++t)
    for (int64_t h = 0; h < H; ++h) {
      float acc = 0.0f;
      for (int64_t j = 0; j < k; ++j) {
        const int64_t row = inv ? inv[t * k + j] : t * k + j;
        if (row < 0 || row >= T * k) continue;
        const float p = y[row * H + h] * scores[t * k + j];
        acc = as_bf16 ? bf16_to_f32(f32_to_bf16(acc + bf16_to_f32(f32_to_bf16(p)))) : acc + p;
      }
      out[t * H + h] = acc;
    }
}
/* fp32 form (the reference declines fp32 there and keeps the unfused chain): (g * sigmoid(g)) * u in fp32. */
QO_API void qo_swiglu_f32(const float* gate, const float* up, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = (gate[i] * sigmoid_f32(gate[i])) * up[i];
}
/* Launchers such as torchrun export OMP_NUM_THREADS=1; a timing run may ask for the host's cores back. */
QO_API void qo_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
QO_API int qo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---- pack / unpack, bits in {2,4,8} (tests/dsv4_imatrix.py:107-153) ----
 * value i of a row sits in word i/(32/bits) at bit (i % (32/bits))*bits. */
QO_API void qo_pack(const uint8_t* q, int64_t rows, int64_t d, int bits, uint32_t* out) {
  const int vpw = 32 / bits;
  const int64_t words = d / vpw;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t w = 0; w < words; ++w) {
      uint32_t word = 0;
      for (int k = 0; k < vpw; ++k) word |= ((uint32_t)q[r * d + w * vpw + k]) << (k * bits);
      out[r * words + w] = word;
    }
}
QO_API void qo_unpack(const uint32_t* w, int64_t rows, int64_t d, int bits, uint8_t* out) {
  const int vpw = 32 / bits;
  const int64_t words = d / vpw;
  const uint32_t mask = (1u << bits) - 1u;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t i = 0; i < d; ++i)
      out[r * d + i] = (uint8_t)((w[r * words + i / vpw] >> ((i % vpw) * bits)) & mask);
}

static inline float unpack1(const uint32_t* row, int64_t i, int bits) {
  const int vpw = 32 / bits;
  return (float)((row[i / vpw] >> ((i % vpw) * bits)) & ((1u << bits) - 1u));
}

/* ---- dequantize (tests/dsv4_imatrix.py:156-163) ----
 * w[r,i] = float(q)*float(s[r,i/gs]) + float(b[r,i/gs]); fp32 out. */
QO_API void qo_dequantize_f32(const uint32_t* w, const uint16_t* s, const uint16_t* b,
                              int64_t rows, int64_t d, int gs, int bits, float* out) {
  const int64_t words = d * bits / 32, groups = d / gs;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t i = 0; i < d; ++i) {
      const float sc = bf16_to_f32(s[r * groups + i / gs]);
      const float bi = bf16_to_f32(b[r * groups + i / gs]);
      const float prod = unpack1(w + r * words, i, bits) * sc; /* rounded fp32 product */
      out[r * d + i] = prod + bi;
    }
}
QO_API void qo_dequantize_bf16(const uint32_t* w, const uint16_t* s, const uint16_t* b,
                               int64_t rows, int64_t d, int gs, int bits, uint16_t* out) {
  const int64_t words = d * bits / 32, groups = d / gs;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t i = 0; i < d; ++i) {
      const float sc = bf16_to_f32(s[r * groups + i / gs]);
      const float bi = bf16_to_f32(b[r * groups + i / gs]);
      const float prod = unpack1(w + r * words, i, bits) * sc;
      out[r * d + i] = f32_to_bf16(prod + bi);
    }
}

/* ---- quantize (tests/dsv4_imatrix.py:169-183 and :264) ----
 * x: fp32 (bf16 inputs are widened by the caller, exactly). */
QO_API void qo_quantize(const float* x, int64_t rows, int64_t d, int gs, int bits,
                        uint32_t* out_q, uint16_t* out_s, uint16_t* out_b) {
  const int vpw = 32 / bits;
  const int64_t words = d / vpw, groups = d / gs;
  const float n_bins = (float)((1 << bits) - 1);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t w = 0; w < words; ++w) out_q[r * words + w] = 0;
    for (int64_t g = 0; g < groups; ++g) {
      const float* X = x + r * d + g * gs;
      float xmin = X[0], xmax = X[0];
      for (int j = 1; j < gs; ++j) {
        xmin = fminf(xmin, X[j]);
        xmax = fmaxf(xmax, X[j]);
      }
      const int mask = fabsf(xmin) > fabsf(xmax);
      float scale = fmaxf((xmax - xmin) / n_bins, 1e-7f);
      scale = mask ? scale : -scale;
      const float edge = mask ? xmin : xmax;
      const float q0 = rintf(edge / scale);
      float bias = 0.0f;
      if (q0 != 0.0f) {
        scale = edge / q0;
        bias = edge;
      }
      for (int j = 0; j < gs; ++j) {
        float v = rintf((X[j] - bias) / scale);
        v = fminf(fmaxf(v, 0.0f), n_bins);
        const int64_t i = g * gs + j;
        out_q[r * words + i / vpw] |= ((uint32_t)v) << ((i % vpw) * bits);
      }
      out_s[r * groups + g] = f32_to_bf16(scale);
      out_b[r * groups + g] = f32_to_bf16(bias);
    }
  }
}

/* ---- quantized_matmul, transpose=true (src/kv_quant.zig:968-1036) ----
 * y[m,n] = sum_k x[m,k] * What[n,k];  W packed [N, K*bits/32], s,b [N, K/gs]. */
QO_API void qo_qmm_t(const float* x, const uint32_t* w, const uint16_t* s, const uint16_t* b,
                     int64_t M, int64_t N, int64_t K, int gs, int bits, float* y) {
  const int64_t words = K * bits / 32, groups = K / gs;
#pragma omp parallel
  {
    float* wrow = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      for (int64_t k = 0; k < K; ++k) {
        const float sc = bf16_to_f32(s[n * groups + k / gs]);
        const float bi = bf16_to_f32(b[n * groups + k / gs]);
        const float prod = unpack1(w + n * words, k, bits) * sc;
        wrow[k] = prod + bi;
      }
      for (int64_t m = 0; m < M; ++m) {
        float acc = 0.0f;
        const float* xr = x + m * K;
        for (int64_t k = 0; k < K; ++k) acc += xr[k] * wrow[k];
        y[m * N + n] = acc;
      }
    }
    free(wrow);
  }
}

/* ---- quantized_matmul through the dense prefill route (src/transformer.zig:20987-21011) ----
 * prefillDqGemm dequantises W to a bf16 [N, K] transient and runs a dense GEMM: the weight
 * term is rounded to bf16 before the dot; accumulation stays fp32. */
QO_API void qo_qmm_t_bf16w(const float* x, const uint32_t* w, const uint16_t* s, const uint16_t* b,
                           int64_t M, int64_t N, int64_t K, int gs, int bits, float* y) {
  const int64_t words = K * bits / 32, groups = K / gs;
#pragma omp parallel
  {
    float* wrow = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      for (int64_t k = 0; k < K; ++k) {
        const float sc = bf16_to_f32(s[n * groups + k / gs]);
        const float bi = bf16_to_f32(b[n * groups + k / gs]);
        const float prod = unpack1(w + n * words, k, bits) * sc;
        wrow[k] = bf16_to_f32(f32_to_bf16(prod + bi));
      }
      for (int64_t m = 0; m < M; ++m) {
        float acc = 0.0f;
        const float* xr = x + m * K;
        for (int64_t k = 0; k < K; ++k) acc += xr[k] * wrow[k];
        y[m * N + n] = acc;
      }
    }
    free(wrow);
  }
}

/* ---- quantized_matmul, transpose=false (src/kv_quant.zig:1038-1094) ----
 * y[m,n] = sum_k x[m,k] * What[k,n];  W packed [K, N*bits/32], s,b [K, N/gs]
 * (groups run along the output axis n). */
QO_API void qo_qmm_n(const float* x, const uint32_t* w, const uint16_t* s, const uint16_t* b,
                     int64_t M, int64_t N, int64_t K, int gs, int bits, float* y) {
  const int64_t words = N * bits / 32, groups = N / gs;
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t n = 0; n < N; ++n) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        const float sc = bf16_to_f32(s[k * groups + n / gs]);
        const float bi = bf16_to_f32(b[k * groups + n / gs]);
        const float prod = unpack1(w + k * words, n, bits) * sc;
        acc += x[m * K + k] * (prod + bi);
      }
      y[m * N + n] = acc;
    }
  }
}

/* ---- gather_qmm, transpose=true (src/transformer.zig:24735-24744, :24799-24808) ----
 * For output batch element i: y[i, m, :] = x[lhs[i], m, :] . What[rhs[i]]^T.
 * x: [XB, M, K]; bank w: [E, N, K*bits/32]; lhs/rhs: [I]. */
QO_API void qo_gather_qmm_t(const float* x, const uint32_t* w, const uint16_t* s, const uint16_t* b,
                            const int64_t* lhs, const int64_t* rhs, int64_t I, int64_t M,
                            int64_t N, int64_t K, int gs, int bits, float* y) {
  const int64_t words = K * bits / 32, groups = K / gs;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t i = 0; i < I; ++i) {
    const int64_t e = rhs[i];
    qo_qmm_t(x + lhs[i] * M * K, w + e * N * words, s + e * N * groups, b + e * N * groups, M, N,
             K, gs, bits, y + i * M * N);
  }
}

/* ---- decode attention over a packed K/V cache ----
 * (src/kv_quant.zig:478-687 semantics with Tq == 1; batch length mask
 *  src/transformer.zig:10216-10249; kernel semantics :4890-5006)
 * q: [B, Hq, D] fp32; K triple: kq [B,Hkv,T,D*bits/32], ks/kb [B,Hkv,T,D/gs];
 * V triple likewise with Dv.  All addressed by explicit (batch, head, token)
 * element strides because cache views are strided slices of capacity buffers
 * (src/transformer.zig:3472-3495).  kv_lens[b] (may be NULL => T) masks
 * positions >= len; mask (may be NULL) is an additive fp32 row [B, T].
 * out: [B, Hq, Dv] fp32. */
QO_API void qo_kv_decode_attention(
    const float* q, const uint32_t* kq, const uint16_t* ks, const uint16_t* kb,
    const uint32_t* vq, const uint16_t* vs, const uint16_t* vb, int64_t B, int64_t Hq,
    int64_t Hkv, int64_t T, int64_t D, int64_t Dv, int gs, int bits,
    const int64_t* kq_str, const int64_t* ksb_str, const int64_t* vq_str, const int64_t* vsb_str,
    float scale, const int32_t* kv_lens, const float* mask, float* out) {
  const int64_t gqa = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int64_t bi = 0; bi < B; ++bi) {
    for (int64_t h = 0; h < Hq; ++h) {
      const int64_t hk = h / gqa;
      const int64_t len = kv_lens ? (int64_t)kv_lens[bi] : T;
      float* sc = (float*)malloc(sizeof(float) * (size_t)(T > 0 ? T : 1));
      const float* qv = q + (bi * Hq + h) * D;
      float mx = -INFINITY;
      for (int64_t t = 0; t < len; ++t) {
        const uint32_t* row = kq + bi * kq_str[0] + hk * kq_str[1] + t * kq_str[2];
        const uint16_t* srow = ks + bi * ksb_str[0] + hk * ksb_str[1] + t * ksb_str[2];
        const uint16_t* brow = kb + bi * ksb_str[0] + hk * ksb_str[1] + t * ksb_str[2];
        float acc = 0.0f;
        for (int64_t e = 0; e < D; ++e) {
          const float prod = unpack1(row, e, bits) * bf16_to_f32(srow[e / gs]);
          acc += qv[e] * (prod + bf16_to_f32(brow[e / gs]));
        }
        float v = acc * scale;
        if (mask) v += mask[bi * T + t];
        sc[t] = v;
        if (v > mx) mx = v;
      }
      float* o = out + (bi * Hq + h) * Dv;
      for (int64_t e = 0; e < Dv; ++e) o[e] = 0.0f;
      float l = 0.0f;
      if (mx == -INFINITY) mx = 0.0f; /* fully masked: weights all zero */
      for (int64_t t = 0; t < len; ++t) {
        const float p = expf(sc[t] - mx);
        l += p;
        const uint32_t* row = vq + bi * vq_str[0] + hk * vq_str[1] + t * vq_str[2];
        const uint16_t* srow = vs + bi * vsb_str[0] + hk * vsb_str[1] + t * vsb_str[2];
        const uint16_t* brow = vb + bi * vsb_str[0] + hk * vsb_str[1] + t * vsb_str[2];
        for (int64_t e = 0; e < Dv; ++e) {
          const float prod = unpack1(row, e, bits) * bf16_to_f32(srow[e / gs]);
          o[e] += p * (prod + bf16_to_f32(brow[e / gs]));
        }
      }
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      for (int64_t e = 0; e < Dv; ++e) o[e] *= inv;
      free(sc);
    }
  }
}


/* ---- mlx_fast_rms_norm (src/mlx.zig:319; callers rmsNorm / rmsNormEps, src/transformer.zig:7770-7779) ----
 * x [rows, d] and w [d] are fp32 carriers of bf16 values when as_bf16; out likewise. */
QO_API void qo_rms_norm(const float* x, const float* w, int64_t rows, int64_t d, float eps, int as_bf16, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * d;
    float acc = 0.f;
    for (int64_t i = 0; i < d; ++i) acc += xr[i] * xr[i];
    const float inv = 1.0f / sqrtf(acc / (float)d + eps);
    for (int64_t i = 0; i < d; ++i) {
      float v = xr[i] * inv;
      if (as_bf16) v = bf16_to_f32(f32_to_bf16(v));
      v = w[i] * v;
      out[r * d + i] = as_bf16 ? bf16_to_f32(f32_to_bf16(v)) : v;
    }
  }
}

/* ---- mlx_fast_rope_dynamic, non-traditional (src/mlx.zig:324; callers src/transformer.zig:9678, :9735) ----
 * x [n, heads, d] at sequence length 1: row n is rotated by the angle of position offsets[n]. */
QO_API void qo_rope(const float* x, int64_t n, int64_t heads, int64_t d, int dims, float base, float scale,
                    const int32_t* offsets, int as_bf16, float* out) {
  const int half = dims / 2;
  const float l2 = log2f(base);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n * heads; ++r) {
    const float pos = scale * (float)offsets[r / heads];
    const float* xr = x + r * d;
    float* o = out + r * d;
    for (int64_t i = 0; i < d; ++i) o[i] = xr[i];
    for (int i = 0; i < half; ++i) {
      const float theta = pos * exp2f(-((float)i / (float)half) * l2);
      const float c = cosf(theta), sn = sinf(theta);
      float a = xr[i] * c - xr[i + half] * sn, b = xr[i] * sn + xr[i + half] * c;
      if (as_bf16) { a = bf16_to_f32(f32_to_bf16(a)); b = bf16_to_f32(f32_to_bf16(b)); }
      o[i] = a;
      o[i + half] = b;
    }
  }
}

/* ---- the rotation of the TurboQuant cache schemes (src/kv_quant.zig:164-403) ----
 * R as TurboState builds it: the Sylvester Hadamard matrix H[N][N] (buildHadamardArray, :284-313) divided by sqrt(N) in
 * fp32 and cast to bf16, then rows and columns multiplied by the +-1 vector of cloneWithSignFlip (:318-360: a 64-bit
 * LCG, bit 33 of the state after every step picks the sign).  out = x @ R with fp32 accumulation in index order and one
 * rounding to bf16 (rotateLastDim is an mlx_matmul on bf16 operands; its summation order is MLX's and is not pinned).
 * signs (optional, N bytes): 1 where the vector is -1. */
QO_API void qo_turbo_rotate(const float* x, int64_t rows, int n, uint64_t seed, float* out, unsigned char* signs_out) {
  float* R = (float*)malloc((size_t)n * n * sizeof(float));
  float* sg = (float*)malloc((size_t)n * sizeof(float));
  R[0] = 1.0f;
  for (int size = 1; size < n; size *= 2)
    for (int r = 0; r < size; ++r)
      for (int c = 0; c < size; ++c) {
        const float tl = R[(size_t)r * n + c];
        R[(size_t)r * n + (c + size)] = tl;
        R[(size_t)(r + size) * n + c] = tl;
        R[(size_t)(r + size) * n + (c + size)] = -tl;
      }
  const float inv = 1.0f / sqrtf((float)n);
  uint64_t st = seed * 6364136223846793005ull;
  for (int e = 0; e < n; ++e) {
    st = st * 6364136223846793005ull + 1442695040888963407ull;
    sg[e] = ((st >> 33) & 1ull) == 0 ? 1.0f : -1.0f;
    if (signs_out) signs_out[e] = sg[e] < 0.0f;
  }
  for (int r = 0; r < n; ++r)
    for (int c = 0; c < n; ++c)
      R[(size_t)r * n + c] = bf16_to_f32(f32_to_bf16(R[(size_t)r * n + c] * inv)) * sg[r] * sg[c];
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < rows; ++i)
    for (int c = 0; c < n; ++c) {
      float acc = 0.0f;
      for (int j = 0; j < n; ++j) acc += x[i * n + j] * R[(size_t)j * n + c];
      out[i * n + c] = bf16_to_f32(f32_to_bf16(acc));
    }
  free(R);
  free(sg);
}

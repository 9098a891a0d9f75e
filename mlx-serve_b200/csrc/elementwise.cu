// dequantize / quantize kernels (bit-exact against the CPU oracle).
//
// dequantize mirrors mlx_dequantize as used by kv_quant.dequantizeAffine
// (mlx-serve src/kv_quant.zig:407-430): w = q*scale + bias with a rounded fp32
// product and a rounded fp32 add (no FMA contraction), then one cast.
// quantize mirrors mlx_quantize as used by kv_quant.quantizeAffine
// (src/kv_quant.zig:126-162); the scale/bias rule is the one restated in
// tests/dsv4_imatrix.py:169-183 and the codes follow :264.
#include "kernels.h"

namespace qb {

namespace {

template <typename T> struct DT;
template <> struct DT<float> { static constexpr int v = QB200_FLOAT32; };
template <> struct DT<__nv_bfloat16> { static constexpr int v = QB200_BFLOAT16; };
template <> struct DT<__half> { static constexpr int v = QB200_FLOAT16; };

template <int BITS, typename ST, typename OT>
__global__ void __launch_bounds__(256) dequant_kernel(DequantArgs a, int64_t words_per_row, int64_t total_words) {
  constexpr int VPW = 32 / BITS;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_words) return;
  const int64_t row = idx / words_per_row;
  const int64_t wi = idx - row * words_per_row;
  const uint32_t word = a.w[a.wmap.offset(row) + wi];
  const int64_t g = (wi * VPW) / a.gs;
  const int64_t sboff = a.sbmap.offset(row) + g;
  const float sc = IO<ST>::load(a.s, sboff);
  const float bi = IO<ST>::load(a.b, sboff);
  const int64_t obase = a.omap.offset(row) + wi * VPW;
  float v[VPW];
#pragma unroll
  for (int k = 0; k < VPW; ++k) {
    const float q = (float)((word >> (k * BITS)) & ((1u << BITS) - 1u));
    v[k] = __fadd_rn(__fmul_rn(q, sc), bi);
  }
  if constexpr (sizeof(OT) == 2 && VPW % 2 == 0) {
    // packed 16-bit stores when the destination is suitably aligned
    OT* op = (OT*)a.out + obase;
    if ((((uintptr_t)op) & (VPW * 2 - 1)) == 0) {
      uint32_t pk[VPW / 2];
#pragma unroll
      for (int k = 0; k < VPW / 2; ++k) {
        OT lo, hi;
        if constexpr (DT<OT>::v == QB200_BFLOAT16) { lo = __float2bfloat16_rn(v[2 * k]); hi = __float2bfloat16_rn(v[2 * k + 1]); }
        else { lo = __float2half_rn(v[2 * k]); hi = __float2half_rn(v[2 * k + 1]); }
        pk[k] = (uint32_t)(*(uint16_t*)&lo) | ((uint32_t)(*(uint16_t*)&hi) << 16);
      }
      if constexpr (VPW == 8) *(uint4*)op = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      else if constexpr (VPW == 4) *(uint2*)op = make_uint2(pk[0], pk[1]);
      else {
#pragma unroll
        for (int k = 0; k < VPW / 2; ++k) ((uint32_t*)op)[k] = pk[k];
      }
      return;
    }
  }
#pragma unroll
  for (int k = 0; k < VPW; ++k) IO<OT>::store(a.out, obase + k, v[k]);
}

template <int BITS, typename ST>
cudaError_t dequant_dispatch_out(const DequantArgs& a, cudaStream_t st) {
  const int64_t wpr = a.d * BITS / 32;
  const int64_t total = a.rows * wpr;
  if (total == 0) return cudaSuccess;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  switch (a.out_dtype) {
    case QB200_BFLOAT16: dequant_kernel<BITS, ST, __nv_bfloat16><<<blocks, 256, 0, st>>>(a, wpr, total); break;
    case QB200_FLOAT32: dequant_kernel<BITS, ST, float><<<blocks, 256, 0, st>>>(a, wpr, total); break;
    case QB200_FLOAT16: dequant_kernel<BITS, ST, __half><<<blocks, 256, 0, st>>>(a, wpr, total); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

template <int BITS>
cudaError_t dequant_dispatch_sb(const DequantArgs& a, cudaStream_t st) {
  switch (a.sb_dtype) {
    case QB200_BFLOAT16: return dequant_dispatch_out<BITS, __nv_bfloat16>(a, st);
    case QB200_FLOAT32: return dequant_dispatch_out<BITS, float>(a, st);
    case QB200_FLOAT16: return dequant_dispatch_out<BITS, __half>(a, st);
    default: return cudaErrorInvalidValue;
  }
}

// One thread per packed output word; the gs/VPW threads of a group are
// consecutive lanes of one warp and share min/max through shuffles.
template <int BITS, typename XT, typename ST>
__global__ void __launch_bounds__(256) quant_kernel(QuantArgs a, int64_t words_per_row, int64_t total_words) {
  constexpr int VPW = 32 / BITS;
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = idx < total_words;
  if (!live) idx = total_words - 1;  // keep the warp converged for the shuffles
  const int64_t row = idx / words_per_row;
  const int64_t wi = idx - row * words_per_row;
  const int64_t xbase = a.xmap.offset(row) + wi * VPW;
  float v[VPW];
#pragma unroll
  for (int k = 0; k < VPW; ++k) v[k] = IO<XT>::load(a.x, xbase + k);
  float xmin = v[0], xmax = v[0];
#pragma unroll
  for (int k = 1; k < VPW; ++k) { xmin = fminf(xmin, v[k]); xmax = fmaxf(xmax, v[k]); }
  const int tpg = a.gs / VPW;  // threads per group: power of two, <= 32
  for (int off = tpg >> 1; off > 0; off >>= 1) {
    xmin = fminf(xmin, __shfl_xor_sync(0xffffffffu, xmin, off));
    xmax = fmaxf(xmax, __shfl_xor_sync(0xffffffffu, xmax, off));
  }
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
  a.q[a.qmap.offset(row) + wi] = word;
  if ((wi % tpg) == 0) {
    const int64_t sboff = a.sbmap.offset(row) + (wi * VPW) / a.gs;
    IO<ST>::store(a.s, sboff, scale);
    IO<ST>::store(a.b, sboff, bias);
  }
}

template <int BITS, typename XT>
cudaError_t quant_dispatch_sb(const QuantArgs& a, cudaStream_t st) {
  const int64_t wpr = a.d * BITS / 32;
  const int64_t total = a.rows * wpr;
  if (total == 0) return cudaSuccess;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  switch (a.sb_dtype) {
    case QB200_BFLOAT16: quant_kernel<BITS, XT, __nv_bfloat16><<<blocks, 256, 0, st>>>(a, wpr, total); break;
    case QB200_FLOAT32: quant_kernel<BITS, XT, float><<<blocks, 256, 0, st>>>(a, wpr, total); break;
    case QB200_FLOAT16: quant_kernel<BITS, XT, __half><<<blocks, 256, 0, st>>>(a, wpr, total); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

template <int BITS>
cudaError_t quant_dispatch_x(const QuantArgs& a, cudaStream_t st) {
  switch (a.x_dtype) {
    case QB200_BFLOAT16: return quant_dispatch_sb<BITS, __nv_bfloat16>(a, st);
    case QB200_FLOAT32: return quant_dispatch_sb<BITS, float>(a, st);
    case QB200_FLOAT16: return quant_dispatch_sb<BITS, __half>(a, st);
    default: return cudaErrorInvalidValue;
  }
}

// One thread per 8 consecutive h of one token: the k rows are read 16 bytes at a time.  bf16: every product is
// rounded to bf16 (the reference multiplies in the activation dtype, src/transformer.zig:15127-15140) and the sum
// over k is an ascending accumulate in bf16, rounded after every add, which is how MLX reduces a bf16 row and what
// the reference's fused down+reduce kernel replicates (src/transformer.zig:20566-20571).
__device__ __forceinline__ float rbf(float x) { return __uint_as_float((uint32_t)f32_to_bf16_bits(x) << 16); }
template <bool F32>
__global__ void __launch_bounds__(256) moe_sum_kernel(MoeSumArgs a) {
  const int64_t per_tok = a.H / 8;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.T * per_tok) return;
  const int64_t t = i / per_tok, h0 = (i - t * per_tok) * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  // top-k entries in batches of 8: first every index and score, then every row (independent loads in flight
  // together), then the products in ascending j
  for (int64_t j0 = 0; j0 < a.topk; j0 += 8) {
    int64_t row[8];
    float sc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int64_t e = t * a.topk + j0 + q;
      row[q] = -1;
      sc[q] = 0.f;
      if (j0 + q < a.topk) {
        row[q] = a.inv ? (a.inv_i64 ? ((const long long*)a.inv)[e] : (long long)((const int*)a.inv)[e]) : e;
        sc[q] = F32 ? ((const float*)a.scores)[e] : __uint_as_float((uint32_t)((const uint16_t*)a.scores)[e] << 16);
        if (row[q] >= a.R) row[q] = -1;   // out-of-range (and negative) entries contribute nothing
      }
    }
    uint4 v0[8], v1[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      v0[q] = v1[q] = make_uint4(0u, 0u, 0u, 0u);
      if (row[q] >= 0) {
        if (F32) {
          v0[q] = *(const uint4*)((const float*)a.y + row[q] * a.H + h0);
          v1[q] = *(const uint4*)((const float*)a.y + row[q] * a.H + h0 + 4);
        } else {
          v0[q] = *(const uint4*)((const uint16_t*)a.y + row[q] * a.H + h0);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (row[q] < 0) continue;
      if (F32) {
        const uint32_t w[8] = {v0[q].x, v0[q].y, v0[q].z, v0[q].w, v1[q].x, v1[q].y, v1[q].z, v1[q].w};
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] += __uint_as_float(w[c]) * sc[q];
      } else {
        const uint32_t w[4] = {v0[q].x, v0[q].y, v0[q].z, v0[q].w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {   // product rounded to bf16, then a bf16 accumulate (rounded after every add)
          acc[2 * c] = rbf(acc[2 * c] + rbf(bf16lo(w[c]) * sc[q]));
          acc[2 * c + 1] = rbf(acc[2 * c + 1] + rbf(bf16hi(w[c]) * sc[q]));
        }
      }
    }
  }
  if (F32) {
    float* o = (float*)a.out + t * a.H + h0;
    *(float4*)o = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *(float4*)(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  } else {
    uint4 o;
    o.x = (uint32_t)f32_to_bf16_bits(acc[0]) | ((uint32_t)f32_to_bf16_bits(acc[1]) << 16);
    o.y = (uint32_t)f32_to_bf16_bits(acc[2]) | ((uint32_t)f32_to_bf16_bits(acc[3]) << 16);
    o.z = (uint32_t)f32_to_bf16_bits(acc[4]) | ((uint32_t)f32_to_bf16_bits(acc[5]) << 16);
    o.w = (uint32_t)f32_to_bf16_bits(acc[6]) | ((uint32_t)f32_to_bf16_bits(acc[7]) << 16);
    *(uint4*)((uint16_t*)a.out + t * a.H + h0) = o;
  }
}

// One warp per row of logits (E <= 1024: up to 32 values per lane, column e in lane e % 32).  The k indices are
// those of the largest logits, larger first, equal logits by lower index (the reference takes them from
// mlx_argpartition, which leaves their order open; everything downstream is indexed alike, src/transformer.zig:17022-17063).
// softmax in fp32 (precise), rounded to the logits' dtype as the reference's array is, then the k entries divided
// by their sum (accumulated in that dtype, larger-first order), each step rounded to that dtype -- the order and the
// accumulation are those of the reference's one-kernel router (src/transformer.zig:17485-17500, :17530-17534).
template <bool F32>
__global__ void __launch_bounds__(128) moe_route_kernel(MoeRouteArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= a.T) return;
  constexpr int kPer = 32;
  float v[kPer];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int e = i * 32 + lane;
    v[i] = -INFINITY;
    if (e < a.E) {
      v[i] = F32 ? ((const float*)a.logits)[row * a.E + e]
                 : __uint_as_float((uint32_t)((const uint16_t*)a.logits)[row * a.E + e] << 16);
      mx = fmaxf(mx, v[i]);
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kPer; ++i)
    if (i * 32 + lane < a.E) sum += expf(v[i] - mx);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  auto round_dt = [](float x) { return F32 ? x : __uint_as_float((uint32_t)f32_to_bf16_bits(x) << 16); };
  float topw = 0.f, wsum = 0.f;   // lane j keeps the j-th selected probability
  int topi = -1;
  uint32_t taken = 0;             // bit i: this lane's value i was selected
  for (int j = 0; j < a.topk; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const int e = i * 32 + lane;
      if (e < a.E && !((taken >> i) & 1u) && (v[i] > bv || (v[i] == bv && e < bi))) { bv = v[i]; bi = e; }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi != 0x7fffffff && (bi & 31) == lane) taken |= 1u << (bi >> 5);
    const float pr = bi != 0x7fffffff ? round_dt(expf(bv - mx) / sum) : 0.f;
    wsum = round_dt(wsum + pr);   // ascending accumulate in the logits' dtype, rounded after every add
                                  // (src/transformer.zig:17530-17534); every lane adds the same values
    if (lane == j) { topw = pr; topi = bi != 0x7fffffff ? bi : 0; }
  }
  if (lane < a.topk) {
    a.inds[row * a.topk + lane] = topi;
    const float ns = round_dt(topw / wsum);
    if (F32) ((float*)a.scores)[row * a.topk + lane] = ns;
    else ((uint16_t*)a.scores)[row * a.topk + lane] = f32_to_bf16_bits(ns);
  }
}

}  // namespace

cudaError_t launch_moe_route(const MoeRouteArgs& a, cudaStream_t st) {
  if (a.T <= 0) return cudaSuccess;
  const unsigned blocks = (unsigned)((a.T + 3) / 4);
  if (a.dtype == QB200_FLOAT32) moe_route_kernel<true><<<blocks, 128, 0, st>>>(a);
  else moe_route_kernel<false><<<blocks, 128, 0, st>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_moe_weighted_sum(const MoeSumArgs& a, cudaStream_t st) {
  const int64_t n = a.T * (a.H / 8);
  if (n <= 0) return cudaSuccess;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (a.dtype == QB200_FLOAT32) moe_sum_kernel<true><<<blocks, 256, 0, st>>>(a);
  else moe_sum_kernel<false><<<blocks, 256, 0, st>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_dequantize(const DequantArgs& a, cudaStream_t st) {
  switch (a.bits) {
    case 2: return dequant_dispatch_sb<2>(a, st);
    case 4: return dequant_dispatch_sb<4>(a, st);
    case 8: return dequant_dispatch_sb<8>(a, st);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_quantize(const QuantArgs& a, cudaStream_t st) {
  switch (a.bits) {
    case 2: return quant_dispatch_x<2>(a, st);
    case 4: return quant_dispatch_x<4>(a, st);
    case 8: return quant_dispatch_x<8>(a, st);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace qb

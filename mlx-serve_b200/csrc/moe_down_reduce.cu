// Down projection of the routed-expert block fused with the router weighting and the sum over top-k, for a
// few tokens: out[t, n] = sum_j round(round(act[t, j, :] . Wdown[inds[t, j]][n, :]) * scores[t, j]).
//
// Replaces gatherQmvDownReduce (mlx-serve src/transformer.zig:20559-20623, :20675-20761), the single-token tail of
// moeDecodeGatherQmv (src/transformer.zig:14692-14817), and keeps its rounding points: every (slot, row) dot
// product is rounded to the activation dtype exactly as the unfused gather_qmm would store it, the product with
// the slot's score is rounded again, and the slots are added in ascending order in that dtype.
//
// One CTA per (token, 16 output rows); warp j of the CTA owns top-k slot j: it converts that slot's activation
// row to 15-bit fixed point (two s8 planes) for itself, streams the 16 rows x K codes of its expert through a
// private cp.async ring and multiplies on the integer tensor cores (the arithmetic of the streaming kernels).
// The k values per row meet in shared memory behind one barrier.
#include <type_traits>

#include <mutex>

#include "kernels.h"
#include "stream_ptx.cuh"

namespace qb {
namespace {

constexpr int kStages = 4;
constexpr int kStageW = 2048;                 // 16 rows x 128 B of packed codes
constexpr int kStageBytes = kStageW + 256;    // + per row: scales | biases
constexpr int kMaxSlots = 16;

struct DRK {
  const void* act; const uint32_t* w; const uint16_t* s; const uint16_t* b; void* y;
  const void* inds; const void* scores;
  int inds_i64;
  int64_t E, wes, ses;     // experts, elements per expert of w and of scales/biases
  int N, K, topk, gshift, f32;
};

__device__ __forceinline__ float rdt(float x, bool f32) { return f32 ? x : __uint_as_float((uint32_t)f32_to_bf16_bits(x) << 16); }

template <int BITS>
__global__ void __launch_bounds__(kMaxSlots * 32) moe_down_reduce_kernel(DRK p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int U = BITS == 4 ? 4 : 2;   // 64-wide groups per unit
  constexpr int CK = 64 * U;             // K values per unit (128 bytes per row)
  __shared__ float s_val[kMaxSlots][16];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int tile = blockIdx.x;
  const int64_t tok = blockIdx.y;
  const int ut = p.K / CK;
  // per warp: ring | fragments of its activation row (16 bytes per 64-group, column and lane quarter) | group scales
  const size_t per_warp = (size_t)kStages * kStageBytes + (size_t)(p.K / 64) * 128 + (size_t)(p.K / 64) * 8;
  unsigned char* mine = smem + (size_t)warp * per_warp;
  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(mine);
  uint2* xfrag = (uint2*)(mine + (size_t)kStages * kStageBytes);
  float* gsc = (float*)(mine + (size_t)kStages * kStageBytes + (size_t)(p.K / 64) * 128);

  const int64_t slot = tok * p.topk + warp;
  const long long e = p.inds_i64 ? ((const long long*)p.inds)[slot] : (long long)((const int*)p.inds)[slot];
  const bool live = e >= 0 && e < p.E;   // an out-of-range expert contributes nothing

  // ---- the weight stream of this warp: units 0 .. ut-1 of the tile's 16 rows of expert e ----
  const int chunk = lane & 7;
  const int64_t ldw = (int64_t)p.K * BITS / 32, lds = p.K >> (6 + p.gshift);
  const unsigned char* wsrc[4];
  uint32_t wdst[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = (lane >> 3) + 4 * r;
    int n = tile * 16 + row;
    n = n < p.N ? n : p.N - 1;
    wsrc[r] = (const unsigned char*)(p.w + (live ? e : 0) * p.wes + (int64_t)n * ldw) + chunk * 16;
    wdst[r] = my_ring + row * 128 + ((chunk ^ swz_w<BITS>(row)) << 4);
  }
  int ns = tile * 16 + (lane & 15);
  ns = ns < p.N ? ns : p.N - 1;
  const uint16_t* sbsrc = ((lane >> 4) ? p.b : p.s) + (live ? e : 0) * p.ses + (int64_t)ns * lds;
  const uint32_t sbdst = my_ring + kStageW + (lane & 15) * 16 + (lane >> 4) * 8;
  int issued = 0;
  auto issue = [&]() {
    const uint32_t off = (uint32_t)(issued % kStages) * kStageBytes;
#pragma unroll
    for (int r = 0; r < 4; ++r) cp_async16(wdst[r] + off, wsrc[r] + (int64_t)issued * 128);
    const uint16_t* ssrc = sbsrc + ((issued * U) >> p.gshift);
    if (BITS == 4 && p.gshift == 0) cp_async8(sbdst + off, ssrc);
    else cp_async4(sbdst + off, ssrc);
  };
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) {
    if (live && issued < ut) issue();
    cp_async_commit();
    ++issued;
  }

  // ---- this slot's activation row as two s8 planes in B-fragment order (one lane: 8 K values per step) ----
  // v = rn(x * 2^(14-E)) per 64-wide group is one FMA onto 1.5 * 2^23 (the low 16 bits of the sum's bit pattern are v
  // in two's complement); the planes are cut out of pairs of values packed into one word.
  for (int c = lane; c < (p.K >> 3); c += 32) {
    float f[8];
    if (!p.f32) {
      const uint4 a = *(const uint4*)((const uint16_t*)p.act + slot * p.K + (int64_t)c * 8);
      f[0] = bf16lo(a.x); f[1] = bf16hi(a.x); f[2] = bf16lo(a.y); f[3] = bf16hi(a.y);
      f[4] = bf16lo(a.z); f[5] = bf16hi(a.z); f[6] = bf16lo(a.w); f[7] = bf16hi(a.w);
    } else {
      const float4 a = *(const float4*)((const float*)p.act + slot * p.K + (int64_t)c * 8);
      const float4 b2 = *(const float4*)((const float*)p.act + slot * p.K + (int64_t)c * 8 + 4);
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b2.x; f[5] = b2.y; f[6] = b2.z; f[7] = b2.w;
    }
    float mx = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmax_nan(mx, fabsf(f[j]));
    mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
    int ex = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 + 1;  // mx < 2^ex
    ex = ex < -100 ? -100 : (ex > 110 ? 110 : ex);
    const float up = __uint_as_float((uint32_t)(127 + 14 - ex) << 23);
    const float down = poison_if(nonfinite(mx), __uint_as_float((uint32_t)(127 + ex - 14) << 23));
    uint32_t w[8], isum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      w[j] = __float_as_uint(fminf(fmaf(f[j], up, 12582912.f), 12599295.f));   // v <= 16383
      isum += w[j];
    }
    isum += __shfl_xor_sync(0xffffffffu, isum, 1);
    isum += __shfl_xor_sync(0xffffffffu, isum, 2);
    isum += __shfl_xor_sync(0xffffffffu, isum, 4);
    const int sum = (int)(isum - 0xD0000000u);   // 64 values: 64 * 0x4B400000 mod 2^32
    const int gi = c >> 3, tt = (c >> 1) & 3, jm = c & 1;
    if ((c & 7) == 0) *(float2*)&gsc[gi * 2] = make_float2(down, down * (float)sum);
    uint32_t o[2][2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t p0 = __byte_perm(w[kslot8<BITS>(h, 0)], w[kslot8<BITS>(h, 1)], 0x5410);
      const uint32_t p1 = __byte_perm(w[kslot8<BITS>(h, 2)], w[kslot8<BITS>(h, 3)], 0x5410);
      o[0][h] = __byte_perm((p0 >> 7) & 0x00FF00FFu, (p1 >> 7) & 0x00FF00FFu, 0x6420);
      o[1][h] = __byte_perm(p0 & 0x007F007Fu, p1 & 0x007F007Fu, 0x6420);
    }
    uint2* d = xfrag + (gi * 8 + tt) * 2 + jm;
    d[0] = make_uint2(o[0][0], o[0][1]);
    d[8] = make_uint2(o[1][0], o[1][1]);
  }
  __syncwarp();

  // ---- stream the units: lanes with t == 0 end up with the dot products of rows g and g+8 ----
  int frag_off[U];
#pragma unroll
  for (int j = 0; j < U; ++j) {
    if (BITS == 4) frag_off[j] = g * 128 + (((2 * j + (t >> 1)) ^ swz_w<4>(g)) << 4) + (t & 1) * 8;
    else frag_off[j] = g * 128 + (((4 * j + t) ^ swz_w<8>(g)) << 4);
  }
  float tot0 = 0.f, tot1 = 0.f;
  for (int u = 0; u < ut; ++u) {
    if (live && issued < ut) issue();
    cp_async_commit();
    ++issued;
    cp_async_wait<kStages - 1>();
    __syncwarp();
    const unsigned char* st = mine + (size_t)(u % kStages) * kStageBytes;
    uint32_t sl[2], sh[2], bl[2], bh[2];
    {
      const uint4 lo = *(const uint4*)(st + kStageW + g * 16), hi = *(const uint4*)(st + kStageW + (g + 8) * 16);
      if (BITS == 4 && p.gshift == 0) {
        sl[0] = lo.x; sl[1] = lo.y; sh[0] = hi.x; sh[1] = hi.y;
        bl[0] = lo.z; bl[1] = lo.w; bh[0] = hi.z; bh[1] = hi.w;
      } else if (BITS == 4) {  // group size 128: each value serves two 64-wide groups
        sl[0] = __byte_perm(lo.x, lo.x, 0x1010); sl[1] = __byte_perm(lo.x, lo.x, 0x3232);
        sh[0] = __byte_perm(hi.x, hi.x, 0x1010); sh[1] = __byte_perm(hi.x, hi.x, 0x3232);
        bl[0] = __byte_perm(lo.z, lo.z, 0x1010); bl[1] = __byte_perm(lo.z, lo.z, 0x3232);
        bh[0] = __byte_perm(hi.z, hi.z, 0x1010); bh[1] = __byte_perm(hi.z, hi.z, 0x3232);
      } else {
        sl[0] = lo.x; sh[0] = hi.x; bl[0] = lo.z; bh[0] = hi.z;
        sl[1] = sh[1] = bl[1] = bh[1] = 0;
      }
    }
    const uint4* xb = (const uint4*)xfrag + (size_t)(u * U) * 8 + (g & 1) * 4 + t;
    const float* gb = gsc + (size_t)(u * U) * 2;
#pragma unroll
    for (int j = 0; j < U; ++j) {
      uint32_t a0[2], a1[2], a2[2], a3[2];
      if constexpr (BITS == 4) {
        const uint2 wl = *(const uint2*)(st + frag_off[j]);
        const uint2 wh = *(const uint2*)(st + frag_off[j] + 1024);
        a0[0] = wl.x & 0x0F0F0F0Fu; a2[0] = (wl.x >> 4) & 0x0F0F0F0Fu;
        a0[1] = wl.y & 0x0F0F0F0Fu; a2[1] = (wl.y >> 4) & 0x0F0F0F0Fu;
        a1[0] = wh.x & 0x0F0F0F0Fu; a3[0] = (wh.x >> 4) & 0x0F0F0F0Fu;
        a1[1] = wh.y & 0x0F0F0F0Fu; a3[1] = (wh.y >> 4) & 0x0F0F0F0Fu;
      } else {
        const uint4 wl = *(const uint4*)(st + frag_off[j]);
        const uint4 wh = *(const uint4*)(st + frag_off[j] + 1024);
        a0[0] = wl.x; a2[0] = wl.y; a0[1] = wl.z; a2[1] = wl.w;
        a1[0] = wh.x; a3[0] = wh.y; a1[1] = wh.z; a3[1] = wh.w;
      }
      const float s_lo = (j & 1) ? bf16hi(sl[j >> 1]) : bf16lo(sl[j >> 1]);
      const float s_hi = (j & 1) ? bf16hi(sh[j >> 1]) : bf16lo(sh[j >> 1]);
      const float b_lo = (j & 1) ? bf16hi(bl[j >> 1]) : bf16lo(bl[j >> 1]);
      const float b_hi = (j & 1) ? bf16hi(bh[j >> 1]) : bf16lo(bh[j >> 1]);
      int acc[4];
      const uint4 bf = xb[j * 8];
      mma_u8s8_z(acc, a0[0], a1[0], a2[0], a3[0], bf.x, bf.y);
      mma_u8s8(acc, a0[1], a1[1], a2[1], a3[1], bf.z, bf.w);
      const float2 gs = *(const float2*)&gb[j * 2];
      const float f_lo = (float)(acc[0] * 128 + acc[1]), f_hi = (float)(acc[2] * 128 + acc[3]);
      tot0 = fmaf(s_lo * gs.x, f_lo, fmaf(b_lo, gs.y, tot0));
      tot1 = fmaf(s_hi * gs.x, f_hi, fmaf(b_hi, gs.y, tot1));
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  // the slot's value of each row, rounded to the activation dtype as the unfused projection would store it
  if (t == 0) {
    s_val[warp][g] = live ? rdt(tot0, p.f32) : 0.f;
    s_val[warp][g + 8] = live ? rdt(tot1, p.f32) : 0.f;
  }
  __syncthreads();
  // rounded product with the slot's score, ascending accumulate in the activation dtype
  if (warp == 0 && lane < 16) {
    const int n = tile * 16 + lane;
    float total = 0.f;
    for (int j = 0; j < p.topk; ++j) {
      const int64_t sj = tok * p.topk + j;
      const float sc = p.f32 ? ((const float*)p.scores)[sj] : bf16_bits_to_f32(((const uint16_t*)p.scores)[sj]);
      total = rdt(total + rdt(s_val[j][lane] * sc, p.f32), p.f32);
    }
    if (n < p.N) {
      if (p.f32) ((float*)p.y)[tok * p.N + n] = total;
      else ((uint16_t*)p.y)[tok * p.N + n] = f32_to_bf16_bits(total);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// gather_qmm for a few rows, each with its own expert (the single-token decode shapes of gatherQmv and
// gatherQmvGateUp, mlx-serve src/transformer.zig:20046-20109, :20303-20396): res[i] = x[lhs(i)] . W[rhs[i]]^T, or
// silu(x . Wgate^T) * (x . Wup^T) in the fused form.  One CTA per (row, 16 output rows); four warps split K in
// units of 128 bytes per weight row (eight warps in the fused form: four per bank), so every unit of a tile is in
// flight at once; the partial sums meet in shared memory in a fixed order (the same order in both forms, so the
// fused result equals the unfused chain bit for bit).
constexpr int kParts = 4;        // warps per bank splitting K

struct GSK {
  const void* x; const uint32_t* w; const uint16_t* s; const uint16_t* b; void* y;
  const uint32_t* w2; const uint16_t* s2; const uint16_t* b2; const uint16_t* sigtab;
  const void* rhs; const void* lhs;
  int rhs_i64, lhs_i64;
  BatchMap xbcast;
  int64_t E, XB, xstride, wes, ses;
  int N, K, gshift, f32;
};

// S: ring depth per warp (2 when a warp has at most two units, so that more CTAs fit an SM; else 4)
template <int BITS, bool FUSED, int S>
__global__ void __launch_bounds__((FUSED ? 2 : 1) * kParts * 32) gather_small_kernel(GSK p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int U = BITS == 4 ? 4 : 2;
  constexpr int CK = 64 * U;
  constexpr int NB = FUSED ? 2 : 1;
  constexpr int kThreads = NB * kParts * 32;
  __shared__ float s_part[NB][kParts][16];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int bank = warp / kParts, part = warp % kParts;
  const int tile = blockIdx.x;
  const int64_t i = blockIdx.y;
  const int ut = p.K / CK;
  const long long e = p.rhs_i64 ? ((const long long*)p.rhs)[i] : (long long)((const uint32_t*)p.rhs)[i];
  long long xi = p.lhs ? (p.lhs_i64 ? ((const long long*)p.lhs)[i] : (long long)((const uint32_t*)p.lhs)[i])
                       : (long long)p.xbcast.offset(i);
  if (e < 0 || e >= p.E || xi < 0 || xi >= p.XB) return;   // the row is left untouched, as in every other form

  // shared memory: the row's fragments and group scales (all warps), then one ring per warp
  uint2* xfrag = (uint2*)smem;
  float* gsc = (float*)(smem + (size_t)(p.K / 64) * 128);
  unsigned char* mine = smem + (size_t)(p.K / 64) * 136 + (size_t)warp * S * kStageBytes;
  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(mine);

  // ---- this warp's units: part, part + 4, ... of the tile's 16 rows of its bank ----
  const uint32_t* wb = (FUSED && bank) ? p.w2 : p.w;
  const uint16_t* sbk = (FUSED && bank) ? p.s2 : p.s;
  const uint16_t* bbk = (FUSED && bank) ? p.b2 : p.b;
  const int chunk = lane & 7;
  const int64_t ldw = (int64_t)p.K * BITS / 32, lds = p.K >> (6 + p.gshift);
  const unsigned char* wsrc[4];
  uint32_t wdst[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = (lane >> 3) + 4 * r;
    int n = tile * 16 + row;
    n = n < p.N ? n : p.N - 1;
    wsrc[r] = (const unsigned char*)(wb + e * p.wes + (int64_t)n * ldw) + chunk * 16;
    wdst[r] = my_ring + row * 128 + ((chunk ^ swz_w<BITS>(row)) << 4);
  }
  int ns = tile * 16 + (lane & 15);
  ns = ns < p.N ? ns : p.N - 1;
  const uint16_t* sbsrc = ((lane >> 4) ? bbk : sbk) + e * p.ses + (int64_t)ns * lds;
  const uint32_t sbdst = my_ring + kStageW + (lane & 15) * 16 + (lane >> 4) * 8;
  const int nu = ut > part ? (ut - part + kParts - 1) / kParts : 0;   // units of this warp
  int issued = 0;
  auto issue = [&]() {
    const int u = part + issued * kParts;
    const uint32_t off = (uint32_t)(issued % S) * kStageBytes;
#pragma unroll
    for (int r = 0; r < 4; ++r) cp_async16(wdst[r] + off, wsrc[r] + (int64_t)u * 128);
    const uint16_t* ssrc = sbsrc + ((u * U) >> p.gshift);
    if (BITS == 4 && p.gshift == 0) cp_async8(sbdst + off, ssrc);
    else cp_async4(sbdst + off, ssrc);
  };
#pragma unroll
  for (int k = 0; k < S; ++k) {   // the whole ring up front: the weights do not depend on the activations
    if (issued < nu) issue();
    cp_async_commit();
    ++issued;
  }

  // ---- the row's activations as two s8 planes in B-fragment order, by all threads ----
  for (int c = tid; c < (p.K >> 3); c += kThreads) {
    float f[8];
    if (!p.f32) {
      const uint4 a = *(const uint4*)((const uint16_t*)p.x + xi * p.xstride + (int64_t)c * 8);
      f[0] = bf16lo(a.x); f[1] = bf16hi(a.x); f[2] = bf16lo(a.y); f[3] = bf16hi(a.y);
      f[4] = bf16lo(a.z); f[5] = bf16hi(a.z); f[6] = bf16lo(a.w); f[7] = bf16hi(a.w);
    } else {
      const float4 a = *(const float4*)((const float*)p.x + xi * p.xstride + (int64_t)c * 8);
      const float4 b2 = *(const float4*)((const float*)p.x + xi * p.xstride + (int64_t)c * 8 + 4);
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b2.x; f[5] = b2.y; f[6] = b2.z; f[7] = b2.w;
    }
    float mx = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmax_nan(mx, fabsf(f[j]));
    mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
    int ex = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 + 1;  // mx < 2^ex
    ex = ex < -100 ? -100 : (ex > 110 ? 110 : ex);
    const float up = __uint_as_float((uint32_t)(127 + 14 - ex) << 23);
    const float down = poison_if(nonfinite(mx), __uint_as_float((uint32_t)(127 + ex - 14) << 23));
    uint32_t w[8], isum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      w[j] = __float_as_uint(fminf(fmaf(f[j], up, 12582912.f), 12599295.f));   // v <= 16383
      isum += w[j];
    }
    isum += __shfl_xor_sync(0xffffffffu, isum, 1);
    isum += __shfl_xor_sync(0xffffffffu, isum, 2);
    isum += __shfl_xor_sync(0xffffffffu, isum, 4);
    const int sum = (int)(isum - 0xD0000000u);   // 64 values: 64 * 0x4B400000 mod 2^32
    const int gi = c >> 3, tt = (c >> 1) & 3, jm = c & 1;
    if ((c & 7) == 0) *(float2*)&gsc[gi * 2] = make_float2(down, down * (float)sum);
    uint32_t o[2][2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t p0 = __byte_perm(w[kslot8<BITS>(h, 0)], w[kslot8<BITS>(h, 1)], 0x5410);
      const uint32_t p1 = __byte_perm(w[kslot8<BITS>(h, 2)], w[kslot8<BITS>(h, 3)], 0x5410);
      o[0][h] = __byte_perm((p0 >> 7) & 0x00FF00FFu, (p1 >> 7) & 0x00FF00FFu, 0x6420);
      o[1][h] = __byte_perm(p0 & 0x007F007Fu, p1 & 0x007F007Fu, 0x6420);
    }
    uint2* d = xfrag + (gi * 8 + tt) * 2 + jm;
    d[0] = make_uint2(o[0][0], o[0][1]);
    d[8] = make_uint2(o[1][0], o[1][1]);
  }
  __syncthreads();

  // ---- this warp's units: lanes with t == 0 end up with the partial dot products of rows g and g+8 ----
  int frag_off[U];
#pragma unroll
  for (int j = 0; j < U; ++j) {
    if (BITS == 4) frag_off[j] = g * 128 + (((2 * j + (t >> 1)) ^ swz_w<4>(g)) << 4) + (t & 1) * 8;
    else frag_off[j] = g * 128 + (((4 * j + t) ^ swz_w<8>(g)) << 4);
  }
  float tot0 = 0.f, tot1 = 0.f;
  for (int k = 0; k < nu; ++k) {
    const int u = part + k * kParts;
    cp_async_wait<S - 1>();
    __syncwarp();
    const unsigned char* st = mine + (size_t)(k % S) * kStageBytes;
    uint32_t sl[2], sh[2], bl[2], bh[2];
    {
      const uint4 lo = *(const uint4*)(st + kStageW + g * 16), hi = *(const uint4*)(st + kStageW + (g + 8) * 16);
      if (BITS == 4 && p.gshift == 0) {
        sl[0] = lo.x; sl[1] = lo.y; sh[0] = hi.x; sh[1] = hi.y;
        bl[0] = lo.z; bl[1] = lo.w; bh[0] = hi.z; bh[1] = hi.w;
      } else if (BITS == 4) {  // group size 128: each value serves two 64-wide groups
        sl[0] = __byte_perm(lo.x, lo.x, 0x1010); sl[1] = __byte_perm(lo.x, lo.x, 0x3232);
        sh[0] = __byte_perm(hi.x, hi.x, 0x1010); sh[1] = __byte_perm(hi.x, hi.x, 0x3232);
        bl[0] = __byte_perm(lo.z, lo.z, 0x1010); bl[1] = __byte_perm(lo.z, lo.z, 0x3232);
        bh[0] = __byte_perm(hi.z, hi.z, 0x1010); bh[1] = __byte_perm(hi.z, hi.z, 0x3232);
      } else {
        sl[0] = lo.x; sh[0] = hi.x; bl[0] = lo.z; bh[0] = hi.z;
        sl[1] = sh[1] = bl[1] = bh[1] = 0;
      }
    }
    const uint4* xb = (const uint4*)xfrag + (size_t)(u * U) * 8 + (g & 1) * 4 + t;
    const float* gb = gsc + (size_t)(u * U) * 2;
#pragma unroll
    for (int j = 0; j < U; ++j) {
      uint32_t a0[2], a1[2], a2[2], a3[2];
      if constexpr (BITS == 4) {
        const uint2 wl = *(const uint2*)(st + frag_off[j]);
        const uint2 wh = *(const uint2*)(st + frag_off[j] + 1024);
        a0[0] = wl.x & 0x0F0F0F0Fu; a2[0] = (wl.x >> 4) & 0x0F0F0F0Fu;
        a0[1] = wl.y & 0x0F0F0F0Fu; a2[1] = (wl.y >> 4) & 0x0F0F0F0Fu;
        a1[0] = wh.x & 0x0F0F0F0Fu; a3[0] = (wh.x >> 4) & 0x0F0F0F0Fu;
        a1[1] = wh.y & 0x0F0F0F0Fu; a3[1] = (wh.y >> 4) & 0x0F0F0F0Fu;
      } else {
        const uint4 wl = *(const uint4*)(st + frag_off[j]);
        const uint4 wh = *(const uint4*)(st + frag_off[j] + 1024);
        a0[0] = wl.x; a2[0] = wl.y; a0[1] = wl.z; a2[1] = wl.w;
        a1[0] = wh.x; a3[0] = wh.y; a1[1] = wh.z; a3[1] = wh.w;
      }
      const float s_lo = (j & 1) ? bf16hi(sl[j >> 1]) : bf16lo(sl[j >> 1]);
      const float s_hi = (j & 1) ? bf16hi(sh[j >> 1]) : bf16lo(sh[j >> 1]);
      const float b_lo = (j & 1) ? bf16hi(bl[j >> 1]) : bf16lo(bl[j >> 1]);
      const float b_hi = (j & 1) ? bf16hi(bh[j >> 1]) : bf16lo(bh[j >> 1]);
      int acc[4];
      const uint4 bf = xb[j * 8];
      mma_u8s8_z(acc, a0[0], a1[0], a2[0], a3[0], bf.x, bf.y);
      mma_u8s8(acc, a0[1], a1[1], a2[1], a3[1], bf.z, bf.w);
      const float2 gs = *(const float2*)&gb[j * 2];
      const float f_lo = (float)(acc[0] * 128 + acc[1]), f_hi = (float)(acc[2] * 128 + acc[3]);
      tot0 = fmaf(s_lo * gs.x, f_lo, fmaf(b_lo, gs.y, tot0));
      tot1 = fmaf(s_hi * gs.x, f_hi, fmaf(b_hi, gs.y, tot1));
    }
    __syncwarp();
    if (issued < nu) issue();   // refill the stage just read
    cp_async_commit();
    ++issued;
  }
  cp_async_wait<0>();
  if (t == 0) { s_part[bank][part][g] = tot0; s_part[bank][part][g + 8] = tot1; }
  __syncthreads();
  if (warp == 0 && lane < 16) {
    const int n = tile * 16 + lane;
    float v[NB];
#pragma unroll
    for (int bk = 0; bk < NB; ++bk) v[bk] = ((s_part[bk][0][lane] + s_part[bk][1][lane]) + s_part[bk][2][lane]) + s_part[bk][3][lane];
    if (n < p.N) {
      if constexpr (FUSED) {
        if (p.f32) {
          const float sy = 1.f / (1.f + expf(fabsf(v[0])));
          ((float*)p.y)[i * p.N + n] = (v[0] * (v[0] < 0.f ? sy : 1.f - sy)) * v[NB - 1];
        } else {
          const uint32_t g16 = f32_to_bf16_bits(v[0]);
          const float gf = __uint_as_float(g16 << 16), sig = __uint_as_float((uint32_t)p.sigtab[g16] << 16);
          const float act = rdt(gf * sig, false), uf = rdt(v[NB - 1], false);
          ((uint16_t*)p.y)[i * p.N + n] = f32_to_bf16_bits(act * uf);
        }
      } else {
        if (p.f32) ((float*)p.y)[i * p.N + n] = v[0];
        else ((uint16_t*)p.y)[i * p.N + n] = f32_to_bf16_bits(v[0]);
      }
    }
  }
}

int small_stages(int K, int bits) {   // units of the busiest warp: 2 stages when they fit, else 4
  const int ut = K / (bits == 4 ? 256 : 128);
  return (ut + kParts - 1) / kParts <= 2 ? 2 : 4;
}
size_t smem_bytes_small(int K, int bits, bool fused) {
  return (size_t)(K / 64) * 136 + (size_t)(fused ? 2 : 1) * kParts * small_stages(K, bits) * kStageBytes;
}

size_t smem_bytes_dr(int K, int topk) {
  return (size_t)topk * ((size_t)kStages * kStageBytes + (size_t)(K / 64) * 128 + (size_t)(K / 64) * 8);
}

}  // namespace

bool moe_down_reduce_supported(const MoeDownReduceArgs& a) {
  if (!((a.bits == 4 && (a.gs == 64 || a.gs == 128)) || (a.bits == 8 && a.gs == 64))) return false;
  if (a.dtype != QB200_BFLOAT16 && a.dtype != QB200_FLOAT32) return false;
  if (a.K % 256 != 0 || a.K <= 0 || a.K > 8192 || a.N <= 0) return false;
  if (a.topk < 1 || a.topk > kMaxSlots || a.T < 1 || a.T > 65535) return false;
  if ((((uintptr_t)a.w) & 15) != 0 || (a.wes * 4) % 16 != 0) return false;
  if ((((uintptr_t)a.s) & 7) != 0 || (((uintptr_t)a.b) & 7) != 0 || (a.ses * 2) % 8 != 0) return false;
  if (a.gs == 64 && (a.K / 64) % 4 != 0) return false;
  if (a.gs == 128 && (a.K / 128) % 2 != 0) return false;
  if ((((uintptr_t)a.act) & 15) != 0) return false;
  return smem_bytes_dr((int)a.K, a.topk) + 2048 <= (size_t)227 * 1024;
}

cudaError_t launch_moe_down_reduce(const MoeDownReduceArgs& a, cudaStream_t st) {
  DRK p;
  p.act = a.act; p.w = a.w; p.s = (const uint16_t*)a.s; p.b = (const uint16_t*)a.b; p.y = a.y;
  p.inds = a.inds; p.scores = a.scores; p.inds_i64 = a.inds_i64;
  p.E = a.E; p.wes = a.wes; p.ses = a.ses;
  p.N = (int)a.N; p.K = (int)a.K; p.topk = a.topk; p.gshift = a.gs == 128 ? 1 : 0; p.f32 = a.dtype == QB200_FLOAT32;
  const size_t smem = smem_bytes_dr(p.K, p.topk);
  const void* kern = a.bits == 4 ? (const void*)moe_down_reduce_kernel<4> : (const void*)moe_down_reduce_kernel<8>;
  static bool done[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int bi = a.bits == 4 ? 0 : 1;
  {
  std::lock_guard<std::mutex> setup_lk(setup_mutex());   // first use on a device, from any thread
  if (dev < 0 || dev >= 64 || !done[bi][dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) done[bi][dev] = true;
  }
  }
  const dim3 grid((unsigned)((p.N + 15) / 16), (unsigned)a.T, 1);
  if (a.bits == 4) moe_down_reduce_kernel<4><<<grid, p.topk * 32, smem, st>>>(p);
  else moe_down_reduce_kernel<8><<<grid, p.topk * 32, smem, st>>>(p);
  return cudaGetLastError();
}

// Rows the small form takes: few enough that streaming one expert tile per (row, tile) CTA beats the expert-centric
// kernel's set-up (single-token decode: top-k rows, each with its own expert).
bool gather_small_supported(const GatherArgs& a) {
  if (!((a.bits == 4 && (a.gs == 64 || a.gs == 128)) || (a.bits == 8 && a.gs == 64))) return false;
  if (a.x_dtype != QB200_BFLOAT16 && a.x_dtype != QB200_FLOAT32) return false;
  if (a.M != 1 || a.K % 256 != 0 || a.K <= 0 || a.K > 16384) return false;
  if (a.N <= 0 || a.I <= 0 || a.I > 16) return false;
  if ((((uintptr_t)a.w) & 15) != 0 || (a.w_expert_stride * 4) % 16 != 0) return false;
  if ((((uintptr_t)a.s) & 7) != 0 || (((uintptr_t)a.b) & 7) != 0 || (a.s_expert_stride * 2) % 8 != 0) return false;
  if (a.w2 && ((((uintptr_t)a.w2) & 15) != 0 || (((uintptr_t)a.s2) & 7) != 0 || (((uintptr_t)a.b2) & 7) != 0)) return false;
  if (a.gs == 64 && (a.K / 64) % 4 != 0) return false;
  if (a.gs == 128 && (a.K / 128) % 2 != 0) return false;
  if ((((uintptr_t)a.x) & 15) != 0 || (a.x_batch_stride * (a.x_dtype == QB200_FLOAT32 ? 4 : 2)) % 16 != 0) return false;
  if (a.rhs_dtype != QB200_INT64 && a.rhs_dtype != QB200_INT32 && a.rhs_dtype != QB200_UINT32) return false;
  if (a.lhs && a.lhs_dtype != QB200_INT64 && a.lhs_dtype != QB200_INT32 && a.lhs_dtype != QB200_UINT32) return false;
  return smem_bytes_small((int)a.K, a.bits, a.w2 != nullptr) + 2048 <= (size_t)227 * 1024;
}

cudaError_t launch_gather_small(const GatherArgs& a, cudaStream_t st) {
  GSK p;
  const bool fused = a.w2 != nullptr;
  p.x = a.x; p.w = a.w; p.s = (const uint16_t*)a.s; p.b = (const uint16_t*)a.b; p.y = a.y;
  p.w2 = a.w2; p.s2 = (const uint16_t*)a.s2; p.b2 = (const uint16_t*)a.b2; p.sigtab = nullptr;
  p.rhs = a.rhs; p.lhs = a.lhs;
  p.rhs_i64 = a.rhs_dtype == QB200_INT64; p.lhs_i64 = a.lhs_dtype == QB200_INT64;
  p.xbcast = a.xbcast;
  p.E = a.E; p.XB = a.XB; p.xstride = a.x_batch_stride; p.wes = a.w_expert_stride; p.ses = a.s_expert_stride;
  p.N = (int)a.N; p.K = (int)a.K; p.gshift = a.gs == 128 ? 1 : 0; p.f32 = a.x_dtype == QB200_FLOAT32;
  if (fused) {
    cudaError_t te;
    p.sigtab = sigmoid_table(st, &te);
    if (!p.sigtab) return te;
  }
  const size_t smem = smem_bytes_small(p.K, a.bits, fused);
  const int S = small_stages(p.K, a.bits);
  const int ki = (a.bits == 4 ? 0 : 1) + (fused ? 2 : 0) + (S == 2 ? 0 : 4);
  const void* kerns[8] = {(const void*)gather_small_kernel<4, false, 2>, (const void*)gather_small_kernel<8, false, 2>,
                          (const void*)gather_small_kernel<4, true, 2>,  (const void*)gather_small_kernel<8, true, 2>,
                          (const void*)gather_small_kernel<4, false, 4>, (const void*)gather_small_kernel<8, false, 4>,
                          (const void*)gather_small_kernel<4, true, 4>,  (const void*)gather_small_kernel<8, true, 4>};
  static bool done[8][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
  std::lock_guard<std::mutex> setup_lk(setup_mutex());   // first use on a device, from any thread
  if (dev < 0 || dev >= 64 || !done[ki][dev]) {
    cudaError_t e = cudaFuncSetAttribute(kerns[ki], cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) done[ki][dev] = true;
  }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((p.N + 15) / 16), (unsigned)a.I, 1);
  cfg.blockDim = dim3((fused ? 2 : 1) * kParts * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  void* args[1] = {(void*)&p};
  return cudaLaunchKernelExC(&cfg, kerns[ki], args);
}

}  // namespace qb

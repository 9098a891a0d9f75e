// Weight-streaming quantized matmul for small M (decode): y = x . What^T.
//
// Replaces mlx_quantized_matmul(transpose=true) as called by qmatmulBits
// (mlx-serve src/transformer.zig:20894-20983) for decode widths, the small-M
// verify lanes (src/transformer.zig:1317-1453) and, in gather form,
// mlx_gather_qmm as called by gatherExpertMm (src/transformer.zig:20763-20784).
//
// Design (HBM-bound; the tensor cores only keep the ALUs out of the way):
//  * A warp owns 16 output rows (one m16 MMA tile) and a slice of K.  For each
//    64-wide group it loads the packed codes of rows g and g+8 with one 64-bit
//    (4-bit) or 128-bit (8-bit) streaming load per row; the four lanes of a
//    quad cover one group's 32/64 contiguous bytes, consecutive groups fill
//    the 128-byte line.
//  * Codes are expanded to bf16 *integers* in registers (LOP3 magic-number
//    trick for 4-bit: (w & 0x000F000F) | 0x43004300 = 128+q per lane; PRMT
//    into an fp32 mantissa for 8-bit) and fed as the A operand of
//    mma.sync.m16n8k16; the B operand is the token block (<= 8 tokens per
//    n-tile) staged once per CTA in shared memory in fragment order.
//    Products q*x are exact in fp32; scale and bias are applied per group on
//    the fp32 accumulators:  y += s*(sum (128+q) x) + (b - 128 s)*(sum x),
//    so the weight term q*s+b is never rounded to bf16.
//  * K is split over the warps of a CTA (and reduced through shared memory);
//    nothing is written to global scratch.
//  * fp32 activations are split into bf16 hi + lo halves that occupy two token
//    slots of the same n-tile, so fp32 inputs keep ~16 significant bits.
#include <mutex>

#include "kernels.h"
#include "qmv_frag.cuh"

namespace qb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
// Activations staged per pass: 16*kc*NT bytes of shared memory (64 KiB).
__host__ __device__ constexpr int kc_for(int nt) { return 4096 / nt; }

struct Shared {
  uint2* xfrag;  // [(group64*4 + step)*NT + nt][32 lanes]
  float* xsum;   // [(group64*NT + nt)*8 + slot]
};

// Stage tokens into fragment order.  `tok_ptr(slot)` gives the row pointer of
// a token slot or nullptr; for fp32 inputs slots 4..7 carry the low halves.
template <int BITS, int NT, typename TokFn>
__device__ __forceinline__ void stage_x(const Shared& sm, int k0, int klen, bool x_f32, TokFn tok_ptr) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int ngroups = klen >> 6;
  for (int item = warp; item < ngroups * NT; item += kWarps) {
    const int gi = item / NT, nt = item - gi * NT;
    const int slot = nt * 8 + g;
    float v[16];
    const void* row = tok_ptr(slot);
    if (row == nullptr) {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = 0.f;
    } else if (!x_f32) {
      const uint16_t* p = (const uint16_t*)row + k0 + gi * 64 + 16 * t;
      if ((((uintptr_t)p) & 15) == 0) {
        const uint4 a = *(const uint4*)p, b = *(const uint4*)(p + 8);
        const uint32_t r[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[2 * j] = bf16lo(r[j]); v[2 * j + 1] = bf16hi(r[j]); }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = bf16_bits_to_f32(p[j]);
      }
    } else {
      const float* p = (const float*)row + k0 + gi * 64 + 16 * t;
      const bool lo_half = (g >= 4);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float f = p[j];
        const float hi = bf16_bits_to_f32(f32_to_bf16_bits(f));
        v[j] = lo_half ? bf16_bits_to_f32(f32_to_bf16_bits(f - hi)) : hi;
      }
    }
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) sum += v[j];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (t == 0) sm.xsum[(gi * NT + nt) * 8 + g] = sum;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint2 f;
      f.x = pack_bf16x2(v[kperm<BITS>(i, 0)], v[kperm<BITS>(i, 1)]);
      f.y = pack_bf16x2(v[kperm<BITS>(i, 2)], v[kperm<BITS>(i, 3)]);
      sm.xfrag[((gi * 4 + i) * NT + nt) * 32 + lane] = f;
    }
  }
}

// One warp, RTPW row tiles, its share of the 64-wide groups of the staged K
// range.  Accumulates into tot[r][nt][4] (MMA C-fragment layout).
template <int BITS, int NT, int RTPW, int KSW>
__device__ __forceinline__ void sweep(const Shared& sm, const uint32_t* (&wlo)[RTPW], const uint32_t* (&whi)[RTPW],
                                      const uint16_t* (&slo)[RTPW], const uint16_t* (&shi)[RTPW],
                                      const uint16_t* (&blo)[RTPW], const uint16_t* (&bhi)[RTPW], int k0, int klen,
                                      int gshift, int ks, float (&tot)[RTPW][NT][4]) {
  using W = typename WReg<BITS>::T;
  constexpr int U = WReg<BITS>::U;
  constexpr int WPG = 64 * BITS / 32;       // packed words per 64-wide group
  constexpr int WPT = WPG / 4;              // words per lane per group
  const int lane = threadIdx.x & 31, t = lane & 3;
  const int nchunks = klen / (64 * U);
  const int g0 = k0 >> 6;                   // first 64-group of this pass (global index)

  W cw_lo[RTPW][U], cw_hi[RTPW][U];
  float cs_lo[RTPW][U], cs_hi[RTPW][U], cb_lo[RTPW][U], cb_hi[RTPW][U];

  auto load_chunk = [&](int c, W (&w_lo)[RTPW][U], W (&w_hi)[RTPW][U], float (&s_lo)[RTPW][U],
                        float (&s_hi)[RTPW][U], float (&b_lo)[RTPW][U], float (&b_hi)[RTPW][U]) {
#pragma unroll
    for (int r = 0; r < RTPW; ++r) {
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const int64_t woff = (int64_t)(g0 + c * U + j) * WPG + t * WPT;
        w_lo[r][j] = load_w<BITS>(wlo[r] + woff);
        w_hi[r][j] = load_w<BITS>(whi[r] + woff);
      }
      const int gidx = g0 + c * U;
      load_sb<U>(slo[r], gidx, gshift, s_lo[r]);
      load_sb<U>(shi[r], gidx, gshift, s_hi[r]);
      load_sb<U>(blo[r], gidx, gshift, b_lo[r]);
      load_sb<U>(bhi[r], gidx, gshift, b_hi[r]);
    }
  };

  int c = ks;
  if (c < nchunks) load_chunk(c, cw_lo, cw_hi, cs_lo, cs_hi, cb_lo, cb_hi);
  for (; c < nchunks; c += KSW) {
    W nw_lo[RTPW][U], nw_hi[RTPW][U];
    float ns_lo[RTPW][U], ns_hi[RTPW][U], nb_lo[RTPW][U], nb_hi[RTPW][U];
    const bool more = (c + KSW) < nchunks;
    if (more) load_chunk(c + KSW, nw_lo, nw_hi, ns_lo, ns_hi, nb_lo, nb_hi);
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const int gl = c * U + j;  // group index inside the staged range
      uint2 bf[4][NT];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) bf[i][nt] = sm.xfrag[((gl * 4 + i) * NT + nt) * 32 + lane];
      float2 xs[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) xs[nt] = *(const float2*)&sm.xsum[(gl * NT + nt) * 8 + 2 * t];
#pragma unroll
      for (int r = 0; r < RTPW; ++r) {
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t a[4];
          expand<BITS>(cw_lo[r][j], i, a[0], a[2]);
          expand<BITS>(cw_hi[r][j], i, a[1], a[3]);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(acc[nt], a, bf[i][nt].x, bf[i][nt].y);
        }
        const float sl = cs_lo[r][j], sh = cs_hi[r][j];
        const float bl = fmaf(-code_base<BITS>(), sl, cb_lo[r][j]);
        const float bh = fmaf(-code_base<BITS>(), sh, cb_hi[r][j]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          tot[r][nt][0] += fmaf(sl, acc[nt][0], bl * xs[nt].x);
          tot[r][nt][1] += fmaf(sl, acc[nt][1], bl * xs[nt].y);
          tot[r][nt][2] += fmaf(sh, acc[nt][2], bh * xs[nt].x);
          tot[r][nt][3] += fmaf(sh, acc[nt][3], bh * xs[nt].y);
        }
      }
    }
    if (more) {
#pragma unroll
      for (int r = 0; r < RTPW; ++r)
#pragma unroll
        for (int j = 0; j < U; ++j) {
          cw_lo[r][j] = nw_lo[r][j]; cw_hi[r][j] = nw_hi[r][j];
          cs_lo[r][j] = ns_lo[r][j]; cs_hi[r][j] = ns_hi[r][j];
          cb_lo[r][j] = nb_lo[r][j]; cb_hi[r][j] = nb_hi[r][j];
        }
    }
  }
}

struct DenseK {
  const void* x; const uint32_t* w; const uint16_t* s; const uint16_t* b; void* y;
  int M, N, K;
  int64_t ldx, ldw, lds, ldy;
  int gshift;   // 0: group size 64, 1: group size 128
  int x_f32;
  BatchMap xb, wb, sb, yb;
};

// Cross-warp reduction of tot through shared memory and the store of y.
// red layout: [warp][r][nt][16 rows][8 cols]
template <int NT, int RTPW, int KSW, typename StoreFn>
__device__ __forceinline__ void reduce_store(float* red, const float (&tot)[RTPW][NT][4], bool x_f32, StoreFn store) {
  constexpr int RTW = kWarps / KSW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int r = 0; r < RTPW; ++r)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float* base = red + (((warp * RTPW + r) * NT + nt) * 16) * 8;
      *(float2*)&base[g * 8 + 2 * t] = make_float2(tot[r][nt][0], tot[r][nt][1]);
      *(float2*)&base[(g + 8) * 8 + 2 * t] = make_float2(tot[r][nt][2], tot[r][nt][3]);
    }
  __syncthreads();
  constexpr int ROWS = 16 * RTW * RTPW;
  const int tok_per_tile = x_f32 ? 4 : 8;
  for (int o = threadIdx.x; o < ROWS * NT * tok_per_tile; o += kThreads) {
    const int row = o % ROWS, col = o / ROWS;        // col: token index inside the CTA's token block
    const int nt = col / tok_per_tile, c = col - nt * tok_per_tile;
    const int rtw = row / (16 * RTPW), rr = row - rtw * 16 * RTPW, r = rr >> 4, ri = rr & 15;
    float v = 0.f;
#pragma unroll
    for (int k = 0; k < KSW; ++k) {
      const float* base = red + ((((rtw * KSW + k) * RTPW + r) * NT + nt) * 16) * 8;
      v += base[ri * 8 + c];
      if (x_f32) v += base[ri * 8 + c + 4];
    }
    store(row, nt * tok_per_tile + c, v);
  }
}

template <int BITS, int NT, int KSW, int RTPW>
__global__ void __launch_bounds__(kThreads) qmv_dense_kernel(DenseK p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int RTW = kWarps / KSW;
  constexpr int ROWS = 16 * RTW * RTPW;
  constexpr int U = WReg<BITS>::U;
  Shared sm;
  sm.xfrag = (uint2*)smem_raw;
  constexpr int KC = kc_for(NT);
  const int kc = p.K < KC ? p.K : KC;
  sm.xsum = (float*)(smem_raw + (size_t)(kc / 16) * NT * 32 * 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2;
  const int ks = warp % KSW, rtw = warp / KSW;
  const int64_t bz = blockIdx.z;
  const char* xbase = (const char*)p.x + p.xb.offset(bz) * (p.x_f32 ? 4 : 2);
  const uint32_t* wbase = p.w + p.wb.offset(bz);
  const int64_t sboff = p.sb.offset(bz);
  const int n_cta = blockIdx.x * ROWS;

  const uint32_t* wlo[RTPW]; const uint32_t* whi[RTPW];
  const uint16_t* slo[RTPW]; const uint16_t* shi[RTPW]; const uint16_t* blo[RTPW]; const uint16_t* bhi[RTPW];
#pragma unroll
  for (int r = 0; r < RTPW; ++r) {
    int n0 = n_cta + (rtw * RTPW + r) * 16 + g, n1 = n0 + 8;
    n0 = n0 < p.N ? n0 : p.N - 1;
    n1 = n1 < p.N ? n1 : p.N - 1;
    wlo[r] = wbase + (int64_t)n0 * p.ldw; whi[r] = wbase + (int64_t)n1 * p.ldw;
    slo[r] = p.s + sboff + (int64_t)n0 * p.lds; shi[r] = p.s + sboff + (int64_t)n1 * p.lds;
    blo[r] = p.b + sboff + (int64_t)n0 * p.lds; bhi[r] = p.b + sboff + (int64_t)n1 * p.lds;
  }
  float tot[RTPW][NT][4];
#pragma unroll
  for (int r = 0; r < RTPW; ++r)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) tot[r][nt][0] = tot[r][nt][1] = tot[r][nt][2] = tot[r][nt][3] = 0.f;

  const int tok_per_tile = p.x_f32 ? 4 : 8;
  auto tok_ptr = [&](int slot) -> const void* {
    const int nt = slot >> 3, s8 = slot & 7;
    const int m = nt * tok_per_tile + (p.x_f32 ? (s8 & 3) : s8);
    if (m >= p.M) return nullptr;
    return xbase + (int64_t)m * p.ldx * (p.x_f32 ? 4 : 2);
  };

  for (int k0 = 0; k0 < p.K; k0 += KC) {
    const int klen = (p.K - k0) < KC ? (p.K - k0) : KC;
    if (k0 > 0) __syncthreads();
    stage_x<BITS, NT>(sm, k0, klen, p.x_f32 != 0, tok_ptr);
    __syncthreads();
    sweep<BITS, NT, RTPW, KSW>(sm, wlo, whi, slo, shi, blo, bhi, k0, klen, p.gshift, ks, tot);
  }
  __syncthreads();
  (void)U;
  char* ybase = (char*)p.y + p.yb.offset(bz) * (p.x_f32 ? 4 : 2);
  reduce_store<NT, RTPW, KSW>((float*)smem_raw, tot, p.x_f32 != 0, [&](int row, int m, float v) {
    const int n = n_cta + row;
    if (n < p.N && m < p.M) {
      if (p.x_f32) ((float*)ybase)[(int64_t)m * p.ldy + n] = v;
      else ((uint16_t*)ybase)[(int64_t)m * p.ldy + n] = f32_to_bf16_bits(v);
    }
  });
}

size_t dense_smem_bytes(int K, int NT, int RTPW) {
  const int kc = K < kc_for(NT) ? K : kc_for(NT);
  const size_t stage = (size_t)(kc / 16) * NT * 32 * 8 + (size_t)(kc / 64) * NT * 8 * 4;
  const size_t red = (size_t)kWarps * RTPW * NT * 16 * 8 * 4;
  return stage > red ? stage : red;
}

template <int BITS, int NT, int KSW, int RTPW>
cudaError_t launch_dense_inst(const DenseK& p, int64_t nbatch, cudaStream_t st) {
  constexpr int ROWS = 16 * (kWarps / KSW) * RTPW;
  const size_t smem = dense_smem_bytes(p.K, NT, RTPW);
  auto kern = qmv_dense_kernel<BITS, NT, KSW, RTPW>;
  static bool attr_done[64] = {};  // per instantiation and device; the call is idempotent
  int dev = 0;
  cudaGetDevice(&dev);
  {
  std::lock_guard<std::mutex> setup_lk(setup_mutex());   // first use on a device, from any thread
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  }
  dim3 grid((unsigned)((p.N + ROWS - 1) / ROWS), 1, (unsigned)nbatch);
  kern<<<grid, kThreads, smem, st>>>(p);
  return cudaGetLastError();
}

template <int BITS, int NT>
cudaError_t launch_dense_tile(const DenseK& p, int64_t nbatch, cudaStream_t st) {
  // Pick the CTA shape: more K-split for short/narrow problems, more rows per
  // CTA (activations staged once per CTA) for tall ones.
  const int64_t tiles = (p.N + 15) / 16;
  const int nchunks = (p.K < kc_for(NT) ? p.K : kc_for(NT)) / (64 * WReg<BITS>::U);
  if constexpr (NT == 4) {
    return launch_dense_inst<BITS, NT, 4, 1>(p, nbatch, st);
  } else {
    if (tiles >= 2048 && nchunks >= 4) return launch_dense_inst<BITS, NT, 4, 2>(p, nbatch, st);
    if (tiles >= 512 && nchunks >= 8) return launch_dense_inst<BITS, NT, 8, 2>(p, nbatch, st);
    return launch_dense_inst<BITS, NT, 8, 1>(p, nbatch, st);
  }
}

template <int BITS>
cudaError_t launch_dense_bits(const DenseK& p, int64_t nbatch, cudaStream_t st) {
  const int tok_per_tile = p.x_f32 ? 4 : 8;
  const int nt = (p.M + tok_per_tile - 1) / tok_per_tile;
  if (nt <= 1) return launch_dense_tile<BITS, 1>(p, nbatch, st);
  if (nt <= 2) return launch_dense_tile<BITS, 2>(p, nbatch, st);
  return launch_dense_tile<BITS, 4>(p, nbatch, st);
}


// ---------------------------------------------------------------------------
// gather form: output row i uses expert rhs[i] and activation row lhs(i).
// A CTA takes a block of 8 output rows (4 for fp32 activations) and 16*RTW
// weight rows; it sweeps once per distinct expert in its block, so rows that
// are sorted by expert (mlx-serve src/transformer.zig:14961-15043) share one
// pass over that expert's weights, and unsorted decode rows
// (src/transformer.zig:15091-15119) cost one pass each, which is the minimum.
struct GatherK {
  const void* x; const uint32_t* w; const uint16_t* s; const uint16_t* b; void* y;
  int64_t I; int N, K;
  int64_t x_stride, XB;        // elements between activation rows; number of rows
  int64_t w_es, s_es; int64_t E;
  const void* lhs; int lhs_i64; const void* rhs; int rhs_i64;
  BatchMap xbcast;
  int gshift, x_f32;
};

template <int BITS, int KSW>
__global__ void __launch_bounds__(kThreads) gather_kernel(GatherK p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int NT = 1, RTPW = 1;
  constexpr int RTW = kWarps / KSW;
  constexpr int ROWS = 16 * RTW;
  constexpr int KC = kc_for(NT);
  __shared__ long long s_eid[8];
  __shared__ long long s_xi[8];
  Shared sm;
  sm.xfrag = (uint2*)smem_raw;
  const int kc = p.K < KC ? p.K : KC;
  sm.xsum = (float*)(smem_raw + (size_t)(kc / 16) * NT * 32 * 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int ks = warp % KSW, rtw = warp / KSW;
  const int tok = p.x_f32 ? 4 : 8;
  const int64_t i0 = (int64_t)blockIdx.y * tok;
  const int n_cta = blockIdx.x * ROWS;
  if (threadIdx.x < 8) {
    const int64_t i = i0 + threadIdx.x;
    long long e = -1, xi = -1;
    if (threadIdx.x < tok && i < p.I) {
      e = p.rhs_i64 ? ((const long long*)p.rhs)[i] : (long long)((const uint32_t*)p.rhs)[i];
      if (p.lhs) xi = p.lhs_i64 ? ((const long long*)p.lhs)[i] : (long long)((const uint32_t*)p.lhs)[i];
      else xi = p.xbcast.offset(i);
      if (e < 0 || e >= p.E || xi < 0 || xi >= p.XB) { e = -1; xi = -1; }
    }
    s_eid[threadIdx.x] = e;
    s_xi[threadIdx.x] = xi;
  }
  __syncthreads();
  auto tok_ptr = [&](int slot) -> const void* {
    const long long xi = s_xi[p.x_f32 ? (slot & 3) : slot];
    if (xi < 0) return nullptr;
    return (const char*)p.x + xi * p.x_stride * (p.x_f32 ? 4 : 2);
  };

  int n0 = n_cta + rtw * 16 + g, n1 = n0 + 8;
  n0 = n0 < p.N ? n0 : p.N - 1;
  n1 = n1 < p.N ? n1 : p.N - 1;
  float fin[RTPW][NT][4];
  fin[0][0][0] = fin[0][0][1] = fin[0][0][2] = fin[0][0][3] = 0.f;
  const int c0 = p.x_f32 ? ((2 * t) & 3) : 2 * t, c1 = p.x_f32 ? ((2 * t + 1) & 3) : 2 * t + 1;

  for (int k0 = 0; k0 < p.K; k0 += KC) {
    const int klen = (p.K - k0) < KC ? (p.K - k0) : KC;
    if (k0 > 0) __syncthreads();
    stage_x<BITS, NT>(sm, k0, klen, p.x_f32 != 0, tok_ptr);
    __syncthreads();
    for (int a = 0; a < tok; ++a) {
      const long long e = s_eid[a];
      if (e < 0) continue;
      bool seen = false;
      for (int q = 0; q < a; ++q) seen |= (s_eid[q] == e);
      if (seen) continue;
      const uint32_t* wlo[1] = {p.w + e * p.w_es + (int64_t)n0 * (p.K * BITS / 32)};
      const uint32_t* whi[1] = {p.w + e * p.w_es + (int64_t)n1 * (p.K * BITS / 32)};
      const int64_t sl = e * p.s_es + (int64_t)n0 * (p.K >> (6 + p.gshift));
      const int64_t sh = e * p.s_es + (int64_t)n1 * (p.K >> (6 + p.gshift));
      const uint16_t* slo[1] = {p.s + sl}; const uint16_t* shi[1] = {p.s + sh};
      const uint16_t* blo[1] = {p.b + sl}; const uint16_t* bhi[1] = {p.b + sh};
      float tot[RTPW][NT][4];
      tot[0][0][0] = tot[0][0][1] = tot[0][0][2] = tot[0][0][3] = 0.f;
      sweep<BITS, NT, RTPW, KSW>(sm, wlo, whi, slo, shi, blo, bhi, k0, klen, p.gshift, ks, tot);
      const bool m0 = s_eid[c0] == e, m1 = s_eid[c1] == e;
      if (m0) { fin[0][0][0] += tot[0][0][0]; fin[0][0][2] += tot[0][0][2]; }
      if (m1) { fin[0][0][1] += tot[0][0][1]; fin[0][0][3] += tot[0][0][3]; }
    }
  }
  __syncthreads();
  reduce_store<NT, RTPW, KSW>((float*)smem_raw, fin, p.x_f32 != 0, [&](int row, int m, float v) {
    const int n = n_cta + row;
    if (n < p.N && m < tok && s_eid[m] >= 0) {
      const int64_t o = (i0 + m) * (int64_t)p.N + n;
      if (p.x_f32) ((float*)p.y)[o] = v;
      else ((uint16_t*)p.y)[o] = f32_to_bf16_bits(v);
    }
  });
}

template <int BITS, int KSW>
cudaError_t launch_gather_inst(const GatherK& p, cudaStream_t st) {
  constexpr int ROWS = 16 * (kWarps / KSW);
  const size_t smem = dense_smem_bytes(p.K, 1, 1);
  auto kern = gather_kernel<BITS, KSW>;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
  std::lock_guard<std::mutex> setup_lk(setup_mutex());   // first use on a device, from any thread
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  }
  const int tok = p.x_f32 ? 4 : 8;
  dim3 grid((unsigned)((p.N + ROWS - 1) / ROWS), (unsigned)((p.I + tok - 1) / tok), 1);
  kern<<<grid, kThreads, smem, st>>>(p);
  return cudaGetLastError();
}

template <int BITS>
cudaError_t launch_gather_bits(const GatherK& p, cudaStream_t st) {
  const int nchunks = (p.K < kc_for(1) ? p.K : kc_for(1)) / (64 * WReg<BITS>::U);
  if (nchunks >= 8) return launch_gather_inst<BITS, 8>(p, st);
  if (nchunks >= 4) return launch_gather_inst<BITS, 4>(p, st);
  return launch_gather_inst<BITS, 2>(p, st);
}

}  // namespace

bool qmv_mma_supported(const QmmArgs& a) {
  if (!a.transpose) return false;
  if (a.bits != 4 && a.bits != 8) return false;
  if (a.gs != 64 && a.gs != 128) return false;
  if (a.x_dtype != QB200_BFLOAT16 && a.x_dtype != QB200_FLOAT32) return false;
  const int U = a.bits == 4 ? 4 : 2;
  if (a.K % (64 * U) != 0 || a.K <= 0 || a.K > (1 << 24)) return false;
  if (a.N <= 0 || a.N > (1 << 30)) return false;
  if (a.M <= 0) return false;
  if ((((uintptr_t)a.w) & 15) != 0 || (a.ldw * 4) % 16 != 0) return false;
  if (a.nbatch > 65535) return false;
  if ((((uintptr_t)a.s) & 7) != 0 || (((uintptr_t)a.b) & 7) != 0) return false;
  for (int d = 0; d < a.wb.nd; ++d)
    if ((a.wb.stride[d] * 4) % 16 != 0 || a.sb.stride[d] % 4 != 0) return false;
  return true;
}

cudaError_t launch_qmv_mma(const QmmArgs& a, cudaStream_t st) {
  DenseK p;
  p.w = a.w; p.s = (const uint16_t*)a.s; p.b = (const uint16_t*)a.b;
  p.N = (int)a.N; p.K = (int)a.K;
  p.ldx = a.ldx; p.ldw = a.ldw; p.lds = a.lds; p.ldy = a.ldy;
  p.gshift = a.gs == 128 ? 1 : 0;
  p.x_f32 = a.x_dtype == QB200_FLOAT32;
  p.xb = a.xb; p.wb = a.wb; p.sb = a.sb; p.yb = a.yb;
  const int esz = p.x_f32 ? 4 : 2;
  const int tok_per_tile = p.x_f32 ? 4 : 8;
  const int64_t block = 4 * tok_per_tile;  // tokens per launch; wider M re-streams the weights per block
  for (int64_t m0 = 0; m0 < a.M; m0 += block) {
    p.x = (const char*)a.x + m0 * a.ldx * esz;
    p.y = (char*)a.y + m0 * a.ldy * esz;
    p.M = (int)((a.M - m0) < block ? (a.M - m0) : block);
    cudaError_t e = a.bits == 4 ? launch_dense_bits<4>(p, a.nbatch, st) : launch_dense_bits<8>(p, a.nbatch, st);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace qb

namespace qb {

bool gather_mma_supported(const GatherArgs& a) {
  if (a.bits != 4 && a.bits != 8) return false;
  if (a.gs != 64 && a.gs != 128) return false;
  if (a.x_dtype != QB200_BFLOAT16 && a.x_dtype != QB200_FLOAT32) return false;
  if (a.M != 1) return false;
  const int U = a.bits == 4 ? 4 : 2;
  if (a.K % (64 * U) != 0 || a.K <= 0 || a.K > (1 << 24)) return false;
  if (a.N <= 0 || a.N > (1 << 30) || a.I <= 0) return false;
  const int tok = a.x_dtype == QB200_FLOAT32 ? 4 : 8;
  if ((a.I + tok - 1) / tok > 65535) return false;
  if ((((uintptr_t)a.w) & 15) != 0 || (a.w_expert_stride * 4) % 16 != 0) return false;
  if ((((uintptr_t)a.s) & 7) != 0 || (((uintptr_t)a.b) & 7) != 0 || a.s_expert_stride % 4 != 0) return false;
  if (a.rhs_dtype != QB200_INT64 && a.rhs_dtype != QB200_INT32 && a.rhs_dtype != QB200_UINT32) return false;
  if (a.lhs && a.lhs_dtype != QB200_INT64 && a.lhs_dtype != QB200_INT32 && a.lhs_dtype != QB200_UINT32) return false;
  return true;
}

cudaError_t launch_gather_mma(const GatherArgs& a, cudaStream_t st) {
  GatherK p;
  p.x = a.x; p.w = a.w; p.s = (const uint16_t*)a.s; p.b = (const uint16_t*)a.b; p.y = a.y;
  p.I = a.I; p.N = (int)a.N; p.K = (int)a.K;
  p.x_stride = a.x_batch_stride; p.XB = a.XB;
  p.w_es = a.w_expert_stride; p.s_es = a.s_expert_stride; p.E = a.E;
  p.lhs = a.lhs; p.lhs_i64 = a.lhs_dtype == QB200_INT64;
  p.rhs = a.rhs; p.rhs_i64 = a.rhs_dtype == QB200_INT64;
  p.xbcast = a.xbcast;
  p.gshift = a.gs == 128 ? 1 : 0;
  p.x_f32 = a.x_dtype == QB200_FLOAT32;
  return a.bits == 4 ? launch_gather_bits<4>(p, st) : launch_gather_bits<8>(p, st);
}

}  // namespace qb

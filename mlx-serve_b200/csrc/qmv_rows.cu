// Quantized matmul with the weight NOT transposed, at attention widths:
//   y[b, m, n] = sum_k x[b, m, k] * (s[b, k, G(n)] * q[b, k, n] + bias[b, k, G(n)]),   m <= 32 rows,
// W [K, N] quantised along N (the output axis), contracted over its rows.
//
// Replaces mlx_quantized_matmul(transpose=false) as quantAttention calls it for attn @ V
// (mlx-serve src/kv_quant.zig:657-674; pinned by the reference test at :1038-1094): x is the
// attention row block [B, Hkv, g*Tq, T], W the packed value cache [B, Hkv, T, D*bits/32], so K = T
// is long, N = D is one or two groups wide and the batch B*Hkv is large.  The work is one pass over
// the packed cache: HBM-bound by intent.
//
// The scale of a code varies along the contraction (every row of W has its own), so it cannot wait
// for the end of the sum as it does when W is transposed.  It is moved onto the activation instead:
//   y = sum_k (x s)[k] * q[k, n]  +  sum_k x[k] * bias[k],
// with one (x s) per (row k, group of n).  The first sum runs on the tensor cores
// (mma.sync m16n8k16 bf16, fp32 accumulate) with the roles swapped: the codes are the 16-row A
// operand (16 outputs n x 16 rows k), the scaled activations the 8-column B operand (8 tokens).
//  * A thread takes one packed word from each of four rows k.  A word holds 8 (4-bit) or 4 (8-bit)
//    outputs n of ONE row k; the MMA wants, per thread, two n by four k.  Both index sets are free
//    to permute (k as long as B follows, n as long as the result is stored where it belongs), so
//    MMA j simply takes byte j of the four words: its low nibbles are A row g, its high nibbles
//    A row g + 8.  No transposition through shared memory.
//  * A nibble c becomes the bf16 value 128 + c by OR-ing it into the mantissa of 0x4300 (one
//    PRMT, one shift and two LOP3 per four codes); the 128 is taken out again in fp32 through
//    the bias term, sum_k x (bias - 128 s).  An 8-bit code is its two nibbles: the high-nibble
//    rows of the accumulator count 16-fold in the epilogue (and the constant is 128 * 17).
//  * (x s) is split into two bf16 values, hi + lo, and each MMA is issued for both: the product
//    keeps 16 significant bits of x s, so that fp32 activations stay far inside the stated
//    tolerance and the 128-fold constant cancels (what is left of it is 2^-18 of |x s| per term).
//    With bf16 activations the split is exact and costs two packed instructions per pair
//    (hi = rn(x s), lo = fma(x, s, -hi)), and the bias term rides on the tensor cores too: the sum
//    of hi + lo against an A operand of ones and the sum of x * bias against an A operand whose rows
//    all hold the biases, both taken from the packed words as loaded -- no fp32 unpacking at all.
//  * The packed codes travel by cp.async (16 bytes per lane, one tile of 16 rows x 32 bytes per
//    instruction) into a ring of shared-memory stages private to the warp, several tiles ahead;
//    a warp only ever waits on its own copies (cp.async.wait_group + __syncwarp), so there is no
//    cross-warp protocol that could hang.  Scales, biases and activations (a quarter of the bytes)
//    come through a ring of registers.  (Sending those through the cp.async ring as well, as
//    4-byte pieces around elements that are only 2-byte aligned, was built and measured: 10 % slower
//    at long T -- four more copy instructions per tile in a kernel bound by instruction issue.)
//  * One CTA = 8 warps on one batch element.  A warp owns one block of 8 packed words of the row
//    (64 outputs at 4 bits, 32 at 8) and every (8 / blocks)-th 16-row tile of the CTA's range of K;
//    the warps add their sums in shared memory in a fixed order.  K is split over the CTAs of a
//    thread-block cluster (up to 8), whose rank 0 adds the partial sums through distributed shared
//    memory, in rank order, and stores: no global scratch, no atomics, a reproducible sum.
#include <type_traits>

#include "kernels.h"
#include "stream_ptx.cuh"

namespace qb {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxTokTiles = 4;        // 8-token tiles per launch
constexpr int kCodeStages = 8;         // ring of packed-code tiles per warp (cp.async; 7 tiles in flight)
constexpr int kCodeTile = 512;        // 16 rows x 32 bytes
constexpr int kSmemLimit = 72 * 1024;  // dynamic shared memory of one CTA (two or three CTAs per SM stay resident)

struct RowsK {
  const void* x; const uint32_t* w; const uint16_t* s; const uint16_t* b; void* y;
  int M, N;
  int64_t K;                     // rows of W: the contraction
  int64_t ldx, ldw, lds, ldy;    // row pitches in elements
  int sgshift;                   // log2(column blocks of 8 words per scale group)
  int ncb;                       // column blocks in a row: 1, 2, 4 or 8
  int tiles, tiles_per_cta;      // 16-row tiles of K, and how many of them one CTA of a cluster takes
  int ksplit;                    // CTAs per cluster
  int x_vec;                     // four consecutive activations may be loaded as one vector
  BatchMap xb, wb, sb, yb;
};



// packed bf16 pair arithmetic, correctly rounded
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// The bias term sum_k x (bias - C s) of a warp's tiles.  With bf16 activations it is two more accumulators of the
// tensor cores, in the token layout of the main ones (TC); otherwise one fp32 sum per token tile, held by the four
// threads that hold the token's activations.
template <int NT, bool TC> struct BiasAcc;
template <int NT> struct BiasAcc<NT, false> { float b[NT]; };
template <int NT> struct BiasAcc<NT, true> { float s[NT][4]; float b[NT][4]; };

// Dynamic shared memory of a CTA: the partial-sum tile [8 * nt][N + 1] (fp32), the per-warp bias sums [warps][8 * nt], the
// scale / bias hand-over [warps][64] (bf16), then, 16-byte aligned, the code rings.
__host__ __device__ inline size_t code_ring_offset(int nt, int N) {
  const size_t b = ((size_t)8 * nt * (N + 1) + (size_t)kWarps * 8 * nt) * sizeof(float) + (size_t)kWarps * 128;
  return (b + 15) & ~(size_t)15;
}

// Loads of the register ring are volatile asm, like the MMAs: the compiler keeps them where they are written, a
// ring's depth ahead of their use, instead of sinking them towards it when registers are short.
__device__ __forceinline__ uint32_t ldg_pin_u16(const void* p) {
  uint16_t v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_pin_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_pin_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// What a thread loads into registers for one 16-row tile (the packed codes go to shared memory instead, by cp.async).
// A ring of kDepth of these lives in registers, so that the loads of the next kDepth - 1 tiles are in flight while one
// tile is computed (3 registers per tile at up to 8 bf16 tokens).  The depth matters: with seven code tiles per warp in
// flight the memory system's queues are long, and a scale or an activation requested only two tiles ahead arrives late
// (measured on the 16 x 8 x 4 x 32768 attention shape: 142 us at depth 3, 127 at 6, 124 at 8).
//   sb: lanes 0-15 hold the scale of row `lane`, lanes 16-31 the bias of row `lane - 16` (bf16 bits)
//   x : activations of token g (per token tile) at rows 4t .. 4t + 3: two packed words for 16-bit types, four floats
template <int NT, int XW>
struct TileRegs {
  uint32_t sb;
  uint32_t x[NT][XW];
};
constexpr int kDepth = 8;
static_assert(kDepth <= kCodeStages, "the code ring is at least as deep as the register ring");

template <typename XT> struct XRaw;   // four consecutive activations, as loaded / as fp32
template <> struct XRaw<float> {
  static constexpr int W = 4;
  static __device__ __forceinline__ void vec(const void* p, int64_t i, uint32_t (&r)[4]) {
    const uint4 q = ldg_pin_u4((const float*)p + i);
    r[0] = q.x; r[1] = q.y; r[2] = q.z; r[3] = q.w;
  }
  static __device__ __forceinline__ void one(const void* p, int64_t i, int e, bool in, uint32_t (&r)[4]) {
    r[e] = in ? __float_as_uint(((const float*)p)[i]) : 0u;   // p is only dereferenced when `in`
  }
  static __device__ __forceinline__ void f32(const uint32_t (&r)[4], float (&v)[4]) {
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = __uint_as_float(r[e]);
  }
};
template <> struct XRaw<__nv_bfloat16> {
  static constexpr int W = 2;
  static __device__ __forceinline__ void vec(const void* p, int64_t i, uint32_t (&r)[2]) {
    const uint2 q = ldg_pin_u2((const uint16_t*)p + i);
    r[0] = q.x; r[1] = q.y;
  }
  static __device__ __forceinline__ void one(const void* p, int64_t i, int e, bool in, uint32_t (&r)[2]) {
    const uint32_t h = in ? (uint32_t)((const uint16_t*)p)[i] : 0u;
    r[e >> 1] = (e & 1) ? (r[e >> 1] | (h << 16)) : h;
  }
  static __device__ __forceinline__ void f32(const uint32_t (&r)[2], float (&v)[4]) {
    v[0] = bf16lo(r[0]); v[1] = bf16hi(r[0]); v[2] = bf16lo(r[1]); v[3] = bf16hi(r[1]);
  }
};
template <> struct XRaw<__half> {
  static constexpr int W = 2;
  static __device__ __forceinline__ void vec(const void* p, int64_t i, uint32_t (&r)[2]) { XRaw<__nv_bfloat16>::vec(p, i, r); }
  static __device__ __forceinline__ void one(const void* p, int64_t i, int e, bool in, uint32_t (&r)[2]) {
    XRaw<__nv_bfloat16>::one(p, i, e, in, r);
  }
  static __device__ __forceinline__ void f32(const uint32_t (&r)[2], float (&v)[4]) {
    const float2 a = __half22float2(*(const __half2*)&r[0]), c = __half22float2(*(const __half2*)&r[1]);
    v[0] = a.x; v[1] = a.y; v[2] = c.x; v[3] = c.y;
  }
};

// The addresses a thread walks, set up once per launch (tile 0; a tile is 16 rows further on).
template <int NT>
struct Walk {
  const uint32_t* w;      // this lane's 16-byte piece of a tile: row lane / 2, half lane % 2 of the warp's column block
  uint32_t ring;          // shared address of the warp's code ring
  uint32_t wdst;          // this lane's piece inside a stage
  uint32_t wsrc;          // this thread's word (row 4t, column g) inside a stage
  const uint16_t* sb;     // lanes 0-15: scale of row `lane`; lanes 16-31: bias of row `lane - 16`
  const char* x[NT];      // activation (token nt * 8 + g, row 4t); a token beyond M reads token 0 (its sums are never stored)
  int ldw16, lds16;       // 16 rows of w / of the scales, in elements
};

// The packed codes of tile `ti` into stage `stage` of the warp's ring: one 16-byte cp.async per lane.  Row r of the tile
// sits at slot (r % 4) * 4 + r / 4, so that the four threads t of a fragment row read four different bank groups.
// A row beyond K is filled with zeros (no bytes are read).
template <int NT>
__device__ __forceinline__ void fetch_codes(const RowsK& p, const Walk<NT>& a, int ti, int stage, int lane) {
  const bool in = (int64_t)ti * 16 + (lane >> 1) < p.K;
  const uint32_t dst = a.ring + (uint32_t)stage * kCodeTile + a.wdst;
  const void* src = in ? (const void*)(a.w + (int64_t)ti * a.ldw16) : (const void*)p.w;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(in ? 16 : 0));
}
template <int NT>
__device__ __forceinline__ void fetch_codes_full(const Walk<NT>& a, int ti, int stage) {
  cp_async16(a.ring + (uint32_t)stage * kCodeTile + a.wdst, a.w + (int64_t)ti * a.ldw16);
}

// A full tile: nothing to predicate (the steady state).
template <int NT, typename XT>
__device__ __forceinline__ void load_full(const Walk<NT>& a, int ti, bool x_vec, TileRegs<NT, XRaw<XT>::W>& r) {
  r.sb = ldg_pin_u16(a.sb + (int64_t)ti * a.lds16);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const char* xp = a.x[nt] + (int64_t)ti * (16 * (int)sizeof(XT));
    if (x_vec) {
      XRaw<XT>::vec(xp, 0, r.x[nt]);
    } else {   // a row pitch or a base that rules the vector load out (a cache length that is not a multiple of four)
#pragma unroll
      for (int i = 0; i < 4; ++i) XRaw<XT>::one(xp, i, i, true, r.x[nt]);
    }
  }
}

// Any tile: rows beyond K read as zero activations; activations loaded one by one.
template <int NT, typename XT>
__device__ __forceinline__ void load_any(const RowsK& p, const Walk<NT>& a, int ti, int lane, TileRegs<NT, XRaw<XT>::W>& r) {
  const int64_t k0 = (int64_t)ti * 16 + 4 * (lane & 3);
  r.sb = ((int64_t)ti * 16 + (lane & 15) < p.K) ? (uint32_t)__ldg(a.sb + (int64_t)ti * a.lds16) : 0u;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const char* xp = a.x[nt] + (int64_t)ti * (16 * (int)sizeof(XT));
#pragma unroll
    for (int i = 0; i < 4; ++i) XRaw<XT>::one(xp, i, i, k0 + i < p.K, r.x[nt]);
  }
}

// One 16-row tile of one column block.  The thread's four packed words come out of the warp's code ring; the warp's 16
// scales and 16 biases go through 64 bytes of shared memory to the threads that need them (rows 4t .. 4t + 3); the scaled activations of those four rows are split hi + lo (the
// bias term stays in fp32); then per byte j of the four words one A fragment and two MMAs per token tile.
template <int BITS, int NT, typename XT>
__device__ __forceinline__ void tile_math(const RowsK& p, const Walk<NT>& a, const TileRegs<NT, XRaw<XT>::W>& r, int stage,
                                          int fetch_ti, bool fetch_full, uint16_t* sbx, int lane, float (&acc)[NT][4][4],
                                          BiasAcc<NT, std::is_same<XT, __nv_bfloat16>::value>& ba) {
  constexpr float kMagic = BITS == 4 ? 128.f : 128.f * 17.f;
  const int t = lane & 3;
  sbx[lane] = (uint16_t)r.sb;
  cp_async_wait<kCodeStages - 2>();   // this lane's piece of the tile has landed ...
  __syncwarp();                       // ... and so has every other lane's
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[i]) : "r"(a.ring + (uint32_t)stage * kCodeTile + a.wsrc + 128u * i));
  const uint2 sraw = *(const uint2*)(sbx + 4 * t), braw = *(const uint2*)(sbx + 16 + 4 * t);
  // The stage read one tile ago is free now (every lane passed the __syncwarp above after reading it): refill it with
  // the tile kCodeStages - 1 ahead.  One group per tile, committed even when empty, keeps the wait count uniform.
  {
    const int fill = stage == 0 ? kCodeStages - 1 : stage - 1;
    if (fetch_full) fetch_codes_full<NT>(a, fetch_ti, fill);
    else if (fetch_ti >= 0) fetch_codes<NT>(p, a, fetch_ti, fill, lane);
    cp_async_commit();
  }
  uint32_t bh[NT][2], bl[NT][2];
  if constexpr (std::is_same<XT, __nv_bfloat16>::value) {
    // bf16 activations times bf16 scales: the product has 16 significant bits, hi = rn(x s) is one packed multiply
    // and lo = x s - hi (exact, then exactly representable) one packed fused multiply-add.  The bias term rides on
    // the tensor cores as well: sum_k (hi + lo) against an A operand of ones, sum_k x bias against an A operand
    // whose 16 rows all hold the biases -- both straight from the packed words as they were loaded.
    const uint32_t ones[4] = {0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u};
    const uint32_t brow[4] = {braw.x, braw.x, braw.y, braw.y};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      bh[nt][0] = mul_bf16x2(r.x[nt][0], sraw.x);
      bh[nt][1] = mul_bf16x2(r.x[nt][1], sraw.y);
      bl[nt][0] = fma_bf16x2(r.x[nt][0], sraw.x, bh[nt][0] ^ 0x80008000u);
      bl[nt][1] = fma_bf16x2(r.x[nt][1], sraw.y, bh[nt][1] ^ 0x80008000u);
      mma_bf16_16816(ba.s[nt], ones, bh[nt][0], bh[nt][1]);
      mma_bf16_16816(ba.s[nt], ones, bl[nt][0], bl[nt][1]);
      mma_bf16_16816(ba.b[nt], brow, r.x[nt][0], r.x[nt][1]);
    }
  } else {
    const float sc[4] = {bf16lo(sraw.x), bf16hi(sraw.x), bf16lo(sraw.y), bf16hi(sraw.y)};
    const float bi[4] = {bf16lo(braw.x), bf16hi(braw.x), bf16lo(braw.y), bf16hi(braw.y)};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float xv[4], v[4];
      XRaw<XT>::f32(r.x[nt], xv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[i] = xv[i] * sc[i];
        ba.b[nt] = fmaf(xv[i], fmaf(-kMagic, sc[i], bi[i]), ba.b[nt]);
      }
      bh[nt][0] = pack2(v[0], v[1]);
      bh[nt][1] = pack2(v[2], v[3]);
      bl[nt][0] = pack2(v[0] - bf16lo(bh[nt][0]), v[1] - bf16hi(bh[nt][0]));
      bl[nt][1] = pack2(v[2] - bf16lo(bh[nt][1]), v[3] - bf16hi(bh[nt][1]));
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t sel = (uint32_t)(j | (j << 4) | ((4 + j) << 8) | ((4 + j) << 12));
    const uint32_t u01 = __byte_perm(w[0], w[1], sel);   // byte j of rows 0 and 1 in bits 0-7 and 16-23
    const uint32_t u23 = __byte_perm(w[2], w[3], sel);
    uint32_t a[4];
    a[0] = lop3_and_or(u01, 0x000F000Fu, 0x43004300u);
    a[1] = lop3_and_or(u01 >> 4, 0x000F000Fu, 0x43004300u);
    a[2] = lop3_and_or(u23, 0x000F000Fu, 0x43004300u);
    a[3] = lop3_and_or(u23 >> 4, 0x000F000Fu, 0x43004300u);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      mma_bf16_16816(acc[nt][j], a, bh[nt][0], bh[nt][1]);
      mma_bf16_16816(acc[nt][j], a, bl[nt][0], bl[nt][1]);
    }
  }
}

template <int BITS, int NT, typename XT>
__global__ void __launch_bounds__(kThreads, NT == 1 ? 2 : 1) qmv_rows_kernel(RowsK p) {
  extern __shared__ __align__(16) float fin[];   // [8 * NT tokens][N + 1] partial sums of this CTA, then sbias, sbx, codes
  constexpr int VPW = 32 / BITS;
  constexpr int NL = 8 * VPW;                     // outputs of one column block
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int64_t bz = blockIdx.y;
  const int crank = p.ksplit > 1 ? (int)cluster_rank() : 0;
  const int pitch = p.N + 1;
  float* sbias = fin + (size_t)8 * NT * pitch;    // [warps][8 * NT]: per-token bias sums of a warp
  uint16_t* sbx = (uint16_t*)(sbias + kWarps * 8 * NT) + warp * 64;   // [warps][2][32]: scale / bias hand-over, two tiles
  unsigned char* codes = (unsigned char*)fin + code_ring_offset(NT, p.N);   // [warps][kCodeStages][512]: packed codes

  const int cb = warp % p.ncb, rsub = warp / p.ncb, rstep = kWarps / p.ncb;
  // the batch element's offsets into x, w, scales/biases and y: worked out by four threads, not by all of them
  __shared__ int64_t boff[4];
  if (tid < 4) boff[tid] = (tid == 0 ? p.xb : (tid == 1 ? p.wb : (tid == 2 ? p.sb : p.yb))).offset(bz);
  __syncthreads();
  Walk<NT> a;
  a.ldw16 = 16 * (int)p.ldw; a.lds16 = 16 * (int)p.lds;
  a.w = p.w + boff[1] + cb * 8 + (lane & 1) * 4 + (int64_t)(lane >> 1) * p.ldw;
  a.ring = (uint32_t)__cvta_generic_to_shared(codes + (size_t)warp * kCodeStages * kCodeTile);
  a.wdst = (uint32_t)(((((lane >> 1) & 3) * 4 + (lane >> 3)) * 32) + (lane & 1) * 16);
  a.wsrc = (uint32_t)(t * 32 + g * 4);
  a.sb = (lane < 16 ? p.s : p.b) + boff[2] + (cb >> p.sgshift) + (int64_t)(lane & 15) * p.lds;
  {
    const char* xb = (const char*)p.x + boff[0] * sizeof(XT);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      a.x[nt] = xb + ((int64_t)(nt * 8 + g < p.M ? nt * 8 + g : 0) * p.ldx + 4 * t) * sizeof(XT);
  }

  constexpr bool TCB = std::is_same<XT, __nv_bfloat16>::value;   // bias term on the tensor cores
  constexpr float kMagic = BITS == 4 ? 128.f : 128.f * 17.f;
  float acc[NT][4][4];
  BiasAcc<NT, TCB> bacc;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    if constexpr (TCB) {
#pragma unroll
      for (int e = 0; e < 4; ++e) bacc.s[nt][e] = bacc.b[nt][e] = 0.f;
    } else {
      bacc.b[nt] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[nt][j][e] = 0.f;
  }

  // This warp's tiles: i = 0 .. n - 1 at t0 + rsub + i * rstep.  The codes of tile i + kCodeStages - 1 and the scales,
  // biases and activations of tile i + kDepth - 1 are requested before tile i is computed.  While the tiles being
  // requested are full (all but the matrix's last one can be) the loop body has no data-dependent branch.
  const int t0 = crank * p.tiles_per_cta;
  const int t1 = min(p.tiles, t0 + p.tiles_per_cta);
  const int first = t0 + rsub;
  const int n = first < t1 ? (t1 - first + rstep - 1) / rstep : 0;
  const bool last_partial = n > 0 && (int64_t)(first + (n - 1) * rstep) * 16 + 16 > p.K;
  const int nfast = last_partial ? n - 1 : n;   // leading tiles the unpredicated loads may fetch
  TileRegs<NT, XRaw<XT>::W> ring[kDepth];
#pragma unroll 1
  for (int d = 0; d < kCodeStages - 1; ++d) {
    if (d < n) fetch_codes<NT>(p, a, first + d * rstep, d, lane);
    cp_async_commit();
  }
#pragma unroll
  for (int d = 0; d < kDepth - 1; ++d)
    if (d < n) load_any<NT, XT>(p, a, first + d * rstep, lane, ring[d]);
  int i = 0, stage = 0;
  for (; i + kDepth - 1 + kCodeStages - 1 < nfast; i += kDepth) {
#pragma unroll
    for (int u = 0; u < kDepth; ++u) {
      load_full<NT, XT>(a, first + (i + u + kDepth - 1) * rstep, p.x_vec != 0, ring[(u + kDepth - 1) % kDepth]);
      tile_math<BITS, NT, XT>(p, a, ring[u], stage, first + (i + u + kCodeStages - 1) * rstep, true, sbx + (u & 1) * 32, lane, acc, bacc);
      stage = stage == kCodeStages - 1 ? 0 : stage + 1;
    }
  }
  while (i < n) {
#pragma unroll
    for (int u = 0; u < kDepth; ++u) {
      if (i < n) {
        if (i + kDepth - 1 < nfast) load_full<NT, XT>(a, first + (i + kDepth - 1) * rstep, p.x_vec != 0, ring[(u + kDepth - 1) % kDepth]);
        else if (i + kDepth - 1 < n) load_any<NT, XT>(p, a, first + (i + kDepth - 1) * rstep, lane, ring[(u + kDepth - 1) % kDepth]);
        const int fj = i + kCodeStages - 1;
        tile_math<BITS, NT, XT>(p, a, ring[u], stage, fj < n ? first + fj * rstep : -1, false, sbx + (u & 1) * 32, lane, acc, bacc);
        stage = stage == kCodeStages - 1 ? 0 : stage + 1;
        ++i;
      }
    }
  }
  cp_async_wait<0>();

  // ---- the warp's bias sums: over the four threads of a token, then to the threads that hold the token's outputs ----
  if constexpr (!TCB) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float v = bacc.b[nt];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      if (t == 0) sbias[warp * 8 * NT + nt * 8 + g] = v;
    }
    __syncwarp();
  }
  // ---- the warps of one column block add their sums into the CTA's tile, one warp per round ----
  for (int r = 0; r < rstep; ++r) {
    if (rsub == r) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float b0, b1;   // bias sums of tokens 2t and 2t + 1 of this token tile
        if constexpr (TCB) {
          b0 = fmaf(-kMagic, bacc.s[nt][0], bacc.b[nt][0]);
          b1 = fmaf(-kMagic, bacc.s[nt][1], bacc.b[nt][1]);
        } else {
          b0 = sbias[warp * 8 * NT + nt * 8 + 2 * t];
          b1 = sbias[warp * 8 * NT + nt * 8 + 2 * t + 1];
        }
        float* row0 = fin + (size_t)(nt * 8 + 2 * t) * pitch + cb * NL;
        float* row1 = row0 + pitch;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float* d = acc[nt][j];
          if (BITS == 4) {
            const int n = 8 * g + 2 * j;
            const float v00 = d[0] + b0, v01 = d[2] + b0, v10 = d[1] + b1, v11 = d[3] + b1;
            if (r == 0) { row0[n] = v00; row0[n + 1] = v01; row1[n] = v10; row1[n + 1] = v11; }
            else { row0[n] += v00; row0[n + 1] += v01; row1[n] += v10; row1[n + 1] += v11; }
          } else {
            const int n = 4 * g + j;
            const float v0 = fmaf(16.f, d[2], d[0]) + b0, v1 = fmaf(16.f, d[3], d[1]) + b1;
            if (r == 0) { row0[n] = v0; row1[n] = v1; }
            else { row0[n] += v0; row1[n] += v1; }
          }
        }
      }
    }
    __syncthreads();
  }
  // ---- across the cluster: rank 0 adds the other ranks' tiles in rank order and stores ----
  if (p.ksplit > 1) cluster_sync_all();
  if (crank == 0) {
    char* yb = (char*)p.y + boff[3] * sizeof(XT);
    const uint32_t fin_s = (uint32_t)__cvta_generic_to_shared(fin);
    for (int idx = tid; idx < p.M * p.N; idx += kThreads) {
      const int m = idx / p.N, n = idx - m * p.N;
      const int off = m * pitch + n;
      float v = fin[off];
      for (int r = 1; r < p.ksplit; ++r) v += ld_cluster_f32(map_to_rank(fin_s + 4u * (uint32_t)off, (uint32_t)r));
      IO<XT>::store(yb, (int64_t)m * p.ldy + n, v);
    }
  }
  if (p.ksplit > 1) cluster_sync_all();   // the other ranks' shared memory stays alive until rank 0 has read it
}

size_t smem_bytes(int nt, int N) { return code_ring_offset(nt, N) + (size_t)kWarps * kCodeStages * kCodeTile; }

template <int BITS, int NT, typename XT>
cudaError_t launch_inst(const RowsK& p, int64_t nbatch, cudaStream_t st) {
  {
    std::lock_guard<std::mutex> lk(setup_mutex());
    static bool done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !done[dev]) {
      const cudaError_t e = cudaFuncSetAttribute(qmv_rows_kernel<BITS, NT, XT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)p.ksplit, (unsigned)nbatch, 1);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem_bytes(NT, p.N);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)p.ksplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.ksplit > 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, qmv_rows_kernel<BITS, NT, XT>, p);
}

template <int BITS, typename XT>
cudaError_t launch_x(const RowsK& p, int64_t nbatch, cudaStream_t st) {
  const int nt = (p.M + 7) / 8;
  if (nt == 1) return launch_inst<BITS, 1, XT>(p, nbatch, st);
  if (nt == 2) return launch_inst<BITS, 2, XT>(p, nbatch, st);
  return launch_inst<BITS, 4, XT>(p, nbatch, st);
}

template <int BITS>
cudaError_t launch_bits(const RowsK& p, int x_dtype, int64_t nbatch, cudaStream_t st) {
  switch (x_dtype) {
    case QB200_BFLOAT16: return launch_x<BITS, __nv_bfloat16>(p, nbatch, st);
    case QB200_FLOAT32: return launch_x<BITS, float>(p, nbatch, st);
    case QB200_FLOAT16: return launch_x<BITS, __half>(p, nbatch, st);
    default: return cudaErrorInvalidValue;
  }
}

bool multiple_of_4(const BatchMap& m) {
  for (int d = 0; d < m.nd; ++d)
    if (m.stride[d] % 4) return false;
  return true;
}

}  // namespace

bool qmv_rows_supported(const QmmArgs& a) {
  if (a.transpose || (a.bits != 4 && a.bits != 8)) return false;
  if (a.M < 1 || a.M > 8 * kMaxTokTiles || a.K < 1 || a.K > (int64_t)1 << 30 || a.nbatch < 1 || a.nbatch > 65535) return false;
  if (a.ldw >= (1 << 26) || a.lds >= (1 << 26)) return false;   // 16 rows of either as a 32-bit element count
  if ((uintptr_t)a.w % 16 || a.ldw % 4 || !multiple_of_4(a.wb)) return false;   // 16-byte pieces of a row by cp.async
  const int vpw = 32 / a.bits, nl = 8 * vpw;
  if (a.N % nl || a.gs % nl) return false;               // a column block of 8 words lies inside one scale group
  const int64_t ncb = a.N / nl;
  if (ncb != 1 && ncb != 2 && ncb != 4 && ncb != 8) return false;
  const int nt = a.M <= 8 ? 1 : (a.M <= 16 ? 2 : 4);
  return smem_bytes(nt, (int)a.N) <= (size_t)kSmemLimit;
}

cudaError_t launch_qmv_rows(const QmmArgs& a, cudaStream_t st) {
  if (!qmv_rows_supported(a)) return cudaErrorInvalidValue;
  RowsK p;
  p.x = a.x; p.w = a.w; p.s = (const uint16_t*)a.s; p.b = (const uint16_t*)a.b; p.y = a.y;
  p.M = (int)a.M; p.N = (int)a.N; p.K = a.K;
  p.ldx = a.ldx; p.ldw = a.ldw; p.lds = a.lds; p.ldy = a.ldy;
  const int nl = 8 * (32 / a.bits);
  p.ncb = (int)(a.N / nl);
  p.sgshift = 0;
  while ((nl << p.sgshift) < a.gs) ++p.sgshift;
  p.tiles = (int)((a.K + 15) / 16);
  // K over the CTAs of a cluster: as many CTAs as fit the GPU at once (three per SM at up to 8 tokens; a second wave
  // would pay the pipeline fill and the reduction again), as long as every warp keeps four tiles
  const int rstep = kWarps / p.ncb;
  const int per_sm = a.M <= 8 ? 2 : 1;
  int64_t ks = (int64_t)per_sm * sm_count() / a.nbatch;
  if (ks > 8) ks = 8;
  while (ks > 1 && p.tiles / ks < 4 * rstep) --ks;
  if (ks < 1) ks = 1;
  p.ksplit = (int)ks;
  p.tiles_per_cta = (p.tiles + ks - 1) / ks;
  const int xa = a.x_dtype == QB200_FLOAT32 ? 16 : 8;
  p.x_vec = ((uintptr_t)a.x % xa == 0) && a.ldx % 4 == 0 && multiple_of_4(a.xb);
  p.xb = a.xb; p.wb = a.wb; p.sb = a.sb; p.yb = a.yb;
  return a.bits == 4 ? launch_bits<4>(p, a.x_dtype, a.nbatch, st) : launch_bits<8>(p, a.x_dtype, a.nbatch, st);
}

}  // namespace qb

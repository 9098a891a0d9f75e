// Batched quantized matmul with a short contraction and many weight rows, at attention widths:
//   y[b, m, n] = sum_k x[b, m, k] * (s[b, n, G(k)] * q[b, n, k] + bias[b, n, G(k)]),   m <= 32, K = 64 / 128 / 256,
// W [N, K] quantised along K in groups of 64, N long, one W per batch element.
//
// Replaces mlx_quantized_matmul(transpose=true) as quantAttention calls it for q @ K^T
// (mlx-serve src/kv_quant.zig:528-533; pinned by the reference test at :968-1036): x is the query
// block [B, Hkv, g*Tq, D], W the packed key cache [B, Hkv, T, D*bits/32], so the contraction is one
// head dimension, N = T is the cache length and the batch B*Hkv is large.  One pass over the packed
// cache, nothing shared between the rows: every warp owns 16-row tiles of one batch element, no
// reduction across warps or CTAs.
//
//  * Tensor cores with the roles swapped: the codes are the 16-row A operand of
//    mma.sync.m16n8k16 (bf16, fp32 accumulate), the activations the 8-column B operand.  A packed
//    word holds 8 (4-bit) or 4 (8-bit) consecutive k of one row, and the position of a k inside the
//    64-wide group is free as long as B follows; so a register of A is simply
//    (word >> 4 i) & 0x000F000F -- nibbles i and i + 4 side by side -- OR-ed into the mantissa of
//    two bf16 128.0: one shift and one LOP3 per two codes, no byte permutation.  The activations are
//    arranged once per CTA into the matching B fragments and stay in registers.
//  * An 8-bit code is its two nibbles on two accumulators (the high one counts 16-fold).
//  * Per 64-wide group the accumulator holds sum (128 + q) x; the group's scale and bias are applied
//    in fp32:  y += s * acc + (bias - C s) * sum_k x  with C = 128 (4-bit) or 128 * 17.  The weight
//    term q s + bias is never rounded.
//  * Activations that are not bf16 are split into two bf16 values, hi + lo, and every MMA is issued
//    for both (16 significant bits of x).
//  * Codes, scales and biases travel by cp.async into a ring of shared-memory stages private to the
//    warp; a warp only ever waits on its own copies (cp.async.wait_group + __syncwarp).
#include <type_traits>

#include "kernels.h"
#include "stream_ptx.cuh"

namespace qb {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;          // tiles per warp in the ring (three in flight)
constexpr int kRowPad = 32;         // bytes added to a row of codes in a stage: fragment reads of rows g, g + 1, .. miss each other's banks

struct ShortK {
  const void* x; const uint32_t* w; const uint16_t* s; const uint16_t* b; void* y;
  int M, K;
  int64_t N;
  int64_t ldx, ldw, lds, ldy;    // row pitches in elements
  int tiles;                     // 16-row tiles of N
  int tiles_per_cta;
  int sb_vec;                    // a batch element's scales and biases start on 4 bytes
  BatchMap xb, wb, sb, yb;
};

template <int BITS, int NG> struct Geo {
  static constexpr int kRowBytes = NG * 64 * BITS / 8;              // packed codes of one row
  static constexpr int kPitch = kRowBytes + kRowPad;                // a row in a stage
  static constexpr int kCodeBytes = 16 * kPitch;
  static constexpr int kSbRow = NG * 2;                             // bytes of a row's scales (= of its biases)
  static constexpr int kSbBytes = 2 * 16 * kSbRow;                  // scales of 16 rows, then their biases
  static constexpr int kStageBytes = (kCodeBytes + kSbBytes + 15) / 16 * 16;
  static constexpr int kCodePieces = 16 * kRowBytes / 16;           // 16-byte pieces of a tile's codes
  static constexpr int kSbWords = 16 * kSbRow / 4;                  // 4-byte pieces of a tile's scales (= biases)
  static constexpr int kWordsPerThread = BITS == 4 ? 2 : 4;         // packed words of one row and group a thread expands
};

__device__ __forceinline__ void cp_async16_if(uint32_t dst, const void* src, bool in) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(in ? 16 : 0));
}
__device__ __forceinline__ uint2 lds_u2(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds_u4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// The k (inside its 64-wide group) that slot `e` (0..3: a0.lo, a0.hi, a2.lo, a2.hi) of MMA `mm` of the group takes
// from thread t.  4 bits: word 2t + mm / 2 of the group, nibbles (2p, 2p + 4) and (2p + 1, 2p + 5) with p = mm % 2.
// 8 bits: word 4t + mm, bytes (0, 2) and (1, 3).
template <int BITS>
__device__ __forceinline__ int k_of_slot(int t, int mm, int e) {
  if (BITS == 4) {
    const int word = 2 * t + (mm >> 1), p = mm & 1;
    return 8 * word + 2 * p + (e >> 1) + 4 * (e & 1);
  }
  return 4 * (4 * t + mm) + (e >> 1) + 2 * (e & 1);
}

// The codes, scales and biases of 16-row tile `tile` of the batch element into stage `stage` of the warp's ring.
template <int BITS, int NG>
__device__ __forceinline__ void fetch_tile(const ShortK& p, const uint32_t* wbase, const uint16_t* sbase, const uint16_t* bbase,
                                           uint32_t ring, int tile, int stage, int lane) {
  using G = Geo<BITS, NG>;
      const int64_t n0 = (int64_t)tile * 16;
      const uint32_t dst = ring + (uint32_t)stage * G::kStageBytes;
  #pragma unroll
      for (int c = 0; c < (G::kCodePieces + 31) / 32; ++c) {
        const int piece = lane + 32 * c;
        if (G::kCodePieces % 32 == 0 || piece < G::kCodePieces) {
          const int row = piece / (G::kRowBytes / 16), col = piece % (G::kRowBytes / 16);
          const bool in = n0 + row < p.N;
          cp_async16_if(dst + row * G::kPitch + col * 16, in ? (const void*)(wbase + (n0 + row) * p.ldw + col * 4) : (const void*)p.w, in);
        }
      }
      // scales of the 16 rows, then their biases: the rows are contiguous (lds == NG), 32 * NG bytes each way, copied as
      // 4-byte pieces (a batch element's scales start on 4 bytes whenever its row count times NG is even)
      if (n0 + 16 <= p.N && p.sb_vec) {
  #pragma unroll
        for (int c = 0; c < (2 * G::kSbWords + 31) / 32; ++c) {
          const int piece = lane + 32 * c;
          if ((2 * G::kSbWords) % 32 == 0 || piece < 2 * G::kSbWords) {
            const int which = piece / G::kSbWords, word = piece % G::kSbWords;
            cp_async4(dst + G::kCodeBytes + which * 16 * G::kSbRow + word * 4, (which ? bbase : sbase) + n0 * NG + word * 2);
          }
        }
      } else {
        // the matrix's last, partial tile (or scales that start on an odd element): entry by entry, so that nothing
        // behind the last row is read; the plain stores are ordered before the reads of this stage by the __syncwarp
        // that precedes them
        for (int idx = lane; idx < 2 * 16 * NG; idx += 32) {
          const int which = idx / (16 * NG), r = (idx % (16 * NG)) / NG;
          const uint16_t v = n0 + r < p.N ? (which ? bbase : sbase)[n0 * NG + idx % (16 * NG)] : (uint16_t)0;
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(dst + G::kCodeBytes + which * 16 * G::kSbRow + (idx % (16 * NG)) * 2), "h"(v) : "memory");
        }
      }
}

template <int BITS, int NG, int NT, typename XT>
__global__ void __launch_bounds__(kThreads, NT == 1 ? 2 : 1) qmv_shortk_kernel(ShortK p) {
  using G = Geo<BITS, NG>;
  constexpr bool SPLIT = !std::is_same<XT, __nv_bfloat16>::value;   // activations as hi + lo
  constexpr int NP = SPLIT ? 2 : 1;
  constexpr float kMagic = BITS == 4 ? 128.f : 128.f * 17.f;
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int64_t bz = blockIdx.y;
  __shared__ int64_t boff[4];
  if (tid < 4) boff[tid] = (tid == 0 ? p.xb : (tid == 1 ? p.wb : (tid == 2 ? p.sb : p.yb))).offset(bz);
  __syncthreads();
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + (uint32_t)warp * kStages * G::kStageBytes;

  // ---- what this lane copies for every tile ----
  const uint32_t* wbase = p.w + boff[1];
  const uint16_t* sbase = p.s + boff[2];
  const uint16_t* bbase = p.b + boff[2];
  auto fetch = [&](int tile, int stage) { fetch_tile<BITS, NG>(p, wbase, sbase, bbase, ring, tile, stage, lane); };

  const int t0 = blockIdx.x * p.tiles_per_cta;
  const int t1 = min(p.tiles, t0 + p.tiles_per_cta);
  const int first = t0 + warp;
  const int n = first < t1 ? (t1 - first + kWarps - 1) / kWarps : 0;
#pragma unroll 1
  for (int d = 0; d < kStages - 1; ++d) {
    if (d < n) fetch(first + d * kWarps, d);
    cp_async_commit();
  }
  // ---- the activations of token g in B-fragment order and the per-group sums of tokens 2t and 2t + 1: the same
  // for every warp, so warp 0 builds them (while the others' first tiles are already on their way) and hands them
  // over through shared memory ----
  constexpr int kFragWords = NP * NG * 8 + NG * 2;   // per token tile
  __shared__ uint32_t xs[NT * kFragWords][32];
  uint32_t bf[NT][NP][NG][4][2];
  float sx[NT][NG][2];
  if (warp == 0) {
    const char* xb = (const char*)p.x + boff[0] * sizeof(XT);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int tok = nt * 8 + g < p.M ? nt * 8 + g : 0;   // a token beyond M repeats token 0: its results are never stored
#pragma unroll
      for (int gi = 0; gi < NG; ++gi) {
        float part = 0.f;
#pragma unroll
        for (int mm = 0; mm < 4; ++mm) {
          float v[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) v[e] = IO<XT>::load(xb, (int64_t)tok * p.ldx + 64 * gi + k_of_slot<BITS>(t, mm, e));
          part += (v[0] + v[1]) + (v[2] + v[3]);
          const uint32_t h0 = pack2(v[0], v[1]), h1 = pack2(v[2], v[3]);
          xs[nt * kFragWords + (gi * 4 + mm) * 2 + 0][lane] = h0;
          xs[nt * kFragWords + (gi * 4 + mm) * 2 + 1][lane] = h1;
          if constexpr (SPLIT) {
            xs[nt * kFragWords + NG * 8 + (gi * 4 + mm) * 2 + 0][lane] = pack2(v[0] - bf16lo(h0), v[1] - bf16hi(h0));
            xs[nt * kFragWords + NG * 8 + (gi * 4 + mm) * 2 + 1][lane] = pack2(v[2] - bf16lo(h1), v[3] - bf16hi(h1));
          }
        }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);            // token nt * 8 + g, the whole group
        xs[nt * kFragWords + NP * NG * 8 + gi * 2 + 0][lane] = __float_as_uint(__shfl_sync(0xffffffffu, part, (2 * t) * 4));   // this thread's accumulator columns
        xs[nt * kFragWords + NP * NG * 8 + gi * 2 + 1][lane] = __float_as_uint(__shfl_sync(0xffffffffu, part, (2 * t + 1) * 4));
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int pl = 0; pl < NP; ++pl)
#pragma unroll
      for (int gi = 0; gi < NG; ++gi)
#pragma unroll
        for (int mm = 0; mm < 4; ++mm) {
          bf[nt][pl][gi][mm][0] = xs[nt * kFragWords + pl * NG * 8 + (gi * 4 + mm) * 2 + 0][lane];
          bf[nt][pl][gi][mm][1] = xs[nt * kFragWords + pl * NG * 8 + (gi * 4 + mm) * 2 + 1][lane];
        }
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
      sx[nt][gi][0] = __uint_as_float(xs[nt * kFragWords + NP * NG * 8 + gi * 2 + 0][lane]);
      sx[nt][gi][1] = __uint_as_float(xs[nt * kFragWords + NP * NG * 8 + gi * 2 + 1][lane]);
    }
  }

  char* yb = (char*)p.y + boff[3] * sizeof(XT);
  int stage = 0;
#pragma unroll 1
  for (int i = 0; i < n; ++i) {
    cp_async_wait<kStages - 2>();   // this lane's pieces of tile i have landed ...
    __syncwarp();                   // ... and so have every other lane's; every lane is done with the stage read last
    if (i + kStages - 1 < n) fetch(first + (i + kStages - 1) * kWarps, stage == 0 ? kStages - 1 : stage - 1);
    cp_async_commit();
    const uint32_t st = ring + (uint32_t)stage * G::kStageBytes;
    float y[NT][4];   // per token tile: rows g, g (tokens 2t, 2t + 1), rows g + 8, g + 8
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) y[nt][e] = 0.f;
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
      // packed words of rows g and g + 8 in this group: words 2t, 2t + 1 (4-bit) or 4t .. 4t + 3 (8-bit)
      uint32_t wq[2][G::kWordsPerThread];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t at = st + (uint32_t)(g + 8 * h) * G::kPitch + gi * (64 * BITS / 8) + t * (4 * G::kWordsPerThread);
        if (BITS == 4) {
          const uint2 q = lds_u2(at);
          wq[h][0] = q.x; wq[h][1] = q.y;
        } else {
          const uint4 q = lds_u4(at);
          wq[h][0] = q.x; wq[h][1] = q.y; wq[h][2] = q.z; wq[h][3] = q.w;
        }
      }
      float d0[NT][4], d1[NT][4];   // low nibbles (all of a 4-bit code) / high nibbles
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) d0[nt][e] = d1[nt][e] = 0.f;
#pragma unroll
      for (int mm = 0; mm < 4; ++mm) {
        uint32_t a[4], ah[4];
        if (BITS == 4) {
          const int wd = mm >> 1, sh = 8 * (mm & 1);   // nibbles (2p, 2p + 4) and (2p + 1, 2p + 5): shifts 8p and 8p + 4
          a[0] = lop3_and_or(wq[0][wd] >> sh, 0x000F000Fu, 0x43004300u);
          a[1] = lop3_and_or(wq[1][wd] >> sh, 0x000F000Fu, 0x43004300u);
          a[2] = lop3_and_or(wq[0][wd] >> (sh + 4), 0x000F000Fu, 0x43004300u);
          a[3] = lop3_and_or(wq[1][wd] >> (sh + 4), 0x000F000Fu, 0x43004300u);
        } else {
          a[0] = lop3_and_or(wq[0][mm], 0x000F000Fu, 0x43004300u);          // bytes 0 and 2, low nibbles
          a[1] = lop3_and_or(wq[1][mm], 0x000F000Fu, 0x43004300u);
          a[2] = lop3_and_or(wq[0][mm] >> 8, 0x000F000Fu, 0x43004300u);     // bytes 1 and 3
          a[3] = lop3_and_or(wq[1][mm] >> 8, 0x000F000Fu, 0x43004300u);
          ah[0] = lop3_and_or(wq[0][mm] >> 4, 0x000F000Fu, 0x43004300u);    // the high nibbles
          ah[1] = lop3_and_or(wq[1][mm] >> 4, 0x000F000Fu, 0x43004300u);
          ah[2] = lop3_and_or(wq[0][mm] >> 12, 0x000F000Fu, 0x43004300u);
          ah[3] = lop3_and_or(wq[1][mm] >> 12, 0x000F000Fu, 0x43004300u);
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int pl = 0; pl < NP; ++pl) {
            mma_bf16_16816(d0[nt], a, bf[nt][pl][gi][mm][0], bf[nt][pl][gi][mm][1]);
            if (BITS == 8) mma_bf16_16816(d1[nt], ah, bf[nt][pl][gi][mm][0], bf[nt][pl][gi][mm][1]);
          }
      }
      // the group's scale and bias of rows g and g + 8
      const uint32_t sat = st + G::kCodeBytes + 2 * gi;
      float sc[2], bi[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint16_t sv, bv;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sv) : "r"(sat + (uint32_t)(g + 8 * h) * G::kSbRow));
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(bv) : "r"(sat + 16 * G::kSbRow + (uint32_t)(g + 8 * h) * G::kSbRow));
        sc[h] = bf16_bits_to_f32(sv);
        bi[h] = fmaf(-kMagic, sc[h], bf16_bits_to_f32(bv));
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1, col = e & 1;
          const float acc = BITS == 4 ? d0[nt][e] : fmaf(16.f, d1[nt][e], d0[nt][e]);
          y[nt][e] = fmaf(sc[h], acc, fmaf(bi[h], sx[nt][gi][col], y[nt][e]));
        }
    }
    const int64_t n0 = (int64_t)(first + i * kWarps) * 16;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t nn = n0 + g + 8 * (e >> 1);
        const int m = nt * 8 + 2 * t + (e & 1);
        if (nn < p.N && m < p.M) IO<XT>::store(yb, (int64_t)m * p.ldy + nn, y[nt][e]);
      }
    stage = stage == kStages - 1 ? 0 : stage + 1;
  }
  cp_async_wait<0>();
}

// ---- up to 8 rows: integer tensor cores ----
// The same kernel with the codes as the u8 A operand of mma.sync.m16n8k32 (s32 accumulate): a packed word is the
// thread's eight k of one MMA as it stands -- 4 bits: its even nibbles (word & 0x0F0F0F0F) and its odd ones; 8 bits: two
// words untouched -- and the activations are 15-bit fixed point, v = rn(x 2^(14 - e)) with one power-of-two scale per
// (token, 64-wide group), split into a signed high and a 7-bit low plane that sit in two columns of the n8 tile (four
// tokens per tile).  sum_k q v is exact in s32; per group  y += (s 2^(e - 14)) (128 d_hi + d_lo) + bias 2^(e - 14) sum v.
// A NaN or an Inf in a group makes its scale NaN, so the row's outputs come out non-finite.
template <int BITS, int NG, int NT, typename XT>
__global__ void __launch_bounds__(kThreads, 2) qmv_shortk_i8_kernel(ShortK p) {
  using G = Geo<BITS, NG>;
  extern __shared__ __align__(16) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int64_t bz = blockIdx.y;
  __shared__ int64_t boff[4];
  if (tid < 4) boff[tid] = (tid == 0 ? p.xb : (tid == 1 ? p.wb : (tid == 2 ? p.sb : p.yb))).offset(bz);
  __syncthreads();
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + (uint32_t)warp * kStages * G::kStageBytes;
  const uint32_t* wbase = p.w + boff[1];
  const uint16_t* sbase = p.s + boff[2];
  const uint16_t* bbase = p.b + boff[2];
  auto fetch = [&](int tile, int stage) { fetch_tile<BITS, NG>(p, wbase, sbase, bbase, ring, tile, stage, lane); };

  const int t0 = blockIdx.x * p.tiles_per_cta;
  const int t1 = min(p.tiles, t0 + p.tiles_per_cta);
  const int first = t0 + warp;
  const int n = first < t1 ? (t1 - first + kWarps - 1) / kWarps : 0;
#pragma unroll 1
  for (int d = 0; d < kStages - 1; ++d) {
    if (d < n) fetch(first + d * kWarps, d);
    cp_async_commit();
  }

  // ---- the activations as B fragments, built by warp 0 and handed over through shared memory.  Lane (g, t) of a
  // token tile holds plane g % 2 of token g / 2 at the eight k of its word: 64 gi + 8 (2t + mm) + (4 bits: even k in
  // b0, odd in b1; 8 bits: k + 0..3 in b0, k + 4..7 in b1) ----
  constexpr int kFragWords = NG * 4 + NG * 2;   // per token tile: [gi][mm][2] fragments, then (scale, scale * sum v) by token
  __shared__ uint32_t xs[NT * kFragWords][32];
  {
    const char* xb = (const char*)p.x + boff[0] * sizeof(XT);
    // 16 consecutive k of a token row as two 16-byte loads where the rows allow it (16-bit activations)
    const bool vec = sizeof(XT) == 2 && (((uintptr_t)xb | (uintptr_t)(p.ldx * 2)) & 15) == 0;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int tk = nt * 4 + (g >> 1);
      const int tok = tk < p.M ? tk : 0;   // a token beyond M repeats token 0: its results are never stored
#pragma unroll
      for (int gi = 0; gi < NG; ++gi) {
        if (warp != (nt * NG + gi) % kWarps) continue;   // one warp per (token tile, group): they work side by side
        float f[2][8];
        float mx = 0.f;
        float lin[16];   // x[tok][64 gi + 16 t + 0..15]
        if (vec) {
          const uint4* src = (const uint4*)(xb + ((int64_t)tok * p.ldx + 64 * gi + 16 * t) * 2);
          const uint4 q0 = src[0], q1 = src[1];
          const uint32_t wds[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (std::is_same<XT, __half>::value) {
              const float2 h2 = __half22float2(*(const __half2*)&wds[j]);
              lin[2 * j] = h2.x; lin[2 * j + 1] = h2.y;
            } else {
              lin[2 * j] = bf16lo(wds[j]); lin[2 * j + 1] = bf16hi(wds[j]);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) lin[j] = IO<XT>::load(xb, (int64_t)tok * p.ldx + 64 * gi + 16 * t + j);
        }
#pragma unroll
        for (int mm = 0; mm < 2; ++mm)
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            f[mm][j] = lin[8 * mm + (BITS == 4 ? 2 * (j & 3) + (j >> 2) : j)];
            mx = fmax_nan(mx, fabsf(f[mm][j]));
          }
        mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        int e = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 + 1;   // mx < 2^e
        e = e < -100 ? -100 : (e > 110 ? 110 : e);
        const float up = __uint_as_float((uint32_t)(127 + 14 - e) << 23);
        const float down = poison_if(nonfinite(mx), __uint_as_float((uint32_t)(127 + e - 14) << 23));
        int isum = 0;
#pragma unroll
        for (int mm = 0; mm < 2; ++mm) {
          uint32_t reg[2] = {0u, 0u};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float r = fmaf(f[mm][j], up, 12582912.f);   // 1.5 * 2^23 + v: the low 16 bits are v in two's complement
            if (sizeof(XT) == 4) r = fminf(r, 12599295.f);   // fp32 inputs may round up to 2^14: v <= 16383
            const int v = (int)(int16_t)(__float_as_uint(r) & 0xFFFFu);
            isum += v;
            const uint32_t byte = (g & 1) ? (uint32_t)(v & 127) : (uint32_t)((v >> 7) & 0xFF);
            reg[j >> 2] |= byte << (8 * (j & 3));
          }
          xs[nt * kFragWords + (gi * 2 + mm) * 2 + 0][lane] = reg[0];
          xs[nt * kFragWords + (gi * 2 + mm) * 2 + 1][lane] = reg[1];
        }
        isum += __shfl_xor_sync(0xffffffffu, isum, 1);
        isum += __shfl_xor_sync(0xffffffffu, isum, 2);
        if ((g & 1) == 0 && t == 0) {   // one lane per token: the scale and scale * sum v, read back by token index
          xs[nt * kFragWords + NG * 4 + gi * 2 + 0][g >> 1] = __float_as_uint(down);
          xs[nt * kFragWords + NG * 4 + gi * 2 + 1][g >> 1] = __float_as_uint(down * (float)isum);
        }
      }
    }
  }
  __syncthreads();
  uint32_t bfr[NT][NG][2][2];
  float dn[NT][NG], ds[NT][NG];   // of token nt * 4 + t: this thread's accumulator columns
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
#pragma unroll
      for (int mm = 0; mm < 2; ++mm) {
        bfr[nt][gi][mm][0] = xs[nt * kFragWords + (gi * 2 + mm) * 2 + 0][lane];
        bfr[nt][gi][mm][1] = xs[nt * kFragWords + (gi * 2 + mm) * 2 + 1][lane];
      }
      dn[nt][gi] = __uint_as_float(xs[nt * kFragWords + NG * 4 + gi * 2 + 0][t]);
      ds[nt][gi] = __uint_as_float(xs[nt * kFragWords + NG * 4 + gi * 2 + 1][t]);
    }

  char* yb = (char*)p.y + boff[3] * sizeof(XT);
  int stage = 0;
#pragma unroll 1
  for (int i = 0; i < n; ++i) {
    cp_async_wait<kStages - 2>();   // this lane's pieces of tile i have landed ...
    __syncwarp();                   // ... and so have every other lane's; every lane is done with the stage read last
    if (i + kStages - 1 < n) fetch(first + (i + kStages - 1) * kWarps, stage == 0 ? kStages - 1 : stage - 1);
    cp_async_commit();
    const uint32_t st = ring + (uint32_t)stage * G::kStageBytes;
    float y[NT][2];   // rows g and g + 8 of token nt * 4 + t
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) y[nt][0] = y[nt][1] = 0.f;
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
      uint32_t wq[2][G::kWordsPerThread];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t at = st + (uint32_t)(g + 8 * h) * G::kPitch + gi * (64 * BITS / 8) + t * (4 * G::kWordsPerThread);
        if (BITS == 4) {
          const uint2 q = lds_u2(at);
          wq[h][0] = q.x; wq[h][1] = q.y;
        } else {
          const uint4 q = lds_u4(at);
          wq[h][0] = q.x; wq[h][1] = q.y; wq[h][2] = q.z; wq[h][3] = q.w;
        }
      }
      int d[NT][4];
#pragma unroll
      for (int mm = 0; mm < 2; ++mm) {
        uint32_t a0, a1, a2, a3;
        if (BITS == 4) {
          a0 = wq[0][mm] & 0x0F0F0F0Fu; a2 = (wq[0][mm] >> 4) & 0x0F0F0F0Fu;
          a1 = wq[1][mm] & 0x0F0F0F0Fu; a3 = (wq[1][mm] >> 4) & 0x0F0F0F0Fu;
        } else {
          a0 = wq[0][2 * mm]; a2 = wq[0][2 * mm + 1];
          a1 = wq[1][2 * mm]; a3 = wq[1][2 * mm + 1];
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          if (mm == 0) mma_u8s8_z(d[nt], a0, a1, a2, a3, bfr[nt][gi][0][0], bfr[nt][gi][0][1]);
          else mma_u8s8(d[nt], a0, a1, a2, a3, bfr[nt][gi][1][0], bfr[nt][gi][1][1]);
        }
      }
      const uint32_t sat = st + G::kCodeBytes + 2 * gi;
      float sc[2], bi[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint16_t sv, bv;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sv) : "r"(sat + (uint32_t)(g + 8 * h) * G::kSbRow));
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(bv) : "r"(sat + 16 * G::kSbRow + (uint32_t)(g + 8 * h) * G::kSbRow));
        sc[h] = bf16_bits_to_f32(sv);
        bi[h] = bf16_bits_to_f32(bv);
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int v = 128 * d[nt][2 * h] + d[nt][2 * h + 1];   // columns 2t, 2t + 1: the two planes of token t
          y[nt][h] = fmaf(sc[h] * dn[nt][gi], (float)v, fmaf(bi[h], ds[nt][gi], y[nt][h]));
        }
    }
    const int64_t n0 = (int64_t)(first + i * kWarps) * 16;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t nn = n0 + g + 8 * h;
        const int m = nt * 4 + t;
        if (nn < p.N && m < p.M) IO<XT>::store(yb, (int64_t)m * p.ldy + nn, y[nt][h]);
      }
    stage = stage == kStages - 1 ? 0 : stage + 1;
  }
  cp_async_wait<0>();
}

template <int BITS, int NG, int NT, typename XT>
cudaError_t launch_i8_inst(const ShortK& p, int ctas_per_batch, int64_t nbatch, cudaStream_t st) {
  using G = Geo<BITS, NG>;
  const size_t smem = (size_t)kWarps * kStages * G::kStageBytes;
  {
    std::lock_guard<std::mutex> lk(setup_mutex());
    static bool done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !done[dev]) {
      const cudaError_t e = cudaFuncSetAttribute(qmv_shortk_i8_kernel<BITS, NG, NT, XT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  return launch_kernel(qmv_shortk_i8_kernel<BITS, NG, NT, XT>, dim3((unsigned)ctas_per_batch, (unsigned)nbatch, 1), dim3(kThreads), smem, st, p);
}

template <int BITS, int NG, int NT, typename XT>
cudaError_t launch_inst(const ShortK& p, int ctas_per_batch, int64_t nbatch, cudaStream_t st) {
  using G = Geo<BITS, NG>;
  const size_t smem = (size_t)kWarps * kStages * G::kStageBytes;
  {
    std::lock_guard<std::mutex> lk(setup_mutex());
    static bool done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !done[dev]) {
      const cudaError_t e = cudaFuncSetAttribute(qmv_shortk_kernel<BITS, NG, NT, XT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  return launch_kernel(qmv_shortk_kernel<BITS, NG, NT, XT>, dim3((unsigned)ctas_per_batch, (unsigned)nbatch, 1), dim3(kThreads), smem, st, p);
}

// Token tiles of 8: fragments of all of them stay in registers, so their number is limited by NT * groups * (2 when the
// activations are split) <= 8 (64 registers of fragments).
constexpr bool inst_ok(int ng, int nt, bool split) { return nt * ng * (split ? 2 : 1) <= 8; }

template <int BITS, int NG, typename XT>
cudaError_t launch_nt(const ShortK& p, int ctas, int64_t nbatch, cudaStream_t st) {
  constexpr bool SPLIT = !std::is_same<XT, __nv_bfloat16>::value;
  if (p.M <= 4) return launch_i8_inst<BITS, NG, 1, XT>(p, ctas, nbatch, st);   // up to 8 rows: the integer tensor-core form
  if (p.M <= 8) return launch_i8_inst<BITS, NG, 2, XT>(p, ctas, nbatch, st);
  const int nt = (p.M + 7) / 8;
  if (nt == 1) return launch_inst<BITS, NG, 1, XT>(p, ctas, nbatch, st);
  if constexpr (inst_ok(NG, 2, SPLIT)) {
    if (nt == 2) return launch_inst<BITS, NG, 2, XT>(p, ctas, nbatch, st);
  }
  if constexpr (inst_ok(NG, 4, SPLIT)) {
    if (nt <= 4) return launch_inst<BITS, NG, 4, XT>(p, ctas, nbatch, st);
  }
  return cudaErrorInvalidValue;
}

template <int BITS, int NG>
cudaError_t launch_x(const ShortK& p, int x_dtype, int ctas, int64_t nbatch, cudaStream_t st) {
  switch (x_dtype) {
    case QB200_BFLOAT16: return launch_nt<BITS, NG, __nv_bfloat16>(p, ctas, nbatch, st);
    case QB200_FLOAT32: return launch_nt<BITS, NG, float>(p, ctas, nbatch, st);
    case QB200_FLOAT16: return launch_nt<BITS, NG, __half>(p, ctas, nbatch, st);
    default: return cudaErrorInvalidValue;
  }
}

template <int BITS>
cudaError_t launch_bits(const ShortK& p, int x_dtype, int ctas, int64_t nbatch, cudaStream_t st) {
  switch (p.K / 64) {
    case 1: return launch_x<BITS, 1>(p, x_dtype, ctas, nbatch, st);
    case 2: return launch_x<BITS, 2>(p, x_dtype, ctas, nbatch, st);
    case 4: return launch_x<BITS, 4>(p, x_dtype, ctas, nbatch, st);
    default: return cudaErrorInvalidValue;
  }
}

bool strides_multiple_of(const BatchMap& m, int64_t q) {
  for (int d = 0; d < m.nd; ++d)
    if (m.stride[d] % q) return false;
  return true;
}

}  // namespace

bool qmv_shortk_supported(const QmmArgs& a) {
  if (!a.transpose || (a.bits != 4 && a.bits != 8) || a.gs != 64) return false;
  if (a.K != 64 && a.K != 128 && a.K != 256) return false;
  if (a.M < 1 || a.M > 32 || a.N < 1 || a.N > ((int64_t)1 << 30) || a.nbatch < 2 || a.nbatch > 65535) return false;
  {
    const int nt = a.M <= 8 ? 1 : (a.M <= 16 ? 2 : 4);
    if (!inst_ok((int)(a.K / 64), nt, a.x_dtype != QB200_BFLOAT16)) return false;
  }
  const int64_t ng = a.K / 64;
  // 16-byte pieces of codes by cp.async: rows start on 16 bytes; a row's scales follow the previous row's (lds == groups)
  if ((uintptr_t)a.w % 16 || a.ldw % 4 || !strides_multiple_of(a.wb, 4)) return false;
  if (a.lds != ng) return false;
  return true;
}

cudaError_t launch_qmv_shortk(const QmmArgs& a, cudaStream_t st) {
  if (!qmv_shortk_supported(a)) return cudaErrorInvalidValue;
  ShortK p;
  p.x = a.x; p.w = a.w; p.s = (const uint16_t*)a.s; p.b = (const uint16_t*)a.b; p.y = a.y;
  p.M = (int)a.M; p.K = (int)a.K; p.N = a.N;
  p.ldx = a.ldx; p.ldw = a.ldw; p.lds = a.lds; p.ldy = a.ldy;
  p.tiles = (int)((a.N + 15) / 16);
  // tiles per CTA: 16 per warp (the ring's fill and the activation set-up are paid once per CTA), halved down to 2 while
  // the grid would have fewer than two CTAs per SM
  int per_warp = 16;
  while (per_warp > 2 && a.nbatch * ((p.tiles + kWarps * per_warp - 1) / (kWarps * per_warp)) < 2LL * sm_count()) per_warp /= 2;
  // the nearest whole number of CTAs, each with an equal share (a cache length just past a multiple of the share must
  // not add a CTA of one tile)
  const int target = kWarps * per_warp;
  const int ctas = p.tiles < target ? 1 : (p.tiles + target / 2) / target;
  p.tiles_per_cta = (p.tiles + ctas - 1) / ctas;
  p.sb_vec = (uintptr_t)a.s % 4 == 0 && (uintptr_t)a.b % 4 == 0 && strides_multiple_of(a.sb, 2);
  p.xb = a.xb; p.wb = a.wb; p.sb = a.sb; p.yb = a.yb;
  return a.bits == 4 ? launch_bits<4>(p, a.x_dtype, ctas, a.nbatch, st) : launch_bits<8>(p, a.x_dtype, ctas, a.nbatch, st);
}

}  // namespace qb

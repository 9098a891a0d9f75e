// Weight-streaming quantized matmul for 9..64 tokens per pass: y[M, N] = x[M, K] . What[N, K]^T with every
// packed word read from HBM once for all tokens, What = bf16(q*s + b).
//
// Replaces mlx_quantized_matmul(transpose=true) as called by qmatmulBits (mlx-serve
// src/transformer.zig:20894-20983) at the widths its scheduler batches (up to 32 slots,
// src/scheduler.zig:5147) and up to the prefill route: the range between the single-digit verify lanes
// (src/transformer.zig:1317-1453) and prefillDqGemm (src/transformer.zig:20987-21011).  Like that dense route --
// and like MLX's own tiled qmm, which dequantises into the activation type -- the weight term is rounded to bf16
// once (one bf16 FMA of the exact code with the group's scale and bias); products are exact and accumulate in
// fp32 inside the MMA.
//
// Why not the narrow kernel's integer form here: its per-(64-group, token tile) fix-up (two integer
// multiply-adds, two conversions, six fp32 operations for two MMAs) grows with the token count and was
// measured at 1000 instructions per 2 KiB ring stage for 32 tokens.  Dequantising the A operand in registers
// costs ~60 instructions per 64-group whatever the token count, after which a token tile is four bf16
// mma.sync.m16n8k16 and two 128-bit shared-memory reads, with no fix-up: the accumulators run over all of K.
//
// Organisation:
//  * A small kernel rewrites the activations once into B-fragment order in a scratch buffer in global
//    memory (it stays in L2), cut into slices of 512 (or 256) K values.  CTAs fetch slices with one bulk
//    copy each (cp.async.bulk + mbarrier, double buffered) instead of every CTA re-staging all of x.
//  * Work is cut stream-K style.  A *step* is one ring stage (16 rows x 128 bytes) per warp for the 16
//    warps of a CTA: 16 consecutive row tiles at the same K offset, so the warps of a step share one
//    activation slice.  The steps of the whole problem -- tile block after tile block, K offset after K
//    offset inside a block -- are divided evenly over the CTAs.  A CTA whose range ends inside a tile block
//    writes its fp32 partial sums to scratch, and the last CTA to arrive for that block (an atomic counter,
//    nobody waits) adds the partial sums in CTA order and stores y.  Every SM gets the same number of steps
//    (+-1) whatever N is, and the result does not depend on timing.
//  * Each warp streams its own tiles through a private cp.async ring, as in the narrow kernel, and keeps
//    its tile's accumulators in registers; nothing is reduced across warps.
// Scratch (activation fragments, partial sums, counters) is a static array inside the library: calls on
// one stream are ordered by the stream; calls that overlap on the GPU from different streams would share
// it and must be serialised by the caller.
#include <mutex>

#include "kernels.h"
#include "stream_ptx.cuh"

namespace qb {
namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;                  // cp.async ring depth per warp
constexpr int kStageW = 2048;               // 16 rows x 128 B of packed codes
constexpr int kStageBytes = kStageW + 256;  // + 16 rows x (scales, biases)
constexpr int kMaxMat = 4;
constexpr int kMaxK = 16384;                // longest contraction the activation scratch holds
constexpr int kMaxTileBlocks = 8192;
constexpr int kMaxGrid = 160;               // CTAs (one per SM)
constexpr int kMaxNT = 8;                   // n8 token tiles per pass (64 tokens)
constexpr uint32_t kSpinLimit = 1u << 22;

// K values per activation slice: 64 bytes per K value at 32 tokens, 128 at 64 -- two slices must fit beside the ring.
__host__ __device__ constexpr int slice_k(int nt) { return nt <= 4 ? 512 : 256; }
// One slice: [64-group][n8 tile][MMA pair][lane][16 B] bf16 B fragments = 1 KiB per (group, tile).
__host__ __device__ constexpr int slice_bytes(int nt) { return (slice_k(nt) / 64) * nt * 1024; }

constexpr size_t kPrepBytes = (size_t)kMaxK * kMaxNT * 16;                                   // 16 bytes per K value and n8 tile
constexpr size_t kPartSlotFloats = (size_t)kWarps * kMaxNT * 4 * 32;                         // one tile block of partial sums
constexpr size_t kPartialBytes = (size_t)2 * kMaxGrid * kPartSlotFloats * sizeof(float);     // two per CTA
constexpr size_t kCounterBytes = (size_t)kMaxTileBlocks * sizeof(int);
constexpr size_t kScratchBytes = kPrepBytes + kPartialBytes + kCounterBytes + 256;
static __device__ __align__(256) unsigned char g_wide_scratch[kScratchBytes];   // zero at load: the counters start at 0

struct PrepK {
  const uint16_t* x; unsigned char* out;
  int M, K, NT;
  int64_t ldx;
};

struct WideK {
  const unsigned char* xprep;
  const uint32_t* w[kMaxMat]; const uint16_t* s[kMaxMat]; const uint16_t* b[kMaxMat]; uint16_t* y[kMaxMat];
  int N[kMaxMat];
  int64_t ldw[kMaxMat], lds[kMaxMat], ldy[kMaxMat];
  int tile0[kMaxMat + 1];
  int nmat, M, K, gshift, ntiles;
  int spb;                 // steps per tile block = K units
  int total_steps;
  float* partial; int* counters; int* status;
};

#define QB_SEL4(arr, i) ((i) == 0 ? (arr)[0] : ((i) == 1 ? (arr)[1] : ((i) == 2 ? (arr)[2] : (arr)[3])))
__device__ __forceinline__ int mat_of_tile(const WideK& p, int tile) {
  int mi = 0;
  if (p.nmat > 1 && tile >= p.tile0[1]) mi = 1;
  if (p.nmat > 2 && tile >= p.tile0[2]) mi = 2;
  if (p.nmat > 3 && tile >= p.tile0[3]) mi = 3;
  return mi;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait; false when the limit expired.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// Contiguous global -> shared copy by the copy engine, completion counted on an mbarrier (no multicast).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// A lane owns 16 consecutive K values of a 64-group (k = 16 t + o) of the rows g and g + 8.  Which of them
// sit in MMA step m (0..3), operand register r (0: a0/a1 with b0, 1: a2/a3 with b1), element e (0, 1) is a
// free permutation of K as long as the activations are staged alike.  4 bits: the pairs one LOP3 cuts out
// of a packed word, (w >> 4i) & 0x000F000F = codes (i, i + 4) of that word.  8 bits: in order.
template <int BITS> __host__ __device__ constexpr int kofs(int m, int r, int e) {
  return BITS == 4 ? 8 * (m >> 1) + 2 * (m & 1) + r + 4 * e : 4 * m + 2 * r + e;
}

// ---- activations -> bf16 B fragments in slices, one thread per (token slot, 16 K values) ----
// Token slots beyond M and K values beyond K (the last slice is padded) are written as zeros.
template <int BITS>
__global__ void __launch_bounds__(256) wide_prep_kernel(PrepK p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int NT = p.NT, SK = slice_k(NT), kpad = (p.K + SK - 1) / SK * SK;
  const int ppt = kpad >> 4;                                   // 16-value pieces per token
  const int idx = blockIdx.x * 256 + threadIdx.x;
  if (idx >= NT * 8 * ppt) return;
  const int m = idx / ppt, pc = idx - m * ppt;                 // token slot, piece
  uint32_t v[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};            // 16 bf16 values, in order
  if (m < p.M && pc * 16 < p.K) {
    const uint16_t* px = p.x + (int64_t)m * p.ldx + pc * 16;
    if ((((uintptr_t)px) & 15) == 0) {
      const uint4 a = *(const uint4*)px, b = *(const uint4*)(px + 8);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (uint32_t)px[2 * j] | ((uint32_t)px[2 * j + 1] << 16);
    }
  }
  auto elem = [&](int o) -> uint32_t { return (o & 1) ? (v[o >> 1] >> 16) : (v[o >> 1] & 0xFFFFu); };
  const int gi_all = pc >> 2, t = pc & 3;
  const int gps = SK / 64, sl = gi_all / gps, gi = gi_all - sl * gps;
  const int nt = m >> 3, g = m & 7;
  unsigned char* base = p.out + (size_t)sl * slice_bytes(NT) + (size_t)((gi * NT + nt) * 2) * 512 + (g * 4 + t) * 16;
#pragma unroll
  for (int h = 0; h < 2; ++h) {   // MMA steps 2h and 2h + 1: (b0, b1) each
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int mm = 2 * h + (q >> 1), r = q & 1;
      o[q] = elem(kofs<BITS>(mm, r, 0)) | (elem(kofs<BITS>(mm, r, 1)) << 16);
    }
    *(uint4*)(base + h * 512) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// CTA that owns step q when S steps are divided over G CTAs as [S*c/G, S*(c+1)/G).
// (S * G stays far below 2^31: at most 2^19 steps, 160 CTAs)
__device__ __forceinline__ int cta_of_step(int q, int S, int G) {
  int c = (q * G) / S;
  while (c + 1 < G && (S * (c + 1)) / G <= q) ++c;
  while (c > 0 && (S * c) / G > q) --c;
  return c;
}

template <int BITS, int NT>
__global__ void __launch_bounds__(kThreads, 1) qmv_wide_kernel(const __grid_constant__ WideK p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int U = BITS == 4 ? 4 : 2;        // 64-wide groups per unit
  constexpr int CK = 64 * U;                  // K values per unit (128 bytes per row)
  constexpr int SB = slice_bytes(NT);
  constexpr int UPS = slice_k(NT) / CK;       // units (= steps) per activation slice, a power of two

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  unsigned char* ring = smem;
  unsigned char* xs = smem + (size_t)kWarps * kStages * kStageBytes;
  uint64_t* mbar = (uint64_t*)(xs + 2 * SB);
  int* s_flag = (int*)(mbar + 2);   // [4]: last arriver?, first and last contributing CTA, slot of the first

  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int S = p.total_steps;
  const int lo = (S * cta) / G, hi = (S * (cta + 1)) / G;
  const int SPB = p.spb;

  if (tid == 0) {
    mbar_init(&mbar[0], 1);
    mbar_init(&mbar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }

  // ---- producer: one ring stage per step, for this warp's tile of the step's tile block ----
  const uint32_t my_ring = smem_u32(ring + (size_t)warp * kStages * kStageBytes);
  const unsigned char* my_ring_p = ring + (size_t)warp * kStages * kStageBytes;
  const int chunk = lane & 7;
  uint32_t wdst[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = (lane >> 3) + 4 * r;
    wdst[r] = my_ring + row * 128 + ((chunk ^ swz_w<BITS>(row)) << 4);
  }
  const uint32_t sbdst = my_ring + kStageW + (lane & 15) * 16 + (lane >> 4) * 8;
  int pq = lo;
  int p_tb = lo / SPB, p_ks = lo - p_tb * SPB;
  int p_tb_set = -1;
  const unsigned char* wsrc = nullptr;   // row slot 0 of this warp's tile, unit 0
  uint32_t roff[3] = {0u, 0u, 0u};
  const uint16_t* sbsrc = nullptr;
  bool p_tile_ok = false;
  uint32_t p_off = 0;
  auto set_tile = [&](int tb) {
    p_tb_set = tb;
    const int tile = tb * kWarps + warp;
    p_tile_ok = tile < p.ntiles;
    if (!p_tile_ok) return;
    const int mi = mat_of_tile(p, tile);
    const int nrows = QB_SEL4(p.N, mi), row0 = (tile - QB_SEL4(p.tile0, mi)) * 16;
    const int64_t ldw = QB_SEL4(p.ldw, mi), lds = QB_SEL4(p.lds, mi);
    int n0 = row0 + (lane >> 3);
    n0 = n0 < nrows ? n0 : nrows - 1;
    wsrc = (const unsigned char*)(QB_SEL4(p.w, mi) + (int64_t)n0 * ldw) + chunk * 16;
#pragma unroll
    for (int r = 1; r < 4; ++r) {
      int n = row0 + (lane >> 3) + 4 * r;
      n = n < nrows ? n : nrows - 1;
      roff[r - 1] = (uint32_t)((n - n0) * (int)ldw * 4);
    }
    int ns = row0 + (lane & 15);
    ns = ns < nrows ? ns : nrows - 1;
    sbsrc = ((lane >> 4) ? QB_SEL4(p.b, mi) : QB_SEL4(p.s, mi)) + (int64_t)ns * lds;
  };
  auto issue = [&]() {
    if (pq < hi) {
      if (p_tb != p_tb_set) set_tile(p_tb);
      if (p_tile_ok) {
        const unsigned char* src = wsrc + (size_t)p_ks * 128;
        cp_async16(wdst[0] + p_off, src);
        cp_async16(wdst[1] + p_off, src + roff[0]);
        cp_async16(wdst[2] + p_off, src + roff[1]);
        cp_async16(wdst[3] + p_off, src + roff[2]);
        const uint16_t* sb = sbsrc + ((p_ks * U) >> p.gshift);
        if (BITS == 4 && p.gshift == 0) cp_async8(sbdst + p_off, sb);
        else cp_async4(sbdst + p_off, sb);
      }
      ++pq;
      if (++p_ks == SPB) { p_ks = 0; ++p_tb; }
    }
    p_off = p_off + kStageBytes == kStages * kStageBytes ? 0u : p_off + kStageBytes;
  };

  // per-lane byte offsets of the code reads of row g (row g + 8 is +1024: same swizzle)
  int frag_off[U];
#pragma unroll
  for (int j = 0; j < U; ++j) {
    if (BITS == 4) frag_off[j] = g * 128 + (((2 * j + (t >> 1)) ^ swz_w<4>(g)) << 4) + (t & 1) * 8;
    else frag_off[j] = g * 128 + (((4 * j + t) ^ swz_w<8>(g)) << 4);
  }

#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) { issue(); cp_async_commit(); }

  // Let the next grid in the stream begin launching; wait for the previous one (the activation fragments,
  // and whatever wrote y last) before touching anything but the weights.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();   // the mbarriers are initialised

  // ---- activation slices: slice i of this CTA's range lives in buffer i & 1 ----
  // first step of the slice after the one that holds step q (ks = q's offset in its tile block)
  auto next_switch = [&](int q, int ks) -> int {
    const int in_slice = UPS - (ks & (UPS - 1)), in_block = SPB - ks;
    return q + (in_slice < in_block ? in_slice : in_block);
  };
  auto load_slice = [&](int q, int buf) {   // thread 0: the slice that holds step q
    const int tb = q / SPB, ks = q - tb * SPB;
    const int sl = ks / UPS;
    mbar_expect_tx(&mbar[buf], (uint32_t)SB);
    bulk_load(smem_u32(xs + (size_t)buf * SB), p.xprep + (size_t)sl * SB, (uint32_t)SB, &mbar[buf]);
  };
  int c_tb = lo / SPB, c_ks = lo - c_tb * SPB;
  int q_next_slice = lo;   // the step at which the next slice switch happens
  int nsl = 0;             // slices switched to so far
  if (tid == 0 && lo < hi) {
    load_slice(lo, 0);
    const int q2 = next_switch(lo, c_ks);
    if (q2 < hi) load_slice(q2, 1);
  }

  float tot[NT][4];   // rows g, g + 8 x tokens 8 nt + 2t, 8 nt + 2t + 1
  float tot2[2][4];   // two token tiles only: a second set for the odd MMA steps (four independent chains)
  int seg_first_ks = c_ks;
  uint32_t c_off = 0;
  int buf = 0;
  const __nv_bfloat162 c128 = __float2bfloat162_rn(128.f);
  for (int q = lo; q < hi; ++q) {
    if (q == lo || c_ks == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) tot2[nt][0] = tot2[nt][1] = tot2[nt][2] = tot2[nt][3] = 0.f;
      seg_first_ks = c_ks;
    }
    if (q == q_next_slice) {   // switch to slice `nsl`
      if (nsl > 0) {
        __syncthreads();       // every warp is done with slice nsl - 1: its buffer may be refilled
        const int q2 = next_switch(q, c_ks);   // the slice after this one goes to the buffer just vacated
        if (tid == 0 && q2 < hi) load_slice(q2, (nsl + 1) & 1);
      }
      buf = nsl & 1;
      if (!mbar_wait(&mbar[buf], (uint32_t)((nsl >> 1) & 1))) atomicExch(p.status, 101);
      q_next_slice = next_switch(q, c_ks);
      ++nsl;
    }
    // keep the ring full, then wait for this step's bytes
    issue();
    cp_async_commit();
    cp_async_wait<kStages - 1>();
    __syncwarp();
    const unsigned char* st = my_ring_p + c_off;
    c_off = c_off + kStageBytes == kStages * kStageBytes ? 0u : c_off + kStageBytes;
    const bool tile_ok = c_tb * kWarps + warp < p.ntiles;
    if (tile_ok) {
      // scales / biases of rows g and g + 8 for the unit's U groups (bf16 pairs): 16 bytes per row
      uint32_t sl[2], sh[2], bl[2], bh[2];
      {
        const uint4 lo4 = *(const uint4*)(st + kStageW + g * 16), hi4 = *(const uint4*)(st + kStageW + (g + 8) * 16);
        if (BITS == 4 && p.gshift == 0) {
          sl[0] = lo4.x; sl[1] = lo4.y; sh[0] = hi4.x; sh[1] = hi4.y;
          bl[0] = lo4.z; bl[1] = lo4.w; bh[0] = hi4.z; bh[1] = hi4.w;
        } else if (BITS == 4) {  // group size 128: each value serves two 64-wide groups
          sl[0] = __byte_perm(lo4.x, lo4.x, 0x1010); sl[1] = __byte_perm(lo4.x, lo4.x, 0x3232);
          sh[0] = __byte_perm(hi4.x, hi4.x, 0x1010); sh[1] = __byte_perm(hi4.x, hi4.x, 0x3232);
          bl[0] = __byte_perm(lo4.z, lo4.z, 0x1010); bl[1] = __byte_perm(lo4.z, lo4.z, 0x3232);
          bh[0] = __byte_perm(hi4.z, hi4.z, 0x1010); bh[1] = __byte_perm(hi4.z, hi4.z, 0x3232);
        } else {
          sl[0] = lo4.x; sh[0] = hi4.x; bl[0] = lo4.z; bh[0] = hi4.z;
          sl[1] = sh[1] = bl[1] = bh[1] = 0;
        }
      }
      const unsigned char* xb = xs + (size_t)buf * SB;
      const int gi0 = (c_ks & (UPS - 1)) * U;   // first 64-group of this unit inside the slice
      const uint4* xfr = (const uint4*)xb + (size_t)(gi0 * NT) * 64 + lane;
#pragma unroll
      for (int j = 0; j < U; ++j) {
        // the group's scale and bias in both bf16 lanes, for row g and row g + 8
        const uint32_t s_lo = __byte_perm(sl[j >> 1], 0, (j & 1) ? 0x3232 : 0x1010), s_hi = __byte_perm(sh[j >> 1], 0, (j & 1) ? 0x3232 : 0x1010);
        const uint32_t b_lo = __byte_perm(bl[j >> 1], 0, (j & 1) ? 0x3232 : 0x1010), b_hi = __byte_perm(bh[j >> 1], 0, (j & 1) ? 0x3232 : 0x1010);
        uint32_t A[4][4];   // [MMA step][a0 row g, a1 row g+8, a2 row g, a3 row g+8]: bf16(q * s + b)
        if constexpr (BITS == 4) {
          const uint2 wl = *(const uint2*)(st + frag_off[j]);
          const uint2 wh = *(const uint2*)(st + frag_off[j] + 1024);
          const __nv_bfloat162 s2l = *(const __nv_bfloat162*)&s_lo, b2l = *(const __nv_bfloat162*)&b_lo;
          const __nv_bfloat162 s2h = *(const __nv_bfloat162*)&s_hi, b2h = *(const __nv_bfloat162*)&b_hi;
#pragma unroll
          for (int m = 0; m < 4; ++m) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              // pair (i, i + 4) of word m / 2 with i = 2 (m % 2) + r: 128 + q in both lanes, exactly; minus 128; one FMA
              const int sh4 = 4 * (2 * (m & 1) + r);
              const uint32_t pl = lop3_and_or(((m >> 1) ? wl.y : wl.x) >> sh4, 0x000F000Fu, 0x43004300u);
              const uint32_t ph = lop3_and_or(((m >> 1) ? wh.y : wh.x) >> sh4, 0x000F000Fu, 0x43004300u);
              __nv_bfloat162 vl = __hfma2(__hsub2(*(const __nv_bfloat162*)&pl, c128), s2l, b2l);
              __nv_bfloat162 vh = __hfma2(__hsub2(*(const __nv_bfloat162*)&ph, c128), s2h, b2h);
              A[m][2 * r] = *(uint32_t*)&vl;
              A[m][2 * r + 1] = *(uint32_t*)&vh;
            }
          }
        } else {
          const uint4 wl = *(const uint4*)(st + frag_off[j]);
          const uint4 wh = *(const uint4*)(st + frag_off[j] + 1024);
          const float sfl = bf16lo(s_lo), bfl = bf16lo(b_lo), sfh = bf16lo(s_hi), bfh = bf16lo(b_hi);
          const uint32_t wlv[4] = {wl.x, wl.y, wl.z, wl.w}, whv[4] = {wh.x, wh.y, wh.z, wh.w};
#pragma unroll
          for (int m = 0; m < 4; ++m) {   // word m holds codes 4m .. 4m + 3: (a0: 4m, 4m+1), (a2: 4m+2, 4m+3)
            const float l0 = __uint_as_float(__byte_perm(wlv[m], 0x4B000000u, 0x7540)) - 8388608.f;
            const float l1 = __uint_as_float(__byte_perm(wlv[m], 0x4B000000u, 0x7541)) - 8388608.f;
            const float l2 = __uint_as_float(__byte_perm(wlv[m], 0x4B000000u, 0x7542)) - 8388608.f;
            const float l3 = __uint_as_float(__byte_perm(wlv[m], 0x4B000000u, 0x7543)) - 8388608.f;
            const float h0 = __uint_as_float(__byte_perm(whv[m], 0x4B000000u, 0x7540)) - 8388608.f;
            const float h1 = __uint_as_float(__byte_perm(whv[m], 0x4B000000u, 0x7541)) - 8388608.f;
            const float h2 = __uint_as_float(__byte_perm(whv[m], 0x4B000000u, 0x7542)) - 8388608.f;
            const float h3 = __uint_as_float(__byte_perm(whv[m], 0x4B000000u, 0x7543)) - 8388608.f;
            A[m][0] = pack_bf16x2(fmaf(l0, sfl, bfl), fmaf(l1, sfl, bfl));
            A[m][2] = pack_bf16x2(fmaf(l2, sfl, bfl), fmaf(l3, sfl, bfl));
            A[m][1] = pack_bf16x2(fmaf(h0, sfh, bfh), fmaf(h1, sfh, bfh));
            A[m][3] = pack_bf16x2(fmaf(h2, sfh, bfh), fmaf(h3, sfh, bfh));
          }
        }
        // Four token tiles at a time: their B fragments first, then the MMA steps with the tiles innermost, so
        // that back-to-back MMAs never wait for each other's accumulator.
#pragma unroll
        for (int n0 = 0; n0 < NT; n0 += 4) {
          constexpr int NB = NT < 4 ? NT : 4;
          uint4 bq[NB][2];
#pragma unroll
          for (int i = 0; i < NB; ++i) {
            bq[i][0] = xfr[(size_t)((j * NT + n0 + i) * 2) * 32];
            bq[i][1] = xfr[(size_t)((j * NT + n0 + i) * 2 + 1) * 32];
          }
#pragma unroll
          for (int m = 0; m < 4; ++m) {
#pragma unroll
            for (int i = 0; i < NB; ++i) {
              const uint32_t b0 = (m & 1) ? bq[i][m >> 1].z : bq[i][m >> 1].x, b1 = (m & 1) ? bq[i][m >> 1].w : bq[i][m >> 1].y;
              if (NT == 2 && (m & 1)) mma_bf16(tot2[i], A[m][0], A[m][1], A[m][2], A[m][3], b0, b1);
              else mma_bf16(tot[n0 + i], A[m][0], A[m][1], A[m][2], A[m][3], b0, b1);
            }
          }
        }
      }
    }
    __syncwarp();

    // ---- end of this CTA's segment of the tile block: store, or hand the partial sums over ----
    if (c_ks == SPB - 1 || q == hi - 1) {
      const bool complete = seg_first_ks == 0 && c_ks == SPB - 1;
      if constexpr (NT == 2) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int r = 0; r < 4; ++r) tot[nt][r] += tot2[nt][r];
      }
      // this warp's tile: rows g and g + 8, tokens 8 nt + 2t (+1)
      const int tile = c_tb * kWarps + warp;
      const int mi = mat_of_tile(p, tile < p.ntiles ? tile : p.ntiles - 1);
      const int nrows = QB_SEL4(p.N, mi), n_lo = (tile - QB_SEL4(p.tile0, mi)) * 16 + g;
      uint16_t* ym = QB_SEL4(p.y, mi);
      const int64_t ldy = QB_SEL4(p.ldy, mi);
      auto store_tile = [&](const float (&v)[NT][4]) {
        if (!tile_ok) return;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int tok = nt * 8 + 2 * t;
          if (tok < p.M) {
            if (n_lo < nrows) ym[(int64_t)tok * ldy + n_lo] = f32_to_bf16_bits(v[nt][0]);
            if (n_lo + 8 < nrows) ym[(int64_t)tok * ldy + n_lo + 8] = f32_to_bf16_bits(v[nt][2]);
          }
          if (tok + 1 < p.M) {
            if (n_lo < nrows) ym[(int64_t)(tok + 1) * ldy + n_lo] = f32_to_bf16_bits(v[nt][1]);
            if (n_lo + 8 < nrows) ym[(int64_t)(tok + 1) * ldy + n_lo + 8] = f32_to_bf16_bits(v[nt][3]);
          }
        }
      };
      if (complete) {
        store_tile(tot);
      } else {
        // partial slot: 0 for the segment that holds this CTA's first step, 1 otherwise; [warp][register][lane]
        float* my_part = p.partial + (size_t)(2 * cta + (lo / SPB == c_tb ? 0 : 1)) * kPartSlotFloats + (size_t)warp * NT * 4 * 32 + lane;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int r = 0; r < 4; ++r) my_part[(nt * 4 + r) * 32] = tot[nt][r];
        // hand-over: the last CTA to arrive for this tile block adds every contributor's partial sums in
        // CTA order and stores; nobody waits
        __syncthreads();
        if (tid == 0) {
          __threadfence();   // release: the barrier ordered every warp's partial sums before this thread
          const int b0 = c_tb * SPB, b1 = b0 + SPB - 1;
          const int c_first = cta_of_step(b0, S, G), c_last = cta_of_step(b1, S, G);
          const int old = atomicAdd(&p.counters[c_tb], 1);
          s_flag[0] = old == c_last - c_first;
          s_flag[1] = c_first;
          s_flag[2] = c_last;
          // every contributor's first step lies in this tile block, except the first contributor's (it may start earlier)
          s_flag[3] = ((S * c_first) / G) / SPB == c_tb ? 0 : 1;
        }
        __syncthreads();
        if (s_flag[0]) {
          __threadfence();
          const int c_first = s_flag[1], c_last = s_flag[2], first_slot = s_flag[3];
          float v[NT][4];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) v[nt][0] = v[nt][1] = v[nt][2] = v[nt][3] = 0.f;
          for (int c = c_first; c <= c_last; ++c) {   // CTA order: the sum does not depend on who arrived when
            const float* part = p.partial + (size_t)(2 * c + (c == c_first ? first_slot : 0)) * kPartSlotFloats + (size_t)warp * NT * 4 * 32 + lane;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int r = 0; r < 4; ++r) v[nt][r] += __ldcg(part + (nt * 4 + r) * 32);
          }
          store_tile(v);
          if (tid == 0) p.counters[c_tb] = 0;   // ready for the next launch
        }
        __syncthreads();   // s_flag may be reused
      }
    }
    if (++c_ks == SPB) { c_ks = 0; ++c_tb; }
  }
  cp_async_wait<0>();
}

// Device address of the scratch array on the current device (looked up once per device).
cudaError_t wide_scratch(unsigned char** out) {
  static unsigned char* addr[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(setup_mutex());
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_wide_scratch);
    if (e != cudaSuccess) return e;
    addr[dev] = (unsigned char*)p;
  }
  *out = addr[dev];
  return cudaSuccess;
}

constexpr size_t smem_wide(int nt) { return (size_t)kWarps * kStages * kStageBytes + (size_t)2 * slice_bytes(nt) + 64; }
static_assert(smem_wide(4) <= 227 * 1024 && smem_wide(8) <= 227 * 1024, "shared memory");

template <int BITS, int NT>
cudaError_t launch_wide_inst(const WideK& p, int grid, cudaStream_t st) {
  auto kern = qmv_wide_kernel<BITS, NT>;
  {
    std::lock_guard<std::mutex> lk(setup_mutex());
    static bool done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !done[dev]) {
      const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_wide(NT));
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem_wide(NT);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace

bool qmv_wide_supported(const QmmArgs& a) {
  if (!a.transpose || a.nbatch != 1) return false;
  if (!((a.bits == 4 && (a.gs == 64 || a.gs == 128)) || (a.bits == 8 && a.gs == 64))) return false;
  if (a.x_dtype != QB200_BFLOAT16) return false;
  if (a.K % 256 != 0 || a.K <= 0 || a.K > kMaxK) return false;
  if (a.N <= 0 || a.N > (int64_t)kMaxTileBlocks * kWarps * 16 || a.M <= 8) return false;
  if ((((uintptr_t)a.w) & 15) != 0 || (a.ldw * 4) % 16 != 0) return false;
  if ((((uintptr_t)a.s) & 7) != 0 || (((uintptr_t)a.b) & 7) != 0) return false;
  if (a.gs == 64 && a.lds % 4 != 0) return false;
  if (a.gs == 128 && (a.lds % 2) != 0) return false;
  return true;
}

// `count` (<= 4) weight matrices on the same activations; more than 64 tokens run in passes of 64.
cudaError_t launch_qmv_wide_multi(const QmmArgs* a, int count, cudaStream_t st) {
  unsigned char* scratch = nullptr;
  cudaError_t e = wide_scratch(&scratch);
  if (e != cudaSuccess) return e;
  const int bits = a[0].bits, CK = bits == 4 ? 256 : 128;
  WideK p;
  p.nmat = count;
  int ntiles = 0;
  for (int i = 0; i < kMaxMat; ++i) {
    const QmmArgs& q = a[i < count ? i : 0];
    p.w[i] = q.w + q.wb.offset(0);
    p.s[i] = (const uint16_t*)q.s + q.sb.offset(0);
    p.b[i] = (const uint16_t*)q.b + q.sb.offset(0);
    p.N[i] = i < count ? (int)q.N : 0;
    p.ldw[i] = q.ldw; p.lds[i] = q.lds; p.ldy[i] = q.ldy;
    p.tile0[i] = ntiles;
    if (i < count) ntiles += ((int)q.N + 15) / 16;
  }
  p.tile0[kMaxMat] = ntiles;
  p.ntiles = ntiles;
  p.K = (int)a[0].K;
  p.gshift = a[0].gs == 128 ? 1 : 0;
  p.xprep = scratch;
  p.partial = (float*)(scratch + kPrepBytes);
  p.counters = (int*)(scratch + kPrepBytes + kPartialBytes);
  p.status = (int*)(scratch + kPrepBytes + kPartialBytes + kCounterBytes);
  const int nsm = sm_count() < kMaxGrid ? sm_count() : kMaxGrid;
  const int ntb = (ntiles + kWarps - 1) / kWarps;
  if (ntb > kMaxTileBlocks) return cudaErrorInvalidConfiguration;
  p.spb = p.K / CK;
  p.total_steps = ntb * p.spb;
  const int grid = p.total_steps < nsm ? p.total_steps : nsm;
  for (int64_t m0 = 0; m0 < a[0].M; m0 += 64) {
    const int M = (int)((a[0].M - m0) < 64 ? (a[0].M - m0) : 64);
    const int NT = M <= 16 ? 2 : (M <= 32 ? 4 : 8);
    PrepK pk;
    pk.x = (const uint16_t*)a[0].x + (a[0].xb.offset(0) + m0 * a[0].ldx);
    pk.out = scratch;
    pk.M = M; pk.K = p.K; pk.NT = NT; pk.ldx = a[0].ldx;
    const int sk = slice_k(NT), kpad = (p.K + sk - 1) / sk * sk;
    const int pblocks = (NT * 8 * (kpad / 16) + 255) / 256;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pblocks);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = bits == 4 ? cudaLaunchKernelEx(&cfg, wide_prep_kernel<4>, pk) : cudaLaunchKernelEx(&cfg, wide_prep_kernel<8>, pk);
    if (e != cudaSuccess) return e;
    for (int i = 0; i < kMaxMat; ++i) {
      const QmmArgs& q = a[i < count ? i : 0];
      p.y[i] = (uint16_t*)q.y + (q.yb.offset(0) + m0 * q.ldy);
    }
    p.M = M;
    if (bits == 4) e = NT == 2 ? launch_wide_inst<4, 2>(p, grid, st) : (NT == 4 ? launch_wide_inst<4, 4>(p, grid, st) : launch_wide_inst<4, 8>(p, grid, st));
    else e = NT == 2 ? launch_wide_inst<8, 2>(p, grid, st) : (NT == 4 ? launch_wide_inst<8, 4>(p, grid, st) : launch_wide_inst<8, 8>(p, grid, st));
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t launch_qmv_wide(const QmmArgs& a, cudaStream_t st) { return launch_qmv_wide_multi(&a, 1, st); }

// 0, or the code of a bounded wait that expired in the wide streaming kernel (synchronises the device).
int qmv_wide_error_code() {
  unsigned char* scratch = nullptr;
  if (wide_scratch(&scratch) != cudaSuccess) return 0;
  int v = 0;
  cudaMemcpy(&v, scratch + kPrepBytes + kPartialBytes + kCounterBytes, sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}
void qmv_wide_error_reset() {
  unsigned char* scratch = nullptr;
  if (wide_scratch(&scratch) != cudaSuccess) return;
  cudaMemset(scratch + kPrepBytes + kPartialBytes + kCounterBytes, 0, sizeof(int));
}

}  // namespace qb

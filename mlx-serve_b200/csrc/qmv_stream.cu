// Persistent weight-streaming quantized matmul for decode widths (M <= 8 per
// launch): y[M, N] = x[M, K] . What[N, K]^T, 4/8-bit affine codes.
//
// Replaces mlx_quantized_matmul(transpose=true) as called by qmatmulBits
// (mlx-serve src/transformer.zig:20894-20983) at decode widths and the small-M
// verify lanes (src/transformer.zig:1317-1453).
//
// The kernel is HBM-bound by construction, so it is organised around (a)
// keeping bytes in flight and (b) spending as few issue slots per packed byte
// as possible -- a first version that expanded codes to bf16 for
// mma.sync.bf16 was measured instruction-bound (INT pipe) at 27% of HBM peak.
//  * One persistent CTA per SM (16 warps = two groups of 8).  Every warp owns a
//    private ring of cp.async (LDGSTS, 128-bit per lane) stages in shared
//    memory; a stage is 16 weight rows x 128 contiguous bytes plus their scales
//    and biases, so ~100 KiB of packed weights are in flight per SM regardless
//    of register pressure.  A warp only ever waits on its own copies
//    (cp.async.wait_group + __syncwarp), so no cross-warp protocol can hang.
//  * Integer tensor cores do the dots exactly: the packed codes are the u8 A
//    operand of mma.sync.m16n8k32.s32.u8.s8 (4-bit: two ANDs and one shift per
//    8 codes; 8-bit: the packed word as is), the activations are the s8 B
//    operand.  Each activation is converted once per CTA to a 15-bit
//    fixed-point value sharing one power-of-two scale per (token, 64-wide
//    group), v = rn(x * 2^(14-E)), split into two 7/8-bit planes
//    v = 128*p0 + p1 that occupy two columns of the n8 tile.  sum_k q*v is
//    therefore exact in s32; the only rounding is that of v (2^-15 of the
//    group's largest |x|: exact for bf16 inputs within 2^-7 of the group
//    maximum, and below fp32 accumulation noise otherwise).
//  * Per 64-wide group the s32 sums are combined (128*acc0 + acc1), converted
//    once to fp32 and scaled:  y += (s 2^(E-14)) * sum(q v) + b * 2^(E-14) * sum(v).
//    The weight term q*s+b is never rounded to bf16.
//  * A group's 8 warps split K for one 16-row tile and reduce through shared
//    memory behind a named barrier, double-buffered so the stream never drains.
//  * Thread-block clusters (M > 1): the CTAs of a cluster either split the
//    conversion of the activations and broadcast the fragments through
//    distributed shared memory, or -- when K is too long for one staging pass --
//    share their tiles and split K, each converting only its own range, with the
//    partial sums added in rank 0 behind one cluster barrier per round.
// Nothing is written to global scratch; the only global writes are y.
#include <type_traits>
#include "kernels.h"
#include "stream_ptx.cuh"

namespace qb {
namespace {

constexpr int kWarpsPerGroup = 8;   // K split inside a group
// Groups (independent tile lists) per CTA.  The single-token kernel keeps its shared memory under half an
// SM (one group, two CTAs per SM) so that, with programmatic dependent launch, a CTA of the next kernel in the
// stream can start filling its weight ring while the previous kernel is still running on the same SM.
__host__ __device__ constexpr int groups_for(bool m1) { return m1 ? 1 : 2; }
__host__ __device__ constexpr int rt_for(int nt, bool m1) { return m1 ? 2 : 4 / nt; }  // tiles reduced per barrier
__host__ __device__ constexpr int stages_for(int nt) { return nt == 1 ? 4 : 3; }  // cp.async ring depth per warp
constexpr int kStageW = 2048;       // 16 rows x 128 B of packed codes
constexpr int kStageBytes = kStageW + 256;  // + 16 rows x (scales, biases)
constexpr int kTokPerTile = 4;      // tokens per n8 tile (two planes each)
constexpr int kMaxTok = 8;          // tokens per launch (two n8 tiles of 4 tokens x 2 planes); wider M in 8-token blocks:
                                    // a 16-token instantiation (K staged in two passes of 2048, partial sums kept in
                                    // shared memory between them) was measured 15% slower than two 8-token launches

__host__ __device__ constexpr int kc_for(int nt) { return nt <= 2 ? 4096 : 1024; }

constexpr int kMaxMat = 4;          // weight matrices served by one launch (same activations)


struct StreamK {
  const void* x;
  const uint32_t* w[kMaxMat]; const uint16_t* s[kMaxMat]; const uint16_t* b[kMaxMat]; void* y[kMaxMat];
  int N[kMaxMat];
  int64_t ldw[kMaxMat], lds[kMaxMat], ldy[kMaxMat];
  int tile0[kMaxMat + 1];  // first 16-row tile of each matrix in the launch-wide tile numbering
  int nmat;
  int M, K;
  int64_t ldx;
  int gshift, x_f32;
  int total_groups;   // groups over the whole grid (tile t belongs to group t % total_groups)
  int ntiles;
  int npass, kc;      // K passes of kc values
  int ntl_max;        // max tiles per group (sizes the multi-pass accumulator)
  int ksplit;         // > 1: the CTAs of a cluster share their tiles and split K (partial sums meet in rank 0)
  int upc;            // K units per CTA in that mode
};

__device__ __forceinline__ void group_barrier(int grp) {
  asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "n"(kWarpsPerGroup * 32) : "memory");
}
// Kernel parameters are indexed with constant subscripts only (a dynamic subscript would force a
// local-memory copy of the parameter block).
#define QB_SEL4(arr, i) ((i) == 0 ? (arr)[0] : ((i) == 1 ? (arr)[1] : ((i) == 2 ? (arr)[2] : (arr)[3])))
__device__ __forceinline__ int mat_of_tile(const StreamK& p, int tile) {
  int mi = 0;
  if (p.nmat > 1 && tile >= p.tile0[1]) mi = 1;
  if (p.nmat > 2 && tile >= p.tile0[2]) mi = 2;
  if (p.nmat > 3 && tile >= p.tile0[3]) mi = 3;
  return mi;
}

template <int BITS, int NT, bool M1>
__global__ void __launch_bounds__(kWarpsPerGroup * groups_for(M1) * 32, M1 ? 2 : 1) qmv_stream_kernel(StreamK p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int U = BITS == 4 ? 4 : 2;        // 64-wide groups per unit
  constexpr int CK = 64 * U;                  // K values per unit (128 bytes per row)
  constexpr int kStages = stages_for(NT);
  constexpr int RT = rt_for(NT, M1);          // tiles reduced per group barrier
  constexpr int kGroups = groups_for(M1);
  constexpr int kThreads = kWarpsPerGroup * kGroups * 32;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int grp = warp / kWarpsPerGroup, ks = warp % kWarpsPerGroup;
  // K-split mode (large K at M > 1): the CTAs of a cluster work on the same tiles, each on its own range of K,
  // so each converts only its range of the activations, once; rank 0 adds the partial sums and stores.
  const bool split = !M1 && p.ksplit > 1;
  const int crank = M1 ? 0 : (int)cluster_rank();
  const int ggrp = (split ? (int)blockIdx.x / p.ksplit : (int)blockIdx.x) * kGroups + grp;  // global group id
  // ---- shared memory carve-up ----
  const int kc = p.kc;
  unsigned char* sp = smem;
  unsigned char* ring = sp;    sp += (size_t)kGroups * kWarpsPerGroup * kStages * kStageBytes;
  uint2* xfrag = (uint2*)sp;   sp += M1 ? (size_t)(kc / 32) * 8 * 8 : (size_t)(kc / 32) * NT * 32 * 8;
  float* gsc = (float*)sp;     sp += M1 ? (size_t)(kc / 64) * 8 : (size_t)(kc / 64) * NT * kTokPerTile * 8;  // (2^(E-14), 2^(E-14)*sum v)
  float* red = (float*)sp;     sp += (size_t)kGroups * 2 * RT * kWarpsPerGroup * NT * 64 * 4;
  sp += 16;
  float* yacc = (float*)sp;    // [kGroups][ntl_max][NT*64], only when npass > 1
  float* xred = (float*)sp;    // K-split mode (npass == 1): [2][ksplit - 1][kGroups][256] partial sums from the peers
  // A CTA's shared memory may only be written by its cluster peers once it is running: arrive now, and
  // wait for every peer's arrival just before the first remote store.
  if constexpr (!M1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(ring + (size_t)warp * kStages * kStageBytes);
  const unsigned char* my_ring_p = ring + (size_t)warp * kStages * kStageBytes;
  const int ntl = ggrp < p.ntiles ? (p.ntiles - ggrp + p.total_groups - 1) / p.total_groups : 0;
  const int k_lo = split ? crank * p.upc * CK : 0;                 // first K value of this CTA's range
  const int k_cta = split ? (p.K - k_lo < p.upc * CK ? (p.K - k_lo > 0 ? p.K - k_lo : 0) : p.upc * CK) : p.K;
  const int ut = k_cta / CK, upk = split ? (ut > 0 ? ut : 1) : kc / CK;
  // ---- producer: this warp's stream of (pass, local tile, K unit) items ----
  // A lane copies 16 bytes of four rows of a stage (rows lane/8 + 4r) and one scale or bias entry.  The source
  // pointers move by constants from unit to unit and from a tile to the group's next tile; only a change of
  // matrix, a last partial tile or a new K pass recomputes them (setup()).
  const int chunk = lane & 7;
  uint32_t wdst[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = (lane >> 3) + 4 * r;
    wdst[r] = my_ring + row * 128 + ((chunk ^ swz_w<BITS>(row)) << 4);
  }
  const uint32_t sbdst = my_ring + kStageW + (lane & 15) * 16 + (lane >> 4) * 8;   // per row: scales | biases
  const int sbstep = (kWarpsPerGroup * U) >> p.gshift;   // scale entries between two units of this warp
  const unsigned char* wp = nullptr;   // row slot 0 of the next item
  const uint16_t* sbp = nullptr;       // scale (lanes 0-15) or bias (16-31) of the next item
  uint32_t roff[3] = {0u, 0u, 0u};     // byte offsets of row slots 1..3 from slot 0
  int64_t tstep_w = 0, tstep_sb = 0;   // from behind a tile's last unit to the next tile's first
  int p_tile = 0, p_fast_end = 0;      // current tile; the group's next tile below p_fast_end is a constant step away
  int p_tl = 0, p_pass = 0, p_j = 0, p_nu = 0;
  uint32_t p_off = 0;                  // byte offset of the stage the next item goes to

  auto setup = [&]() {
    for (;;) {
      if (p_pass >= p.npass || ntl <= 0) { p_pass = p.npass; p_tl = ntl; return; }   // stream exhausted
      const int left = ut - p_pass * upk, upt_p = left < upk ? left : upk;
      p_nu = upt_p > ks ? (upt_p - ks + kWarpsPerGroup - 1) / kWarpsPerGroup : 0;
      if (p_nu > 0) break;
      ++p_pass;   // this warp has no unit in this pass
    }
    p_tile = ggrp + p_tl * p.total_groups;
    const int mi = mat_of_tile(p, p_tile);
    const int t0 = QB_SEL4(p.tile0, mi), nrows = QB_SEL4(p.N, mi);
    const int row0 = (p_tile - t0) * 16;
    const int64_t ldw = QB_SEL4(p.ldw, mi), lds = QB_SEL4(p.lds, mi);
    const int k0 = k_lo + p_pass * kc + ks * CK;
    int n0 = row0 + (lane >> 3);
    n0 = n0 < nrows ? n0 : nrows - 1;
    wp = (const unsigned char*)(QB_SEL4(p.w, mi) + (int64_t)n0 * ldw) + chunk * 16 + k0 * BITS / 8;
#pragma unroll
    for (int r = 1; r < 4; ++r) {
      int n = row0 + (lane >> 3) + 4 * r;
      n = n < nrows ? n : nrows - 1;
      roff[r - 1] = (uint32_t)((n - n0) * (int)ldw * 4);
    }
    int ns = row0 + (lane & 15);
    ns = ns < nrows ? ns : nrows - 1;
    sbp = ((lane >> 4) ? QB_SEL4(p.b, mi) : QB_SEL4(p.s, mi)) + (int64_t)ns * lds + ((k0 >> 6) >> p.gshift);
    tstep_w = (int64_t)p.total_groups * 16 * ldw * 4 - (int64_t)p_nu * (kWarpsPerGroup * 128);
    tstep_sb = (int64_t)p.total_groups * 16 * lds - (int64_t)p_nu * sbstep;
    p_fast_end = t0 + nrows / 16;
  };
  auto prod_valid = [&]() { return p_tl < ntl; };
  // copy the next item into its stage and step to the one after it
  auto issue = [&]() {
    cp_async16(wdst[0] + p_off, wp);
    cp_async16(wdst[1] + p_off, wp + roff[0]);
    cp_async16(wdst[2] + p_off, wp + roff[1]);
    cp_async16(wdst[3] + p_off, wp + roff[2]);
    if (BITS == 4 && p.gshift == 0) cp_async8(sbdst + p_off, sbp);
    else cp_async4(sbdst + p_off, sbp);
    p_off = p_off + kStageBytes == kStages * kStageBytes ? 0u : p_off + kStageBytes;
    wp += kWarpsPerGroup * 128;
    sbp += sbstep;
    if (++p_j == p_nu) {
      p_j = 0;
      ++p_tl;
      p_tile += p.total_groups;
      wp += tstep_w;
      sbp += tstep_sb;
      if (p_tl >= ntl) { p_tl = 0; ++p_pass; setup(); }
      else if (p_tile >= p_fast_end) setup();
    }
  };

  // per-lane byte offsets of the fragment reads of row g (row g+8 is +1024: same swizzle)
  int frag_off[U];
#pragma unroll
  for (int j = 0; j < U; ++j) {
    if (BITS == 4) frag_off[j] = g * 128 + (((2 * j + (t >> 1)) ^ swz_w<4>(g)) << 4) + (t & 1) * 8;
    else frag_off[j] = g * 128 + (((4 * j + t) ^ swz_w<8>(g)) << 4);
  }

  setup();
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) {
    if (prod_valid()) issue();
    cp_async_commit();
  }

  // Let the next grid in the stream begin launching, then wait for the previous grid to complete (and
  // its writes to be visible) before reading activations or writing outputs.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if constexpr (!M1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");

  uint32_t c_off = 0;   // byte offset of the stage the next unit is read from
  int red_buf = 0;

  for (int pass = 0; pass < p.npass; ++pass) {
    const int k_base = k_lo + pass * kc;
    const int klen = split ? k_cta : ((p.K - k_base) < kc ? (p.K - k_base) : kc);
    if (pass > 0) {  // every reader of the previous pass's fragments (cluster-wide) is done
      if constexpr (M1) __syncthreads(); else cluster_sync_all();
    }
    // ---- stage this pass's activations as s8 planes in B-fragment order ----
    // One thread converts 8 consecutive K values of one token; the 8 lanes that cover a 64-wide
    // group agree on the group's power-of-two scale (|x| * up < 2^14) through shuffles.  The conversion
    // v = rn(x * up) is one FMA onto 1.5 * 2^23: the low 16 bits of the sum's bit pattern are v in two's
    // complement, so the planes are cut out of pairs of values packed into one word.
    {
      const int cpt = klen >> 3;                         // 8-value chunks per token
      constexpr int PF = (M1 || NT == 2) ? 4 : 2;  // chunks fetched per thread before any is converted (loads in flight together)
      const bool al16 = ((((uintptr_t)p.x) | (uintptr_t)(p.ldx * (p.x_f32 ? 4 : 2))) & 15) == 0;  // k_base * element size is
      // The CTAs of a cluster take the tokens in turn and write what they convert into the shared memory of
      // all of them (K-split mode: every CTA converts its own K range of every token for itself).
      const int CS = (M1 || split) ? 1 : (int)cluster_size(), crank_b = (M1 || split) ? 0 : crank;
      uint32_t xdst[4] = {0u, 0u, 0u, 0u}, gdelta = 0u;   // a peer's gsc is the same distance behind its xfrag
      if constexpr (!M1) {
        const uint32_t xfrag_s = (uint32_t)__cvta_generic_to_shared(xfrag), gsc_s = (uint32_t)__cvta_generic_to_shared(gsc);
#pragma unroll
        for (int cr = 0; cr < 4; ++cr) {
          const uint32_t rk = split ? (uint32_t)crank : (uint32_t)(cr < CS ? cr : 0);
          xdst[cr] = map_to_rank(xfrag_s, rk);
        }
        gdelta = gsc_s - xfrag_s;
      }
      auto load = [&](auto f32tag, int m, int c, uint4& r0, uint4& r1) {
        constexpr bool F32 = decltype(f32tag)::value;
        const int64_t off = (int64_t)m * p.ldx + k_base + c * 8;
        if constexpr (!F32) {
          const uint16_t* px = (const uint16_t*)p.x + off;
          if (al16) {
            r0 = *(const uint4*)px;
          } else {
            uint32_t r[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) r[j] = (uint32_t)px[2 * j] | ((uint32_t)px[2 * j + 1] << 16);
            r0 = make_uint4(r[0], r[1], r[2], r[3]);
          }
        } else {
          const float* px = (const float*)p.x + off;
          if (al16) {
            r0 = *(const uint4*)px;
            r1 = *(const uint4*)(px + 4);
          } else {
            r0 = make_uint4(__float_as_uint(px[0]), __float_as_uint(px[1]), __float_as_uint(px[2]), __float_as_uint(px[3]));
            r1 = make_uint4(__float_as_uint(px[4]), __float_as_uint(px[5]), __float_as_uint(px[6]), __float_as_uint(px[7]));
          }
        }
      };
      // every lane of the warp calls this (shuffles); `ok` gates the stores
      auto convert = [&](auto f32tag, const uint4& a, const uint4& b2, int c, int m, bool ok) {
        constexpr bool F32 = decltype(f32tag)::value;
        float f[8];
        if constexpr (!F32) {
          f[0] = bf16lo(a.x); f[1] = bf16hi(a.x); f[2] = bf16lo(a.y); f[3] = bf16hi(a.y);
          f[4] = bf16lo(a.z); f[5] = bf16hi(a.z); f[6] = bf16lo(a.w); f[7] = bf16hi(a.w);
        } else {
          f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
          f[4] = __uint_as_float(b2.x); f[5] = __uint_as_float(b2.y); f[6] = __uint_as_float(b2.z); f[7] = __uint_as_float(b2.w);
        }
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) mx = fmax_nan(mx, fabsf(f[j]));
        mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        int e = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 + 1;  // mx < 2^e
        e = e < -100 ? -100 : (e > 110 ? 110 : e);
        const float up = __uint_as_float((uint32_t)(127 + 14 - e) << 23);
        const float down = poison_if(nonfinite(mx), __uint_as_float((uint32_t)(127 + e - 14) << 23));
        uint32_t w[8];   // bit patterns of 1.5 * 2^23 + v: 0x4B400000 + v
        uint32_t isum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float r = fmaf(f[j], up, 12582912.f);
          if constexpr (F32) r = fminf(r, 12599295.f);   // fp32 inputs may round up to 2^14: v <= 16383 (-2^14 fits the high plane)
          w[j] = __float_as_uint(r);
          isum += w[j];
        }
        isum += __shfl_xor_sync(0xffffffffu, isum, 1);
        isum += __shfl_xor_sync(0xffffffffu, isum, 2);
        isum += __shfl_xor_sync(0xffffffffu, isum, 4);
        const int sum = (int)(isum - 0xD0000000u);   // 64 values: 64 * 0x4B400000 mod 2^32
        if (!ok) return;
        uint32_t o[2][2];   // [plane][operand register]
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t p0 = __byte_perm(w[kslot8<BITS>(h, 0)], w[kslot8<BITS>(h, 1)], 0x5410);   // two 16-bit values
          const uint32_t p1 = __byte_perm(w[kslot8<BITS>(h, 2)], w[kslot8<BITS>(h, 3)], 0x5410);
          o[0][h] = __byte_perm((p0 >> 7) & 0x00FF00FFu, (p1 >> 7) & 0x00FF00FFu, 0x6420);   // (v >> 7) & 0xFF
          o[1][h] = __byte_perm(p0 & 0x007F007Fu, p1 & 0x007F007Fu, 0x6420);                 // v & 127
        }
        const int gi = c >> 3, tt = (c >> 1) & 3, jm = c & 1;  // 64-group, lane quarter, MMA of the group
        if constexpr (M1) {
          if ((c & 7) == 0) *(float2*)&gsc[gi * 2] = make_float2(down, down * (float)sum);
          uint2* d = xfrag + (gi * 8 + tt) * 2 + jm;   // 16 bytes per (group, column, lane quarter): both MMAs' operands
          d[0] = make_uint2(o[0][0], o[0][1]);
          d[8] = make_uint2(o[1][0], o[1][1]);
        } else {
          const int nt = m / kTokPerTile, ml = m - nt * kTokPerTile;
          const uint32_t xo = (uint32_t)((gi * NT + nt) * 32 + 2 * ml * 4 + tt) * 16u + (uint32_t)jm * 8u;
          const uint32_t go = (uint32_t)(((gi * kTokPerTile + ml) * NT + nt) * 2) * 4u;
#pragma unroll
          for (int cr = 0; cr < 4; ++cr) {
            if (cr < CS) {
              st_cluster_v2(xdst[cr] + xo, o[0][0], o[0][1]);
              st_cluster_v2(xdst[cr] + xo + 64u, o[1][0], o[1][1]);
              if ((c & 7) == 0) st_cluster_v2(xdst[cr] + gdelta + go, __float_as_uint(down), __float_as_uint(down * (float)sum));
            }
          }
        }
      };
      auto stage_all = [&](auto f32tag) {
        if constexpr (M1) {
          for (int c0 = 0; c0 < cpt; c0 += kThreads * PF) {
            uint4 raw[PF][2];
#pragma unroll
            for (int q = 0; q < PF; ++q) {
              const int c = c0 + q * kThreads + tid;
              raw[q][0] = raw[q][1] = make_uint4(0u, 0u, 0u, 0u);
              if (c < cpt) load(f32tag, 0, c, raw[q][0], raw[q][1]);
            }
#pragma unroll
            for (int q = 0; q < PF; ++q) {
              if (c0 + q * kThreads >= cpt) continue;
              const int c = c0 + q * kThreads + tid;
              convert(f32tag, raw[q][0], raw[q][1], c, 0, c < cpt);
            }
          }
        } else {
          for (int c0 = 0; c0 < cpt; c0 += kThreads) {
            const int c = c0 + tid;
            for (int m0 = crank_b; m0 < p.M; m0 += PF * CS) {
              uint4 raw[PF][2];
#pragma unroll
              for (int q = 0; q < PF; ++q) {
                const int m = m0 + q * CS;
                raw[q][0] = raw[q][1] = make_uint4(0u, 0u, 0u, 0u);
                if (m < p.M && c < cpt) load(f32tag, m, c, raw[q][0], raw[q][1]);
              }
#pragma unroll
              for (int q = 0; q < PF; ++q) {
                const int m = m0 + q * CS;
                if (m >= p.M) continue;
                convert(f32tag, raw[q][0], raw[q][1], c, m, c < cpt);
              }
            }
          }
        }
      };
      if (p.x_f32) stage_all(std::true_type{}); else stage_all(std::false_type{});
    }
    if constexpr (M1) __syncthreads(); else cluster_sync_all();
    const int upt = (ut - pass * upk) < upk ? (ut - pass * upk) : upk;
    const int ntl_rounds = split ? p.ntl_max : ntl;   // K-split: the same number of rounds in every group and CTA
    for (int tl0 = 0; tl0 < ntl_rounds; tl0 += RT) {
     const int rcnt = (ntl - tl0) < RT ? ((ntl - tl0) > 0 ? (ntl - tl0) : 0) : RT;
     float* rb = red + ((size_t)(grp * 2 + red_buf) * RT * kWarpsPerGroup) * NT * 64;
     for (int r = 0; r < rcnt; ++r) {

      float tot[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = 0.f;

      for (int u = ks; u < upt; u += kWarpsPerGroup) {
        // keep the ring full, then wait for this item's bytes
        if (prod_valid()) issue();
        cp_async_commit();
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const unsigned char* st = my_ring_p + c_off;
        c_off = c_off + kStageBytes == kStages * kStageBytes ? 0u : c_off + kStageBytes;

        // scales / biases of rows g and g+8 for the unit's U groups (bf16 pairs): 16 bytes per row
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
        // Fragments and group scales of this unit's U groups; every offset below is a compile-time constant.
        // Single token: only the two plane columns 0 and 1 of the n8 tile are read back (by the lanes
        // with t == 0), so the lanes that feed columns 2..7 may load anything: they re-read columns 0/1.
        const uint4* xb = M1 ? (const uint4*)xfrag + (size_t)(u * U) * 8 + (g & 1) * 4 + t
                             : (const uint4*)xfrag + (size_t)(u * U * NT) * 32 + lane;
        const float* gb = M1 ? gsc + (size_t)(u * U) * 2 : gsc + (size_t)((u * U * kTokPerTile + t) * NT) * 2;
        float2 gs1[U];   // single token: the unit's group scales, two groups per load
        if constexpr (M1) {
#pragma unroll
          for (int j = 0; j < U; j += 2) {
            const float4 v = *(const float4*)&gb[j * 2];
            gs1[j] = make_float2(v.x, v.y); gs1[j + 1] = make_float2(v.z, v.w);
          }
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
          uint32_t a0[2], a1[2], a2[2], a3[2];  // [mma]: row g lo, row g+8 lo, row g hi, row g+8 hi
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
          if constexpr (M1) {
            int acc[4];
            const uint4 bf = xb[j * 8];
            mma_u8s8_z(acc, a0[0], a1[0], a2[0], a3[0], bf.x, bf.y);
            mma_u8s8(acc, a0[1], a1[1], a2[1], a3[1], bf.z, bf.w);
            const float2 gs = gs1[j];
            const float f_lo = (float)(acc[0] * 128 + acc[1]), f_hi = (float)(acc[2] * 128 + acc[3]);
            tot[0][0] = fmaf(s_lo * gs.x, f_lo, fmaf(b_lo, gs.y, tot[0][0]));
            tot[0][1] = fmaf(s_hi * gs.x, f_hi, fmaf(b_hi, gs.y, tot[0][1]));
          } else {
            float2 gsn[NT];   // this lane's token of every tile
            if constexpr (NT == 2) {
              const float4 v = *(const float4*)&gb[j * kTokPerTile * NT * 2];
              gsn[0] = make_float2(v.x, v.y); gsn[NT - 1] = make_float2(v.z, v.w);
            } else {
              gsn[0] = *(const float2*)&gb[j * kTokPerTile * NT * 2];
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              int acc[4];
              const uint4 bf = xb[(j * NT + nt) * 32];
              mma_u8s8_z(acc, a0[0], a1[0], a2[0], a3[0], bf.x, bf.y);
              mma_u8s8(acc, a0[1], a1[1], a2[1], a3[1], bf.z, bf.w);
              const float2 gs = gsn[nt];
              const float f_lo = (float)(acc[0] * 128 + acc[1]), f_hi = (float)(acc[2] * 128 + acc[3]);
              tot[nt][0] = fmaf(s_lo * gs.x, f_lo, fmaf(b_lo, gs.y, tot[nt][0]));
              tot[nt][1] = fmaf(s_hi * gs.x, f_hi, fmaf(b_hi, gs.y, tot[nt][1]));
            }
          }
        }
        __syncwarp();
      }

      // partial sums of this tile: red[buf][r][ks][nt][row 16][token 4]
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float* base = rb + (((size_t)r * kWarpsPerGroup + ks) * NT + nt) * 64;
        base[g * 4 + t] = tot[nt][0];
        base[(g + 8) * 4 + t] = tot[nt][1];
      }
     }
     // ---- one barrier per round: reduce the group's 8 K-slices of up to RT tiles ----
     group_barrier(grp);
     const int gt = tid - grp * (kWarpsPerGroup * 32);  // thread index inside the group
     const int ncols = M1 ? 1 : NT * kTokPerTile;
     if (split) {
       // RT * NT == 4, so a round has at most 256 outputs per group: one per thread
       const int o = gt;
       const int row = o & 15, rc = o >> 4;
       const int r = rc / ncols, col = rc - r * ncols;
       const int nt = col / kTokPerTile, c = col - nt * kTokPerTile;
       const bool live = o < rcnt * 16 * ncols;
       float v = 0.f;
       if (live) {
#pragma unroll
         for (int k = 0; k < kWarpsPerGroup; ++k) v += rb[(((size_t)r * kWarpsPerGroup + k) * NT + nt) * 64 + row * 4 + c];
       }
       float* slot0 = xred + ((size_t)red_buf * (p.ksplit - 1) * kGroups + grp) * 256 + gt;  // peer 1's slot of this round
       if (crank != 0)
         st_cluster_f32(map_to_rank((uint32_t)__cvta_generic_to_shared(slot0 + (size_t)(crank - 1) * kGroups * 256), 0), v);
       cluster_sync_all();
       if (crank == 0 && live) {
         for (int k = 0; k + 1 < p.ksplit; ++k) v += slot0[(size_t)k * kGroups * 256];
         const int tile = ggrp + (tl0 + r) * p.total_groups;
         const int mi = mat_of_tile(p, tile);
         const int n = (tile - QB_SEL4(p.tile0, mi)) * 16 + row;
         if (n < QB_SEL4(p.N, mi) && col < p.M) {
           void* ym = QB_SEL4(p.y, mi);
           const int64_t ldy = QB_SEL4(p.ldy, mi);
           if (p.x_f32) ((float*)ym)[(int64_t)col * ldy + n] = v;
           else ((uint16_t*)ym)[(int64_t)col * ldy + n] = f32_to_bf16_bits(v);
         }
       }
     } else
     for (int o = gt; o < rcnt * 16 * ncols; o += kWarpsPerGroup * 32) {
        const int row = o & 15, rc = o >> 4;
        const int r = rc / ncols, col = rc - r * ncols;
        const int nt = col / kTokPerTile, c = col - nt * kTokPerTile;
        const int tl = tl0 + r;
        const int tile = ggrp + tl * p.total_groups;
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < kWarpsPerGroup; ++k) v += rb[(((size_t)r * kWarpsPerGroup + k) * NT + nt) * 64 + row * 4 + c];
        if (p.npass > 1) {
          float* ya = yacc + ((size_t)(grp * p.ntl_max + tl) * NT * 64) + col * 16 + row;
          if (pass > 0) v += *ya;
          if (pass + 1 < p.npass) { *ya = v; continue; }
        }
        const int mi = mat_of_tile(p, tile);
        const int n = (tile - QB_SEL4(p.tile0, mi)) * 16 + row;
        if (n < QB_SEL4(p.N, mi) && col < p.M) {
          void* ym = QB_SEL4(p.y, mi);
          const int64_t ldy = QB_SEL4(p.ldy, mi);
          if (p.x_f32) ((float*)ym)[(int64_t)col * ldy + n] = v;
          else ((uint16_t*)ym)[(int64_t)col * ldy + n] = f32_to_bf16_bits(v);
        }
     }
     red_buf ^= 1;
    }
  }
  cp_async_wait<0>();
}



// Grid, K passes and shared-memory footprint of one instantiation; false when it does not fit.
bool plan_stream(StreamK& p, int NT, bool M1, int* grid_out, size_t* smem_out, int* cluster_out = nullptr, int cluster = 1,
                 int max_ctas = 0, int ck = 256, int split_cluster = 0, int split_ctas = 0) {
  int nsm = sm_count() * (M1 ? 2 : 1);  // CTA slots
  if (max_ctas > 0 && max_ctas < nsm) nsm = max_ctas;
  const int kGroups = groups_for(M1);
  int ntiles = 0;
  for (int i = 0; i < p.nmat; ++i) { p.tile0[i] = ntiles; ntiles += (p.N[i] + 15) / 16; }
  for (int i = p.nmat; i <= kMaxMat; ++i) p.tile0[i] = ntiles;
  p.ntiles = ntiles;
  p.ksplit = 1;
  p.upc = 0;
  // K-split across the cluster: when K does not fit one staging pass, but a cluster's share of it does
  // and still gives every warp of a group at least one unit per tile.
  if (!M1 && split_cluster > 1 && p.K > kc_for(NT)) {
    const int ut = p.K / ck, upc = (ut + split_cluster - 1) / split_cluster;
    if (upc * ck <= kc_for(NT) && upc >= kWarpsPerGroup) { p.ksplit = split_cluster; p.upc = upc; }
  }
  int grid;
  if (p.ksplit > 1) {
    cluster = split_cluster;
    const int nclus = (split_ctas > 0 ? split_ctas : nsm) / cluster;
    const int groups = ntiles < kGroups * nclus ? ntiles : kGroups * nclus;
    const int used = (groups + kGroups - 1) / kGroups;
    grid = used * cluster;
    p.total_groups = used * kGroups;
    p.kc = p.upc * ck;
  } else {
    const int total_groups = ntiles < kGroups * nsm ? ntiles : kGroups * nsm;
    grid = (total_groups + kGroups - 1) / kGroups;
    grid = (grid + cluster - 1) / cluster * cluster;   // whole clusters; CTAs beyond the tiles only help staging
    p.total_groups = grid * kGroups;
    p.kc = p.K < kc_for(NT) ? p.K : kc_for(NT);
    if (M1) p.kc = p.K;
  }
  p.ntl_max = (ntiles + p.total_groups - 1) / p.total_groups;
  p.npass = p.ksplit > 1 ? 1 : (p.K + p.kc - 1) / p.kc;
  size_t smem = (size_t)kGroups * kWarpsPerGroup * stages_for(NT) * kStageBytes;
  smem += M1 ? (size_t)(p.kc / 32) * 64 : (size_t)(p.kc / 32) * NT * 256;
  smem += M1 ? (size_t)(p.kc / 64) * 8 : (size_t)(p.kc / 64) * NT * kTokPerTile * 8;
  smem += (size_t)kGroups * 2 * rt_for(NT, M1) * kWarpsPerGroup * NT * 256;
  smem += 16;
  if (p.npass > 1) smem += (size_t)kGroups * p.ntl_max * NT * 256;
  if (p.ksplit > 1) smem += (size_t)2 * (p.ksplit - 1) * kGroups * 256 * 4;
  *grid_out = grid;
  *smem_out = smem;
  if (cluster_out) *cluster_out = cluster;
  return smem <= (size_t)(M1 ? 113 : 227) * 1024;
}

void pick_inst(const StreamK& p, int* NT, bool* M1) {
  const int nt = (p.M + kTokPerTile - 1) / kTokPerTile;
  *M1 = (p.M == 1 && p.K <= 65536);
  *NT = nt <= 1 ? 1 : 2;
}

template <int BITS, int NT, bool M1>
cudaError_t launch_inst(StreamK p, cudaStream_t st) {
  auto kern = qmv_stream_kernel<BITS, NT, M1>;
  static bool attr_done[64] = {};
  static int cluster_of[64] = {}, max_ctas_of[64] = {}, split_cluster_of[64] = {}, split_ctas_of[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int di = (dev >= 0 && dev < 64) ? dev : 0;
  std::unique_lock<std::mutex> setup_lk(setup_mutex());   // first use on a device, from any thread
  if (!attr_done[di] || di != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    // Cluster size for the shared activation staging: the largest of 4, 2 whose co-resident clusters (at the
    // full shared-memory footprint) still cover at least 97% of the SMs; 1 otherwise.  The K-split mode
    // needs 4 and accepts losing up to 15% of the SMs to cluster placement.
    int cs = 1, ctas = sm_count(), scs = 0, sctas = 0;
    if (!M1) {
      for (int c = 4; c >= 2; c >>= 1) {
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3((sm_count() / c) * c);
        q.blockDim = dim3(kWarpsPerGroup * groups_for(M1) * 32);
        q.dynamicSmemBytes = 227 * 1024;
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = c; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
        q.attrs = qa;
        q.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        const int covered = n * c < sm_count() ? n * c : (sm_count() / c) * c;
        if (c == 4 && covered * 100 >= sm_count() * 85) { scs = 4; sctas = covered; }
        if (cs == 1 && covered * 100 >= sm_count() * 97) { cs = c; ctas = covered; }
      }
    }
    cluster_of[di] = cs; max_ctas_of[di] = ctas; split_cluster_of[di] = scs; split_ctas_of[di] = sctas;
    attr_done[di] = true;
  }
  int cs = cluster_of[di];
  const int max_ctas = max_ctas_of[di];
  const int split_cluster = split_cluster_of[di], split_ctas = split_ctas_of[di];
  setup_lk.unlock();
  int grid = 0;
  size_t smem = 0;
  if (!plan_stream(p, NT, M1, &grid, &smem, &cs, cs, M1 ? 0 : max_ctas, BITS == 4 ? 256 : 128, split_cluster, split_ctas))
    return cudaErrorInvalidConfiguration;
  // Programmatic dependent launch: this grid may start (and prefetch weights, which no kernel writes)
  // before the previous grid in the stream has finished; it waits for that grid before touching x or y.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kWarpsPerGroup * groups_for(M1) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cs; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (!M1 && cs > 1) ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int BITS>
cudaError_t launch_bits(const StreamK& p, cudaStream_t st) {
  int nt; bool m1;
  pick_inst(p, &nt, &m1);
  if (m1) return launch_inst<BITS, 1, true>(p, st);
  if (nt == 1) return launch_inst<BITS, 1, false>(p, st);
  return launch_inst<BITS, 2, false>(p, st);
}

}  // namespace

bool qmv_stream_supported(const QmmArgs& a) {
  if (!a.transpose) return false;
  if (!((a.bits == 4 && (a.gs == 64 || a.gs == 128)) || (a.bits == 8 && a.gs == 64))) return false;
  if (a.x_dtype != QB200_BFLOAT16 && a.x_dtype != QB200_FLOAT32) return false;
  if (a.K % 256 != 0 || a.K <= 0 || a.K > (1 << 20)) return false;
  if (a.N <= 0 || a.N > (1 << 24) || a.M <= 0) return false;
  if (a.nbatch != 1) return false;
  if ((((uintptr_t)a.w) & 15) != 0 || (a.ldw * 4) % 16 != 0) return false;
  if ((((uintptr_t)a.s) & 7) != 0 || (((uintptr_t)a.b) & 7) != 0) return false;
  if (a.gs == 64 && a.lds % 4 != 0) return false;
  if (a.gs == 128 && (a.lds % 2) != 0) return false;
  StreamK p;
  p.nmat = 1; p.N[0] = (int)a.N; p.K = (int)a.K; p.x_f32 = a.x_dtype == QB200_FLOAT32;
  p.M = (int)(a.M < kMaxTok ? a.M : kMaxTok);
  int nt, grid; bool m1; size_t smem;
  pick_inst(p, &nt, &m1);
  if (!plan_stream(p, nt, m1, &grid, &smem)) return false;
  return true;
}

// `count` (<= 4) weight matrices applied to the same activations in one launch.  Every entry must
// have passed qmv_stream_supported and share x, M, K, dtype, bits and group size with the first.
cudaError_t launch_qmv_stream_multi(const QmmArgs* a, int count, cudaStream_t st) {
  StreamK p;
  p.nmat = count;
  for (int i = 0; i < kMaxMat; ++i) {
    const QmmArgs& q = a[i < count ? i : 0];
    p.w[i] = q.w + q.wb.offset(0);
    p.s[i] = (const uint16_t*)q.s + q.sb.offset(0);
    p.b[i] = (const uint16_t*)q.b + q.sb.offset(0);
    p.N[i] = i < count ? (int)q.N : 0;
    p.ldw[i] = q.ldw; p.lds[i] = q.lds; p.ldy[i] = q.ldy;
  }
  p.K = (int)a[0].K;
  p.ldx = a[0].ldx;
  p.gshift = a[0].gs == 128 ? 1 : 0;
  p.x_f32 = a[0].x_dtype == QB200_FLOAT32;
  const int esz = p.x_f32 ? 4 : 2;
  // wider M re-streams the weights once per block of kMaxTok tokens
  for (int64_t m0 = 0; m0 < a[0].M; m0 += kMaxTok) {
    p.x = (const char*)a[0].x + (a[0].xb.offset(0) + m0 * a[0].ldx) * esz;
    for (int i = 0; i < kMaxMat; ++i) {
      const QmmArgs& q = a[i < count ? i : 0];
      p.y[i] = (char*)q.y + (q.yb.offset(0) + m0 * q.ldy) * esz;
    }
    p.M = (int)((a[0].M - m0) < kMaxTok ? (a[0].M - m0) : kMaxTok);
    cudaError_t e = a[0].bits == 4 ? launch_bits<4>(p, st) : launch_bits<8>(p, st);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t launch_qmv_stream(const QmmArgs& a, cudaStream_t st) { return launch_qmv_stream_multi(&a, 1, st); }

}  // namespace qb

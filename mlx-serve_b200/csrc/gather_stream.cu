// Routed-MoE gather_qmm at decode widths: res[i] = x[lhs(i)] . What[rhs[i]]^T.
//
// Replaces mlx_gather_qmm as called by gatherExpertMm (mlx-serve
// src/transformer.zig:20763-20784) for both call shapes of moeMLP2 -- rows
// sorted by expert ([N,1,D] + rhs [N], src/transformer.zig:15007-15035) and the
// stock decode shape (x [B,S,1,1,D] + rhs [B,S,K], src/transformer.zig:15091-15119)
// -- and, like the reference's single-token gatherQmv kernels
// (src/transformer.zig:20046-20109), it reads each routed expert's packed bank
// in place, once.
//
// Decomposition (HBM-bound, one pass over every expert that is hit):
//  * a persistent grid (one CTA of 16 warps per SM).  Every CTA derives the same
//    per-expert row counts from rhs.  An expert with c rows costs ceil(c/8)
//    sweeps over its N/16 row tiles; the (expert, sweep, tile) triples are
//    numbered in that order and CTA i takes the i-th equal share of the
//    numbering, so every SM streams the same number of tiles however the
//    router spread the rows.
//  * for each (expert, sweep) segment of its share the CTA looks up the sweep's
//    output rows (in ascending order of their position in rhs, so that all CTAs
//    agree; `sorted_indices` is never needed for correctness), stages their
//    activations as two s8 fixed-point planes per row (8 rows per sweep), and
//    each warp owns whole 16-row tiles: it streams the tile's K range through a
//    private cp.async ring, multiplies on the integer tensor cores
//    (mma.m16n8k32.u8.s8, codes as the A operand) and stores its 16 x rows
//    results straight from registers.  No cross-warp reduction, no barriers in
//    the streaming loop, nothing written to global scratch.
// Arithmetic is that of the dense streaming kernel: exact s32 dots of codes with
// 15-bit fixed-point activations, scale and bias applied per 64-wide group in
// fp32; the weight term q*s+b is never rounded to bf16.
#include <cmath>
#include <cstring>
#include <type_traits>

#include <mutex>

#include "kernels.h"
#include "stream_ptx.cuh"

namespace qb {
namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;
constexpr int kStageW = 2048;                 // 16 rows x 128 B of packed codes
constexpr int kStageBytes = kStageW + 256;    // + scales, biases
constexpr int kRowsPerSweep = 8;              // two n8 tiles of (4 rows x 2 planes)
constexpr int kMaxExperts = 1024;
constexpr int kMaxRows = 2048;                // rows of one expert kept in shared memory

struct GK {
  const void* x; const uint32_t* w; const uint16_t* s; const uint16_t* b; void* y;
  const void* rhs; const void* lhs;
  int rhs_i64, lhs_i64;
  BatchMap xbcast;
  int64_t I, E, XB, xstride, wes, ses;
  int N, K, gshift, x_f32;
  int nsb;   // (expert, sweep) segments staged together: 2 when their fragments fit beside the ring, else 1
  // fused gate/up form: a second bank of the same geometry; y = silu(x . gate^T) * (x . up^T)
  const uint32_t* w2; const uint16_t* s2; const uint16_t* b2;
  const uint16_t* sigtab;   // sigmoid of every bf16 pattern, as bf16
};

__device__ __forceinline__ long long load_index(const void* p, int is64, int64_t i) {
  return is64 ? ((const long long*)p)[i] : (long long)((const uint32_t*)p)[i];
}


template <int BITS, bool FUSED>
__global__ void __launch_bounds__(kThreads, 1) gather_stream_kernel(GK p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int U = BITS == 4 ? 4 : 2;   // 64-wide groups per unit
  constexpr int CK = 64 * U;             // K values per unit (128 bytes per row)
  constexpr int NT = 2;
  __shared__ int s_cum[kMaxExperts + 1];        // tiles of work before expert e (exclusive prefix), [E] = total
  __shared__ int s_cnt[kMaxExperts];            // rows routed to expert e
  __shared__ unsigned short s_rhs[kMaxRows];    // expert of every output row (0xFFFF: out of range)
  __shared__ long long s_xi[2 * kRowsPerSweep]; // activation row of each slot of each staged segment (-1: empty)
  __shared__ int s_orow[2 * kRowsPerSweep];     // output row of each slot (-1: empty)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  unsigned char* sp = smem;
  unsigned char* ring = sp;    sp += (size_t)kWarps * kStages * kStageBytes;
  uint2* xfrag = (uint2*)sp;   sp += (size_t)p.nsb * (p.K / 32) * NT * 32 * 8;   // per staged segment
  float* gsc = (float*)sp;     sp += (size_t)p.nsb * (p.K / 64) * NT * 4 * 8;   // [(group*NT + nt)*4 + row][2]: (2^(E-14), 2^(E-14) * sum v)
  float* red = (float*)sp;     // [warp][nt][2][lane]: partial sums of warps that share a tile's K range
  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(ring + (size_t)warp * kStages * kStageBytes);
  const unsigned char* my_ring_p = ring + (size_t)warp * kStages * kStageBytes;

  // The indices (and activations) may come from the previous kernel in the stream.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- every CTA derives the same per-expert row counts and the prefix of their cost in tiles ----
  const int E = (int)p.E, I = (int)p.I;
  const int tiles_n = (p.N + 15) / 16;
  for (int i = tid; i < E; i += kThreads) s_cnt[i] = 0;
  __syncthreads();
  for (int i = tid; i < I; i += kThreads) {
    const long long e = load_index(p.rhs, p.rhs_i64, i);
    const bool in = e >= 0 && e < p.E;
    s_rhs[i] = in ? (unsigned short)e : (unsigned short)0xFFFF;
    if (in) atomicAdd(&s_cnt[(int)e], 1);
  }
  __syncthreads();
  if (warp == 0) {
    int base = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int cost = e < E ? ((s_cnt[e] + kRowsPerSweep - 1) / kRowsPerSweep) * tiles_n : 0;
      int inc = cost;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
      }
      if (e < E) s_cum[e] = base + inc - cost;
      base += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) s_cum[E] = base;
  }
  __syncthreads();
  const int W = s_cum[E];
  if (W == 0) return;
  // This CTA's share [lo, hi) of the numbering.  With many (expert, sweep) segments: equal shares, which
  // may straddle two segments.  With few (single-token decode): every segment is cut into the same number
  // of chunks so that no CTA pays the per-segment set-up twice.
  int lo, hi;
  const int nseg = W / tiles_n;
  if (nseg * 2 <= (int)gridDim.x) {
    const int cps = (int)gridDim.x / nseg;                 // chunks per segment
    const int c = (tiles_n + cps - 1) / cps;               // tiles per chunk
    const int seg = blockIdx.x / cps, ch = blockIdx.x - seg * cps;
    if (seg >= nseg || ch * c >= tiles_n) return;
    lo = seg * tiles_n + ch * c;
    hi = (ch + 1) * c < tiles_n ? lo + c : (seg + 1) * tiles_n;
  } else {
    lo = (int)((long long)W * blockIdx.x / gridDim.x);
    hi = (int)((long long)W * (blockIdx.x + 1) / gridDim.x);
  }
  const int ut = p.K / CK;

  // per-lane constants of the ring
  const int chunk = lane & 7;
  uint32_t wdst[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = (lane >> 3) + 4 * r;
    wdst[r] = row * 128 + ((chunk ^ swz_w<BITS>(row)) << 4);
  }
  const uint32_t sbdst = kStageW + (lane & 15) * 16 + (lane >> 4) * 8;   // per row: scales | biases
  int frag_off[U];
#pragma unroll
  for (int j = 0; j < U; ++j) {
    if (BITS == 4) frag_off[j] = g * 128 + (((2 * j + (t >> 1)) ^ swz_w<4>(g)) << 4) + (t & 1) * 8;
    else frag_off[j] = g * 128 + (((4 * j + t) ^ swz_w<8>(g)) << 4);
  }

  int e = 0;
  {  // first expert whose share of the numbering reaches past lo (s_cum is non-decreasing)
    int a = 0, b = E;  // invariant: s_cum[a] <= lo < s_cum[b]
    while (b - a > 1) {
      const int m = (a + b) >> 1;
      if (s_cum[m] <= lo) a = m; else b = m;
    }
    e = a;
  }
  const int64_t ldw = (int64_t)p.K * BITS / 32, lds = p.K >> (6 + p.gshift);
  // fused form: the second bank has the first one's geometry, so its stage sources are a constant away
  const int64_t wdelta = FUSED ? (const unsigned char*)p.w2 - (const unsigned char*)p.w : 0;           // bytes
  const int64_t sbdelta = FUSED ? ((lane >> 4) ? p.b2 - p.b : p.s2 - p.s) : 0;                          // entries
  const int xf_stride = (p.K / 32) * NT * 32;       // uint2 elements of one segment's fragments
  const int gs_stride = (p.K / 64) * NT * 4 * 2;    // floats of one segment's group scales
  for (int pos = lo; pos < hi;) {
    // ---- up to p.nsb consecutive (expert, sweep) segments of the share are staged together, so that the
    //      weight stream does not drain at the boundary between two experts ----
    int e0 = 0, r00 = 0, t00 = 0, nt0 = 0, e1 = 0, r01 = 0, t01 = 0, nt1 = 0;
    {
      while (s_cum[e + 1] <= pos) ++e;           // skips experts without rows
      int off = pos - s_cum[e];
      int sweep = off / tiles_n;
      e0 = e; r00 = sweep * kRowsPerSweep; t00 = off - sweep * tiles_n;
      nt0 = (t00 + (hi - pos)) < tiles_n ? (hi - pos) : tiles_n - t00;
      pos += nt0;
      if (p.nsb > 1 && pos < hi) {
        while (s_cum[e + 1] <= pos) ++e;
        off = pos - s_cum[e];
        sweep = off / tiles_n;
        e1 = e; r01 = sweep * kRowsPerSweep; t01 = off - sweep * tiles_n;
        nt1 = (t01 + (hi - pos)) < tiles_n ? (hi - pos) : tiles_n - t01;
        pos += nt1;
      }
    }
    const int ntb = nt0 + nt1;                    // tiles of this batch, numbered j = 0 .. ntb-1
    const uint32_t* wexp0 = p.w + (int64_t)e0 * p.wes;
    const uint16_t* sexp0 = p.s + (int64_t)e0 * p.ses;
    const uint16_t* bexp0 = p.b + (int64_t)e0 * p.ses;
    const uint32_t* wexp1 = p.w + (int64_t)e1 * p.wes;
    const uint16_t* sexp1 = p.s + (int64_t)e1 * p.ses;
    const uint16_t* bexp1 = p.b + (int64_t)e1 * p.ses;
    const int nte0 = (s_cnt[e0] - r00) > 4 ? 2 : 1;             // n8 tiles in use per segment
    const int nte1 = nt1 > 0 && (s_cnt[e1] - r01) > 4 ? 2 : 1;

    // ---- start streaming this warp's weights right away: they do not depend on the activations.
    //      Each warp owns whole 16-row tiles; when the batch has fewer tiles than the CTA has warps,
    //      `ksplit` warps share a tile's K range and reduce through shared memory ----
    int ksplit = 1;
    while (ksplit * 2 * ntb <= kWarps && ksplit * 2 <= ut) ksplit *= 2;
    const int kp = warp % ksplit;
    const int first = ksplit == 1 ? warp : warp / ksplit;
    const int my_tiles = first < ntb ? (ksplit == 1 ? (ntb - first + kWarps - 1) / kWarps : 1) : 0;
    const int nu = (ut - kp + ksplit - 1) / ksplit;   // units of one tile handled by this warp
    const int total = my_tiles * nu * (FUSED ? 2 : 1);   // fused form: every unit of both banks, first bank first
    int issued = 0, ptile = 0, pu = kp;  // producer position: (tile index, unit)
    int pbank = 0;                       // fused form: bank of the next item
    uint32_t p_off = 0, c_off = 0;       // byte offsets of the stages the next item is copied to / read from
    // per-lane source pointers of the producer's current tile (recomputed when the tile changes)
    const unsigned char* wsrc[4] = {nullptr, nullptr, nullptr, nullptr};
    const uint16_t* sbsrc = nullptr;
    int cached_tile = -1;
    auto issue = [&]() {
      if (ptile != cached_tile) {
        cached_tile = ptile;
        const int j = first + ptile * kWarps;
        const bool sg = j >= nt0;
        const int tile = sg ? t01 + (j - nt0) : t00 + j;
        const uint32_t* wexp = sg ? wexp1 : wexp0;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          int n = tile * 16 + (lane >> 3) + 4 * r;
          n = n < p.N ? n : p.N - 1;
          wsrc[r] = (const unsigned char*)(wexp + (int64_t)n * ldw) + chunk * 16;
        }
        int n = tile * 16 + (lane & 15);
        n = n < p.N ? n : p.N - 1;
        sbsrc = ((lane >> 4) ? (sg ? bexp1 : bexp0) : (sg ? sexp1 : sexp0)) + (int64_t)n * lds;
      }
      const uint32_t st = my_ring + p_off;
      p_off = p_off + kStageBytes == kStages * kStageBytes ? 0u : p_off + kStageBytes;
      const int64_t woff = (int64_t)pu * 128 + ((FUSED && pbank) ? wdelta : 0);
#pragma unroll
      for (int r = 0; r < 4; ++r) cp_async16(st + wdst[r], wsrc[r] + woff);
      const uint16_t* ssrc = sbsrc + ((pu * U) >> p.gshift) + ((FUSED && pbank) ? sbdelta : 0);
      if (BITS == 4 && p.gshift == 0) cp_async8(st + sbdst, ssrc);
      else cp_async4(st + sbdst, ssrc);
      if (FUSED) { pbank ^= 1; if (pbank) return; }
      pu += ksplit;
      if (pu >= ut) { pu = kp; ++ptile; }
    };
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {
      if (issued < total) issue();
      cp_async_commit();
      ++issued;
    }

    __syncthreads();  // the previous batch has finished with the fragments and the slots
    // ---- rows r0 .. r0+7 of each segment's expert in ascending rhs position (one warp per segment) ----
    if (warp < 2 && (warp == 0 || nt1 > 0)) {
      const int es = warp ? e1 : e0, r0 = warp ? r01 : r00;
      long long* xi_s = s_xi + warp * kRowsPerSweep;
      int* orow_s = s_orow + warp * kRowsPerSweep;
      if (lane < kRowsPerSweep) { xi_s[lane] = -1; orow_s[lane] = -1; }
      __syncwarp();
      int seen = 0;
      for (int i0 = 0; i0 < I && seen < r0 + kRowsPerSweep; i0 += 32) {
        const int i = i0 + lane;
        const bool hit = i < I && s_rhs[i] == (unsigned short)es;
        const unsigned bal = __ballot_sync(0xffffffffu, hit);
        const int rank = seen + __popc(bal & ((1u << lane) - 1u));
        if (hit && rank >= r0 && rank < r0 + kRowsPerSweep) {
          long long xi = p.lhs ? load_index(p.lhs, p.lhs_i64, i) : (long long)p.xbcast.offset(i);
          int orow = i;
          if (xi < 0 || xi >= p.XB) { xi = -1; orow = -1; }
          xi_s[rank - r0] = xi;
          orow_s[rank - r0] = orow;
        }
        seen += __popc(bal);
      }
    }
    __syncthreads();
    // ---- stage the rows' activations as s8 planes in B-fragment order (one thread: 8 K values) ----
    // v = rn(x * up) is one FMA onto 1.5 * 2^23 (the low 16 bits of the sum's bit pattern are v in two's
    // complement); the two planes are cut out of pairs of values packed into one word.
    // thread -> (row of the pass, 8-value chunk); K <= 4096, so one pass covers every chunk of a row
    const int st_cpt = p.K >> 3;
    const int st_rpp = kThreads / st_cpt;               // rows converted per pass
    const int st_mr = tid / st_cpt, st_cr = tid - st_mr * st_cpt;
    for (int sg = 0; sg < (nt1 > 0 ? 2 : 1); ++sg) {
      const int nrows = (sg ? nte1 : nte0) * 4;
      uint2* xf = xfrag + sg * xf_stride;
      float* gsb = gsc + sg * gs_stride;
      const long long* xi_s = s_xi + sg * kRowsPerSweep;
      constexpr int PF = 2;   // rows fetched per thread before any is converted
      for (int mb = 0; mb < nrows; mb += PF * st_rpp) {
        uint4 raw[PF][2];
        bool okq[PF];
#pragma unroll
        for (int q = 0; q < PF; ++q) {
          const int m = mb + q * st_rpp + st_mr;
          okq[q] = st_mr < st_rpp && m < nrows;
          raw[q][0] = raw[q][1] = make_uint4(0u, 0u, 0u, 0u);
          const long long xi = okq[q] ? xi_s[m] : -1;
          if (xi >= 0) {
            const int64_t off = xi * p.xstride + (int64_t)st_cr * 8;
            if (!p.x_f32) {
              raw[q][0] = *(const uint4*)((const uint16_t*)p.x + off);
            } else {
              raw[q][0] = *(const uint4*)((const float*)p.x + off);
              raw[q][1] = *(const uint4*)((const float*)p.x + off + 4);
            }
          }
        }
#pragma unroll
        for (int q = 0; q < PF; ++q) {
          if (mb + q * st_rpp >= nrows) continue;
          const int m = mb + q * st_rpp + st_mr, c = st_cr;
          float f[8];
          const uint4 a = raw[q][0], b2 = raw[q][1];
          if (!p.x_f32) {
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
          int ex = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 + 1;  // mx < 2^ex
          ex = ex < -100 ? -100 : (ex > 110 ? 110 : ex);
          const float up = __uint_as_float((uint32_t)(127 + 14 - ex) << 23);
          const float down = poison_if(nonfinite(mx), __uint_as_float((uint32_t)(127 + ex - 14) << 23));
          uint32_t w[8], isum = 0;   // bit patterns 0x4B400000 + v
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            w[j] = __float_as_uint(fminf(fmaf(f[j], up, 12582912.f), 12599295.f));   // v <= 16383 (fp32 inputs may round up to 2^14)
            isum += w[j];
          }
          isum += __shfl_xor_sync(0xffffffffu, isum, 1);
          isum += __shfl_xor_sync(0xffffffffu, isum, 2);
          isum += __shfl_xor_sync(0xffffffffu, isum, 4);
          const int sum = (int)(isum - 0xD0000000u);   // 64 values: 64 * 0x4B400000 mod 2^32
          if (!okq[q]) continue;
          const int gi = c >> 3, tt = (c >> 1) & 3, jm = c & 1;
          const int nt = m >> 2, ml = m & 3;
          if ((c & 7) == 0) *(float2*)&gsb[((gi * 4 + ml) * NT + nt) * 2] = make_float2(down, down * (float)sum);
          uint32_t o[2][2];   // [plane][operand register]
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t p0 = __byte_perm(w[kslot8<BITS>(h, 0)], w[kslot8<BITS>(h, 1)], 0x5410);   // two 16-bit values
            const uint32_t p1 = __byte_perm(w[kslot8<BITS>(h, 2)], w[kslot8<BITS>(h, 3)], 0x5410);
            o[0][h] = __byte_perm((p0 >> 7) & 0x00FF00FFu, (p1 >> 7) & 0x00FF00FFu, 0x6420);   // (v >> 7) & 0xFF
            o[1][h] = __byte_perm(p0 & 0x007F007Fu, p1 & 0x007F007Fu, 0x6420);                 // v & 127
          }
          // 16 bytes per (group, tile, column, lane quarter): the operands of both MMAs of the group
          uint2* d = xf + (((gi * NT + nt) * 32 + 2 * ml * 4 + tt) * 2 + jm);
          d[0] = make_uint2(o[0][0], o[0][1]);
          d[8] = make_uint2(o[1][0], o[1][1]);
        }
      }
    }
    __syncthreads();
    // lane (g, t) holds weight rows g, g+8 of a tile for the row in slot nt*4 + t of the tile's segment
    // fused form: silu(gate) * up with the reference's rounding points (src/transformer.zig:19842-19851): the
    // sigmoid of the rounded gate from the table of all bf16 patterns, each product rounded to the output type
    auto swiglu16 = [&](float gate, float up) -> uint16_t {
      const uint32_t g16 = f32_to_bf16_bits(gate);
      const float gf = __uint_as_float(g16 << 16), sig = __uint_as_float((uint32_t)p.sigtab[g16] << 16);
      const float act = __uint_as_float((uint32_t)f32_to_bf16_bits(gf * sig) << 16);
      const float uf = __uint_as_float((uint32_t)f32_to_bf16_bits(up) << 16);
      return f32_to_bf16_bits(act * uf);
    };
    auto swiglu32 = [&](float gate, float up) -> float {
      const float sy = 1.f / (1.f + expf(fabsf(gate)));
      return (gate * (gate < 0.f ? sy : 1.f - sy)) * up;
    };
    auto store_tile = [&](int j, const float (&tot)[NT][2], const float (&tot2)[NT][2]) {
      const bool sg = j >= nt0;
      const int tile = sg ? t01 + (j - nt0) : t00 + j;
      const int nte = sg ? nte1 : nte0;
      const int n_lo = tile * 16 + g;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int orow = s_orow[(sg ? kRowsPerSweep : 0) + nt * 4 + t];
        if (nt < nte && orow >= 0) {
          const int64_t o = (int64_t)orow * p.N;
          if (p.x_f32) {
            if (n_lo < p.N) ((float*)p.y)[o + n_lo] = FUSED ? swiglu32(tot[nt][0], tot2[nt][0]) : tot[nt][0];
            if (n_lo + 8 < p.N) ((float*)p.y)[o + n_lo + 8] = FUSED ? swiglu32(tot[nt][1], tot2[nt][1]) : tot[nt][1];
          } else {
            if (n_lo < p.N) ((uint16_t*)p.y)[o + n_lo] = FUSED ? swiglu16(tot[nt][0], tot2[nt][0]) : f32_to_bf16_bits(tot[nt][0]);
            if (n_lo + 8 < p.N) ((uint16_t*)p.y)[o + n_lo + 8] = FUSED ? swiglu16(tot[nt][1], tot2[nt][1]) : f32_to_bf16_bits(tot[nt][1]);
          }
        }
      }
    };
    {
      float tot[NT][2], tot2[NT][2];   // tot2: the second bank's sums (fused form)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = tot2[nt][0] = tot2[nt][1] = 0.f;
      for (int ti = 0; ti < my_tiles; ++ti) {
        const int j = first + ti * kWarps;
        const bool sg = j >= nt0;
        const int nte = sg ? nte1 : nte0;
        const uint2* xf = xfrag + (sg ? xf_stride : 0);
        const float* gsb = gsc + (sg ? gs_stride : 0);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = tot2[nt][0] = tot2[nt][1] = 0.f;
        // one ring stage (16 rows x 128 bytes of codes) against the staged rows; NTE n8 tiles in use
        auto unit = [&](auto nte_c, const unsigned char* st, int u, float (&tt)[NT][2]) {
          constexpr int NTE = decltype(nte_c)::value;
          // fragments and group scales of this unit's U groups: every offset below is a compile-time constant
          const uint4* xb = (const uint4*)xf + (size_t)(u * U * NT) * 32 + lane;
          const float* gb = gsb + (size_t)((u * U * 4 + t) * NT) * 2;
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
#pragma unroll
          for (int jj = 0; jj < U; ++jj) {
            uint32_t a0[2], a1[2], a2[2], a3[2];
            if constexpr (BITS == 4) {
              const uint2 wl = *(const uint2*)(st + frag_off[jj]);
              const uint2 wh = *(const uint2*)(st + frag_off[jj] + 1024);
              a0[0] = wl.x & 0x0F0F0F0Fu; a2[0] = (wl.x >> 4) & 0x0F0F0F0Fu;
              a0[1] = wl.y & 0x0F0F0F0Fu; a2[1] = (wl.y >> 4) & 0x0F0F0F0Fu;
              a1[0] = wh.x & 0x0F0F0F0Fu; a3[0] = (wh.x >> 4) & 0x0F0F0F0Fu;
              a1[1] = wh.y & 0x0F0F0F0Fu; a3[1] = (wh.y >> 4) & 0x0F0F0F0Fu;
            } else {
              const uint4 wl = *(const uint4*)(st + frag_off[jj]);
              const uint4 wh = *(const uint4*)(st + frag_off[jj] + 1024);
              a0[0] = wl.x; a2[0] = wl.y; a0[1] = wl.z; a2[1] = wl.w;
              a1[0] = wh.x; a3[0] = wh.y; a1[1] = wh.z; a3[1] = wh.w;
            }
            const float s_lo = (jj & 1) ? bf16hi(sl[jj >> 1]) : bf16lo(sl[jj >> 1]);
            const float s_hi = (jj & 1) ? bf16hi(sh[jj >> 1]) : bf16lo(sh[jj >> 1]);
            const float b_lo = (jj & 1) ? bf16hi(bl[jj >> 1]) : bf16lo(bl[jj >> 1]);
            const float b_hi = (jj & 1) ? bf16hi(bh[jj >> 1]) : bf16lo(bh[jj >> 1]);
            float2 gsn[NT];   // this lane's row of every n8 tile
            if constexpr (NTE == 2) {
              const float4 v = *(const float4*)&gb[jj * 4 * NT * 2];
              gsn[0] = make_float2(v.x, v.y); gsn[1] = make_float2(v.z, v.w);
            } else {
              gsn[0] = *(const float2*)&gb[jj * 4 * NT * 2];
            }
#pragma unroll
            for (int nt = 0; nt < NTE; ++nt) {
              int acc[4];
              const uint4 bf = xb[(jj * NT + nt) * 32];
              mma_u8s8_z(acc, a0[0], a1[0], a2[0], a3[0], bf.x, bf.y);
              mma_u8s8(acc, a0[1], a1[1], a2[1], a3[1], bf.z, bf.w);
              const float2 gs = gsn[nt];
              const float f_lo = (float)(acc[0] * 128 + acc[1]), f_hi = (float)(acc[2] * 128 + acc[3]);
              tt[nt][0] = fmaf(s_lo * gs.x, f_lo, fmaf(b_lo, gs.y, tt[nt][0]));
              tt[nt][1] = fmaf(s_hi * gs.x, f_hi, fmaf(b_hi, gs.y, tt[nt][1]));
            }
          }
        };
        auto sweep_k = [&](auto nte_c) {
          auto step = [&](int u, float (&tt)[NT][2]) {
            if (issued < total) issue();
            cp_async_commit();
            ++issued;
            cp_async_wait<kStages - 1>();
            __syncwarp();
            const unsigned char* st = my_ring_p + c_off;
            c_off = c_off + kStageBytes == kStages * kStageBytes ? 0u : c_off + kStageBytes;
            unit(nte_c, st, u, tt);
            __syncwarp();
          };
          for (int u = kp; u < ut; u += ksplit) {
            step(u, tot);
            if constexpr (FUSED) step(u, tot2);   // the same unit of the second bank, against the same fragments
          }
        };
        if (nte == 1) sweep_k(std::integral_constant<int, 1>{});
        else sweep_k(std::integral_constant<int, 2>{});
        if (ksplit == 1) store_tile(j, tot, tot2);
      }
      cp_async_wait<0>();
      if (ksplit > 1) {   // uniform over the CTA: every warp reaches the barrier
        float* mine = red + (size_t)warp * (NT * 2 * 32);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { mine[(nt * 2 + 0) * 32 + lane] = tot[nt][0]; mine[(nt * 2 + 1) * 32 + lane] = tot[nt][1]; }
        __syncthreads();
        if (kp == 0 && my_tiles > 0) {
          for (int k = 1; k < ksplit; ++k) {
            const float* o = red + (size_t)(warp + k) * (NT * 2 * 32);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) { tot[nt][0] += o[(nt * 2 + 0) * 32 + lane]; tot[nt][1] += o[(nt * 2 + 1) * 32 + lane]; }
          }
        }
        if constexpr (FUSED) {   // the second bank's sums through the same buffer
          __syncthreads();
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) { mine[(nt * 2 + 0) * 32 + lane] = tot2[nt][0]; mine[(nt * 2 + 1) * 32 + lane] = tot2[nt][1]; }
          __syncthreads();
          if (kp == 0 && my_tiles > 0) {
            for (int k = 1; k < ksplit; ++k) {
              const float* o = red + (size_t)(warp + k) * (NT * 2 * 32);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) { tot2[nt][0] += o[(nt * 2 + 0) * 32 + lane]; tot2[nt][1] += o[(nt * 2 + 1) * 32 + lane]; }
            }
          }
        }
        if (kp == 0 && my_tiles > 0) store_tile(first, tot, tot2);
      }
    }
  }
}

// sigmoid of every bf16 bit pattern, rounded to bf16 (the reference tabulates mlx_sigmoid the same way,
// src/transformer.zig:19853-19885); filled from the host once per device.
__device__ uint16_t g_sigtab[1 << 16];

}  // namespace

const uint16_t* sigmoid_table(cudaStream_t st, cudaError_t* err) {
  static const uint16_t* ptr[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
  std::lock_guard<std::mutex> setup_lk(setup_mutex());   // the table and its host staging buffer are built once
  if (!ptr[dev]) {
    // the upload is a synchronous copy: not possible while `st` is being captured into a graph (call once before)
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
      (void)cudaGetLastError();
      *err = cudaErrorStreamCaptureUnsupported;
      return nullptr;
    }
    static uint16_t host[1 << 16];
    for (uint32_t i = 0; i < (1u << 16); ++i) {
      uint32_t bits = i << 16;
      float x;
      memcpy(&x, &bits, 4);
      // the two-sided form of MLX's Sigmoid, as the reference quotes it (src/transformer.zig:17566-17570)
      const float sy = 1.0f / (1.0f + expf(fabsf(x)));
      const float sg = x < 0.0f ? sy : 1.0f - sy;
      uint32_t u;
      memcpy(&u, &sg, 4);
      host[i] = (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);   // round to nearest even
    }
    void* d = nullptr;
    if ((*err = cudaGetSymbolAddress(&d, g_sigtab)) != cudaSuccess) return nullptr;
    if ((*err = cudaMemcpy(d, host, sizeof(host), cudaMemcpyHostToDevice)) != cudaSuccess) return nullptr;
    ptr[dev] = (const uint16_t*)d;
  }
  *err = cudaSuccess;
  return ptr[dev];
}

namespace {


constexpr size_t kStaticSmem = 14 * 1024;   // upper bound of the kernel's static shared arrays
size_t smem_bytes(int K, int nsb) {
  return (size_t)kWarps * kStages * kStageBytes + (size_t)nsb * ((size_t)(K / 32) * 2 * 256 + (size_t)(K / 64) * 2 * 4 * 8) +
         (size_t)kWarps * 2 * 2 * 32 * 4 + 64;
}
int pick_nsb(int K) { return smem_bytes(K, 2) + kStaticSmem <= 227 * 1024 ? 2 : 1; }

}  // namespace

bool gather_stream_supported(const GatherArgs& a) {
  if (!((a.bits == 4 && (a.gs == 64 || a.gs == 128)) || (a.bits == 8 && a.gs == 64))) return false;
  if (a.x_dtype != QB200_BFLOAT16 && a.x_dtype != QB200_FLOAT32) return false;
  if (a.M != 1 || a.K % 256 != 0 || a.K <= 0 || a.K > 4096) return false;
  if (a.N <= 0 || a.N > (1 << 24) || a.I <= 0 || a.I > kMaxRows || a.E > kMaxExperts) return false;
  if ((((uintptr_t)a.w) & 15) != 0 || (a.w_expert_stride * 4) % 16 != 0) return false;
  if ((((uintptr_t)a.s) & 7) != 0 || (((uintptr_t)a.b) & 7) != 0 || (a.s_expert_stride * 2) % 8 != 0) return false;
  if (a.gs == 64 && (a.K / 64) % 4 != 0) return false;
  if (a.gs == 128 && (a.K / 128) % 2 != 0) return false;
  if ((((uintptr_t)a.x) & 15) != 0 || (a.x_batch_stride * (a.x_dtype == QB200_FLOAT32 ? 4 : 2)) % 16 != 0) return false;
  if (a.rhs_dtype != QB200_INT64 && a.rhs_dtype != QB200_INT32 && a.rhs_dtype != QB200_UINT32) return false;
  if (a.lhs && a.lhs_dtype != QB200_INT64 && a.lhs_dtype != QB200_INT32 && a.lhs_dtype != QB200_UINT32) return false;
  return smem_bytes((int)a.K, 1) + kStaticSmem <= 227 * 1024;
}

cudaError_t launch_gather_stream(const GatherArgs& a, cudaStream_t st) {
  GK p;
  p.x = a.x; p.w = a.w; p.s = (const uint16_t*)a.s; p.b = (const uint16_t*)a.b; p.y = a.y;
  p.rhs = a.rhs; p.lhs = a.lhs;
  p.rhs_i64 = a.rhs_dtype == QB200_INT64; p.lhs_i64 = a.lhs_dtype == QB200_INT64;
  p.xbcast = a.xbcast;
  p.I = a.I; p.E = a.E; p.XB = a.XB; p.xstride = a.x_batch_stride;
  p.wes = a.w_expert_stride; p.ses = a.s_expert_stride;
  p.N = (int)a.N; p.K = (int)a.K; p.gshift = a.gs == 128 ? 1 : 0; p.x_f32 = a.x_dtype == QB200_FLOAT32;
  p.nsb = pick_nsb(p.K);
  const bool fused = a.w2 != nullptr;
  p.w2 = a.w2; p.s2 = (const uint16_t*)a.s2; p.b2 = (const uint16_t*)a.b2; p.sigtab = nullptr;
  if (fused) {
    cudaError_t te;
    p.sigtab = sigmoid_table(st, &te);
    if (!p.sigtab) return te;
  }
  const size_t smem = smem_bytes(p.K, p.nsb);
  static bool done[4][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int bi = (a.bits == 4 ? 0 : 1) + (fused ? 2 : 0);
  const void* kern = a.bits == 4 ? (fused ? (const void*)gather_stream_kernel<4, true> : (const void*)gather_stream_kernel<4, false>)
                                 : (fused ? (const void*)gather_stream_kernel<8, true> : (const void*)gather_stream_kernel<8, false>);
  {
  std::lock_guard<std::mutex> setup_lk(setup_mutex());   // first use on a device, from any thread
  if (dev < 0 || dev >= 64 || !done[bi][dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024 - kStaticSmem));
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) done[bi][dev] = true;
  }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sm_count());
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (fused) {
    if (a.bits == 4) return cudaLaunchKernelEx(&cfg, gather_stream_kernel<4, true>, p);
    return cudaLaunchKernelEx(&cfg, gather_stream_kernel<8, true>, p);
  }
  if (a.bits == 4) return cudaLaunchKernelEx(&cfg, gather_stream_kernel<4, false>, p);
  return cudaLaunchKernelEx(&cfg, gather_stream_kernel<8, false>, p);
}

}  // namespace qb

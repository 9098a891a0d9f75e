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
#include "kernels.h"

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
                                    // a 16-token instantiation needed four staging passes over K = 4096 and was
                                    // measured slower than two 8-token launches

__host__ __device__ constexpr int kc_for(int nt) { return nt <= 2 ? 4096 : 1024; }

constexpr int kMaxMat = 4;          // weight matrices served by one launch (same activations)

// Optional timeline of one launch (a build with -DQB_STREAM_PROFILE; not part of the library build):
// nanosecond timestamps of thread 0 of every CTA at the phase boundaries
// (0 start, 1 first ring stages issued, 2 previous grid complete, 3 activations staged, 4 end).
#ifdef QB_STREAM_PROFILE
__device__ unsigned long long g_stream_tl[512][8];
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define TL(i) do { if (threadIdx.x == 0 && blockIdx.x < 512) g_stream_tl[blockIdx.x][i] = gtime(); } while (0)
#else
#define TL(i)
#endif

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

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void group_barrier(int grp) {
  asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "n"(kWarpsPerGroup * 32) : "memory");
}
// Thread-block cluster helpers (distributed shared memory): the CTAs of a cluster split the conversion of
// the activations and write every converted fragment into the shared memory of all of them.
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v2(uint32_t addr, uint32_t x, uint32_t y) {
  asm volatile("st.shared::cluster.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// All threads of all CTAs of the cluster (a hardware barrier: no spinning in software).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// D(16x8,s32) += A(16x32,u8,row) * B(32x8,s8,col)
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same with a zero C operand (no accumulator initialisation in registers).
__device__ __forceinline__ void mma_u8s8_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// 16-byte chunk swizzle inside a 128-byte stage row so that the fragment reads
// (64-bit per lane at 4 bits, 128-bit at 8 bits) are bank-conflict free.
template <int BITS> __device__ __forceinline__ int swz(int row) {
  return BITS == 4 ? 2 * (row & 3) : 4 * (row & 1);
}

// A lane owns 16 consecutive K values of a group, 8 per MMA.  Offset (0..7)
// inside those 8 of the byte that sits in operand register h (0: k-slots 4t..,
// 1: k-slots 16+4t..), byte i.  4-bit words split into even and odd nibbles;
// 8-bit words are in order.
template <int BITS> __device__ __forceinline__ int kslot8(int h, int i) {
  return BITS == 4 ? 2 * i + h : 4 * h + i;
}

// Fixed-point value of one activation: v = clamp(rn(x * up)), |v| < 2^14.
// Round-to-nearest through the fp32 magic number 1.5*2^23 (one FMA, one integer subtract).
__device__ __forceinline__ int fix15(float x, float up) {
  const int v = __float_as_int(fmaf(x, up, 12582912.f)) - 0x4B400000;
  return v > 16383 ? 16383 : v;  // fp32 inputs may round up to 2^14; -2^14 still fits the high plane
}
__device__ __forceinline__ uint32_t plane_byte(int v, int plane) {
  return plane == 0 ? (uint32_t)((v >> 7) & 0xFF) : (uint32_t)(v & 127);
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

// Position of a warp in its stream of (pass, local tile, K unit) items.
struct ItemIter {
  int pass, tl, u;
  int ks, ntl, npass, upk, ut;  // ut: units per tile over all of K; upk: units per full pass
  __device__ __forceinline__ int upt(int p) const {
    const int left = ut - p * upk;
    return left < upk ? left : upk;
  }
  __device__ __forceinline__ void normalize() {
    while (pass < npass && u >= upt(pass)) {
      u = ks;
      if (++tl >= ntl) { tl = 0; ++pass; }
    }
  }
  __device__ __forceinline__ void init(int ks_, int ntl_, int npass_, int upk_, int ut_) {
    ks = ks_; ntl = ntl_; npass = npass_; upk = upk_; ut = ut_;
    pass = 0; tl = 0; u = ks;
    if (ntl <= 0) pass = npass;
    normalize();
  }
  __device__ __forceinline__ bool valid() const { return pass < npass; }
  __device__ __forceinline__ void next() { u += kWarpsPerGroup; normalize(); }
};

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
  TL(0);

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
  if constexpr (!M1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(ring + (size_t)warp * kStages * kStageBytes);
  const unsigned char* my_ring_p = ring + (size_t)warp * kStages * kStageBytes;
  const int ntl = ggrp < p.ntiles ? (p.ntiles - ggrp + p.total_groups - 1) / p.total_groups : 0;
  const int k_lo = split ? crank * p.upc * CK : 0;                 // first K value of this CTA's range
  const int k_cta = split ? (p.K - k_lo < p.upc * CK ? (p.K - k_lo > 0 ? p.K - k_lo : 0) : p.upc * CK) : p.K;
  const int ut = k_cta / CK, upk = split ? (ut > 0 ? ut : 1) : kc / CK;

  // ---- producer state: per-lane source pointers of the current tile ----
  const int chunk = lane & 7;
  const unsigned char* wsrc[4];
  const uint16_t* sbsrc;
  uint32_t wdst[4];
  uint32_t sbdst;
  int prod_tile = -1;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = (lane >> 3) + 4 * r;
    wdst[r] = row * 128 + ((chunk ^ swz<BITS>(row)) << 4);
  }
  sbdst = kStageW + (lane >> 4) * 128 + (lane & 15) * 8;

  auto issue = [&](const ItemIter& it, int stage) {
    const int tile = ggrp + it.tl * p.total_groups;
    if (tile != prod_tile) {
      prod_tile = tile;
      const int mi = mat_of_tile(p, tile);
      const int row0 = (tile - QB_SEL4(p.tile0, mi)) * 16, nrows = QB_SEL4(p.N, mi);
      const uint32_t* wm = QB_SEL4(p.w, mi);
      const int64_t ldw = QB_SEL4(p.ldw, mi), lds = QB_SEL4(p.lds, mi);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        int n = row0 + (lane >> 3) + 4 * r;
        n = n < nrows ? n : nrows - 1;
        wsrc[r] = (const unsigned char*)(wm + (int64_t)n * ldw) + chunk * 16;
      }
      int n = row0 + (lane & 15);
      n = n < nrows ? n : nrows - 1;
      sbsrc = ((lane >> 4) ? QB_SEL4(p.b, mi) : QB_SEL4(p.s, mi)) + (int64_t)n * lds;
    }
    const uint32_t st = my_ring + stage * kStageBytes;
    const int k0 = k_lo + it.pass * kc + it.u * CK;
    const int woff = k0 * BITS / 8;
#pragma unroll
    for (int r = 0; r < 4; ++r) cp_async16(st + wdst[r], wsrc[r] + woff);
    const uint16_t* ssrc = sbsrc + ((k0 >> 6) >> p.gshift);
    if (BITS == 4 && p.gshift == 0) cp_async8(st + sbdst, ssrc);
    else cp_async4(st + sbdst, ssrc);
  };

  // per-lane byte offsets of the fragment reads of row g (row g+8 is +1024: same swizzle)
  int frag_off[U];
#pragma unroll
  for (int j = 0; j < U; ++j) {
    if (BITS == 4) frag_off[j] = g * 128 + (((2 * j + (t >> 1)) ^ swz<4>(g)) << 4) + (t & 1) * 8;
    else frag_off[j] = g * 128 + (((4 * j + t) ^ swz<8>(g)) << 4);
  }

  ItemIter prod;
  prod.init(ks, ntl, p.npass, upk, ut);
  int issued = 0;
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) {
    if (prod.valid()) { issue(prod, issued % kStages); prod.next(); }
    cp_async_commit();
    ++issued;
  }

  // Let the next grid in the stream begin launching, then wait for the previous grid to complete (and
  // its writes to be visible) before reading activations or writing outputs.
  TL(1);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  TL(2);
  if constexpr (!M1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");

  int consumed = 0;
  int red_buf = 0;

  for (int pass = 0; pass < p.npass; ++pass) {
    const int k_base = k_lo + pass * kc;
    const int klen = split ? k_cta : ((p.K - k_base) < kc ? (p.K - k_base) : kc);
    if (pass > 0) {  // every reader of the previous pass's fragments (cluster-wide) is done
      if constexpr (M1) __syncthreads(); else cluster_sync_all();
    }
    // ---- stage this pass's activations as s8 planes in B-fragment order ----
    // One thread converts 8 consecutive K values of one token; the 8 lanes that cover a 64-wide
    // group agree on the group's power-of-two scale (|x| * up < 2^14) through shuffles.
    {
      const int cpt = klen >> 3;                         // 8-value chunks per token
      const int slots = M1 ? 1 : NT * kTokPerTile;
      const int total = slots * cpt;
      constexpr int PF = 4;  // chunks fetched per thread before any is converted (loads in flight together)
      // The CTAs of a cluster take interleaved blocks of kThreads chunks and broadcast what they convert.
      // (K-split mode: every CTA converts its own K range for itself)
      const int CS = (M1 || split) ? 1 : (int)cluster_size(), crank_b = (M1 || split) ? 0 : crank;
      const uint32_t xfrag_s = (uint32_t)__cvta_generic_to_shared(xfrag), gsc_s = (uint32_t)__cvta_generic_to_shared(gsc);
      for (int base0 = 0; base0 < total; base0 += kThreads * PF * CS) {
       uint4 raw[PF][2];
#pragma unroll
       for (int q = 0; q < PF; ++q) {
        const int it = base0 + (q * CS + crank_b) * kThreads + tid;
        raw[q][0] = make_uint4(0u, 0u, 0u, 0u);
        raw[q][1] = make_uint4(0u, 0u, 0u, 0u);
        if (it < total) {
          const int m = it / cpt, c = it - m * cpt;
          if (m < p.M) {
            const int64_t off = (int64_t)m * p.ldx + k_base + c * 8;
            if (!p.x_f32) {
              const uint16_t* px = (const uint16_t*)p.x + off;
              if ((((uintptr_t)px) & 15) == 0) {
                raw[q][0] = *(const uint4*)px;
              } else {
                uint32_t r[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) r[j] = (uint32_t)px[2 * j] | ((uint32_t)px[2 * j + 1] << 16);
                raw[q][0] = make_uint4(r[0], r[1], r[2], r[3]);
              }
            } else {
              const float* px = (const float*)p.x + off;
              if ((((uintptr_t)px) & 15) == 0) {
                raw[q][0] = *(const uint4*)px;
                raw[q][1] = *(const uint4*)(px + 4);
              } else {
                raw[q][0] = make_uint4(__float_as_uint(px[0]), __float_as_uint(px[1]), __float_as_uint(px[2]), __float_as_uint(px[3]));
                raw[q][1] = make_uint4(__float_as_uint(px[4]), __float_as_uint(px[5]), __float_as_uint(px[6]), __float_as_uint(px[7]));
              }
            }
          }
        }
       }
#pragma unroll
       for (int q = 0; q < PF; ++q) {
        const int base = base0 + (q * CS + crank_b) * kThreads;
        if (base >= total) continue;
        const int it = base + tid;
        const bool ok = it < total;
        const int m = ok ? it / cpt : 0;
        const int c = ok ? it - m * cpt : 0;             // chunk index inside the pass
        float f[8];
        if (!p.x_f32) {
          const uint4 a = raw[q][0];
          f[0] = bf16lo(a.x); f[1] = bf16hi(a.x); f[2] = bf16lo(a.y); f[3] = bf16hi(a.y);
          f[4] = bf16lo(a.z); f[5] = bf16hi(a.z); f[6] = bf16lo(a.w); f[7] = bf16hi(a.w);
        } else {
          const uint4 a = raw[q][0], b2 = raw[q][1];
          f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
          f[4] = __uint_as_float(b2.x); f[5] = __uint_as_float(b2.y); f[6] = __uint_as_float(b2.z); f[7] = __uint_as_float(b2.w);
        }
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(f[j]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        int e = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 + 1;  // mx < 2^e
        e = e < -100 ? -100 : (e > 110 ? 110 : e);
        const float up = __uint_as_float((uint32_t)(127 + 14 - e) << 23);
        const float down = __uint_as_float((uint32_t)(127 + e - 14) << 23);
        int v[8];
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[j] = fix15(f[j], up); sum += v[j]; }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (ok) {
          const int gi = c >> 3, tt = (c >> 1) & 3, jm = c & 1;  // 64-group, lane quarter, MMA of the group
          const int nt = m / kTokPerTile, ml = m - nt * kTokPerTile;
          if ((c & 7) == 0) {
            if constexpr (M1) {
              gsc[gi * 2] = down;
              gsc[gi * 2 + 1] = down * (float)sum;
            } else {
              const uint32_t a = gsc_s + (uint32_t)(((gi * NT + nt) * kTokPerTile + ml) * 2) * 4u;
              for (int cr = 0; cr < CS; ++cr)
                st_cluster_v2(map_to_rank(a, split ? crank : cr), __float_as_uint(down), __float_as_uint(down * (float)sum));
            }
          }
#pragma unroll
          for (int pl = 0; pl < 2; ++pl) {
            uint2 o;
            o.x = plane_byte(v[kslot8<BITS>(0, 0)], pl) | (plane_byte(v[kslot8<BITS>(0, 1)], pl) << 8) |
                  (plane_byte(v[kslot8<BITS>(0, 2)], pl) << 16) | (plane_byte(v[kslot8<BITS>(0, 3)], pl) << 24);
            o.y = plane_byte(v[kslot8<BITS>(1, 0)], pl) | (plane_byte(v[kslot8<BITS>(1, 1)], pl) << 8) |
                  (plane_byte(v[kslot8<BITS>(1, 2)], pl) << 16) | (plane_byte(v[kslot8<BITS>(1, 3)], pl) << 24);
            if constexpr (M1) {
              xfrag[(gi * 2 + jm) * 8 + pl * 4 + tt] = o;
            } else {
              const uint32_t a = xfrag_s + (uint32_t)(((gi * 2 + jm) * NT + nt) * 32 + (2 * ml + pl) * 4 + tt) * 8u;
              for (int cr = 0; cr < CS; ++cr) st_cluster_v2(map_to_rank(a, split ? crank : cr), o.x, o.y);
            }
          }
        }
       }
      }
    }
    if constexpr (M1) __syncthreads(); else cluster_sync_all();
    if (pass == 0) TL(3);

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
        if (prod.valid()) { issue(prod, issued % kStages); prod.next(); }
        cp_async_commit();
        ++issued;
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const unsigned char* st = my_ring_p + (consumed % kStages) * kStageBytes;
        ++consumed;

        // scales / biases of rows g and g+8 for the unit's U groups (bf16 pairs)
        uint32_t sl[2], sh[2], bl[2], bh[2];
        {
          const unsigned char* sb = st + kStageW;
          if (BITS == 4 && p.gshift == 0) {
            const uint2 a = *(const uint2*)(sb + g * 8), c = *(const uint2*)(sb + (g + 8) * 8);
            const uint2 d = *(const uint2*)(sb + 128 + g * 8), e = *(const uint2*)(sb + 128 + (g + 8) * 8);
            sl[0] = a.x; sl[1] = a.y; sh[0] = c.x; sh[1] = c.y;
            bl[0] = d.x; bl[1] = d.y; bh[0] = e.x; bh[1] = e.y;
          } else {
            const uint32_t a = *(const uint32_t*)(sb + g * 8), c = *(const uint32_t*)(sb + (g + 8) * 8);
            const uint32_t d = *(const uint32_t*)(sb + 128 + g * 8), e = *(const uint32_t*)(sb + 128 + (g + 8) * 8);
            if (BITS == 4) {  // group size 128: each value serves two 64-wide groups
              sl[0] = __byte_perm(a, a, 0x1010); sl[1] = __byte_perm(a, a, 0x3232);
              sh[0] = __byte_perm(c, c, 0x1010); sh[1] = __byte_perm(c, c, 0x3232);
              bl[0] = __byte_perm(d, d, 0x1010); bl[1] = __byte_perm(d, d, 0x3232);
              bh[0] = __byte_perm(e, e, 0x1010); bh[1] = __byte_perm(e, e, 0x3232);
            } else {
              sl[0] = a; sh[0] = c; bl[0] = d; bh[0] = e;
              sl[1] = sh[1] = bl[1] = bh[1] = 0;
            }
          }
        }
        // Fragments and group scales of this unit's U groups; every offset below is a compile-time constant.
        // Single token: only the two plane columns 0 and 1 of the n8 tile are read back (by the lanes
        // with t == 0), so the lanes that feed columns 2..7 may load anything: they re-read columns 0/1.
        const uint2* xb = M1 ? xfrag + (size_t)(u * U * 2) * 8 + (g & 1) * 4 + t
                             : xfrag + (size_t)(u * U * 2 * NT) * 32 + lane;
        const float* gb = M1 ? gsc + (size_t)(u * U) * 2 : gsc + (size_t)(u * U * NT * kTokPerTile + t) * 2;
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
            const uint2 bf0 = xb[(j * 2 + 0) * 8], bf1 = xb[(j * 2 + 1) * 8];
            mma_u8s8_z(acc, a0[0], a1[0], a2[0], a3[0], bf0.x, bf0.y);
            mma_u8s8(acc, a0[1], a1[1], a2[1], a3[1], bf1.x, bf1.y);
            const float2 gs = *(const float2*)&gb[j * 2];
            const float f_lo = (float)(acc[0] * 128 + acc[1]), f_hi = (float)(acc[2] * 128 + acc[3]);
            tot[0][0] = fmaf(s_lo * gs.x, f_lo, fmaf(b_lo, gs.y, tot[0][0]));
            tot[0][1] = fmaf(s_hi * gs.x, f_hi, fmaf(b_hi, gs.y, tot[0][1]));
          } else {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              int acc[4];
              const uint2 bf0 = xb[((j * 2 + 0) * NT + nt) * 32], bf1 = xb[((j * 2 + 1) * NT + nt) * 32];
              mma_u8s8_z(acc, a0[0], a1[0], a2[0], a3[0], bf0.x, bf0.y);
              mma_u8s8(acc, a0[1], a1[1], a2[1], a3[1], bf1.x, bf1.y);
              const float2 gs = *(const float2*)&gb[(j * NT + nt) * kTokPerTile * 2];
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
  TL(4);
}

#ifdef QB_STREAM_PROFILE
extern "C" __attribute__((visibility("default"))) void qb200_debug_stream_timeline(unsigned long long* out) {
  cudaMemcpyFromSymbol(out, g_stream_tl, sizeof(unsigned long long) * 512 * 8);
}
#endif

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
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
  int grid = 0;
  size_t smem = 0;
  if (!plan_stream(p, NT, M1, &grid, &smem, &cs, cs, M1 ? 0 : max_ctas, BITS == 4 ? 256 : 128, split_cluster_of[di],
                   split_ctas_of[di]))
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

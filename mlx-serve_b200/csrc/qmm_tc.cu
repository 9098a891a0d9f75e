// Prefill-width quantized matmul on the 5th-generation tensor cores:
// y[M, N] = x[M, K] . What[N, K]^T with What = bf16(q*s + b).
//
// Replaces the dense prefill route of qmatmulBits: prefillDqGemm (dequantize to
// a bf16 [N, K] transient, then a dense GEMM; mlx-serve
// src/transformer.zig:20987-21011) and stock qmm_t for large M
// (src/transformer.zig:20894-20983).  The weight term is rounded to bf16 once,
// exactly as that route's dequantised transient is (src/transformer.zig:20872-20873);
// accumulation is fp32 in tensor memory.  No [N, K] transient ever reaches HBM:
// each CTA dequantises the weight tile it is about to multiply straight into the
// swizzled shared-memory operand.
//
// Persistent, warp-specialised CTAs (one per SM) walk the output tiles of
// 256 tokens x BN weight rows (BN chosen per problem so that the last wave of
// tiles is full), K in steps of 64 through a 3- or 4-stage ring (and a ring of packed codes beside it).  Two tile
// forms: BN <= 128 with two accumulator sets in tensor memory (the epilogue of
// tile i overlaps the main loop of tile i+1; used below 257 tokens and by the
// grouped form), and BN <= 208 with one set (fewer shared-memory operand bytes
// per MAC -- the resource that bounds this kernel -- at the price of an
// epilogue that is not overlapped; used for wide prefill).  Roles:
//   warps 0-15 : dequantisers in groups that take k-blocks in turn (four groups of four warps
//                for tiles of up to 128 weight rows, two of eight for the wide form): a group's
//                per-k-block latency -- two barrier polls, scale selection, proxy fence, arrival
//                -- is several times its arithmetic, so several k-blocks are always being
//                converted side by side.  One thread per weight row: packed codes -> exact bf16
//                integers (byte shuffles) -> one bf16 FMA with the group's scale and bias ->
//                the K-major SWIZZLE_128B operand row.  The packed codes come
//                from a shared-memory ring that TMA fills (below); scales and
//                biases are fetched eight k-groups at a time, one window ahead.
//   warps 16-19: epilogue: tcgen05.ld of a finished accumulator, bf16 rows of y.
//                Tensor memory holds two accumulator sets (2 x 2 x 128 columns),
//                so the epilogue of tile i overlaps the main loop of tile i+1.
//   warp 20    : TMA producer -- two 128x64 bf16 boxes of x per stage
//                (cp.async.bulk.tensor.2d, SWIZZLE_128B, no multicast).
//   warp 21    : TMA producer for the packed codes: 128 bytes of each of the
//                tile's BN weight rows per copy (SWIZZLE_128B, no multicast),
//                double-buffered.  Per-lane global loads of the codes would
//                touch 32 cache lines per instruction and saturate the L1 data
//                path that the tensor core's operand reads share.
//   warp 22    : the single-thread tcgen05.mma issuer (M=128, N=BN, K=16 x4 per
//                stage and accumulator) and its tcgen05.commit arrivals.
//   warp 23    : the issuer's scout.  The issuing thread is held for as long as its MMAs execute, so
//                whatever else it executes adds to the k-block time, and a poll of an mbarrier costs it
//                ~130 cycles even when the phase is already complete (measured: 4 MMAs of N <= 128 per
//                k-block issue in 256 cycles, with the two polls and the commit in 624).  The scout polls
//                the two "stage full" barriers of the next k-block while the issuer is busy and the
//                two meet at a named barrier, which costs the issuer a few cycles.
// Every mbarrier wait is bounded: on expiry the kernel records an error code,
// every role leaves its loops, the CTA frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "kernels.h"

namespace qb {
namespace {

constexpr int BM = 256, BN_MAX = 128, BK = 64;
// ring depth: the grouped (routed-expert) form gives one stage's room to its row-offset tables.  The few-token form
// (at most 128 tokens, no second token half) puts TWO k-blocks into a stage -- the stage's second x box holds the
// next 64 columns of K instead of the next 128 tokens, and B has two sub-tiles, one per dequant group: what a
// k-block costs there is the hand-over of a stage between the roles (~800 cycles with nothing to compute), not any
// role's work, so it is paid half as often.
__host__ __device__ constexpr int stages_of(bool grouped, bool wide = false, bool half = false) { return half ? 3 : ((grouped || wide) ? 3 : 4); }
__host__ __device__ constexpr int kb_per_stage_of(bool half) { return half ? 2 : 1; }
// Buffers of the packed-code ring (each holds 128 bytes of every weight row of the tile: four k-blocks at 4 bits,
// two at 8).  Two are enough: trading pipeline stages for a ring of five or six buffers was measured and changed
// nothing at few tokens (the refills are not what the k-loop waits for).
__host__ __device__ constexpr int raw_bufs_of(bool grouped, bool wide = false, bool half = false) { return 2; }
// The wide form multiplies one B tile of up to 208 weight rows per stage against both token halves: fewer
// operand bytes per MAC through shared memory (the resource that bounds this kernel), at the price of a
// single accumulator set in tensor memory (2 x 256 columns), i.e. an epilogue that is not overlapped.
constexpr int BN_WIDE = 208, BN_WIDE_GROUPED = 192;   // the grouped form keeps 8 KiB for its tables
__host__ __device__ constexpr int bn_max_of(bool wide, bool grouped = false) { return wide ? (grouped ? BN_WIDE_GROUPED : BN_WIDE) : BN_MAX; }
constexpr int kMaxGroupExperts = 1024;
// The sixteen dequant warps work in groups; group g converts the k-blocks with (index % groups) == g, one thread per
// weight row (both halves of the row's 64 codes).  What a group spends per k-block is mostly not arithmetic -- two
// barrier polls of ~130 cycles each, the scale selection, the proxy fence, the arrival: ~1500 cycles around ~400 of
// conversion -- and the k-loop of a few-token tile ran at exactly (that sum) / groups.  Tiles of up to 128 weight
// rows therefore use four groups of four warps; the wide form needs eight warps to cover its 208 rows.  A group must
// not step further than the stage ring holds (groups <= stages x k-blocks per stage): its wait on a stage's "empty"
// barrier names a phase by parity, and a group that is two completions ahead of the barrier reads the previous
// round's completion as its own.  The grouped form has three one-k-block stages and so keeps two groups.
__host__ __device__ constexpr int dq_groups_of(bool wide, bool grouped) { return (wide || grouped) ? 2 : 4; }
constexpr int kDequantWarps = 16, kEpiWarps = 4;
constexpr int kEpiWarp0 = kDequantWarps;            // warps 16..19: warp % 4 = TMEM lane quarter
constexpr int kTmaWarp = kEpiWarp0 + kEpiWarps, kWTmaWarp = kTmaWarp + 1, kMmaWarp = kWTmaWarp + 1;
constexpr int kScoutWarp = kMmaWarp + 1;            // waits on the stage barriers on the issuer's behalf (below)
constexpr int kThreads = (kScoutWarp + 1) * 32;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // two 128-row boxes
constexpr int B_STAGE_BYTES = BN_MAX * BK * 2;
constexpr int RAW_BYTES = BN_MAX * 128;      // one super-block of packed codes: 128 bytes of every weight row
constexpr uint32_t kSpinLimit = 1u << 24;

__device__ int g_tc_error = 0;   // 0 = ok; otherwise the code of the wait that expired

constexpr int kMaxTcMat = 4;   // weight matrices multiplied against the same activations by one launch (dense forms)
struct TcMaps { CUtensorMap m[kMaxTcMat]; };   // their packed codes as tensor maps
struct TcK {
  // per matrix (the grouped form has one: the banks seen as a matrix of E * N rows)
  const uint16_t* sv[kMaxTcMat]; const uint16_t* bv[kMaxTcMat]; uint16_t* yv[kMaxTcMat];
  int Nv[kMaxTcMat];
  int64_t ldsv[kMaxTcMat], ldyv[kMaxTcMat];
  int tstart[kMaxTcMat + 1];   // first tile of each matrix in the launch-wide tile numbering
  int nmat;
  int M, N, K;                 // N: rows of matrix 0 (the grouped form: of ONE expert's matrix)
  int gshift;   // scale column = (k / 64) >> gshift
  int BN;       // weight rows per tile (multiple of 16, <= 128)
  int tiles_m, ntiles;
  int sb_vec;   // scales / biases can be fetched 8 at a time (16-byte aligned rows, whole windows)
  // grouped form (gather_qmm with rows sorted by expert): M = routed rows, N = rows of ONE expert's matrix,
  // w/s/b are the banks [E][N][.] seen as one matrix of E*N rows, rhs[i] = expert of row i (ascending)
  const void* rhs; int rhs_i64; int E;
  // split-K form (few tokens, few tiles): the `ksplit` CTAs of a cluster share one tile, each multiplies its own
  // K range, and rank 0 adds the partial accumulators it receives through distributed shared memory
  int ksplit;
};

// Kernel parameters are indexed with constant subscripts only (a dynamic subscript would force a local copy).
#define TC_SEL4(arr, i) ((i) == 0 ? (arr)[0] : ((i) == 1 ? (arr)[1] : ((i) == 2 ? (arr)[2] : (arr)[3])))

struct TileCoord {
  int mi;                // matrix of the tile (0 in the grouped form)
  int row0, row_end;     // token rows [row0, min(row0 + 256, row_end)) of x / y
  int n0, nend;          // output columns [n0, nend) of y
  int wrow0, wrow_last;  // first weight row of the tile in the (stacked) weight matrix; last row that may be read
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait; returns false when the limit expired.
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
// The same for waits that are off the critical path (producers running ahead, the epilogue waiting for a
// whole tile): after a few polls the thread sleeps between polls, so that it does not take issue slots
// from the warps that convert weights.  Still bounded: 2^22 polls of at least 100 ns.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t it = 0; it < (kSpinLimit >> 2); ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (it >= 4) __nanosleep(100);
  }
  return false;
}
// Wait of the dequant warps: they run several stages ahead of the tensor core, so a poll that fails is followed
// by a short sleep -- sixteen warps polling in a tight loop take issue slots from the one thread that issues MMAs.
__device__ __forceinline__ bool mbar_wait_backoff(uint64_t* bar, uint32_t parity) {
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
    __nanosleep(40);
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank_tc() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_tc() {   // all threads of all CTAs of the cluster (hardware barrier)
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t rank, float4 v) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(addr), "r"(rank));
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(ra), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// K-major, SWIZZLE_128B operand descriptor: rows of 128 bytes, 8-row atoms 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);   // start address
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset
  d |= (uint64_t)1 << 46;                    // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return d;
}
// bf16 x bf16 -> f32, A and B K-major, M = 128, N = bn
__device__ __forceinline__ uint32_t make_idesc(int bn) {
  uint32_t d = 0;
  d |= 1u << 4;                  // c format f32
  d |= 1u << 7;                  // a format bf16
  d |= 1u << 10;                 // b format bf16
  d |= (uint32_t)(bn >> 3) << 17;
  d |= (uint32_t)(128 >> 4) << 24;
  return d;
}
// Both are executed by every lane of the issuing warp with the same operands (so that the compiler can keep
// them in uniform registers and the loop around them stays convergent); only the lane with `issue` set
// issues the instruction.
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %6, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum), "r"(0u), "r"(issue)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(smem_u32(bar)), "r"(issue) : "memory");
}
__device__ __forceinline__ void umma_commit_addr(uint32_t bar_smem, uint32_t issue) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(bar_smem), "r"(issue) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

// 32 codes (half of a k-block) of one weight row -> 32 bf16 values q*s+b (one rounding), written as
// chunks 4h..4h+3 of the 128-byte row `r` of a K-major SWIZZLE_128B tile (16-byte chunk c lands at
// chunk c ^ (r & 7)).
template <int BITS>
__device__ __forceinline__ void dequant_half(const uint32_t* codes, uint32_t sb2, uint32_t bb2, unsigned char* tile, int r,
                                             int h) {
  // sb2 / bb2: the group's scale / bias replicated in both bf16 lanes
  const __nv_bfloat162 s2 = *(const __nv_bfloat162*)&sb2, b2 = *(const __nv_bfloat162*)&bb2;
  unsigned char* row = tile + r * 128;
  const int xr = ((4 * h) ^ (r & 7)) << 4;   // chunk (4h + c) ^ (r & 7) = ((4h) ^ (r & 7)) ^ c for c < 4
  if constexpr (BITS == 4) {
    const __nv_bfloat162 c128 = __float2bfloat162_rn(128.f);
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // one packed word = 8 values = one 16-byte chunk of bf16
      const uint32_t w = codes[c];
      // bytes (q1q0, q3q2, q5q4, q7q6) -> bytes q0,q1,q2,q3 and q4,q5,q6,q7 in order
      const uint32_t lo = __byte_perm(w, 0, 0x4140), hi = __byte_perm(w, 0, 0x4342);
      const uint32_t nl = (lo | (lo << 4)) & 0x0F0F0F0Fu, nh = (hi | (hi << 4)) & 0x0F0F0F0Fu;
      uint32_t o[4];
      // 0x43 in the high byte of a bf16 lane: 128 + q, exact
      o[0] = __byte_perm(nl, 0x43434343u, 0x5140);
      o[1] = __byte_perm(nl, 0x43434343u, 0x5342);
      o[2] = __byte_perm(nh, 0x43434343u, 0x5140);
      o[3] = __byte_perm(nh, 0x43434343u, 0x5342);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 v = *(__nv_bfloat162*)&o[j];
        v = __hsub2(v, c128);         // exact q
        v = __hfma2(v, s2, b2);       // q*s + b, rounded once
        o[j] = *(uint32_t*)&v;
      }
      *(uint4*)(row + (xr ^ (c << 4))) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    const float sf = bf16lo(sb2), bf = bf16lo(bb2);
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // two packed words = 8 values
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const uint32_t w = codes[2 * c + q];
        const float f0 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)) - 8388608.f;
        const float f1 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)) - 8388608.f;
        const float f2 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7542)) - 8388608.f;
        const float f3 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7543)) - 8388608.f;
        o[2 * q] = pack_bf16x2(fmaf(f0, sf, bf), fmaf(f1, sf, bf));
        o[2 * q + 1] = pack_bf16x2(fmaf(f2, sf, bf), fmaf(f3, sf, bf));
      }
      *(uint4*)(row + (xr ^ (c << 4))) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Tile t -> coordinates.  Dense: token block t % tiles_m (fastest, so that CTAs running side by side share
// a weight tile through L2), weight block t / tiles_m.  Grouped: the expert whose tile range holds t, then
// the same order inside the expert (s_off: first routed row of every expert, s_tcum: prefix of their tile counts).
template <bool GROUPED>
__device__ __forceinline__ TileCoord tile_coords(const TcK& p, int BN, const int* s_off, const int* s_tcum, int tile) {
  TileCoord c;
  if constexpr (GROUPED) {
    int a = 0, b = p.E;   // s_tcum[a] <= tile < s_tcum[b]
    while (b - a > 1) {
      const int m = (a + b) >> 1;
      if (s_tcum[m] <= tile) a = m; else b = m;
    }
    const int local = tile - s_tcum[a];
    const int rows = s_off[a + 1] - s_off[a], tm = (rows + BM - 1) / BM;
    const int nb = local / tm, mb = local - nb * tm;
    c.mi = 0;
    c.row0 = s_off[a] + mb * BM;
    c.row_end = s_off[a + 1];
    c.n0 = nb * BN;
    c.nend = (c.n0 + BN) < p.N ? (c.n0 + BN) : p.N;
    c.wrow0 = a * p.N + c.n0;
    c.wrow_last = a * p.N + p.N - 1;
  } else {
    int mi = 0;
    if (p.nmat > 1 && tile >= p.tstart[1]) mi = 1;
    if (p.nmat > 2 && tile >= p.tstart[2]) mi = 2;
    if (p.nmat > 3 && tile >= p.tstart[3]) mi = 3;
    const int t = tile - TC_SEL4(p.tstart, mi), Nm = TC_SEL4(p.Nv, mi);
    c.mi = mi;
    c.row0 = (t % p.tiles_m) * BM;
    c.row_end = p.M;
    c.n0 = (t / p.tiles_m) * BN;
    c.nend = (c.n0 + BN) < Nm ? (c.n0 + BN) : Nm;
    c.wrow0 = c.n0;
    c.wrow_last = Nm - 1;
  }
  return c;
}

// The MMA issuer's walk over this CTA's tiles and k-blocks, kept out of line: as part of the kernel's one big
// function its loop was compiled into something three times slower than the same loop on its own (4 MMAs issued in
// ~700 cycles against ~260).  Every lane of the warp runs it; `lead` marks the lane that issues.
struct IssuerArgs {
  uint32_t tmem_base, a_smem, b_smem, empty_smem, acc_full_smem;
  int tile0, ntiles, tstride, nkb, BN;
  const int* s_off; const int* s_tcum;
};
template <bool GROUPED, bool WIDE, bool HALF>
__device__ __noinline__ void issuer_walk(const TcK& p, const IssuerArgs a, uint32_t lead) {
  constexpr int STAGES = stages_of(GROUPED, WIDE, HALF);
  constexpr int KPST = kb_per_stage_of(HALF);          // k-blocks per stage
  constexpr int A_STAGE = A_STAGE_BYTES;               // two x boxes: two token halves, or (few-token form) two k-blocks
  constexpr int B_SUB = bn_max_of(WIDE, GROUPED) * BK * 2, B_STAGE = KPST * B_SUB;
  constexpr int HALF_COLS = WIDE ? 256 : 128;
  const uint32_t idesc = make_idesc(a.BN);
  const uint64_t adesc0 = make_desc(a.a_smem), bdesc0 = make_desc(a.b_smem);
  int it = 0, ti = 0;
  for (int tile = a.tile0; tile < a.ntiles; tile += a.tstride, ++ti) {
    const TileCoord tc = tile_coords<GROUPED>(p, a.BN, a.s_off, a.s_tcum, tile);
    const bool two_halves = tc.row0 + 128 < tc.row_end;  // the second 128 token rows hold real tokens
    // dense form: two accumulator sets used alternately; wide form: one set, reused by every tile
    const int buf = WIDE ? 0 : ti & 1;
    const uint32_t d0 = a.tmem_base + buf * 256;   // (buf is 0 in the wide form)
    for (int kb = 0; kb < a.nkb; kb += KPST, ++it) {   // `it` counts stages
      const int st = it % STAGES;
      // the scout has seen both "full" barriers of this stage (and, before a tile's first k-block, that the
      // epilogue has drained the accumulator set)
      asm volatile("bar.sync 1, 64;" ::: "memory");
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // descriptors of the stage: the start-address field counts 16-byte units, so a K step of
      // 16 values (32 bytes) adds 2 and the stage's second x box adds 16 KiB / 16
      const uint64_t ad0 = adesc0 + (uint64_t)(st * (A_STAGE >> 4)), bd0 = bdesc0 + (uint64_t)(st * (B_STAGE >> 4));
      // A tile without a second token half keeps two partial sums over K, in the columns the second
      // half would use (odd K steps go there; the epilogue adds them).
#pragma unroll
      for (int sub = 0; sub < KPST; ++sub) {
#pragma unroll
        for (int k16 = 0; k16 < BK / 16; ++k16) {
          if (!HALF && two_halves) {
            const uint32_t accum = (kb > 0 || k16 > 0) ? 1u : 0u;
            umma(d0, ad0 + 2 * k16, bd0 + 2 * k16, idesc, accum, lead);
            umma(d0 + HALF_COLS, ad0 + ((128 * BK * 2) >> 4) + 2 * k16, bd0 + 2 * k16, idesc, accum, lead);
          } else {
            const uint32_t accum = (kb > 0 || sub > 0 || k16 > 1) ? 1u : 0u;
            umma(d0 + (k16 & 1) * HALF_COLS, ad0 + sub * ((128 * BK * 2) >> 4) + 2 * k16, bd0 + sub * (B_SUB >> 4) + 2 * k16, idesc,
                 accum, lead);
          }
        }
      }
      umma_commit_addr(a.empty_smem + (uint32_t)st * 8u, lead);  // frees this stage (A and B) once the MMAs above have read it
    }
    umma_commit_addr(a.acc_full_smem + (uint32_t)buf * 8u, lead);
  }
}

template <int BITS, bool GROUPED, bool WIDE, bool HALF = false>
__global__ void __launch_bounds__(kThreads, 1) qmm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ TcMaps wmaps, TcK p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // 1024-byte alignment for the swizzled tiles.  The wide form has no room for the slack: the kernel has no
  // static shared memory, so its dynamic window starts aligned; that is verified below.
  unsigned char* smem = WIDE ? smem_raw : (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int STAGES = stages_of(GROUPED, WIDE, HALF);
  constexpr int KPST = kb_per_stage_of(HALF);          // k-blocks per stage (2 in the few-token form)
  constexpr int DQG = dq_groups_of(WIDE, GROUPED);     // dequant groups, kDequantWarps / DQG warps each
  static_assert(DQG <= STAGES * KPST, "a dequant group would run more than one ring round ahead of its barrier");
  constexpr int A_STAGE = A_STAGE_BYTES;               // two x boxes: two token halves, or (few-token form) two k-blocks
  constexpr int B_SUB = bn_max_of(WIDE, GROUPED) * BK * 2, B_STAGE = KPST * B_SUB, RAW_B = bn_max_of(WIDE, GROUPED) * 128;
  constexpr int HALF_COLS = WIDE ? 256 : 128;      // tensor-memory columns between the two token halves
  unsigned char* a_tiles = smem;                                   // [STAGES][2][128 x 64 bf16]
  unsigned char* b_tiles = smem + STAGES * A_STAGE;                // [STAGES][BN x 64 bf16]
  constexpr int RAW_BUFS = raw_bufs_of(GROUPED, WIDE, HALF);
  unsigned char* raw = b_tiles + STAGES * B_STAGE;                 // [RAW_BUFS][BN x 128 B of packed codes]
  uint64_t* bars = (uint64_t*)(raw + RAW_BUFS * RAW_B);
  uint64_t* full_a = bars, *full_b = bars + STAGES, *empty = bars + 2 * STAGES;
  uint64_t* acc_full = bars + 3 * STAGES, *acc_empty = bars + 3 * STAGES + 2;
  uint64_t* raw_full = bars + 3 * STAGES + 4, *raw_empty = raw_full + RAW_BUFS;
  uint32_t* tmem_slot = (uint32_t*)(raw_empty + RAW_BUFS);
  volatile int& s_fail = *(volatile int*)(tmem_slot + 1);
  // grouped form: first routed row of every expert and the prefix of their tile counts
  int* s_off = (int*)(tmem_slot + 4);               // [E + 1]
  int* s_tcum = s_off + (kMaxGroupExperts + 1);     // [E + 1]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr bool CAN_SPLIT = !GROUPED && !WIDE;
  const int S = CAN_SPLIT ? p.ksplit : 1;                  // CTAs per tile (cluster size)
  const int crank = S > 1 ? (int)cluster_rank_tc() : 0;
  const int nkb = p.K / BK / S;                            // k-blocks of this CTA
  const int kb0 = crank * nkb;                             // its first k-block
  const int tile0 = (int)blockIdx.x / S, tstride = (int)gridDim.x / S;
  const int BN = p.BN;
  constexpr int WPH = (BK / 2) * BITS / 32;  // packed words per half row per k-block (4 or 8)
  constexpr int KPS = 128 * 8 / (BK * BITS);  // k-blocks per 128-byte super-block of codes (4 or 2)

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full_a[i], 1); mbar_init(&full_b[i], KPST * kDequantWarps / DQG); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], kEpiWarps * 32); }
    for (int i = 0; i < RAW_BUFS; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], (kDequantWarps / DQG) * (DQG < KPS ? DQG : KPS)); }
    s_fail = (WIDE && (smem_u32(smem) & 1023u) != 0) ? 8 : 0;   // misaligned window: every role leaves at once
    if (s_fail) atomicCAS(&g_tc_error, 0, 8);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {  // tensor memory: 512 columns = two sets of two 128x128 fp32 accumulators
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_nn = (p.N + BN - 1) / BN;   // weight-row blocks of one matrix
  int ntiles = p.ntiles;
  if constexpr (GROUPED) {
    // rhs is ascending: expert e owns rows [lower_bound(e), lower_bound(e + 1)); each expert contributes
    // ceil(rows / 256) * tiles_nn tiles.  Every CTA builds the same tables.
    for (int e = tid; e <= p.E; e += kThreads) {
      int lo = 0, hi = p.M;   // first index whose expert is >= e
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        const long long v = p.rhs_i64 ? ((const long long*)p.rhs)[mid] : (long long)((const int*)p.rhs)[mid];
        if (v < e) lo = mid + 1; else hi = mid;
      }
      s_off[e] = lo;
    }
    __syncthreads();
    if (warp == 0) {
      int base = 0;
      for (int e0 = 0; e0 < p.E; e0 += 32) {
        const int e = e0 + lane;
        const int cnt = e < p.E ? s_off[e + 1] - s_off[e] : 0;
        const int nt = ((cnt + BM - 1) / BM) * tiles_nn;
        int inc = nt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int o = __shfl_up_sync(0xffffffffu, inc, d);
          if (lane >= d) inc += o;
        }
        if (e < p.E) s_tcum[e] = base + inc - nt;
        base += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) s_tcum[p.E] = base;
    }
    __syncthreads();
    ntiles = s_tcum[p.E];
  }
  // Tile t -> coordinates.  Dense: token block t % tiles_m (fastest, so that CTAs running side by side share
  // a weight tile through L2), weight block t / tiles_m.  Grouped: the expert whose tile range holds t, then
  // the same order inside the expert.
  auto coords = [&](int tile) { return tile_coords<GROUPED>(p, BN, s_off, s_tcum, tile); };
  if (warp == kTmaWarp) {
    if (lane == 0) {
      // ---------------- TMA producer (one thread) ----------------
      int it = 0, fail = 0;
      for (int tile = tile0; tile < ntiles && !fail && !s_fail; tile += tstride) {
        const TileCoord tc = coords(tile);
        const int m0 = tc.row0;
        const bool two = m0 + 128 < tc.row_end;   // the second 128-row box holds real tokens (else it is not multiplied)
        for (int kb = 0; kb < nkb; kb += KPST, ++it) {   // `it` counts stages
          const int st = it % STAGES;
          if (it >= STAGES && !mbar_wait_relaxed(&empty[st], ((it / STAGES) - 1) & 1)) { fail = 3; break; }
          const uint32_t dst = smem_u32(a_tiles + st * A_STAGE);
          if constexpr (HALF) {   // the second box is the next k-block of the same 128 tokens
            mbar_expect_tx(&full_a[st], A_STAGE_BYTES);
            tma_load_2d(dst, &xmap, &full_a[st], (kb0 + kb) * BK, m0);
            tma_load_2d(dst + 128 * BK * 2, &xmap, &full_a[st], (kb0 + kb + 1) * BK, m0);
          } else {
            mbar_expect_tx(&full_a[st], two ? A_STAGE_BYTES : A_STAGE_BYTES / 2);
            tma_load_2d(dst, &xmap, &full_a[st], (kb0 + kb) * BK, m0);
            if (two) tma_load_2d(dst + 128 * BK * 2, &xmap, &full_a[st], (kb0 + kb) * BK, m0 + 128);
          }
        }
      }
      if (fail) { s_fail = fail; atomicCAS(&g_tc_error, 0, fail); }
    }
  } else if (warp == kWTmaWarp) {
    if (lane == 0) {
      // ---------------- TMA producer of the packed codes (one thread) ----------------
      const int sb_per_tile = nkb / KPS;
      int sbk = 0, fail = 0;
      for (int tile = tile0; tile < ntiles && !fail && !s_fail; tile += tstride) {
        const TileCoord tcw = coords(tile);
        const int n0 = tcw.wrow0;
        const CUtensorMap* wmap = &wmaps.m[tcw.mi];
        for (int sbl = 0; sbl < sb_per_tile; ++sbl, ++sbk) {
          const int buf = sbk % RAW_BUFS;
          if (sbk >= RAW_BUFS && !mbar_wait_relaxed(&raw_empty[buf], ((sbk / RAW_BUFS) - 1) & 1)) { fail = 7; break; }
          mbar_expect_tx(&raw_full[buf], (uint32_t)BN * 128u);
          tma_load_2d(smem_u32(raw + buf * RAW_B), wmap, &raw_full[buf], (kb0 / KPS + sbl) * 32, n0);
        }
      }
      if (fail) { s_fail = fail; atomicCAS(&g_tc_error, 0, fail); }
    }
  } else if (warp == kMmaWarp) {
    {
      // ---------------- MMA issuer (the whole warp walks the loop, lane 0 issues) ----------------
      // The issuer waits on nothing but its scout: the two walk the same (tile, k-block) sequence and meet at named
      // barrier 1 once per k-block, whatever happens.  When a wait of the scout runs out it records the failure and
      // stops waiting; the issuer then multiplies stale stages into an accumulator nobody trusts (the status word
      // says so) and every role still reaches the end of the kernel.
      IssuerArgs ia;
      ia.tmem_base = tmem_base; ia.a_smem = smem_u32(a_tiles); ia.b_smem = smem_u32(b_tiles);
      ia.empty_smem = smem_u32(empty); ia.acc_full_smem = smem_u32(acc_full);
      ia.tile0 = tile0; ia.ntiles = ntiles; ia.tstride = tstride; ia.nkb = nkb; ia.BN = BN;
      ia.s_off = s_off; ia.s_tcum = s_tcum;
      issuer_walk<GROUPED, WIDE, HALF>(p, ia, lane == 0 ? 1u : 0u);
    }
  } else if (warp == kScoutWarp) {
    // ---------------- the issuer's scout: the same walk, one meeting per k-block ----------------
    int it = 0, ti = 0, fail = 0;
    for (int tile = tile0; tile < ntiles; tile += tstride, ++ti) {
      const int buf = WIDE ? 0 : ti & 1;
      const int use = WIDE ? ti : ti >> 1;     // how many times this accumulator set was used before
      if (!fail && s_fail) fail = 9;           // another role gave up
      if (!fail && use >= 1 && !mbar_wait_relaxed(&acc_empty[buf], (use - 1) & 1)) fail = 6;
      for (int kb = 0; kb < nkb; kb += KPST, ++it) {   // `it` counts stages
        const int st = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!fail && s_fail) fail = 9;
        if (!fail && !mbar_wait(&full_a[st], ph)) fail = 1;
        if (!fail && !mbar_wait(&full_b[st], ph)) fail = 2;
        if (fail && fail != 9 && !s_fail && lane == 0) { s_fail = fail; atomicCAS(&g_tc_error, 0, fail); }
        asm volatile("bar.sync 1, 64;" ::: "memory");
      }
    }
  } else if (warp < kDequantWarps) {
    // ---------------- dequant producers: DQG groups, one thread per weight row ----------------
    constexpr int WPG = kDequantWarps / DQG;   // warps per group
    constexpr int TPR = (WPG * 32) / bn_max_of(WIDE, GROUPED);   // threads per weight row: 1, or 2 (a half of the k-block each)
    static_assert(TPR == 1 || TPR == 2, "dequant thread layout");
    const int grp = warp / WPG, wg = warp % WPG;
    const int r = (wg % (WPG / TPR)) * 32 + lane, h = wg / (WPG / TPR);
    const bool active = r < BN;
    const int ntl = ntiles > tile0 ? (ntiles - tile0 + tstride - 1) / tstride : 0;  // tiles of this CTA
    const int total_it = ntl * nkb;
    // Scales and biases of this thread's row: windows of 8 values (8 << gshift k-blocks), the next
    // window prefetched while the current one is used.  f_* is the prefetch cursor (tile, k-block).
    const int WL = 8 << p.gshift;
    uint4 s_cur = make_uint4(0, 0, 0, 0), b_cur = s_cur, s_nxt = s_cur, b_nxt = s_cur;
    int f_tl = 0, f_kb = 0;
    // this thread's row of scales and of biases in tile `tl` (looked up once per tile: coords() divides, and
    // searches in the grouped form)
    auto row_ptrs = [&](int tl, const uint16_t*& sp, const uint16_t*& bp) {
      const int tile = tile0 + tl * tstride;
      const TileCoord tc = coords(tile);
      int n = tc.wrow0 + r;
      n = n < tc.wrow_last ? n : tc.wrow_last;
      const int64_t off = (int64_t)n * TC_SEL4(p.ldsv, tc.mi);
      sp = TC_SEL4(p.sv, tc.mi) + off;
      bp = TC_SEL4(p.bv, tc.mi) + off;
    };
    const uint16_t* f_sp = nullptr; const uint16_t* f_bp = nullptr;   // prefetch cursor's row
    const uint16_t* c_sp = nullptr; const uint16_t* c_bp = nullptr;   // current tile's row (scalar path)
    if (ntl > 0) { row_ptrs(0, f_sp, f_bp); c_sp = f_sp; c_bp = f_bp; }
    auto prefetch_window = [&]() {
      if (f_kb >= nkb) {
        f_kb = 0;
        ++f_tl;
        if (f_tl < ntl) row_ptrs(f_tl, f_sp, f_bp);
      }
      if (active && f_tl < ntl) {
        const int off = (kb0 + f_kb) >> p.gshift;
        s_nxt = __ldg((const uint4*)(f_sp + off));
        b_nxt = __ldg((const uint4*)(f_bp + off));
      }
      f_kb += WL;
    };
    if (p.sb_vec) prefetch_window();
    bool ok = true;
    // (tile, k-block) of iteration `it`, stepped without dividing (nkb is a multiple of four)
    int tl = 0, kb = grp - DQG;
    for (int it = grp; it < total_it; it += DQG) {   // `it` counts k-blocks
      const int sit = it / KPST, st = sit % STAGES;   // stage iteration and stage (few-token form: group g fills sub-tile g)
      kb += DQG;
      if (kb >= nkb) {
        kb -= nkb;
        ++tl;
        if (!p.sb_vec) row_ptrs(tl, c_sp, c_bp);
      }
      const int sbk = it / KPS, kbl = it % KPS, buf = sbk % RAW_BUFS;   // nkb is a multiple of KPS
      uint32_t sv2, bv2;
      if (p.sb_vec) {
        if ((kb & (WL - 1)) == grp) {   // this group's first k-block of a window
          s_cur = s_nxt; b_cur = b_nxt;
          prefetch_window();
        }
        const int e = ((kb0 + kb) >> p.gshift) & 7;
        const uint32_t sw = e < 4 ? (e < 2 ? s_cur.x : s_cur.y) : (e < 6 ? s_cur.z : s_cur.w);
        const uint32_t bw = e < 4 ? (e < 2 ? b_cur.x : b_cur.y) : (e < 6 ? b_cur.z : b_cur.w);
        sv2 = (e & 1) ? __byte_perm(sw, sw, 0x3232) : __byte_perm(sw, sw, 0x1010);
        bv2 = (e & 1) ? __byte_perm(bw, bw, 0x3232) : __byte_perm(bw, bw, 0x1010);
      }
      else {
        const int off = (kb0 + kb) >> p.gshift;
        const uint32_t sv = active ? __ldg(c_sp + off) : 0u, bv = active ? __ldg(c_bp + off) : 0u;
        sv2 = sv | (sv << 16);
        bv2 = bv | (bv << 16);
      }
      ok = mbar_wait_backoff(&raw_full[buf], (sbk / RAW_BUFS) & 1);
      if (!ok || s_fail) { ok = false; break; }
      constexpr int NH = 2 / TPR;   // halves of the k-block this thread converts
      uint32_t c[NH][WPH];
      if (active) {
        const unsigned char* rrow = raw + buf * RAW_B + r * 128;
#pragma unroll
        for (int hh = 0; hh < NH; ++hh)
#pragma unroll
          for (int i = 0; i < WPH / 4; ++i) {
            const int chunk = kbl * (2 * WPH / 4) + (h + hh) * (WPH / 4) + i;
            const uint4 v = *(const uint4*)(rrow + ((chunk ^ (r & 7)) << 4));
            c[hh][4 * i] = v.x; c[hh][4 * i + 1] = v.y; c[hh][4 * i + 2] = v.z; c[hh][4 * i + 3] = v.w;
          }
      }
      if (sit >= STAGES) ok = mbar_wait_backoff(&empty[st], ((sit / STAGES) - 1) & 1);
      if (!ok || s_fail) { ok = false; break; }
      if (active)
      {
#pragma unroll
        for (int hh = 0; hh < NH; ++hh) dequant_half<BITS>(c[hh], sv2, bv2, b_tiles + st * B_STAGE + (it % KPST) * B_SUB, r, h + hh);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> async proxy (UMMA)
      // One arrival per warp: every lane has written its part of the stage and made it visible to the async
      // proxy above; the warp barrier orders those behind lane 0's arrival.  (256 threads arriving one by one on
      // the same barrier word kept the stage from completing for several hundred cycles.)
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&full_b[st]);
        // Release the codes buffer only now that the loaded words have been consumed: the arrival is not
        // ordered behind a shared-memory load whose result no instruction has waited for yet, and the
        // TMA refill must not overtake the warp's last read.
        if (kbl + DQG >= KPS) mbar_arrive(&raw_empty[buf]);
      }
    }
    if (!ok && !s_fail) { s_fail = 4; atomicCAS(&g_tc_error, 0, 4); }
  } else {
    // ---------------- epilogue: TMEM -> registers -> bf16 rows of y ----------------
    const int q = warp & 3;   // TMEM lane quarter this warp may read
    int ti = 0;
    bool ok = true;
    for (int tile = tile0; tile < ntiles && ok; tile += tstride, ++ti) {
      const TileCoord tc = coords(tile);
      const int m0 = tc.row0, n0 = tc.n0, nend = tc.nend, mend = tc.row_end;
      const bool ksum = m0 + 128 >= mend;   // (same test as the MMA issuer's two_halves)
      const int buf = WIDE ? 0 : ti & 1;
      ok = mbar_wait_relaxed(&acc_full[buf], (WIDE ? ti : ti >> 1) & 1);
      if (!ok || s_fail) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (S > 1) break;   // split-K: one tile per cluster; the partial accumulators are exchanged below
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        if (half == 1 && m0 + 128 >= mend) break;
        const int m = m0 + half * 128 + q * 32 + lane;  // TMEM lane = token row
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256 + half * HALF_COLS + c0, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (ksum) {   // single-half tile: the other half's columns hold the second partial sum over K
            uint32_t w[32];
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256 + HALF_COLS + c0, w);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
          }
          if (m < mend) {
            uint16_t* yrow = TC_SEL4(p.yv, tc.mi) + (int64_t)m * TC_SEL4(p.ldyv, tc.mi) + n0 + c0;
            const int nvalid = nend - (n0 + c0);   // columns of this chunk inside the matrix and the tile
            const bool aligned = (((uintptr_t)yrow) & 15) == 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (aligned && 8 * j + 8 <= nvalid) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
                o.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                o.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                o.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                *(uint4*)(yrow + 8 * j) = o;
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (8 * j + i < nvalid) yrow[8 * j + i] = f32_to_bf16_bits(__uint_as_float(v[8 * j + i]));
              }
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&acc_empty[buf]);  // this accumulator set may be overwritten
    }
    if (!ok && !s_fail) { s_fail = 5; atomicCAS(&g_tc_error, 0, 5); }
  }
  if constexpr (CAN_SPLIT) {
    if (S > 1) {
      // Every role of every CTA of the cluster has left its loops (the epilogue warps after their own CTA's
      // accumulator was complete), so the pipeline buffers of rank 0 are free: ranks 1.. write their fp32
      // partial tiles there (rows padded by 16 bytes against bank conflicts), rank 0 adds them to its own
      // accumulator and stores, one or two 128-token halves.
      const bool epi = warp >= kEpiWarp0 && warp < kEpiWarp0 + kEpiWarps;
      const int q = warp & 3;
      const int pitch = (BN + 31) / 32 * 32 * 4 + 16;      // bytes per partial row: whole 32-column chunks + padding
      const bool have_tile = tile0 < ntiles && !s_fail;
      const TileCoord tc = coords(have_tile ? tile0 : 0);
      const int nhalf = tc.row0 + 128 < tc.row_end ? 2 : 1;   // token halves in use (the host keeps the buffer in bounds)
      cluster_sync_tc();
      if (epi && crank != 0 && have_tile) {
#pragma unroll 1
        for (int half = 0; half < nhalf; ++half) {
          const uint32_t dst0 = smem_u32(smem) + (uint32_t)(((crank - 1) * nhalf * 128 + half * 128 + q * 32 + lane) * pitch);
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + half * HALF_COLS + c0, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (nhalf == 1) {   // second partial sum over K
              uint32_t w[32];
              tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + HALF_COLS + c0, w);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
              st_cluster_v4(dst0 + (uint32_t)(c0 + 4 * j) * 4u, 0u,
                            make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                        __uint_as_float(v[4 * j + 3])));
          }
        }
      }
      cluster_sync_tc();
      if (epi && crank == 0 && have_tile) {
#pragma unroll 1
        for (int half = 0; half < nhalf; ++half) {
          const int m = tc.row0 + half * 128 + q * 32 + lane;
          const unsigned char* src0 = smem + (size_t)(half * 128 + q * 32 + lane) * pitch;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + half * HALF_COLS + c0, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
            if (nhalf == 1) {   // second partial sum over K
              tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + HALF_COLS + c0, v);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] += __uint_as_float(v[j]);
            }
            for (int k = 0; k + 1 < S; ++k) {
              const float4* pr = (const float4*)(src0 + (size_t)k * nhalf * 128 * pitch + (size_t)c0 * 4);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 a = pr[j];
                f[4 * j] += a.x; f[4 * j + 1] += a.y; f[4 * j + 2] += a.z; f[4 * j + 3] += a.w;
              }
            }
            if (m < tc.row_end) {
              uint16_t* yrow = TC_SEL4(p.yv, tc.mi) + (int64_t)m * TC_SEL4(p.ldyv, tc.mi) + tc.n0 + c0;
              const int nvalid = tc.nend - (tc.n0 + c0);
              const bool aligned = (((uintptr_t)yrow) & 15) == 0;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (aligned && 8 * j + 8 <= nvalid) {
                  uint4 o;
                  o.x = pack_bf16x2(f[8 * j], f[8 * j + 1]);
                  o.y = pack_bf16x2(f[8 * j + 2], f[8 * j + 3]);
                  o.z = pack_bf16x2(f[8 * j + 4], f[8 * j + 5]);
                  o.w = pack_bf16x2(f[8 * j + 6], f[8 * j + 7]);
                  *(uint4*)(yrow + 8 * j) = o;
                } else {
#pragma unroll
                  for (int i = 0; i < 8; ++i)
                    if (8 * j + i < nvalid) yrow[8 * j + i] = f32_to_bf16_bits(f[8 * j + i]);
                }
              }
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u));
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static bool tried = false;
  std::lock_guard<std::mutex> setup_lk(setup_mutex());
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeFn)sym;
  }
  return fn;
}

constexpr size_t pipe_bytes_tc(bool grouped, bool wide, bool half = false) {   // stages + code ring
  return (size_t)stages_of(grouped, wide, half) * (A_STAGE_BYTES + kb_per_stage_of(half) * bn_max_of(wide, grouped) * BK * 2) +
         (size_t)raw_bufs_of(grouped, wide, half) * bn_max_of(wide, grouped) * 128;
}
constexpr size_t smem_bytes_tc(bool grouped, bool wide, bool half = false) {
  return pipe_bytes_tc(grouped, wide, half) + (3 * stages_of(grouped, wide, half) + 4 + 2 * raw_bufs_of(grouped, wide, half)) * 8 + 16 +
         (grouped ? (size_t)2 * (kMaxGroupExperts + 1) * 4 : 0) + (wide ? 0 : 1024);
}
static_assert(smem_bytes_tc(false, true) <= 227 * 1024 && smem_bytes_tc(true, true) <= 227 * 1024, "wide form does not fit in shared memory");
static_assert(smem_bytes_tc(false, false) <= 227 * 1024 && smem_bytes_tc(true, false) <= 227 * 1024, "shared memory");
static_assert(smem_bytes_tc(false, false, true) <= 227 * 1024, "few-token form does not fit in shared memory");

// pipeline buffers reused by the split-K exchange (either few-token form)
constexpr size_t STAGES_DENSE_BYTES = pipe_bytes_tc(false, false) < pipe_bytes_tc(false, false, true) ? pipe_bytes_tc(false, false) : pipe_bytes_tc(false, false, true);


// Weight rows per tile: the candidate whose tile count fills the last wave best.  Time per tile ~ rows + 40:
// the activation traffic of a k-block through shared memory does not shrink with the tile, so narrow tiles
// only pay when they put otherwise idle SMs to work (few weight rows, long K, few tokens).
int64_t count_tiles(const int64_t* N, int nmat, int bn) {   // weight-row blocks of all matrices (tiles never straddle two)
  int64_t t = 0;
  for (int i = 0; i < nmat; ++i) t += (N[i] + bn - 1) / bn;
  return t;
}
int pick_bn(int64_t M, const int64_t* N, int nmat, int nsm, int bn_max = BN_MAX) {
  const int64_t tiles_m = (M + BM - 1) / BM;
  int best = bn_max;
  int64_t best_cost = -1;
  for (int bn = bn_max; bn >= 32; bn -= 16) {
    const int64_t tiles = tiles_m * count_tiles(N, nmat, bn);
    const int64_t waves = (tiles + nsm - 1) / nsm;
    const int64_t cost = waves * (bn + 40);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

}  // namespace

bool qmm_tc_supported(const QmmArgs& a) {
  if (!a.transpose || a.nbatch != 1) return false;
  if (a.bits != 4 && a.bits != 8) return false;
  if (a.gs != 64 && a.gs != 128) return false;
  if (a.x_dtype != QB200_BFLOAT16) return false;
  if (a.K % 256 != 0 || a.K < 256 || a.N < 1 || a.M < 1) return false;   // whole 128-byte super-blocks of codes
  if (a.M > (1 << 24) || a.N > (1 << 24)) return false;
  if ((((uintptr_t)a.x) & 15) != 0 || (a.ldx * 2) % 16 != 0) return false;
  if ((((uintptr_t)a.w) & 15) != 0 || (a.ldw * 4) % 16 != 0) return false;
  if (get_encode() == nullptr) return false;
  return true;
}

namespace {

// One launch of either form.  x: [M rows][K] bf16 with row pitch ldx; weights: `wrows` rows (N for the dense
// form, E * N stacked expert rows for the grouped form) with pitches ldw / lds.
struct TcLaunch {
  const void* x; int64_t M, K, ldx;
  const uint32_t* w; const uint16_t* s; const uint16_t* b; int64_t wrows, N, ldw, lds;
  uint16_t* y; int64_t ldy;
  int bits, gs;
  const void* rhs; int rhs_i64; int E;   // grouped form only
};

template <int BITS, bool GROUPED, bool WIDE, bool HALF = false>
cudaError_t launch_tc_inst(const CUtensorMap& xmap, const TcMaps& wmap, const TcK& p, dim3 grid, cudaStream_t st,
                           int cluster = 1) {
  static bool done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  constexpr size_t smem = smem_bytes_tc(GROUPED, WIDE, HALF);
  {
  std::lock_guard<std::mutex> setup_lk(setup_mutex());   // first use on a device, from any thread
  if (dev < 0 || dev >= 64 || !done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(qmm_tc_kernel<BITS, GROUPED, WIDE, HALF>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) done[dev] = true;
  }
  }
  if (cluster > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, qmm_tc_kernel<BITS, GROUPED, WIDE, HALF>, xmap, wmap, p);
  }
  qmm_tc_kernel<BITS, GROUPED, WIDE, HALF><<<grid, kThreads, smem, st>>>(xmap, wmap, p);
  return cudaGetLastError();
}

// CTAs that clusters of `cluster` CTAs of the dense form can keep resident at once (cluster placement is per GPC,
// so this is less than the SM count for clusters of 4).
template <int BITS>
int split_capacity(int cluster) {
  static int cached[64][5] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  std::lock_guard<std::mutex> setup_lk(setup_mutex());
  if (cached[dev][cluster] == 0) {
    constexpr size_t smem = smem_bytes_tc(false, false);
    int n = 0;
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3((unsigned)(sm_count() / cluster * cluster));
    q.blockDim = dim3(kThreads);
    q.dynamicSmemBytes = smem;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = cluster; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
    q.attrs = qa;
    q.numAttrs = 1;
    if (cudaFuncSetAttribute(qmm_tc_kernel<BITS, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, qmm_tc_kernel<BITS, false, false>, &q) != cudaSuccess) {
      (void)cudaGetLastError();
      n = 0;
    }
    cached[dev][cluster] = n > 0 ? n * cluster : -1;
  }
  return cached[dev][cluster] > 0 ? cached[dev][cluster] : 0;
}

// `nmat` matrices against the same activations (dense forms; every entry shares x, M, K, bits and group size with
// the first; the grouped form takes one).
cudaError_t launch_tc(const TcLaunch* av, int nmat, bool grouped, cudaStream_t st) {
  const TcLaunch& a = av[0];
  int64_t Nv[kMaxTcMat];
  for (int i = 0; i < nmat; ++i) Nv[i] = av[i].N;
  int64_t Ntot = 0, Nmin = a.N;
  for (int i = 0; i < nmat; ++i) { Ntot += Nv[i]; Nmin = Nv[i] < Nmin ? Nv[i] : Nmin; }
  EncodeFn enc = get_encode();
  if (!enc) return cudaErrorNotSupported;
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
  const cuuint64_t strides[1] = {(cuuint64_t)a.ldx * 2};
  const cuuint32_t box[2] = {BK, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)a.x, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  TcK p;
  const int nsm = sm_count();
  // Wide tiles when both 128-token halves of a tile are in use and there are enough weight rows to fill the GPU
  // with them; the grouped form does not know its tile count on the host and takes full-width dense tiles.
  // (grouped: many rows per expert on average, so that most tiles have both halves)
  const bool wide = grouped ? (a.M >= 192 * (int64_t)a.E && a.N >= 256) : (a.M > 256 && Nmin >= 1024);
  if (grouped) {
    // tile width with the best product of (rows used / rows multiplied) and the width's own efficiency
    // (time per tile ~ width + 40, as in pick_bn)
    const int cap = bn_max_of(wide, true);
    int best = cap;
    double best_score = -1.0;
    for (int bn = cap; bn >= 64; bn -= 16) {
      const double used = (double)a.N / (double)((a.N + bn - 1) / bn * bn);
      const double score = used * bn / (bn + 40.0);
      if (score > best_score) { best_score = score; best = bn; }
    }
    p.BN = a.N >= 64 ? best : (int)((a.N + 15) / 16 * 16);
  } else {
    p.BN = pick_bn(a.M, Nv, nmat, nsm, bn_max_of(wide));
  }
  // Split-K over a cluster when a few-token problem has too few tiles to occupy the GPU: with one tile per CTA
  // the time is the number of k-blocks a CTA walks (plus ~6 k-block times for the exchange), whatever the tile
  // width, so K is cut in 4 or 2 and the tile is made just wide enough for tiles x ranks to fit the SMs.
  p.ksplit = 1;
  const bool half = !grouped && !wide && a.M <= 128;   // no tile has a second token half: stages of one x box
  if (!grouped && !wide && a.M <= 256) {
    const int gshift = a.gs == 128 ? 1 : 0;
    const int nkb_all = (int)(a.K / BK);
    const int64_t plain_tiles = count_tiles(Nv, nmat, p.BN);
    const int64_t plain_cost = ((plain_tiles + nsm - 1) / nsm) * nkb_all;
    for (int sp = 4; sp >= 2; sp >>= 1) {
      if (nkb_all % (sp * (8 << gshift)) != 0 || nkb_all / sp < 8) continue;   // whole scale windows per rank
      const int cap = a.bits == 4 ? split_capacity<4>(sp) : split_capacity<8>(sp);   // resident CTAs in clusters of sp
      const int max_tiles = cap / sp;
      if (max_tiles < 1) continue;
      int bn = (int)((Ntot + max_tiles - 1) / max_tiles);
      bn = (bn + 15) / 16 * 16;
      if (bn < 32) bn = 32;
      while (bn <= BN_MAX && count_tiles(Nv, nmat, bn) > max_tiles) bn += 16;   // (tiles do not straddle matrices)
      if (bn > BN_MAX) continue;
      if ((size_t)(sp - 1) * (a.M > 128 ? 256 : 128) * ((bn + 31) / 32 * 32 * 4 + 16) > (size_t)STAGES_DENSE_BYTES) continue;   // exchange buffer
      if (nkb_all / sp + 6 < plain_cost) { p.ksplit = sp; p.BN = bn; break; }
    }
  }
  // packed codes as a [rows][K * bits / 32] array of 32-bit words: 128 bytes of BN rows per copy
  TcMaps wmap;
  for (int i = 0; i < kMaxTcMat; ++i) {
    const TcLaunch& m = av[i < nmat ? i : 0];
    const cuuint64_t wdims[2] = {(cuuint64_t)(m.K * m.bits / 32), (cuuint64_t)m.wrows};
    const cuuint64_t wstrides[1] = {(cuuint64_t)m.ldw * 4};
    const cuuint32_t wbox[2] = {32, (cuuint32_t)p.BN};
    r = enc(&wmap.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)m.w, wdims, wstrides, wbox, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  }
  p.nmat = nmat;
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.gshift = a.gs == 128 ? 1 : 0;
  p.tiles_m = (int)((a.M + BM - 1) / BM);
  p.sb_vec = (a.K % (512 << p.gshift)) == 0;
  p.tstart[0] = 0;
  for (int i = 0; i < kMaxTcMat; ++i) {
    const TcLaunch& m = av[i < nmat ? i : 0];
    p.sv[i] = m.s; p.bv[i] = m.b; p.yv[i] = m.y;
    p.Nv[i] = (int)m.N; p.ldsv[i] = m.lds; p.ldyv[i] = m.ldy;
    p.tstart[i + 1] = p.tstart[i] + (i < nmat ? p.tiles_m * (int)((m.N + p.BN - 1) / p.BN) : 0);
    if (i < nmat && !((m.lds % 8 == 0) && ((((uintptr_t)m.s) | ((uintptr_t)m.b)) & 15) == 0)) p.sb_vec = 0;
  }
  p.ntiles = p.tstart[nmat];   // dense forms; the grouped form counts on the device
  p.rhs = a.rhs; p.rhs_i64 = a.rhs_i64; p.E = a.E;
  dim3 grid((unsigned)((!grouped && p.ntiles < nsm) ? p.ntiles : nsm), 1, 1);
  if (p.ksplit > 1) {
    grid = dim3((unsigned)(p.ntiles * p.ksplit), 1, 1);   // one tile per cluster
    if (half) return a.bits == 4 ? launch_tc_inst<4, false, false, true>(map, wmap, p, grid, st, p.ksplit)
                                 : launch_tc_inst<8, false, false, true>(map, wmap, p, grid, st, p.ksplit);
    return a.bits == 4 ? launch_tc_inst<4, false, false>(map, wmap, p, grid, st, p.ksplit)
                       : launch_tc_inst<8, false, false>(map, wmap, p, grid, st, p.ksplit);
  }
  if (grouped && wide) return a.bits == 4 ? launch_tc_inst<4, true, true>(map, wmap, p, grid, st) : launch_tc_inst<8, true, true>(map, wmap, p, grid, st);
  if (grouped) return a.bits == 4 ? launch_tc_inst<4, true, false>(map, wmap, p, grid, st) : launch_tc_inst<8, true, false>(map, wmap, p, grid, st);
  if (wide) return a.bits == 4 ? launch_tc_inst<4, false, true>(map, wmap, p, grid, st) : launch_tc_inst<8, false, true>(map, wmap, p, grid, st);
  if (half) return a.bits == 4 ? launch_tc_inst<4, false, false, true>(map, wmap, p, grid, st) : launch_tc_inst<8, false, false, true>(map, wmap, p, grid, st);
  return a.bits == 4 ? launch_tc_inst<4, false, false>(map, wmap, p, grid, st) : launch_tc_inst<8, false, false>(map, wmap, p, grid, st);
}

}  // namespace

cudaError_t launch_qmm_tc(const QmmArgs& a, cudaStream_t st) {
  TcLaunch l;
  l.x = (const char*)a.x + a.xb.offset(0) * 2; l.M = a.M; l.K = a.K; l.ldx = a.ldx;
  l.w = a.w + a.wb.offset(0);
  l.s = (const uint16_t*)a.s + a.sb.offset(0);
  l.b = (const uint16_t*)a.b + a.sb.offset(0);
  l.wrows = a.N; l.N = a.N; l.ldw = a.ldw; l.lds = a.lds;
  l.y = (uint16_t*)a.y + a.yb.offset(0); l.ldy = a.ldy;
  l.bits = a.bits; l.gs = a.gs;
  l.rhs = nullptr; l.rhs_i64 = 0; l.E = 0;
  return launch_tc(&l, 1, false, st);
}

// `count` (<= 4) matrices against the same activations in one launch: every entry has passed qmm_tc_supported
// and shares x, M, K, bits and group size with the first.  Few-token forms only (M <= 256): that is where a
// launch is short enough for its fixed part and its partly filled wave to matter.
bool qmm_tc_multi_supported(const QmmArgs* a, int count) {
  if (count < 2 || count > kMaxTcMat || a[0].M > 256) return false;
  for (int i = 0; i < count; ++i) {
    if (!qmm_tc_supported(a[i])) return false;
    if (a[i].x != a[0].x || a[i].M != a[0].M || a[i].K != a[0].K || a[i].bits != a[0].bits || a[i].gs != a[0].gs ||
        a[i].ldx != a[0].ldx || a[i].xb.offset(0) != a[0].xb.offset(0))
      return false;
  }
  return true;
}
cudaError_t launch_qmm_tc_multi(const QmmArgs* a, int count, cudaStream_t st) {
  TcLaunch l[kMaxTcMat];
  for (int i = 0; i < count; ++i) {
    l[i].x = (const char*)a[i].x + a[i].xb.offset(0) * 2; l[i].M = a[i].M; l[i].K = a[i].K; l[i].ldx = a[i].ldx;
    l[i].w = a[i].w + a[i].wb.offset(0);
    l[i].s = (const uint16_t*)a[i].s + a[i].sb.offset(0);
    l[i].b = (const uint16_t*)a[i].b + a[i].sb.offset(0);
    l[i].wrows = a[i].N; l[i].N = a[i].N; l[i].ldw = a[i].ldw; l[i].lds = a[i].lds;
    l[i].y = (uint16_t*)a[i].y + a[i].yb.offset(0); l[i].ldy = a[i].ldy;
    l[i].bits = a[i].bits; l[i].gs = a[i].gs;
    l[i].rhs = nullptr; l[i].rhs_i64 = 0; l[i].E = 0;
  }
  return launch_tc(l, count, false, st);
}

// gather_qmm with the rows sorted by expert (the reference's prefill MoE path: x [I, 1, K] already gathered,
// rhs [I] ascending, mlx-serve src/transformer.zig:15007-15035) as a grouped GEMM: every expert's run of rows
// is a dense problem against that expert's matrix.
bool gather_tc_supported(const GatherArgs& a) {
  if (!a.sorted || a.lhs != nullptr || a.M != 1) return false;
  if (a.XB != a.I) return false;                       // one activation row per output row, in order
  for (int d = 0; d < a.xbcast.nd; ++d)
    if (a.xbcast.shape[d] != 1 && a.xbcast.stride[d] == 0) return false;   // no broadcast of x
  if (a.bits != 4 && a.bits != 8) return false;
  if (a.gs != 64 && a.gs != 128) return false;
  if (a.x_dtype != QB200_BFLOAT16) return false;
  if (a.K % 256 != 0 || a.K < 256 || a.N < 16 || a.I < 1 || a.I > (1 << 24) || a.E < 1 || a.E > kMaxGroupExperts) return false;
  if (a.E * a.N > (int64_t)1 << 30) return false;
  if ((((uintptr_t)a.x) & 15) != 0 || (a.K * 2) % 16 != 0) return false;
  if ((((uintptr_t)a.w) & 15) != 0 || (a.K * a.bits / 8) % 16 != 0) return false;
  if (a.w_expert_stride != a.N * (a.K * a.bits / 32) || a.s_expert_stride != a.N * (a.K / a.gs)) return false;
  if (a.rhs_dtype != QB200_INT64 && a.rhs_dtype != QB200_INT32 && a.rhs_dtype != QB200_UINT32) return false;
  if (get_encode() == nullptr) return false;
  return true;
}

cudaError_t launch_gather_tc(const GatherArgs& a, cudaStream_t st) {
  TcLaunch l;
  l.x = a.x; l.M = a.I; l.K = a.K; l.ldx = a.K;
  l.w = a.w; l.s = (const uint16_t*)a.s; l.b = (const uint16_t*)a.b;
  l.wrows = a.E * a.N; l.N = a.N; l.ldw = a.K * a.bits / 32; l.lds = a.K / a.gs;
  l.y = (uint16_t*)a.y; l.ldy = a.N;
  l.bits = a.bits; l.gs = a.gs;
  l.rhs = a.rhs; l.rhs_i64 = a.rhs_dtype == QB200_INT64; l.E = (int)a.E;
  return launch_tc(&l, 1, true, st);
}


void qmm_tc_error_reset() {
  const int zero = 0;
  cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
}

int qmm_tc_error_code() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int));
  return v;
}

}  // namespace qb

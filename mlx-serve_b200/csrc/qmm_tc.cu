// Prefill-width quantized matmul on the 5th-generation tensor cores:
// y[M, N] = x[M, K] . What[N, K]^T with What = bf16(q*s + b).
//
// Replaces the dense prefill route of qmatmulBits: prefillDqGemm (dequantize to
// a bf16 [N, K] transient, then a dense GEMM; mlx-serve
// src/transformer.zig:20987-21011) and stock qmm_t for large M
// (src/transformer.zig:20894-20983).  The weight term is rounded to bf16 once,
// exactly as that route's dequantised transient is (src/transformer.zig:20872-20873);
// accumulation is fp32 in tensor memory.  No [N, K] transient ever reaches HBM:
// each CTA dequantises the 128 x 64 weight tile it is about to multiply
// straight into the swizzled shared-memory operand.
//
// CTA tile: 256 tokens x 128 weight rows, K in steps of 64.
//   warp 4 lane 0 : TMA producer -- two 128x64 bf16 boxes of x per stage
//                   (cp.async.bulk.tensor.2d, SWIZZLE_128B, no multicast), then
//                   the single-thread tcgen05.mma issuer (M=128, N=128, K=16 x4,
//                   two accumulators of 128 columns in TMEM) and tcgen05.commit.
//   warps 0-3     : one thread per weight row: packed codes -> exact bf16
//                   integers (byte shuffles) -> one bf16 FMA with the group's
//                   scale and bias -> the K-major SWIZZLE_128B operand row;
//                   after the main loop the same warps drain TMEM
//                   (tcgen05.ld 32x32b) and store bf16 rows of y.
// Every mbarrier wait is bounded: on expiry the kernel records an error code,
// leaves its loops, frees its tensor memory and returns.
#include <cuda.h>

#include "kernels.h"

namespace qb {
namespace {

constexpr int BM = 256, BN = 128, BK = 64, STAGES = 4;
constexpr int kDequantThreads = 128;
constexpr int kThreads = kDequantThreads + 32;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // two 128-row boxes
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr uint32_t kSpinLimit = 1u << 24;

__device__ int g_tc_error = 0;  // 0 = ok; otherwise the code of the wait that expired

struct TcK {
  const uint32_t* w; const uint16_t* s; const uint16_t* b; uint16_t* y;
  int M, N, K;
  int64_t ldw, lds, ldy;
  int gshift;   // scale column = (k / 64) >> gshift
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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
               : "memory");
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
// bf16 x bf16 -> f32, A and B K-major, M = 128, N = 128
__device__ __forceinline__ uint32_t make_idesc() {
  uint32_t d = 0;
  d |= 1u << 4;                  // c format f32
  d |= 1u << 7;                  // a format bf16
  d |= 1u << 10;                 // b format bf16
  d |= (uint32_t)(BN >> 3) << 17;
  d |= (uint32_t)(128 >> 4) << 24;
  return d;
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
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

// 64 codes of one weight row -> 64 bf16 values q*s+b (one rounding), written as the 128-byte row
// `r` of a K-major SWIZZLE_128B tile (16-byte chunk c lands at chunk c ^ (r & 7)).
template <int BITS>
__device__ __forceinline__ void dequant_row(const uint32_t* codes, uint32_t sb2, uint32_t bb2, unsigned char* tile, int r) {
  // sb2 / bb2: the group's scale / bias replicated in both bf16 lanes
  const __nv_bfloat162 s2 = *(const __nv_bfloat162*)&sb2, b2 = *(const __nv_bfloat162*)&bb2;
  unsigned char* row = tile + r * 128;
  if constexpr (BITS == 4) {
    const __nv_bfloat162 c128 = __float2bfloat162_rn(128.f);
#pragma unroll
    for (int c = 0; c < 8; ++c) {  // one packed word = 8 values = one 16-byte chunk of bf16
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
      *(uint4*)(row + ((c ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    const float sf = bf16lo(sb2), bf = bf16lo(bb2);
#pragma unroll
    for (int c = 0; c < 8; ++c) {  // two packed words = 8 values
      uint32_t o[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t w = codes[2 * c + h];
        const float f0 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)) - 8388608.f;
        const float f1 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)) - 8388608.f;
        const float f2 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7542)) - 8388608.f;
        const float f3 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7543)) - 8388608.f;
        o[2 * h] = pack_bf16x2(fmaf(f0, sf, bf), fmaf(f1, sf, bf));
        o[2 * h + 1] = pack_bf16x2(fmaf(f2, sf, bf), fmaf(f3, sf, bf));
      }
      *(uint4*)(row + ((c ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

template <int BITS>
__global__ void __launch_bounds__(kThreads, 1) qmm_tc_kernel(const __grid_constant__ CUtensorMap xmap, TcK p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* a_tiles = smem;                                   // [STAGES][2][128 x 64 bf16]
  unsigned char* b_tiles = smem + STAGES * A_STAGE_BYTES;          // [STAGES][128 x 64 bf16]
  uint64_t* bars = (uint64_t*)(b_tiles + STAGES * B_STAGE_BYTES);  // full_a[S], full_b[S], empty[S], acc
  uint64_t* full_a = bars, *full_b = bars + STAGES, *empty = bars + 2 * STAGES, *acc_bar = bars + 3 * STAGES;
  uint32_t* tmem_slot = (uint32_t*)(bars + 3 * STAGES + 1);
  __shared__ int s_fail;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int nkb = p.K / BK;
  constexpr int WPK = BK * BITS / 32;  // packed words per row per k-block

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full_a[i], 1); mbar_init(&full_b[i], kDequantThreads); mbar_init(&empty[i], 1); }
    mbar_init(acc_bar, 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {  // tensor-memory allocation: 256 columns (two 128x128 fp32 accumulators)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      // ---------------- TMA producer + MMA issuer (one thread) ----------------
      const uint32_t idesc = make_idesc();
      const bool two_halves = m0 + 128 < p.M;  // the second 128 token rows hold real tokens
      int fail = 0;
      // prologue: fill the pipeline
      int loaded = 0;
      for (; loaded < STAGES && loaded < nkb; ++loaded) {
        mbar_expect_tx(&full_a[loaded], A_STAGE_BYTES);
        const uint32_t dst = smem_u32(a_tiles + loaded * A_STAGE_BYTES);
        tma_load_2d(dst, &xmap, &full_a[loaded], loaded * BK, m0);
        tma_load_2d(dst + 128 * BK * 2, &xmap, &full_a[loaded], loaded * BK, m0 + 128);
      }
      for (int kb = 0; kb < nkb && !fail; ++kb) {
        const int st = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&full_a[st], ph)) { fail = 1; break; }
        if (!mbar_wait(&full_b[st], ph)) { fail = 2; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(a_tiles + st * A_STAGE_BYTES), b_addr = smem_u32(b_tiles + st * B_STAGE_BYTES);
#pragma unroll
        for (int k16 = 0; k16 < BK / 16; ++k16) {
          const uint64_t bd = make_desc(b_addr + k16 * 32);
          const uint32_t accum = (kb > 0 || k16 > 0) ? 1u : 0u;
          umma(tmem_base, make_desc(a_addr + k16 * 32), bd, idesc, accum);
          if (two_halves) umma(tmem_base + 128, make_desc(a_addr + 128 * BK * 2 + k16 * 32), bd, idesc, accum);
        }
        umma_commit(&empty[st]);  // frees this stage once the MMAs above have read it
        // refill the stage of the PREVIOUS k-block (its MMAs finish while the ones just issued are queued)
        if (kb >= 1 && loaded < nkb) {
          const int ls = (kb - 1) % STAGES;
          if (!mbar_wait(&empty[ls], ((kb - 1) / STAGES) & 1)) { fail = 3; break; }
          mbar_expect_tx(&full_a[ls], A_STAGE_BYTES);
          const uint32_t dst = smem_u32(a_tiles + ls * A_STAGE_BYTES);
          tma_load_2d(dst, &xmap, &full_a[ls], loaded * BK, m0);
          tma_load_2d(dst + 128 * BK * 2, &xmap, &full_a[ls], loaded * BK, m0 + 128);
          ++loaded;
        }
      }
      umma_commit(acc_bar);
      if (fail) { s_fail = fail; atomicExch(&g_tc_error, fail); }
    }
  } else {
    // ---------------- dequant producers: thread = weight row ----------------
    const int r = tid;
    int n = n0 + r;
    n = n < p.N ? n : p.N - 1;
    const uint32_t* wrow = p.w + (int64_t)n * p.ldw;
    const uint16_t* srow = p.s + (int64_t)n * p.lds;
    const uint16_t* brow = p.b + (int64_t)n * p.lds;
    uint32_t codes[WPK], ncodes[WPK];
    uint32_t sc = 0, bi = 0, nsc = 0, nbi = 0;
    auto fetch = [&](int kb, uint32_t (&c)[WPK], uint32_t& s2, uint32_t& b2) {
      const uint4* src = (const uint4*)(wrow + (int64_t)kb * WPK);
#pragma unroll
      for (int i = 0; i < WPK / 4; ++i) {
        const uint4 v = __ldg(src + i);
        c[4 * i] = v.x; c[4 * i + 1] = v.y; c[4 * i + 2] = v.z; c[4 * i + 3] = v.w;
      }
      const uint32_t sv = __ldg(srow + (kb >> p.gshift)), bv = __ldg(brow + (kb >> p.gshift));
      s2 = sv | (sv << 16);
      b2 = bv | (bv << 16);
    };
    if (nkb > 0) fetch(0, codes, sc, bi);
    bool ok = true;
    for (int kb = 0; kb < nkb; ++kb) {
      const int st = kb % STAGES;
      if (kb + 1 < nkb) fetch(kb + 1, ncodes, nsc, nbi);
      if (kb >= STAGES && ok) ok = mbar_wait(&empty[st], ((kb / STAGES) - 1) & 1);
      if (!ok) break;
      dequant_row<BITS>(codes, sc, bi, b_tiles + st * B_STAGE_BYTES, r);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> async proxy (UMMA)
      mbar_arrive(&full_b[st]);
#pragma unroll
      for (int i = 0; i < WPK; ++i) codes[i] = ncodes[i];
      sc = nsc; bi = nbi;
    }
    if (!ok) atomicExch(&g_tc_error, 4);
    // ---------------- epilogue: TMEM -> registers -> bf16 rows of y ----------------
    bool acc_ok = ok && mbar_wait(acc_bar, 0);
    if (!acc_ok) atomicExch(&g_tc_error, 5);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (acc_ok && s_fail == 0) {
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        if (half == 1 && m0 + 128 >= p.M) break;
        const int m = m0 + half * 128 + warp * 32 + lane;  // TMEM lane = token row
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + half * 128 + c0, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (m < p.M) {
            uint16_t* yrow = p.y + (int64_t)m * p.ldy + n0 + c0;
            if (n0 + c0 + 32 <= p.N && (((uintptr_t)yrow) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
                o.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                o.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                o.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                *(uint4*)(yrow + 8 * j) = o;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (n0 + c0 + j < p.N) yrow[j] = f32_to_bf16_bits(__uint_as_float(v[j]));
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u));
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static bool tried = false;
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

constexpr size_t kSmemBytes = (size_t)STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + (3 * STAGES + 1) * 8 + 16 + 1024;

}  // namespace

bool qmm_tc_supported(const QmmArgs& a) {
  if (!a.transpose || a.nbatch != 1) return false;
  if (a.bits != 4 && a.bits != 8) return false;
  if (a.gs != 64 && a.gs != 128) return false;
  if (a.x_dtype != QB200_BFLOAT16) return false;
  if (a.K % BK != 0 || a.K < BK || a.N < 1 || a.M < 1) return false;
  if (a.M > (1 << 24) || a.N > (1 << 24)) return false;
  if ((((uintptr_t)a.x) & 15) != 0 || (a.ldx * 2) % 16 != 0) return false;
  if ((((uintptr_t)a.w) & 15) != 0 || (a.ldw * 4) % 16 != 0) return false;
  if (get_encode() == nullptr) return false;
  return true;
}

cudaError_t launch_qmm_tc(const QmmArgs& a, cudaStream_t st) {
  EncodeFn enc = get_encode();
  if (!enc) return cudaErrorNotSupported;
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
  const cuuint64_t strides[1] = {(cuuint64_t)a.ldx * 2};
  const cuuint32_t box[2] = {BK, 128};
  const cuuint32_t estr[2] = {1, 1};
  const void* xptr = (const char*)a.x + a.xb.offset(0) * 2;
  CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)xptr, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  TcK p;
  p.w = a.w + a.wb.offset(0);
  p.s = (const uint16_t*)a.s + a.sb.offset(0);
  p.b = (const uint16_t*)a.b + a.sb.offset(0);
  p.y = (uint16_t*)a.y + a.yb.offset(0);
  p.M = (int)a.M; p.N = (int)a.N; p.K = (int)a.K;
  p.ldw = a.ldw; p.lds = a.lds; p.ldy = a.ldy;
  p.gshift = a.gs == 128 ? 1 : 0;
  dim3 grid((unsigned)((a.N + BN - 1) / BN), (unsigned)((a.M + BM - 1) / BM), 1);
  static bool done[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int bi = a.bits == 4 ? 0 : 1;
  if (dev < 0 || dev >= 64 || !done[bi][dev]) {
    cudaError_t e = a.bits == 4
        ? cudaFuncSetAttribute(qmm_tc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes)
        : cudaFuncSetAttribute(qmm_tc_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) done[bi][dev] = true;
  }
  if (a.bits == 4) qmm_tc_kernel<4><<<grid, kThreads, kSmemBytes, st>>>(map, p);
  else qmm_tc_kernel<8><<<grid, kThreads, kSmemBytes, st>>>(map, p);
  return cudaGetLastError();
}

int qmm_tc_error_code() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int));
  return v;
}

}  // namespace qb

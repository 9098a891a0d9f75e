// Persistent weight-streaming quantized matmul for decode widths (M <= 32):
// y[M, N] = x[M, K] . What[N, K]^T, 4/8-bit affine codes, fp32 accumulate.
//
// Replaces mlx_quantized_matmul(transpose=true) as called by qmatmulBits
// (mlx-serve src/transformer.zig:20894-20983) at decode widths and the small-M
// verify lanes (src/transformer.zig:1317-1453).
//
// The kernel is HBM-bound by construction, so it is organised around keeping
// bytes in flight rather than around the math:
//  * one persistent CTA per SM (16 warps = two groups of 8); every warp owns a
//    private ring of cp.async (LDGSTS, 128-bit per lane) stages in shared
//    memory, each stage = 16 weight rows x 128 contiguous bytes plus their
//    scales and biases, so ~100 KiB of packed weights are in flight per SM
//    independent of register pressure; no thread ever waits on another warp
//    for data (cp.async.wait_group + __syncwarp only), so there is no
//    barrier-protocol that could hang;
//  * activations are staged once per CTA (per 4096-wide K pass) in MMA
//    fragment order; a group's 8 warps split K for one 16-row tile and reduce
//    through shared memory behind a named barrier, double-buffered so the
//    weight stream never drains;
//  * codes are expanded in registers (LOP3 magic number for 4-bit, PRMT into an
//    fp32 mantissa for 8-bit) to exact bf16 integers and contracted with
//    mma.sync.m16n8k16; scale and bias are applied per 64-wide group to the
//    fp32 accumulators:  y += s*(sum (c+q) x) + (b - c s)*(sum x), c = 128 or 0,
//    so the weight term q*s+b keeps fp32 precision;
//  * fp32 activations ride as bf16 hi + lo halves in two token slots.
// Nothing is written to global scratch; the only global writes are y.
#include "kernels.h"
#include "qmv_frag.cuh"

namespace qb {
namespace {

constexpr int kWarpsPerGroup = 8;   // K split inside a group
constexpr int kGroups = 2;          // groups (independent tile lists) per CTA
constexpr int kThreads = kWarpsPerGroup * kGroups * 32;
constexpr int kStages = 4;          // cp.async ring depth per warp
constexpr int kStageW = 2048;       // 16 rows x 128 B of packed codes
constexpr int kStageBytes = kStageW + 256;  // + 16 rows x (scales, biases)

__host__ __device__ constexpr int kc_for(int nt) { return 4096 / nt; }

struct StreamK {
  const void* x; const uint32_t* w; const uint16_t* s; const uint16_t* b; void* y;
  int M, N, K;
  int64_t ldx, ldw, lds, ldy;
  int gshift, x_f32;
  int total_groups;   // groups over the whole grid (tile t belongs to group t % total_groups)
  int ntiles;
  int npass, kc;      // K passes of kc values
  int ntl_max;        // max tiles per group (sizes the multi-pass accumulator)
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async8(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void group_barrier(int grp) {
  asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "n"(kWarpsPerGroup * 32) : "memory");
}

// 16-byte chunk swizzle inside a 128-byte stage row so that the fragment reads
// (64-bit per lane at 4 bits, 128-bit at 8 bits) are bank-conflict free.
template <int BITS> __device__ __forceinline__ int swz(int row) {
  return BITS == 4 ? 2 * (row & 3) : 4 * (row & 1);
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
__global__ void __launch_bounds__(kThreads, 1) qmv_stream_kernel(StreamK p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int U = WReg<BITS>::U;            // 64-wide groups per unit
  constexpr int CK = 64 * U;                  // K values per unit (128 bytes per row)
  constexpr int SLOTS = M1 ? 1 : 8 * NT;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int grp = warp / kWarpsPerGroup, ks = warp % kWarpsPerGroup;
  const int ggrp = blockIdx.x * kGroups + grp;  // global group id

  // ---- shared memory carve-up ----
  const int kc = p.kc;
  unsigned char* sp = smem;
  unsigned char* ring = sp;                   sp += (size_t)kGroups * kWarpsPerGroup * kStages * kStageBytes;
  uint2* xfrag = (uint2*)sp;                  sp += M1 ? (size_t)(kc / 16) * 4 * 8 : (size_t)(kc / 16) * NT * 32 * 8;
  float* xsum = (float*)sp;                   sp += (size_t)(kc / 64) * SLOTS * 4;
  float* red = (float*)sp;                    sp += (size_t)kGroups * 2 * kWarpsPerGroup * NT * 128 * 4;
  float* yacc = (float*)sp;                   // [kGroups][ntl_max][NT*128], only when npass > 1

  unsigned char* my_ring = ring + (size_t)warp * kStages * kStageBytes;
  const int ntl = ggrp < p.ntiles ? (p.ntiles - ggrp + p.total_groups - 1) / p.total_groups : 0;
  const int ut = p.K / CK, upk = kc / CK;

  // ---- producer: cp.async one item (16 rows x 128 B + scales/biases) into a ring stage ----
  auto issue = [&](const ItemIter& it, int stage) {
    unsigned char* st = my_ring + stage * kStageBytes;
    const int tile = ggrp + it.tl * p.total_groups;
    const int64_t k0 = (int64_t)it.pass * kc + (int64_t)it.u * CK;
    const int chunk = lane & 7;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = (lane >> 3) + 4 * r;
      int n = tile * 16 + row;
      n = n < p.N ? n : p.N - 1;
      const unsigned char* src = (const unsigned char*)(p.w + (int64_t)n * p.ldw) + k0 * BITS / 8 + chunk * 16;
      cp_async16(st + row * 128 + ((chunk ^ swz<BITS>(row)) << 4), src);
    }
    {
      const int row = lane & 15;
      int n = tile * 16 + row;
      n = n < p.N ? n : p.N - 1;
      const uint16_t* base = (lane >> 4) ? p.b : p.s;
      const uint16_t* src = base + (int64_t)n * p.lds + ((k0 >> 6) >> p.gshift);
      unsigned char* dst = st + kStageW + (lane >> 4) * 128 + row * 8;
      if (BITS == 4 && p.gshift == 0) cp_async8(dst, src);
      else cp_async4(dst, src);
    }
  };

  ItemIter prod;
  prod.init(ks, ntl, p.npass, upk, ut);
  int issued = 0;
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) {
    if (prod.valid()) { issue(prod, issued % kStages); prod.next(); }
    cp_async_commit();
    ++issued;
  }

  const int tok_per_tile = p.x_f32 ? 4 : 8;
  const int esz = p.x_f32 ? 4 : 2;
  int consumed = 0;
  int red_buf = 0;

  for (int pass = 0; pass < p.npass; ++pass) {
    const int k_base = pass * kc;
    const int klen = (p.K - k_base) < kc ? (p.K - k_base) : kc;
    if (pass > 0) __syncthreads();
    // ---- stage activations of this pass in fragment order ----
    if constexpr (M1) {
      const int nitems = klen / 16;
      for (int base = 0; base < nitems; base += kThreads) {
        const int it = base + tid;
        const bool ok = it < nitems;
        float v[16];
        if (ok) {
          const uint16_t* px = (const uint16_t*)p.x + k_base + it * 16;
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = bf16_bits_to_f32(px[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) sum += v[j];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (ok) {
          const int gi = it >> 2, tt = it & 3;
          if (tt == 0) xsum[gi] = sum;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint2 f;
            f.x = pack_bf16x2(v[kperm<BITS>(i, 0)], v[kperm<BITS>(i, 1)]);
            f.y = pack_bf16x2(v[kperm<BITS>(i, 2)], v[kperm<BITS>(i, 3)]);
            xfrag[(gi * 4 + i) * 4 + tt] = f;
          }
        }
      }
    } else {
      const int ngroups = klen >> 6;
      for (int item = warp; item < ngroups * NT; item += kThreads / 32) {
        const int gi = item / NT, nt = item - gi * NT;
        const int m = nt * tok_per_tile + (p.x_f32 ? (g & 3) : g);
        float v[16];
        if (m >= p.M) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        } else if (!p.x_f32) {
          const uint16_t* px = (const uint16_t*)p.x + (int64_t)m * p.ldx + k_base + gi * 64 + 16 * t;
          if ((((uintptr_t)px) & 15) == 0) {
            const uint4 a = *(const uint4*)px, c = *(const uint4*)(px + 8);
            const uint32_t r[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) { v[2 * j] = bf16lo(r[j]); v[2 * j + 1] = bf16hi(r[j]); }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = bf16_bits_to_f32(px[j]);
          }
        } else {
          const float* px = (const float*)p.x + (int64_t)m * p.ldx + k_base + gi * 64 + 16 * t;
          const bool lo_half = g >= 4;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float f = px[j];
            const float hi = bf16_bits_to_f32(f32_to_bf16_bits(f));
            v[j] = lo_half ? bf16_bits_to_f32(f32_to_bf16_bits(f - hi)) : hi;
          }
        }
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) sum += v[j];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (t == 0) xsum[(gi * NT + nt) * 8 + g] = sum;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint2 f;
          f.x = pack_bf16x2(v[kperm<BITS>(i, 0)], v[kperm<BITS>(i, 1)]);
          f.y = pack_bf16x2(v[kperm<BITS>(i, 2)], v[kperm<BITS>(i, 3)]);
          xfrag[((gi * 4 + i) * NT + nt) * 32 + lane] = f;
        }
      }
    }
    __syncthreads();

    const int upt = (ut - pass * upk) < upk ? (ut - pass * upk) : upk;
    for (int tl = 0; tl < ntl; ++tl) {
      float tot[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.f;

      for (int u = ks; u < upt; u += kWarpsPerGroup) {
        // keep the ring full, then wait for this item's bytes
        if (prod.valid()) { issue(prod, issued % kStages); prod.next(); }
        cp_async_commit();
        ++issued;
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const unsigned char* st = my_ring + (consumed % kStages) * kStageBytes;
        ++consumed;

        float s_lo[U], s_hi[U], b_lo[U], b_hi[U];
        {
          const unsigned char* sb = st + kStageW;
          if (BITS == 4 && p.gshift == 0) {
            const uint2 a = *(const uint2*)(sb + g * 8), c = *(const uint2*)(sb + (g + 8) * 8);
            const uint2 d = *(const uint2*)(sb + 128 + g * 8), e = *(const uint2*)(sb + 128 + (g + 8) * 8);
            const uint32_t ra[2] = {a.x, a.y}, rc[2] = {c.x, c.y}, rd[2] = {d.x, d.y}, re[2] = {e.x, e.y};
#pragma unroll
            for (int j = 0; j < U; ++j) {
              s_lo[j] = (j & 1) ? bf16hi(ra[(j >> 1) & 1]) : bf16lo(ra[(j >> 1) & 1]);
              s_hi[j] = (j & 1) ? bf16hi(rc[(j >> 1) & 1]) : bf16lo(rc[(j >> 1) & 1]);
              b_lo[j] = (j & 1) ? bf16hi(rd[(j >> 1) & 1]) : bf16lo(rd[(j >> 1) & 1]);
              b_hi[j] = (j & 1) ? bf16hi(re[(j >> 1) & 1]) : bf16lo(re[(j >> 1) & 1]);
            }
          } else {
            // U values at stride (1 >> gshift): 4-bit g128 -> 2 distinct, 8-bit g64 -> 2 distinct
            const uint32_t a = *(const uint32_t*)(sb + g * 8), c = *(const uint32_t*)(sb + (g + 8) * 8);
            const uint32_t d = *(const uint32_t*)(sb + 128 + g * 8), e = *(const uint32_t*)(sb + 128 + (g + 8) * 8);
#pragma unroll
            for (int j = 0; j < U; ++j) {
              const int idx = BITS == 4 ? (j >> 1) : j;  // 4-bit reaches here only with group size 128
              s_lo[j] = idx ? bf16hi(a) : bf16lo(a);
              s_hi[j] = idx ? bf16hi(c) : bf16lo(c);
              b_lo[j] = idx ? bf16hi(d) : bf16lo(d);
              b_hi[j] = idx ? bf16hi(e) : bf16lo(e);
            }
          }
        }
        const int gl0 = u * U;  // first 64-group of this unit inside the staged pass
#pragma unroll
        for (int j = 0; j < U; ++j) {
          typename WReg<BITS>::T wl, wh;
          if constexpr (BITS == 4) {
            const int c = 2 * j + (t >> 1), off = (t & 1) * 8;
            wl = *(const uint2*)(st + g * 128 + ((c ^ swz<4>(g)) << 4) + off);
            wh = *(const uint2*)(st + (g + 8) * 128 + ((c ^ swz<4>(g + 8)) << 4) + off);
          } else {
            const int c = 4 * j + t;
            wl = *(const uint4*)(st + g * 128 + ((c ^ swz<8>(g)) << 4));
            wh = *(const uint4*)(st + (g + 8) * 128 + ((c ^ swz<8>(g + 8)) << 4));
          }
          float acc[NT][4];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
          const int gl = gl0 + j;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t a[4];
            expand<BITS>(wl, i, a[0], a[2]);
            expand<BITS>(wh, i, a[1], a[3]);
            if constexpr (M1) {
              uint2 bf = make_uint2(0u, 0u);
              if (g == 0) bf = xfrag[(gl * 4 + i) * 4 + t];
              mma_bf16_16816(acc[0], a, bf.x, bf.y);
            } else {
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                const uint2 bf = xfrag[((gl * 4 + i) * NT + nt) * 32 + lane];
                mma_bf16_16816(acc[nt], a, bf.x, bf.y);
              }
            }
          }
          const float sl = s_lo[j], sh = s_hi[j];
          const float bl = fmaf(-code_base<BITS>(), sl, b_lo[j]);
          const float bh = fmaf(-code_base<BITS>(), sh, b_hi[j]);
          if constexpr (M1) {
            const float xs = xsum[gl];
            tot[0][0] += fmaf(sl, acc[0][0], bl * xs);
            tot[0][2] += fmaf(sh, acc[0][2], bh * xs);
          } else {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const float2 xs = *(const float2*)&xsum[(gl * NT + nt) * 8 + 2 * t];
              tot[nt][0] += fmaf(sl, acc[nt][0], bl * xs.x);
              tot[nt][1] += fmaf(sl, acc[nt][1], bl * xs.y);
              tot[nt][2] += fmaf(sh, acc[nt][2], bh * xs.x);
              tot[nt][3] += fmaf(sh, acc[nt][3], bh * xs.y);
            }
          }
        }
        __syncwarp();
      }

      // ---- reduce the group's 8 K-slices for this tile ----
      float* rb = red + ((size_t)(grp * 2 + red_buf) * kWarpsPerGroup) * NT * 128;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float* base = rb + ((size_t)ks * NT + nt) * 128;
        *(float2*)&base[g * 8 + 2 * t] = make_float2(tot[nt][0], tot[nt][1]);
        *(float2*)&base[(g + 8) * 8 + 2 * t] = make_float2(tot[nt][2], tot[nt][3]);
      }
      group_barrier(grp);
      const int tile = ggrp + tl * p.total_groups;
      const int gt = tid - grp * (kWarpsPerGroup * 32);  // thread index inside the group
      const int ncols = M1 ? 1 : NT * tok_per_tile;
      for (int o = gt; o < 16 * ncols; o += kWarpsPerGroup * 32) {
        const int row = o & 15, col = o >> 4;
        const int nt = M1 ? 0 : col / tok_per_tile, c = M1 ? 0 : col - nt * tok_per_tile;
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < kWarpsPerGroup; ++k) {
          const float* base = rb + ((size_t)k * NT + nt) * 128;
          v += base[row * 8 + c];
          if (!M1 && p.x_f32) v += base[row * 8 + c + 4];
        }
        if (p.npass > 1) {
          float* ya = yacc + ((size_t)(grp * p.ntl_max + tl) * NT * 128) + col * 16 + row;
          if (pass > 0) v += *ya;
          if (pass + 1 < p.npass) { *ya = v; continue; }
        }
        const int n = tile * 16 + row;
        if (n < p.N && col < p.M) {
          if (p.x_f32) ((float*)p.y)[(int64_t)col * p.ldy + n] = v;
          else ((uint16_t*)p.y)[(int64_t)col * p.ldy + n] = f32_to_bf16_bits(v);
        }
      }
      red_buf ^= 1;
    }
  }
  cp_async_wait<0>();
  (void)esz;
}

struct LaunchCfg { int grid; size_t smem; int ntl_max; int total_groups; };

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
bool plan_stream(StreamK& p, int NT, bool M1, int* grid_out, size_t* smem_out) {
  const int nsm = sm_count();
  const int ntiles = (p.N + 15) / 16;
  const int per = (ntiles + kGroups * nsm - 1) / (kGroups * nsm);
  const int total_groups = (ntiles + per - 1) / per;
  const int grid = (total_groups + kGroups - 1) / kGroups;
  p.ntiles = ntiles;
  p.total_groups = grid * kGroups;
  p.ntl_max = (ntiles + p.total_groups - 1) / p.total_groups;
  p.kc = p.K < kc_for(NT) ? p.K : kc_for(NT);
  if (M1) p.kc = p.K;
  p.npass = (p.K + p.kc - 1) / p.kc;
  const int slots = M1 ? 1 : 8 * NT;
  size_t smem = (size_t)kGroups * kWarpsPerGroup * kStages * kStageBytes;
  smem += M1 ? (size_t)(p.kc / 16) * 32 : (size_t)(p.kc / 16) * NT * 256;
  smem += (size_t)(p.kc / 64) * slots * 4;
  smem += (size_t)kGroups * 2 * kWarpsPerGroup * NT * 512;
  if (p.npass > 1) smem += (size_t)kGroups * p.ntl_max * NT * 512;
  *grid_out = grid;
  *smem_out = smem;
  return smem <= 227 * 1024;
}

void pick_inst(const StreamK& p, int* NT, bool* M1) {
  const int tok = p.x_f32 ? 4 : 8;
  const int nt = (p.M + tok - 1) / tok;
  *M1 = (p.M == 1 && !p.x_f32 && p.K <= 32768);
  *NT = nt <= 1 ? 1 : (nt <= 2 ? 2 : 4);
}

template <int BITS, int NT, bool M1>
cudaError_t launch_inst(StreamK p, cudaStream_t st) {
  int grid = 0;
  size_t smem = 0;
  if (!plan_stream(p, NT, M1, &grid, &smem)) return cudaErrorInvalidConfiguration;
  auto kern = qmv_stream_kernel<BITS, NT, M1>;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  kern<<<grid, kThreads, smem, st>>>(p);
  return cudaGetLastError();
}

template <int BITS>
cudaError_t launch_bits(const StreamK& p, cudaStream_t st) {
  int nt; bool m1;
  pick_inst(p, &nt, &m1);
  if (m1) return launch_inst<BITS, 1, true>(p, st);
  if (nt == 1) return launch_inst<BITS, 1, false>(p, st);
  if (nt == 2) return launch_inst<BITS, 2, false>(p, st);
  return launch_inst<BITS, 4, false>(p, st);
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
  p.N = (int)a.N; p.K = (int)a.K; p.x_f32 = a.x_dtype == QB200_FLOAT32;
  const int tok = p.x_f32 ? 4 : 8;
  p.M = (int)(a.M < 4 * tok ? a.M : 4 * tok);
  int nt, grid; bool m1; size_t smem;
  pick_inst(p, &nt, &m1);
  if (!plan_stream(p, nt, m1, &grid, &smem)) return false;
  return true;
}

cudaError_t launch_qmv_stream(const QmmArgs& a, cudaStream_t st) {
  StreamK p;
  p.w = a.w + a.wb.offset(0); p.s = (const uint16_t*)a.s + a.sb.offset(0); p.b = (const uint16_t*)a.b + a.sb.offset(0);
  p.N = (int)a.N; p.K = (int)a.K;
  p.ldx = a.ldx; p.ldw = a.ldw; p.lds = a.lds; p.ldy = a.ldy;
  p.gshift = a.gs == 128 ? 1 : 0;
  p.x_f32 = a.x_dtype == QB200_FLOAT32;
  const int esz = p.x_f32 ? 4 : 2;
  const int tok = p.x_f32 ? 4 : 8;
  const int64_t block = 4 * tok;  // wider M re-streams the weights once per token block
  for (int64_t m0 = 0; m0 < a.M; m0 += block) {
    p.x = (const char*)a.x + (a.xb.offset(0) + m0 * a.ldx) * esz;
    p.y = (char*)a.y + (a.yb.offset(0) + m0 * a.ldy) * esz;
    p.M = (int)((a.M - m0) < block ? (a.M - m0) : block);
    cudaError_t e = a.bits == 4 ? launch_bits<4>(p, st) : launch_bits<8>(p, st);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace qb

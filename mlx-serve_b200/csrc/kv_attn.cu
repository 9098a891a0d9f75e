// Decode attention read directly from the affine-quantized KV cache.
//
// Semantics: kv_quant.quantAttention with T_q == 1 (mlx-serve
// src/kv_quant.zig:478-687) = softmax(scale * q.K^T + mask) . V over the
// dequantised cache, K/V kept in fp32 as the packed decode kernel does
// (src/transformer.zig:4890-5006), extended to a batch with per-sequence
// lengths (the additive length mask of src/transformer.zig:10216-10249).
// Two phases like the reference kernel: split-KV partials (m, l,
// unnormalised O) then the merge of src/transformer.zig:5194-5203.
#include <math.h>

#include <type_traits>

#include <cstdlib>

#include "kernels.h"

namespace qb {
namespace {

constexpr int kMaxGqa = 8;
constexpr float kNegBig = -1e30f;  // clamp for fully masked blocks (src/transformer.zig:4957-4958)

struct SplitPlan {
  int nsplit;
  int64_t tokens_per_split;  // multiple of 128
};

// Deterministic in (B, Hkv, T) so that the workspace query and the launch agree.
// A split is served by one CTA of 8 warps that take its 128-token blocks round-robin.  The plan minimises
//   waves of CTAs over the GPU x (blocks per warp + a fixed per-CTA cost of ~0.7 block times)
// summed over the two residencies the fast kernel has (one CTA per SM at 8 bits, two at 4 bits; the bit
// width is not an input here because the workspace query does not know it).
__host__ SplitPlan plan_splits(int64_t B, int64_t Hkv, int64_t T) {
  SplitPlan p;
  const int nsm = sm_count();   // CTA slots: one CTA per SM at 8 bits, two at 4 bits
  const int64_t pairs = B * Hkv > 0 ? B * Hkv : 1;
  int64_t max_ns = (T + 255) / 256;  // at least 256 tokens per split
  if (max_ns < 1) max_ns = 1;
  if (max_ns > 1024) max_ns = 1024;
  double best = -1.0;
  int64_t best_ns = 1, best_tps = 128;
  for (int64_t ns = 1; ns <= max_ns; ++ns) {
    int64_t tps = (T + ns - 1) / ns;
    tps = (tps + 127) / 128 * 128;
    if (tps < 128) tps = 128;
    const int64_t ns_eff = (T + tps - 1) / tps > 0 ? (T + tps - 1) / tps : 1;
    const double per_cta = (double)((tps / 128 + 7) / 8) + 0.7;
    double cost = 0.0;
    for (int slots = nsm; slots <= 2 * nsm; slots += nsm) cost += (double)((pairs * ns_eff + slots - 1) / slots) * per_cta;
    if (best < 0.0 || cost < best - 1e-9) { best = cost; best_ns = ns_eff; best_tps = tps; }
  }
  p.nsplit = (int)best_ns;
  p.tokens_per_split = best_tps;
  return p;
}

struct KvK {
  KvAttnArgs a;
  int nsplit;
  int64_t tps;
  int gqa;
  float* part_m;  // [B, Hq, nsplit]
  float* part_l;  // [B, Hq, nsplit]
  float* part_o;  // [B, Hq, nsplit, Dv]
};

__device__ __forceinline__ float load_mask(const KvK& p, int64_t b, int64_t t) {
  if (!p.a.mask) return 0.f;
  const int64_t off = b * p.a.mask_bstride + t;
  if (p.a.mask_dtype == QB200_FLOAT32) return ((const float*)p.a.mask)[off];
  return bf16_bits_to_f32(((const uint16_t*)p.a.mask)[off]);
}

// Generic CUDA-core path: any head dim that is a multiple of 32, any group
// size, GQA <= 8.  One warp per token; lanes stride over the packed words.
template <int BITS, class TAB>
__global__ void __launch_bounds__(128) kv_split_generic(KvK p, const __grid_constant__ TAB tab) {
  constexpr bool PTRS = std::is_same<TAB, KvSeqTable>::value;
  constexpr int VPW = 32 / BITS;
  extern __shared__ float smem[];
  const KvAttnArgs& a = p.a;
  const int split = blockIdx.x, hk = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int g = p.gqa;
  const int D = (int)a.D, Dv = (int)a.Dv;
  float* qs = smem;                       // [g][D]
  float* red_m = qs + g * D;              // [nwarp][g]
  float* red_l = red_m + nwarp * g;       // [nwarp][g]
  float* red_o = red_l + nwarp * g;       // [nwarp][g][Dv]
  for (int i = threadIdx.x; i < g * D; i += blockDim.x) {
    const int h = i / D, e = i - h * D;
    const int64_t off = b * a.q_str[0] + (int64_t)(hk * g + h) * a.q_str[1] + e;
    qs[i] = a.q_dtype == QB200_FLOAT32 ? ((const float*)a.q)[off] : bf16_bits_to_f32(((const uint16_t*)a.q)[off]);
  }
  __syncthreads();
  // this sequence's cache view: its own pointers and strides, or a slice of the batched tensors
  const uint32_t* kq_b; const uint32_t* vq_b;
  const uint16_t* ks_b; const uint16_t* kb_b; const uint16_t* vs_b; const uint16_t* vb_b;
  int64_t kq_tok, ksb_tok, vq_tok, vsb_tok, T_seq;
  if constexpr (PTRS) {
    const KvSeq& q = tab.s[b];
    kq_b = q.kq + hk * q.kq_str[0]; vq_b = q.vq + hk * q.vq_str[0];
    ks_b = (const uint16_t*)q.ks + hk * q.ksb_str[0]; kb_b = (const uint16_t*)q.kb + hk * q.ksb_str[0];
    vs_b = (const uint16_t*)q.vs + hk * q.vsb_str[0]; vb_b = (const uint16_t*)q.vb + hk * q.vsb_str[0];
    kq_tok = q.kq_str[1]; ksb_tok = q.ksb_str[1]; vq_tok = q.vq_str[1]; vsb_tok = q.vsb_str[1];
    T_seq = q.T;
  } else {
    kq_b = a.kq + b * a.kq_str[0] + hk * a.kq_str[1]; vq_b = a.vq + b * a.vq_str[0] + hk * a.vq_str[1];
    ks_b = (const uint16_t*)a.ks + b * a.ksb_str[0] + hk * a.ksb_str[1]; kb_b = (const uint16_t*)a.kb + b * a.ksb_str[0] + hk * a.ksb_str[1];
    vs_b = (const uint16_t*)a.vs + b * a.vsb_str[0] + hk * a.vsb_str[1]; vb_b = (const uint16_t*)a.vb + b * a.vsb_str[0] + hk * a.vsb_str[1];
    kq_tok = a.kq_str[2]; ksb_tok = a.ksb_str[2]; vq_tok = a.vq_str[2]; vsb_tok = a.vsb_str[2];
    T_seq = a.T;
  }
  int64_t len = a.kv_lens ? (int64_t)a.kv_lens[b] : T_seq;
  if (len > T_seq) len = T_seq;
  const int64_t t0 = (int64_t)split * p.tps;
  int64_t t1 = t0 + p.tps;
  if (t1 > len) t1 = len;

  const int kwords = D / VPW, vwords = Dv / VPW;
  const int vw_per_lane = (vwords + 31) / 32;  // <= 2 for Dv <= 256 at 8 bits
  float m[kMaxGqa], l[kMaxGqa];
  float o[kMaxGqa][2][VPW];
#pragma unroll
  for (int h = 0; h < kMaxGqa; ++h) {
    m[h] = kNegBig; l[h] = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int k = 0; k < VPW; ++k) o[h][j][k] = 0.f;
  }
  for (int64_t t = t0 + warp; t < t1; t += nwarp) {
    const uint32_t* krow = kq_b + t * kq_tok;
    const uint16_t* ksr = ks_b + t * ksb_tok;
    const uint16_t* kbr = kb_b + t * ksb_tok;
    float dot[kMaxGqa];
#pragma unroll
    for (int h = 0; h < kMaxGqa; ++h) dot[h] = 0.f;
    for (int w = lane; w < kwords; w += 32) {
      const uint32_t word = krow[w];
      const int e0 = w * VPW;
      const float sc = bf16_bits_to_f32(ksr[e0 / a.gs]), bi = bf16_bits_to_f32(kbr[e0 / a.gs]);
#pragma unroll
      for (int k = 0; k < VPW; ++k) {
        const float kv = __fadd_rn(__fmul_rn((float)((word >> (k * BITS)) & ((1u << BITS) - 1u)), sc), bi);
#pragma unroll
        for (int h = 0; h < kMaxGqa; ++h)
          if (h < g) dot[h] = fmaf(qs[h * D + e0 + k], kv, dot[h]);
      }
    }
    const float mk = load_mask(p, b, t);
    float pw[kMaxGqa];
#pragma unroll
    for (int h = 0; h < kMaxGqa; ++h) {
      if (h < g) {
        float d = dot[h];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        float sv = d * a.scale + mk;
        if (!(sv > kNegBig)) sv = kNegBig;  // -inf mask entries and NaN guards
        const float mn = fmaxf(m[h], sv);
        const float alpha = __expf(m[h] - mn);
        pw[h] = sv <= kNegBig ? 0.f : __expf(sv - mn);
        l[h] = l[h] * alpha + pw[h];
        m[h] = mn;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int k = 0; k < VPW; ++k) o[h][j][k] *= alpha;
      }
    }
    const uint32_t* vrow = vq_b + t * vq_tok;
    const uint16_t* vsr = vs_b + t * vsb_tok;
    const uint16_t* vbr = vb_b + t * vsb_tok;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int w = lane + 32 * j;
      if (j < vw_per_lane && w < vwords) {
        const uint32_t word = vrow[w];
        const int e0 = w * VPW;
        const float sc = bf16_bits_to_f32(vsr[e0 / a.gs]), bi = bf16_bits_to_f32(vbr[e0 / a.gs]);
#pragma unroll
        for (int k = 0; k < VPW; ++k) {
          const float vv = __fadd_rn(__fmul_rn((float)((word >> (k * BITS)) & ((1u << BITS) - 1u)), sc), bi);
#pragma unroll
          for (int h = 0; h < kMaxGqa; ++h)
            if (h < g) o[h][j][k] = fmaf(pw[h], vv, o[h][j][k]);
        }
      }
    }
  }
  // merge the warps of this CTA
  if (lane == 0)
    for (int h = 0; h < g; ++h) { red_m[warp * g + h] = m[h]; red_l[warp * g + h] = l[h]; }
#pragma unroll
  for (int h = 0; h < kMaxGqa; ++h)
    if (h < g)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int w = lane + 32 * j;
        if (j < vw_per_lane && w < vwords)
#pragma unroll
          for (int k = 0; k < VPW; ++k) red_o[(warp * g + h) * Dv + w * VPW + k] = o[h][j][k];
      }
  __syncthreads();
  for (int i = threadIdx.x; i < g * Dv; i += blockDim.x) {
    const int h = i / Dv, e = i - h * Dv;
    float M = kNegBig;
    for (int w = 0; w < nwarp; ++w) M = fmaxf(M, red_m[w * g + h]);
    float L = 0.f, O = 0.f;
    for (int w = 0; w < nwarp; ++w) {
      const float sc = __expf(red_m[w * g + h] - M);
      L += red_l[w * g + h] * sc;
      O += red_o[(w * g + h) * Dv + e] * sc;
    }
    const int64_t pi = (b * a.Hq + hk * g + h) * p.nsplit + split;
    p.part_o[pi * Dv + e] = O;
    if (e == 0) { p.part_m[pi] = M; p.part_l[pi] = L; }
  }
}

// out = (sum_b o_b w_b) / (sum_b l_b w_b), w_b = exp(m_b - max m)  (src/transformer.zig:5194-5203)
__global__ void kv_merge(KvK p) {
  const KvAttnArgs& a = p.a;
  const int h = blockIdx.x;
  const int64_t b = blockIdx.y;
  const int64_t base = (b * a.Hq + h) * p.nsplit;
  float M = kNegBig;
  for (int s = 0; s < p.nsplit; ++s) M = fmaxf(M, p.part_m[base + s]);
  float L = 0.f;
  for (int s = 0; s < p.nsplit; ++s) L += p.part_l[base + s] * __expf(p.part_m[base + s] - M);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int e = threadIdx.x; e < a.Dv; e += blockDim.x) {
    float O = 0.f;
    for (int s = 0; s < p.nsplit; ++s) O += p.part_o[(base + s) * a.Dv + e] * __expf(p.part_m[base + s] - M);
    const int64_t off = b * a.o_str[0] + (int64_t)h * a.o_str[1] + e;
    const float v = O * inv;
    if (a.q_dtype == QB200_FLOAT32) ((float*)a.out)[off] = v;
    else ((uint16_t*)a.out)[off] = f32_to_bf16_bits(v);
  }
}

}  // namespace

cudaError_t launch_kv_fast(const KvAttnArgs& a, int nsplit, int64_t tps, float* pm, float* pl, float* po,
                           cudaStream_t st, const KvSeqTable* seqs, bool fused);
constexpr int kMaxFusedSplits = 8;   // the portable cluster size

size_t kv_attn_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t T, int64_t Dv) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || T <= 0 || Dv <= 0) return 0;
  const SplitPlan sp = plan_splits(B, Hkv, T);
  return (size_t)B * Hq * sp.nsplit * (2 + Dv) * sizeof(float);
}

bool kv_attn_supported(const KvAttnArgs& a) {
  if (a.bits != 4 && a.bits != 8) return false;
  if (a.D % 32 != 0 || a.Dv % 32 != 0) return false;
  if (a.Dv * a.bits / 32 > 64) return false;
  const int64_t gqa = a.Hq / a.Hkv;
  if (gqa < 1 || gqa > kMaxGqa) return false;
  if (a.Hkv > 65535 || a.B > 65535) return false;
  return true;
}

// QB200_KV_FUSED_MERGE=0 in the environment keeps the partials-plus-merge-kernel path for every split count (a
// diagnostic for measuring the two against each other on one GPU; read once).
static bool fused_merge_enabled() {
  static const bool v = [] {
    const char* e = getenv("QB200_KV_FUSED_MERGE");
    return !(e && e[0] == '0');
  }();
  return v;
}

cudaError_t launch_kv_attn(const KvAttnArgs& a, cudaStream_t st, const KvSeqTable* seqs) {
  KvK p;
  p.a = a;
  if (a.B <= 0 || a.Hq <= 0 || a.Hkv <= 0 || a.T <= 0 || a.Dv <= 0 || a.workspace == nullptr) return cudaErrorInvalidValue;
  const SplitPlan sp = plan_splits(a.B, a.Hkv, a.T);
  p.nsplit = sp.nsplit;
  p.tps = sp.tokens_per_split;
  p.gqa = (int)(a.Hq / a.Hkv);
  float* ws = (float*)a.workspace;
  p.part_m = ws;
  p.part_l = ws + a.B * a.Hq * sp.nsplit;
  p.part_o = ws + 2 * a.B * a.Hq * sp.nsplit;
  cudaError_t e;
  if (kv_fast_supported(a, seqs)) {
    // Up to 8 splits per (sequence, kv head) run as one thread-block cluster whose rank 0 merges the partial results
    // through distributed shared memory and writes the output: no partials in global memory, no merge launch.
    // Measured against the merge kernel on one GPU (16 sequences, 8 kv heads): 4-bit caches 23.4 against 24.0 us at
    // 4096 tokens and 132.8 against 134.0 us at 32768; 8-bit caches, whose CTAs fill an SM alone, 33.0 against 31.8 us
    // at 4096 tokens -- so only the 4-bit kernel takes the cluster form.
    if (sp.nsplit <= kMaxFusedSplits && a.bits == 4 && fused_merge_enabled()) {
      e = launch_kv_fast(a, sp.nsplit, sp.tokens_per_split, p.part_m, p.part_l, p.part_o, st, seqs, true);
      if (e == cudaSuccess) return e;
      (void)cudaGetLastError();   // a cluster this launch could not place: fall back to partials and the merge kernel
    }
    e = launch_kv_fast(a, sp.nsplit, sp.tokens_per_split, p.part_m, p.part_l, p.part_o, st, seqs, false);
  } else {
    const int nwarp = 4;
    const size_t smem = (size_t)(p.gqa * a.D + 2 * nwarp * p.gqa + nwarp * p.gqa * a.Dv) * sizeof(float);
    dim3 grid((unsigned)sp.nsplit, (unsigned)a.Hkv, (unsigned)a.B);
    const dim3 blk(nwarp * 32);
    if (seqs) {
      e = a.bits == 4 ? launch_kernel(kv_split_generic<4, KvSeqTable>, grid, blk, smem, st, p, *seqs)
                      : launch_kernel(kv_split_generic<8, KvSeqTable>, grid, blk, smem, st, p, *seqs);
    } else {
      e = a.bits == 4 ? launch_kernel(kv_split_generic<4, KvNoTable>, grid, blk, smem, st, p, KvNoTable{})
                      : launch_kernel(kv_split_generic<8, KvNoTable>, grid, blk, smem, st, p, KvNoTable{});
    }
  }
  if (e != cudaSuccess) return e;
  dim3 mgrid((unsigned)a.Hq, (unsigned)a.B, 1);
  return launch_kernel(kv_merge, mgrid, dim3(128), 0, st, p);
}

}  // namespace qb

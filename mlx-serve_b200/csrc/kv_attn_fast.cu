// Split-KV flash-decode over the affine-quantized KV cache, head dim 128,
// group size 64, 4- or 8-bit, GQA <= 4, on the integer tensor cores.
//
// Semantics: kv_quant.quantAttention at T_q == 1 (mlx-serve
// src/kv_quant.zig:478-687) with K/V kept in fp32 (q*s+b) exactly as the packed
// decode kernel does (src/transformer.zig:4890-5006); per-sequence lengths as
// the batched path's additive mask (src/transformer.zig:10216-10249); partials
// merged as src/transformer.zig:5194-5203.
//
// Organisation (HBM-bound: the packed bytes are read once, straight from the
// strided cache views):
//  * grid (split, kv head, sequence); 8 warps per CTA, each warp walks blocks
//    of 128 tokens with its own online softmax and its own cp.async ring of
//    32-token K and V stages (codes + scales + biases), so no warp waits on
//    another for data and nothing can dead-lock.
//  * scores: K codes are the u8 A operand of mma.m16n8k32.s32.u8.s8 (two ANDs
//    and a shift per 8 codes at 4 bits, none at 8 bits); q is staged once per
//    CTA as 15-bit fixed point in two s8 planes per head (the 4 heads of a GQA
//    group x 2 planes fill the n8 tile).  Scale and bias of each (token,
//    64-group) are applied to the s32 sums in fp32.
//  * values: p * v_scale is converted per 128-token block to two s8 planes
//    (the B operand); the V codes become the A operand through
//    ldmatrix.m16n16.trans.b8, which hands each lane four tokens of one byte
//    column -- the transposition the packed layout (codes packed along the head
//    dim, contraction along tokens) otherwise makes expensive.  s32 sums are
//    kept for a whole block and folded into fp32 once per block; the V bias
//    term is a plain fp32 dot of p with the biases.
#include <mutex>

#include <type_traits>

#include "kernels.h"
#include "stream_ptx.cuh"

namespace qb {
namespace {

constexpr int kWarps = 8;
constexpr int kChunk = 32;            // tokens per ring stage
constexpr int kBlockTok = 128;        // tokens per softmax block (4 chunks)
constexpr int kD = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegBig = -1e30f;

template <int BITS> struct Geo {
  static constexpr int ROWB = kD * BITS / 8;              // code bytes per token row
  static constexpr int CHUNKS = ROWB / 16;                // 16-byte chunks per row
  static constexpr int STAGE_BYTES = kChunk * ROWB;       // one ring stage: the codes of 32 tokens
  static constexpr int STAGES = 4;
  // scales and biases travel per 128-token block, double buffered: [2][ks, kb, vs, vb][128 tokens][2 groups] bf16
  static constexpr int SB_BYTES = 2 * 4 * kBlockTok * 4;
};

struct FastK {
  KvAttnArgs a;
  int nsplit;
  int64_t tps;  // tokens per split, multiple of 128
  int gqa;
  int fused;    // the splits of a (sequence, kv head) are the CTAs of one cluster: rank 0 merges them and writes the output
  float* part_m; float* part_l; float* part_o;
};

// Two 16x16 byte matrices, transposed: lanes 0-15 give the row addresses of the first, 16-31 of the
// second.  Lane (g, t) receives for each matrix: r0 = rows 4t..4t+3 of byte column g, r1 = of column g+8.
__device__ __forceinline__ void ldmatrix_b8_trans_x2(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// 16-byte chunk swizzle of a stage row; keeps both the 64/128-bit fragment reads of the score phase and
// the ldmatrix row reads of the value phase at the minimum number of shared-memory wavefronts.
template <int BITS> __device__ __forceinline__ int swz(int row) {
  int f = (((row >> 1) & 1) << 1) ^ ((row >> 3) & 3);
  if (BITS == 8) f ^= (row & 1) << 2;
  return f;
}

__device__ __forceinline__ int fix15(float x, float up) {
  const int v = __float_as_int(fmaf(x, up, 12582912.f)) - 0x4B400000;
  return v > 16383 ? 16383 : v;
}
__device__ __forceinline__ uint32_t plane_byte(int v, int plane) {
  return plane == 0 ? (uint32_t)((v >> 7) & 0xFF) : (uint32_t)(v & 127);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// TAB = KvSeqTable: sequence b reads its own cache view from the table; KvNoTable: one strided [B, Hkv, T, .] tensor.
template <int BITS, class TAB>
__global__ void __launch_bounds__(kWarps * 32, BITS == 4 ? 2 : 1) kv_fast_kernel(FastK p, const __grid_constant__ TAB tab) {
  constexpr bool PTRS = std::is_same<TAB, KvSeqTable>::value;
  using G = Geo<BITS>;
  extern __shared__ __align__(128) unsigned char smem[];
  const KvAttnArgs& a = p.a;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, hk = blockIdx.y;
  const int64_t b = blockIdx.z;

  unsigned char* sp = smem;
  unsigned char* ring = sp;     sp += (size_t)kWarps * G::STAGES * G::STAGE_BYTES;
  unsigned char* sbbuf = sp;    sp += (size_t)kWarps * G::SB_BYTES;
  uint2* qfrag = (uint2*)sp;    sp += 4 * 32 * 8;       // [(grp*2 + mma)][lane]
  float2* qgs = (float2*)sp;    sp += 2 * 4 * 8;        // [grp][head]: (2^(E-14), 2^(E-14) * sum v)
  // after the main loop the ring is reused for the cross-warp merge

  // ---- stage q * scale * log2(e) as two s8 planes per head (one warp; tiny) ----
  if (warp == 0) {
    // item = (head h, 8-value chunk c of the 128-wide row): 4 x 16 = 64 items, two per lane
#pragma unroll
    for (int rep = 0; rep < 2; ++rep) {
      const int item = rep * 32 + lane;
      const int h = item >> 4, c = item & 15;
      float f[8];
      if (h < p.gqa) {
        const int64_t off = b * a.q_str[0] + (int64_t)(hk * p.gqa + h) * a.q_str[1] + c * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          f[j] = (a.q_dtype == QB200_FLOAT32 ? ((const float*)a.q)[off + j] : bf16_bits_to_f32(((const uint16_t*)a.q)[off + j])) *
                 (a.scale * kLog2e);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = 0.f;
      }
      float mx = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmax_nan(mx, fabsf(f[j]));
      mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      int e = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 + 1;
      e = e < -100 ? -100 : (e > 110 ? 110 : e);
      const float up = __uint_as_float((uint32_t)(127 + 14 - e) << 23);
      const float down = poison_if(nonfinite(mx), __uint_as_float((uint32_t)(127 + e - 14) << 23));
      int v[8], sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { v[j] = fix15(f[j], up); sum += v[j]; }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      const int grp = c >> 3, tt = (c >> 1) & 3, jm = c & 1;
      if ((c & 7) == 0) qgs[grp * 4 + h] = make_float2(down, down * (float)sum);
#pragma unroll
      for (int pl = 0; pl < 2; ++pl) {
        uint2 o;
        o.x = plane_byte(v[kslot8<BITS>(0, 0)], pl) | (plane_byte(v[kslot8<BITS>(0, 1)], pl) << 8) |
              (plane_byte(v[kslot8<BITS>(0, 2)], pl) << 16) | (plane_byte(v[kslot8<BITS>(0, 3)], pl) << 24);
        o.y = plane_byte(v[kslot8<BITS>(1, 0)], pl) | (plane_byte(v[kslot8<BITS>(1, 1)], pl) << 8) |
              (plane_byte(v[kslot8<BITS>(1, 2)], pl) << 16) | (plane_byte(v[kslot8<BITS>(1, 3)], pl) << 24);
        qfrag[(grp * 2 + jm) * 32 + (2 * h + pl) * 4 + tt] = o;
      }
    }
  }
  __syncthreads();

  // this sequence's cache view
  const unsigned char* kq_base; const unsigned char* vq_base;
  const uint16_t* ks_base; const uint16_t* kb_base; const uint16_t* vs_base; const uint16_t* vb_base;
  int64_t kq_tok, ksb_tok, vq_tok, vsb_tok, T_seq;
  if constexpr (PTRS) {
    const KvSeq& q = tab.s[b];
    kq_base = (const unsigned char*)(q.kq + hk * q.kq_str[0]);
    vq_base = (const unsigned char*)(q.vq + hk * q.vq_str[0]);
    ks_base = (const uint16_t*)q.ks + hk * q.ksb_str[0]; kb_base = (const uint16_t*)q.kb + hk * q.ksb_str[0];
    vs_base = (const uint16_t*)q.vs + hk * q.vsb_str[0]; vb_base = (const uint16_t*)q.vb + hk * q.vsb_str[0];
    kq_tok = q.kq_str[1]; ksb_tok = q.ksb_str[1]; vq_tok = q.vq_str[1]; vsb_tok = q.vsb_str[1];
    T_seq = q.T;
  } else {
    kq_base = (const unsigned char*)(a.kq + b * a.kq_str[0] + hk * a.kq_str[1]);
    vq_base = (const unsigned char*)(a.vq + b * a.vq_str[0] + hk * a.vq_str[1]);
    ks_base = (const uint16_t*)a.ks + b * a.ksb_str[0] + hk * a.ksb_str[1];
    kb_base = (const uint16_t*)a.kb + b * a.ksb_str[0] + hk * a.ksb_str[1];
    vs_base = (const uint16_t*)a.vs + b * a.vsb_str[0] + hk * a.vsb_str[1];
    vb_base = (const uint16_t*)a.vb + b * a.vsb_str[0] + hk * a.vsb_str[1];
    kq_tok = a.kq_str[2]; ksb_tok = a.ksb_str[2]; vq_tok = a.vq_str[2]; vsb_tok = a.vsb_str[2];
    T_seq = a.T;
  }
  int64_t len = a.kv_lens ? (int64_t)a.kv_lens[b] : T_seq;
  len = len > T_seq ? T_seq : (len < 0 ? 0 : len);
  const int64_t t_begin = (int64_t)split * p.tps;
  int64_t t_end = t_begin + p.tps;
  t_end = t_end > len ? len : t_end;
  const int nblocks = t_end > t_begin ? (int)((t_end - t_begin + kBlockTok - 1) / kBlockTok) : 0;
  const int my_blocks = warp < nblocks ? (nblocks - warp + kWarps - 1) / kWarps : 0;
  const int my_items = my_blocks * 8;  // per block: 4 K chunks then 4 V chunks

  const int64_t last_tok = T_seq > 0 ? T_seq - 1 : 0;

  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(ring + (size_t)warp * G::STAGES * G::STAGE_BYTES);
  const unsigned char* my_ring_p = ring + (size_t)warp * G::STAGES * G::STAGE_BYTES;

  // ---- producer: item i -> (block, K or V, chunk) ----
  auto issue = [&](int item, int stage) {
    const int blk = warp + (item >> 3) * kWarps;
    const int isv = (item >> 2) & 1, ch = item & 3;
    const int64_t tok0 = t_begin + (int64_t)blk * kBlockTok + ch * kChunk;
    const uint32_t st = my_ring + stage * G::STAGE_BYTES;
    const unsigned char* cbase = isv ? vq_base : kq_base;
    const int64_t cstr = (isv ? vq_tok : kq_tok) * 4;  // bytes per token row
    constexpr int RPI = 32 / G::CHUNKS;                          // rows covered per instruction
    const int cc = lane % G::CHUNKS, r0 = lane / G::CHUNKS;
#pragma unroll
    for (int r = 0; r < kChunk / RPI; ++r) {
      const int row = r0 + r * RPI;
      int64_t tok = tok0 + row;
      tok = tok > last_tok ? last_tok : tok;
      cp_async16(st + row * G::ROWB + ((cc ^ swz<BITS>(row)) << 4), cbase + tok * cstr + cc * 16);
    }
  };
  // scales/biases of one 128-token block: lane g of the consumer reads tokens g, g+8, g+16, g+24 of a
  // chunk with one 128-bit load, so token (chunk c, row r) goes to word c*32 + (r&7)*4 + (r>>3).
  const uint32_t my_sb = (uint32_t)__cvta_generic_to_shared(sbbuf + (size_t)warp * G::SB_BYTES);
  const unsigned char* my_sb_p = sbbuf + (size_t)warp * G::SB_BYTES;
  auto issue_sb = [&](int bi) {
    const int blk = warp + bi * kWarps;
    const uint32_t dst0 = my_sb + (bi & 1) * (4 * kBlockTok * 4);
    const uint32_t pos = ((lane & 7) * 4 + (lane >> 3)) * 4;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      int64_t tok = t_begin + (int64_t)blk * kBlockTok + ch * kChunk + lane;
      tok = tok > last_tok ? last_tok : tok;
      const uint32_t d = dst0 + ch * 128 + pos;
      cp_async4(d, ks_base + tok * ksb_tok);
      cp_async4(d + 512, kb_base + tok * ksb_tok);
      cp_async4(d + 1024, vs_base + tok * vsb_tok);
      cp_async4(d + 1536, vb_base + tok * vsb_tok);
    }
  };

  if (my_blocks > 0) issue_sb(0);
  int issued = 0;
#pragma unroll
  for (int i = 0; i < G::STAGES - 1; ++i) {
    if (issued < my_items) issue(issued, issued % G::STAGES);
    cp_async_commit();
    ++issued;
  }
  int consumed = 0;
  auto acquire = [&]() -> const unsigned char* {
    if (issued < my_items) issue(issued, issued % G::STAGES);
    if ((consumed & 7) == 0 && (consumed >> 3) + 1 < my_blocks) issue_sb((consumed >> 3) + 1);
    cp_async_commit();
    ++issued;
    cp_async_wait<G::STAGES - 1>();
    __syncwarp();
    const unsigned char* st = my_ring_p + (consumed % G::STAGES) * G::STAGE_BYTES;
    ++consumed;
    return st;
  };

  // per-lane constants
  const float2 qg0 = qgs[0 * 4 + t], qg1 = qgs[1 * 4 + t];  // this lane's head is t
  uint2 qf[2][2];
#pragma unroll
  for (int grp = 0; grp < 2; ++grp)
#pragma unroll
    for (int j = 0; j < 2; ++j) qf[grp][j] = qfrag[(grp * 2 + j) * 32 + lane];

  float m_run = kNegBig, l_part = 0.f;
  float O[16];   // [mma tile 0..7][row half]: fp32 partial output for head t
  float ob[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 16; ++i) O[i] = 0.f;

  const float* maskrow = a.mask ? (const float*)a.mask : nullptr;

  for (int bi = 0; bi < my_blocks; ++bi) {
    const int blk = warp + bi * kWarps;
    const int64_t tok_blk = t_begin + (int64_t)blk * kBlockTok;
    float sc[16];       // scores (log2 domain) of tokens chunk*32 + g + 8j, head t
    // ---------------- phase 1: scores of 4 chunks ----------------
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      const unsigned char* st = acquire();
      const unsigned char* sbb = my_sb_p + (bi & 1) * (4 * kBlockTok * 4);
      const uint4 sraw = *(const uint4*)(sbb + ch * 128 + g * 16);
      const uint4 braw = *(const uint4*)(sbb + 512 + ch * 128 + g * 16);
      const uint32_t sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w}, bw[4] = {braw.x, braw.y, braw.z, braw.w};
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int tile = 0; tile < 2; ++tile) {
        const int row_lo = tile * 16 + g, row_hi = row_lo + 8;  // tokens j = 2*tile, 2*tile+1 of this lane
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
          uint32_t a0[2], a1[2], a2[2], a3[2];
          if constexpr (BITS == 4) {
            const int c = 2 * grp + (t >> 1), off = (t & 1) * 8;
            const uint2 wl = *(const uint2*)(st + row_lo * G::ROWB + ((c ^ swz<4>(row_lo)) << 4) + off);
            const uint2 wh = *(const uint2*)(st + row_hi * G::ROWB + ((c ^ swz<4>(row_hi)) << 4) + off);
            a0[0] = wl.x & 0x0F0F0F0Fu; a2[0] = (wl.x >> 4) & 0x0F0F0F0Fu;
            a0[1] = wl.y & 0x0F0F0F0Fu; a2[1] = (wl.y >> 4) & 0x0F0F0F0Fu;
            a1[0] = wh.x & 0x0F0F0F0Fu; a3[0] = (wh.x >> 4) & 0x0F0F0F0Fu;
            a1[1] = wh.y & 0x0F0F0F0Fu; a3[1] = (wh.y >> 4) & 0x0F0F0F0Fu;
          } else {
            const int c = 4 * grp + t;
            const uint4 wl = *(const uint4*)(st + row_lo * G::ROWB + ((c ^ swz<8>(row_lo)) << 4));
            const uint4 wh = *(const uint4*)(st + row_hi * G::ROWB + ((c ^ swz<8>(row_hi)) << 4));
            a0[0] = wl.x; a2[0] = wl.y; a0[1] = wl.z; a2[1] = wl.w;
            a1[0] = wh.x; a3[0] = wh.y; a1[1] = wh.z; a3[1] = wh.w;
          }
          int acc[4] = {0, 0, 0, 0};
          mma_u8s8_ordered(acc, a0[0], a1[0], a2[0], a3[0], qf[grp][0].x, qf[grp][0].y);
          mma_u8s8_ordered(acc, a0[1], a1[1], a2[1], a3[1], qf[grp][1].x, qf[grp][1].y);
          const float2 qg = grp == 0 ? qg0 : qg1;
          const float f_lo = (float)(acc[0] * 128 + acc[1]), f_hi = (float)(acc[2] * 128 + acc[3]);
          // token j = 2*tile (row g) and 2*tile+1 (row g+8): scale/bias pair words sw[j], bw[j]; group = half
          const uint32_t swl = sw[2 * tile], swh = sw[2 * tile + 1], bwl = bw[2 * tile], bwh = bw[2 * tile + 1];
          const float s_lo = grp ? bf16hi(swl) : bf16lo(swl), s_hi = grp ? bf16hi(swh) : bf16lo(swh);
          const float b_lo = grp ? bf16hi(bwl) : bf16lo(bwl), b_hi = grp ? bf16hi(bwh) : bf16lo(bwh);
          s4[2 * tile] = fmaf(s_lo * qg.x, f_lo, fmaf(b_lo, qg.y, s4[2 * tile]));
          s4[2 * tile + 1] = fmaf(s_hi * qg.x, f_hi, fmaf(b_hi, qg.y, s4[2 * tile + 1]));
        }
      }
      __syncwarp();
      // token of slot j: chunk base + g + 8*j  (tile = j>>1, row half = j&1)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t tok = tok_blk + ch * kChunk + (j >> 1) * 16 + (j & 1) * 8 + g;
        float v = s4[j];
        if (tok >= t_end) v = kNegBig;
        else if (a.mask) {
          const int64_t mo = b * a.mask_bstride + tok;
          const float mk = a.mask_dtype == QB200_FLOAT32 ? maskrow[mo] : bf16_bits_to_f32(((const uint16_t*)a.mask)[mo]);
          v = fmaf(mk, kLog2e, v);
          if (!(v > kNegBig)) v = kNegBig;
        }
        sc[ch * 4 + j] = v;
      }
    }
    // ---------------- block softmax bookkeeping ----------------
    float mb = sc[0];
#pragma unroll
    for (int i = 1; i < 16; ++i) mb = fmaxf(mb, sc[i]);
    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 4));
    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 8));
    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 16));
    const float m_new = fmaxf(m_run, mb);
    const float alpha = ex2(m_run - m_new);  // both finite (>= -1e30); 0 when the running max was empty
    float psum = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float pv = sc[i] <= kNegBig ? 0.f : ex2(sc[i] - m_new);
      sc[i] = pv;
      psum += pv;
    }
    l_part = l_part * alpha + psum;
    m_run = m_new;
    ob[0] *= alpha;
    ob[1] *= alpha;

    // ---------------- phase 2: values of 4 chunks ----------------
    int accv[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) accv[i][0] = accv[i][1] = accv[i][2] = accv[i][3] = 0;
    // one power-of-two scale per (block, 64-group) for p * v_scale, from the largest |v_scale| of the block
    int emax[2] = {0, 0};
    uint32_t vsw[16];  // v_scale words (two bf16 groups) of this lane's 16 tokens
    {
      const unsigned char* sbb = my_sb_p + (bi & 1) * (4 * kBlockTok * 4);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        const uint4 sraw = *(const uint4*)(sbb + 1024 + ch * 128 + g * 16);
        const uint4 braw = *(const uint4*)(sbb + 1536 + ch * 128 + g * 16);
        const uint32_t sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w}, bw[4] = {braw.x, braw.y, braw.z, braw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          vsw[ch * 4 + j] = sw[j];
          emax[0] = max(emax[0], (int)((sw[j] >> 7) & 0xFF));
          emax[1] = max(emax[1], (int)((sw[j] >> 23) & 0xFF));
          const float pj = sc[ch * 4 + j];
          ob[0] = fmaf(pj, bf16lo(bw[j]), ob[0]);
          ob[1] = fmaf(pj, bf16hi(bw[j]), ob[1]);
        }
      }
    }
    emax[0] = __reduce_max_sync(0xffffffffu, emax[0]);
    emax[1] = __reduce_max_sync(0xffffffffu, emax[1]);
    // the largest weight of the block for head t (long, flat contexts have p << 1: without this the
    // fixed-point grid would be sized for p = 1 and keep only a few bits of p * v_scale)
    int pexp = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) pexp = max(pexp, (int)((__float_as_uint(sc[i]) >> 23) & 0xFF));
    pexp = max(pexp, __shfl_xor_sync(0xffffffffu, pexp, 4));
    pexp = max(pexp, __shfl_xor_sync(0xffffffffu, pexp, 8));
    pexp = max(pexp, __shfl_xor_sync(0xffffffffu, pexp, 16));
    // (per head: lane (g, t) builds and reads back only head t's columns, so up/down may differ by t)
    const int ep = pexp - 126 < 0 ? pexp - 126 : 0;   // p < 2^ep (p <= 1 always)
    float up[2], down[2];
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
      int e = emax[grp] - 127 + 1 + ep;  // |v_scale| < 2^(e - ep) and p < 2^ep
      e = e < -100 ? -100 : (e > 110 ? 110 : e);
      up[grp] = __uint_as_float((uint32_t)(127 + 14 - e) << 23);
      down[grp] = __uint_as_float((uint32_t)(127 + e - 14) << 23);
    }
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      const unsigned char* vstage = acquire();
      // this lane's 4 tokens (k-slots 4g..4g+3) of head t, both groups, both planes
      uint32_t W[2][2];
#pragma unroll
      for (int grp = 0; grp < 2; ++grp) {
        int v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          v[j] = fix15(sc[ch * 4 + j] * (grp ? bf16hi(vsw[ch * 4 + j]) : bf16lo(vsw[ch * 4 + j])), up[grp]);
#pragma unroll
        for (int pl = 0; pl < 2; ++pl)
          W[grp][pl] = plane_byte(v[0], pl) | (plane_byte(v[1], pl) << 8) | (plane_byte(v[2], pl) << 16) |
                       (plane_byte(v[3], pl) << 24);
      }
      // B fragments: column g = (head g>>1, plane g&1); k-slots 4t.. come from lane (g'=t, t'=head),
      // k-slots 16+4t.. from lane (g'=4+t, t'=head)
      const int src_lo = t * 4 + (g >> 1), src_hi = (4 + t) * 4 + (g >> 1);
      uint32_t bfr[2][2];
#pragma unroll
      for (int grp = 0; grp < 2; ++grp) {
        const uint32_t l0 = __shfl_sync(0xffffffffu, W[grp][0], src_lo), l1 = __shfl_sync(0xffffffffu, W[grp][1], src_lo);
        const uint32_t h0 = __shfl_sync(0xffffffffu, W[grp][0], src_hi), h1 = __shfl_sync(0xffffffffu, W[grp][1], src_hi);
        bfr[grp][0] = (g & 1) ? l1 : l0;
        bfr[grp][1] = (g & 1) ? h1 : h0;
      }
      // A fragments: ldmatrix rows = tokens in k-slot order: slot s -> token (s>>2) + 8*(s&3)
      const int slot = lane & 15, half = lane >> 4;
      const int tokrow = half * 4 + (slot >> 2) + 8 * (slot & 3);  // slots 16.. -> tokens 4 + ..
      const uint32_t stv = (uint32_t)__cvta_generic_to_shared(vstage);
#pragma unroll
      for (int kb = 0; kb < G::CHUNKS; ++kb) {
        uint32_t r[4];
        ldmatrix_b8_trans_x2(r, stv + tokrow * G::ROWB + ((kb ^ swz<BITS>(tokrow)) << 4));
        const int grp = kb / (G::CHUNKS / 2);
        if constexpr (BITS == 4) {
          // byte column c holds head-dim values 32kb + 2c (low nibble) and 2c+1 (high nibble)
          mma_u8s8_ordered(accv[2 * kb], r[0] & 0x0F0F0F0Fu, r[1] & 0x0F0F0F0Fu, r[2] & 0x0F0F0F0Fu, r[3] & 0x0F0F0F0Fu,
                   bfr[grp][0], bfr[grp][1]);
          mma_u8s8_ordered(accv[2 * kb + 1], (r[0] >> 4) & 0x0F0F0F0Fu, (r[1] >> 4) & 0x0F0F0F0Fu, (r[2] >> 4) & 0x0F0F0F0Fu,
                   (r[3] >> 4) & 0x0F0F0F0Fu, bfr[grp][0], bfr[grp][1]);
        } else {
          mma_u8s8_ordered(accv[kb], r[0], r[1], r[2], r[3], bfr[grp][0], bfr[grp][1]);
        }
      }
      __syncwarp();
    }
    // ---------------- fold the block's s32 sums into the fp32 output ----------------
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int grp = i >> 2;  // tiles 0-3 cover head-dim values 0..63, tiles 4-7 cover 64..127 (both widths)
      const float f_lo = (float)(accv[i][0] * 128 + accv[i][1]), f_hi = (float)(accv[i][2] * 128 + accv[i][3]);
      O[2 * i] = fmaf(O[2 * i], alpha, f_lo * down[grp]);
      O[2 * i + 1] = fmaf(O[2 * i + 1], alpha, f_hi * down[grp]);
    }
  }
  cp_async_wait<0>();

  // ---- finish the warp: l and the bias dot are partial over the 8 lanes that share a head ----
  l_part += __shfl_xor_sync(0xffffffffu, l_part, 4);
  l_part += __shfl_xor_sync(0xffffffffu, l_part, 8);
  l_part += __shfl_xor_sync(0xffffffffu, l_part, 16);
#pragma unroll
  for (int grp = 0; grp < 2; ++grp) {
    ob[grp] += __shfl_xor_sync(0xffffffffu, ob[grp], 4);
    ob[grp] += __shfl_xor_sync(0xffffffffu, ob[grp], 8);
    ob[grp] += __shfl_xor_sync(0xffffffffu, ob[grp], 16);
  }
  __syncthreads();  // every warp is done with its ring
  // merge buffers (reuse the ring): wm[warp][head], wl[warp][head], wo[warp][head][128]
  float* wm = (float*)ring;
  float* wl = wm + kWarps * 4;
  float* wo = wl + kWarps * 4;
  if (g == 0) { wm[warp * 4 + t] = m_run; wl[warp * 4 + t] = l_part; }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int grp = i >> 2;
    int e_lo, e_hi;  // head-dim index of rows g and g+8 of tile i
    if (BITS == 4) { const int kb = i >> 1, odd = i & 1; e_lo = 32 * kb + 2 * g + odd; e_hi = e_lo + 16; }
    else { e_lo = 16 * i + g; e_hi = e_lo + 8; }
    wo[(warp * 4 + t) * kD + e_lo] = O[2 * i] + ob[grp];
    wo[(warp * 4 + t) * kD + e_hi] = O[2 * i + 1] + ob[grp];
  }
  __syncthreads();
  // this CTA's split: (M, L, O) per head, either to the workspace (a merge kernel follows) or, when the splits of
  // this (sequence, kv head) form a cluster, to shared memory, where rank 0 reads them through distributed shared memory
  float* cm = wo + kWarps * 4 * kD;   // [4] running maxima (log2 domain), [4] sums, [4][128] outputs of this CTA
  float* cl = cm + 4;
  float* co = cl + 4;
  for (int i = tid; i < p.gqa * kD; i += kWarps * 32) {
    const int h = i / kD, e = i - h * kD;
    float M = kNegBig;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, wm[w * 4 + h]);
    float L = 0.f, Ov = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float scl = ex2(wm[w * 4 + h] - M);
      L += wl[w * 4 + h] * scl;
      Ov += wo[(w * 4 + h) * kD + e] * scl;
    }
    if (p.fused) {
      co[i] = Ov;
      if (e == 0) { cm[h] = M; cl[h] = L; }
    } else {
      const int64_t pi = (b * a.Hq + hk * p.gqa + h) * p.nsplit + split;
      p.part_o[pi * kD + e] = Ov;
      if (e == 0) { p.part_m[pi] = M * 0.6931471805599453f; p.part_l[pi] = L; }  // natural-log domain for the merge
    }
  }
  if (p.fused) {
    // out = (sum_r o_r w_r) / (sum_r l_r w_r), w_r = 2^(m_r - max m)  (src/transformer.zig:5194-5203), r over the cluster
    if (p.nsplit > 1) cluster_sync_all(); else __syncthreads();
    if (split == 0) {   // the cluster spans the grid's x dimension: its rank is the split index
      const uint32_t cm_s = (uint32_t)__cvta_generic_to_shared(cm), cl_s = (uint32_t)__cvta_generic_to_shared(cl),
                     co_s = (uint32_t)__cvta_generic_to_shared(co);
      for (int i = tid; i < p.gqa * kD; i += kWarps * 32) {
        const int h = i / kD, e = i - h * kD;
        float M = kNegBig;
        for (int r = 0; r < p.nsplit; ++r) M = fmaxf(M, ld_cluster_f32(map_to_rank(cm_s + 4u * h, (uint32_t)r)));
        float L = 0.f, Ov = 0.f;
        for (int r = 0; r < p.nsplit; ++r) {
          const float wgt = ex2(ld_cluster_f32(map_to_rank(cm_s + 4u * h, (uint32_t)r)) - M);
          L += ld_cluster_f32(map_to_rank(cl_s + 4u * h, (uint32_t)r)) * wgt;
          Ov += ld_cluster_f32(map_to_rank(co_s + 4u * i, (uint32_t)r)) * wgt;
        }
        const float v = Ov * (L > 0.f ? 1.f / L : 0.f);
        const int64_t off = b * a.o_str[0] + (int64_t)(hk * p.gqa + h) * a.o_str[1] + e;
        if (a.q_dtype == QB200_FLOAT32) ((float*)a.out)[off] = v;
        else ((uint16_t*)a.out)[off] = f32_to_bf16_bits(v);
      }
    }
    if (p.nsplit > 1) cluster_sync_all();   // the other ranks' shared memory stays alive until rank 0 has read it
  }
}

}  // namespace

bool kv_fast_supported(const KvAttnArgs& a, const KvSeqTable* seqs) {
  if (a.bits != 4 && a.bits != 8) return false;
  if (a.D != kD || a.Dv != kD || a.gs != 64) return false;
  const int64_t gqa = a.Hq / a.Hkv;
  if (gqa < 1 || gqa > 4) return false;
  if (a.q_dtype != QB200_BFLOAT16 && a.q_dtype != QB200_FLOAT32) return false;
  if (a.Hkv > 65535 || a.B > 65535 || a.T < 1) return false;
  // 16-byte aligned code rows, 4-byte aligned scale/bias rows
  if (seqs) {
    if (a.B > kMaxSeqPtrs) return false;
    for (int64_t b = 0; b < a.B; ++b) {
      const KvSeq& q = seqs->s[b];
      if (q.T < 1) return false;
      if ((((uintptr_t)q.kq) & 15) || (((uintptr_t)q.vq) & 15)) return false;
      if ((((uintptr_t)q.ks) & 3) || (((uintptr_t)q.kb) & 3) || (((uintptr_t)q.vs) & 3) || (((uintptr_t)q.vb) & 3)) return false;
      for (int d = 0; d < 2; ++d) {
        if ((q.kq_str[d] * 4) % 16 != 0 || (q.vq_str[d] * 4) % 16 != 0) return false;
        if ((q.ksb_str[d] * 2) % 4 != 0 || (q.vsb_str[d] * 2) % 4 != 0) return false;
      }
    }
    return true;
  }
  if ((((uintptr_t)a.kq) & 15) || (((uintptr_t)a.vq) & 15)) return false;
  for (int d = 0; d < 3; ++d) {
    if ((a.kq_str[d] * 4) % 16 != 0 || (a.vq_str[d] * 4) % 16 != 0) return false;
    if ((a.ksb_str[d] * 2) % 4 != 0 || (a.vsb_str[d] * 2) % 4 != 0) return false;
  }
  if ((((uintptr_t)a.ks) & 3) || (((uintptr_t)a.kb) & 3) || (((uintptr_t)a.vs) & 3) || (((uintptr_t)a.vb) & 3)) return false;
  return true;
}

namespace {
template <int BITS, class TAB>
cudaError_t launch_fast_inst(const FastK& p, const TAB& tab, dim3 grid, cudaStream_t st) {
  const size_t smem = (size_t)kWarps * (Geo<BITS>::STAGES * Geo<BITS>::STAGE_BYTES + Geo<BITS>::SB_BYTES) + 4 * 32 * 8 + 64;
  static bool done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> setup_lk(setup_mutex());   // first use on a device, from any thread
    if (dev < 0 || dev >= 64 || !done[dev]) {
      const cudaError_t e = cudaFuncSetAttribute(kv_fast_kernel<BITS, TAB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  if (p.fused && p.nsplit > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)p.nsplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kv_fast_kernel<BITS, TAB>, p, tab);
  }
  return launch_kernel(kv_fast_kernel<BITS, TAB>, grid, dim3(kWarps * 32), smem, st, p, tab);
}
}  // namespace

cudaError_t launch_kv_fast(const KvAttnArgs& a, int nsplit, int64_t tps, float* pm, float* pl, float* po,
                           cudaStream_t st, const KvSeqTable* seqs, bool fused) {
  FastK p;
  p.a = a; p.nsplit = nsplit; p.tps = tps; p.gqa = (int)(a.Hq / a.Hkv);
  p.fused = fused ? 1 : 0;
  p.part_m = pm; p.part_l = pl; p.part_o = po;
  const dim3 grid((unsigned)nsplit, (unsigned)a.Hkv, (unsigned)a.B);
  if (seqs) return a.bits == 4 ? launch_fast_inst<4, KvSeqTable>(p, *seqs, grid, st) : launch_fast_inst<8, KvSeqTable>(p, *seqs, grid, st);
  return a.bits == 4 ? launch_fast_inst<4, KvNoTable>(p, KvNoTable{}, grid, st) : launch_fast_inst<8, KvNoTable>(p, KvNoTable{}, grid, st);
}

}  // namespace qb

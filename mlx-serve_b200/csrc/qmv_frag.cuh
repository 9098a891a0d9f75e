// Device helpers shared by the weight-streaming kernels: packed-code expansion
// into bf16 MMA fragments and the matching order of the activation fragments.
#pragma once
#include "common.cuh"

namespace qb {

template <int BITS> struct WReg;
template <> struct WReg<4> { using T = uint2; static constexpr int U = 4; };
template <> struct WReg<8> { using T = uint4; static constexpr int U = 2; };

template <int BITS>
__device__ __forceinline__ typename WReg<BITS>::T load_w(const uint32_t* p) {
  if constexpr (BITS == 4) return ldg_stream_u2(p);
  else return ldg_stream_u4(p);
}

// A-operand registers of MMA step i (0..3) of one 64-wide group.
// 4-bit: value lanes hold 128+q (bias folded later); 8-bit: exact q.
template <int BITS>
__device__ __forceinline__ void expand(const typename WReg<BITS>::T& v, int i, uint32_t& lo, uint32_t& hi) {
  if constexpr (BITS == 4) {
    const uint32_t word = (i >> 1) ? v.y : v.x;
    const uint32_t sh = (i & 1) * 8;
    lo = lop3_and_or(word >> sh, 0x000F000Fu, 0x43004300u);
    hi = lop3_and_or(word >> (sh + 4), 0x000F000Fu, 0x43004300u);
  } else {
    const uint32_t word = i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
    const float f0 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540)) - 8388608.f;
    const float f1 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7541)) - 8388608.f;
    const float f2 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7542)) - 8388608.f;
    const float f3 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7543)) - 8388608.f;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(f0, f1);
    __nv_bfloat162 p1 = __floats2bfloat162_rn(f2, f3);
    lo = *(uint32_t*)&p0;
    hi = *(uint32_t*)&p1;
  }
}
template <int BITS> __device__ __forceinline__ float code_base() { return BITS == 4 ? 128.f : 0.f; }

// Order in which the 16 values a lane owns (k = 16t .. 16t+15 of a group) are
// consumed by the four MMA steps; the B fragments are staged in this order.
template <int BITS>
__device__ __forceinline__ int kperm(int i, int j) {  // step i, slot j (0..3) -> offset 0..15
  if constexpr (BITS == 4) {
    const int base = 8 * (i >> 1) + 2 * (i & 1);
    return base + ((j & 1) ? 4 : 0) + (j >> 1);  // {0,4,1,5}
  } else {
    return 4 * i + j;
  }
}

// Scales (or biases) of U consecutive 64-wide groups starting at group `gidx`
// (a multiple of U) of one row; gshift = 1 when the group size is 128.
template <int U>
__device__ __forceinline__ void load_sb(const uint16_t* row, int gidx, int gshift, float (&out)[U]) {
  if constexpr (U == 4) {
    if (gshift == 0) {
      const uint2 v = __ldg((const uint2*)(row + gidx));
      out[0] = bf16lo(v.x); out[1] = bf16hi(v.x); out[2] = bf16lo(v.y); out[3] = bf16hi(v.y);
    } else {
      const uint32_t v = __ldg((const uint32_t*)(row + (gidx >> 1)));
      out[0] = out[1] = bf16lo(v); out[2] = out[3] = bf16hi(v);
    }
  } else {
    if (gshift == 0) {
      const uint32_t v = __ldg((const uint32_t*)(row + gidx));
      out[0] = bf16lo(v); out[1] = bf16hi(v);
    } else {
      out[0] = out[1] = bf16_bits_to_f32(__ldg(row + (gidx >> 1)));
    }
  }
}


}  // namespace qb

// Shared device/host helpers for libqb200 (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qb200.h"

namespace qb {

constexpr int kMaxLead = QB200_MAX_DIMS - 1;  // leading (row) dims of a tensor

// Maps a linear row index (row-major over `nd` leading dims) to an element
// offset using explicit strides.  Cache views are strided slices of capacity
// buffers (mlx-serve src/transformer.zig:3472-3495), so every kernel that
// walks rows of a caller tensor goes through one of these.
struct RowMap {
  int nd;
  int64_t shape[kMaxLead];
  int64_t stride[kMaxLead];
  int contiguous;      // rows are `row_pitch` elements apart, no gaps
  int64_t row_pitch;
  __host__ __device__ inline int64_t offset(int64_t row) const {
    if (contiguous) return row * row_pitch;
    int64_t off = 0;
    for (int d = nd - 1; d >= 0; --d) {
      const int64_t q = row / shape[d];
      off += (row - q * shape[d]) * stride[d];
      row = q;
    }
    return off;
  }
};

// Broadcast batch addressing for matmul operands: batch index -> element offset.
struct BatchMap {
  int nd;
  int64_t shape[kMaxLead];    // broadcast batch shape
  int64_t stride[kMaxLead];   // 0 where the operand is broadcast
  __host__ __device__ inline int64_t offset(int64_t bidx) const {
    int64_t off = 0;
    for (int d = nd - 1; d >= 0; --d) {
      const int64_t q = bidx / shape[d];
      off += (bidx - q * shape[d]) * stride[d];
      bidx = q;
    }
    return off;
  }
};

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) { return __uint_as_float(((uint32_t)h) << 16); }
__device__ __forceinline__ float bf16lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  return (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
}

// two fp32 -> packed bf16 (round to nearest even), `lo` in the low half: one conversion instruction
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *(const uint32_t*)&h;
}

template <typename T> struct IO;
template <> struct IO<float> {
  __device__ static __forceinline__ float load(const void* p, int64_t i) { return ((const float*)p)[i]; }
  __device__ static __forceinline__ void store(void* p, int64_t i, float v) { ((float*)p)[i] = v; }
};
template <> struct IO<__nv_bfloat16> {
  __device__ static __forceinline__ float load(const void* p, int64_t i) {
    return bf16_bits_to_f32(((const uint16_t*)p)[i]);
  }
  __device__ static __forceinline__ void store(void* p, int64_t i, float v) {
    ((uint16_t*)p)[i] = f32_to_bf16_bits(v);
  }
};
template <> struct IO<__half> {
  __device__ static __forceinline__ float load(const void* p, int64_t i) { return __half2float(((const __half*)p)[i]); }
  __device__ static __forceinline__ void store(void* p, int64_t i, float v) { ((__half*)p)[i] = __float2half_rn(v); }
};

// Streaming 64/128-bit loads of packed weights: read-only path, do not keep in L1.
__device__ __forceinline__ uint2 ldg_stream_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// (a & b) | c in one LOP3
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}

}  // namespace qb

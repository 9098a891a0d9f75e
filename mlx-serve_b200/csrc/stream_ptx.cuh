// Inline-PTX helpers shared by the weight-streaming kernels (dense, gather, single-token MoE) and the
// packed-KV attention kernel: cp.async copies into a per-warp ring, the integer MMA the packed codes
// feed, thread-block cluster addressing, and the 15-bit fixed-point staging of activations.
#pragma once
#include "common.cuh"

namespace qb {

// ---- cp.async (LDGSTS): 16-byte copies bypass L1, the small ones keep it ----
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

// ---- D(16x8,s32) += A(16x32,u8,row) * B(32x8,s8,col) ----
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The same with a zero C operand (no accumulator initialisation in registers).
__device__ __forceinline__ void mma_u8s8_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {0,0,0,0};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Kept in program order (the attention kernel interleaves it with ldmatrix reads of the same stage).
__device__ __forceinline__ void mma_u8s8_ordered(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16-byte chunk swizzle inside a 128-byte ring-stage row of the weight-streaming kernels, so that the
// fragment reads (64-bit per lane at 4 bits, 128-bit at 8 bits) are bank-conflict free.
template <int BITS> __device__ __forceinline__ int swz_w(int row) { return BITS == 4 ? 2 * (row & 3) : 4 * (row & 1); }

// A lane owns 16 consecutive K values of a group, 8 per MMA.  Offset (0..7) inside those 8 of the byte
// that sits in operand register h (0: k-slots 4t.., 1: k-slots 16+4t..), byte i.  4-bit words split into
// even and odd nibbles; 8-bit words are in order.
template <int BITS> __device__ __forceinline__ int kslot8(int h, int i) { return BITS == 4 ? 2 * i + h : 4 * h + i; }

// ---- thread-block clusters (distributed shared memory) ----
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
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
// All threads of all CTAs of the cluster (a hardware barrier: no spinning in software).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- 15-bit block fixed point ----
// A group of 64 activations shares one power-of-two scale: v = rn(x * 2^(14-e)) with |x| < 2^e, so
// |v| <= 2^14 and v = 128 * p0 + p1 splits into a signed high plane and a 7-bit low plane, both s8.
// The group's largest |x| is taken with a NaN-propagating maximum, so an Inf or a NaN anywhere in the
// group shows in the exponent field of the maximum; the group's fp32 scale is then replaced by NaN and
// every output that depends on the group becomes NaN instead of a finite number.
__device__ __forceinline__ float fmax_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ bool nonfinite(float mx) { return ((__float_as_uint(mx) >> 23) & 0xFF) == 0xFF; }
__device__ __forceinline__ float poison_if(bool bad, float v) { return bad ? __uint_as_float(0x7FC00000u) : v; }

}  // namespace qb

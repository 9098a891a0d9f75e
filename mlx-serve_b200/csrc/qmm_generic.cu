// Shape-agnostic quantized matmul / gather on CUDA cores.
//
// This is the safety net behind the tuned kernels: any (bits in {2,4,8},
// group size, M, N, K, dtype, batch broadcast) the C ABI accepts but the
// streaming tensor-core kernels decline is served here, so a request is never
// mis-computed or silently dropped.  It also carries transpose_w=false, the
// form quantAttention uses for attn @ V (mlx-serve src/kv_quant.zig:657-674).
// fp32 accumulate, weight term q*s+b kept in fp32.
#include "kernels.h"

namespace qb {
namespace {

// transpose=true: one warp per output element (m, n); lanes stride over the
// packed words of row n.
template <int BITS, typename XT, typename ST>
__global__ void __launch_bounds__(256) qmm_t_generic(QmmArgs a) {
  constexpr int VPW = 32 / BITS;
  const int lane = threadIdx.x & 31;
  const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t m = blockIdx.y;
  const int64_t bz = blockIdx.z;
  if (n >= a.N) return;
  const char* xb = (const char*)a.x + a.xb.offset(bz) * sizeof(XT);
  const uint32_t* w = a.w + a.wb.offset(bz) + n * a.ldw;
  const int64_t sboff = a.sb.offset(bz) + n * a.lds;
  const int64_t words = a.K / VPW;
  float acc = 0.f;
  for (int64_t wi = lane; wi < words; wi += 32) {
    const uint32_t word = w[wi];
    const int64_t k0 = wi * VPW;
    const float sc = IO<ST>::load(a.s, sboff + k0 / a.gs);
    const float bi = IO<ST>::load(a.b, sboff + k0 / a.gs);
#pragma unroll
    for (int k = 0; k < VPW; ++k) {
      const float q = (float)((word >> (k * BITS)) & ((1u << BITS) - 1u));
      const float wv = __fadd_rn(__fmul_rn(q, sc), bi);
      acc = fmaf(IO<XT>::load(xb, m * a.ldx + k0 + k), wv, acc);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) IO<XT>::store((char*)a.y + a.yb.offset(bz) * sizeof(XT), m * a.ldy + n, acc);
}

// transpose=false: one thread per (m, packed output word); walks the K rows.
template <int BITS, typename XT, typename ST>
__global__ void __launch_bounds__(256) qmm_n_generic(QmmArgs a) {
  constexpr int VPW = 32 / BITS;
  const int64_t words = a.N / VPW;
  const int64_t wi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t m = blockIdx.y;
  const int64_t bz = blockIdx.z;
  if (wi >= words) return;
  const char* xb = (const char*)a.x + a.xb.offset(bz) * sizeof(XT);
  const uint32_t* w = a.w + a.wb.offset(bz);
  const int64_t sbase = a.sb.offset(bz);
  const int64_t g = (wi * VPW) / a.gs;
  float acc[VPW];
#pragma unroll
  for (int k = 0; k < VPW; ++k) acc[k] = 0.f;
  for (int64_t kk = 0; kk < a.K; ++kk) {
    const uint32_t word = w[kk * a.ldw + wi];
    const float sc = IO<ST>::load(a.s, sbase + kk * a.lds + g);
    const float bi = IO<ST>::load(a.b, sbase + kk * a.lds + g);
    const float xv = IO<XT>::load(xb, m * a.ldx + kk);
#pragma unroll
    for (int k = 0; k < VPW; ++k) {
      const float q = (float)((word >> (k * BITS)) & ((1u << BITS) - 1u));
      acc[k] = fmaf(xv, __fadd_rn(__fmul_rn(q, sc), bi), acc[k]);
    }
  }
  char* yb = (char*)a.y + a.yb.offset(bz) * sizeof(XT);
#pragma unroll
  for (int k = 0; k < VPW; ++k) IO<XT>::store(yb, m * a.ldy + wi * VPW + k, acc[k]);
}

template <int BITS, typename XT>
cudaError_t launch_bits_x(const QmmArgs& a, cudaStream_t st) {
  if (a.M == 0 || a.N == 0 || a.nbatch == 0) return cudaSuccess;
  if (a.M > 65535 || a.nbatch > 65535) return cudaErrorInvalidValue;
  if (a.transpose) {
    dim3 grid((unsigned)((a.N + 7) / 8), (unsigned)a.M, (unsigned)a.nbatch);
    qmm_t_generic<BITS, XT, __nv_bfloat16><<<grid, 256, 0, st>>>(a);
  } else {
    const int64_t words = a.N * BITS / 32;
    dim3 grid((unsigned)((words + 127) / 128), (unsigned)a.M, (unsigned)a.nbatch);
    qmm_n_generic<BITS, XT, __nv_bfloat16><<<grid, 128, 0, st>>>(a);
  }
  return cudaGetLastError();
}

template <int BITS>
cudaError_t launch_bits(const QmmArgs& a, cudaStream_t st) {
  switch (a.x_dtype) {
    case QB200_BFLOAT16: return launch_bits_x<BITS, __nv_bfloat16>(a, st);
    case QB200_FLOAT32: return launch_bits_x<BITS, float>(a, st);
    case QB200_FLOAT16: return launch_bits_x<BITS, __half>(a, st);
    default: return cudaErrorInvalidValue;
  }
}

// gather: one warp per (output batch element i, row m, output n).
template <int BITS, typename XT, typename IT>
__global__ void __launch_bounds__(256) gather_t_generic(GatherArgs a) {
  constexpr int VPW = 32 / BITS;
  const int lane = threadIdx.x & 31;
  const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t i = blockIdx.y;
  if (n >= a.N) return;
  int64_t e = (int64_t)((const IT*)a.rhs)[i];
  if (e < 0 || e >= a.E) return;  // out-of-range expert: leave the row untouched
  int64_t xi;
  if (a.lhs) {
    if (a.lhs_dtype == QB200_INT64) xi = ((const int64_t*)a.lhs)[i];
    else xi = (int64_t)((const uint32_t*)a.lhs)[i];
  } else {
    xi = a.xbcast.offset(i);
  }
  if (xi < 0 || xi >= a.XB) return;
  const uint32_t* w = a.w + e * a.w_expert_stride + n * (a.K / VPW);
  const int64_t sboff = e * a.s_expert_stride + n * (a.K / a.gs);
  const int64_t words = a.K / VPW;
  for (int64_t m = 0; m < a.M; ++m) {
    const int64_t xoff = xi * a.x_batch_stride + m * a.K;
    float acc = 0.f;
    for (int64_t wi = lane; wi < words; wi += 32) {
      const uint32_t word = w[wi];
      const int64_t k0 = wi * VPW;
      const float sc = IO<__nv_bfloat16>::load(a.s, sboff + k0 / a.gs);
      const float bi = IO<__nv_bfloat16>::load(a.b, sboff + k0 / a.gs);
#pragma unroll
      for (int k = 0; k < VPW; ++k) {
        const float q = (float)((word >> (k * BITS)) & ((1u << BITS) - 1u));
        acc = fmaf(IO<XT>::load(a.x, xoff + k0 + k), __fadd_rn(__fmul_rn(q, sc), bi), acc);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) IO<XT>::store(a.y, (i * a.M + m) * a.N + n, acc);
  }
}

template <int BITS, typename XT>
cudaError_t gather_bits_x(const GatherArgs& a, cudaStream_t st) {
  if (a.I == 0 || a.N == 0 || a.M == 0) return cudaSuccess;
  if (a.I > 65535 * 1024LL) return cudaErrorInvalidValue;
  // grid.y is limited to 65535: fold long index lists over several launches
  for (int64_t i0 = 0; i0 < a.I; i0 += 65535) {
    GatherArgs b = a;
    const int64_t cnt = (a.I - i0 < 65535) ? (a.I - i0) : 65535;
    const int isz = (a.rhs_dtype == QB200_INT64) ? 8 : 4;
    b.rhs = (const char*)a.rhs + i0 * isz;
    if (a.lhs) b.lhs = (const char*)a.lhs + i0 * ((a.lhs_dtype == QB200_INT64) ? 8 : 4);
    b.y = (char*)a.y + i0 * a.M * a.N * sizeof(XT);
    if (!a.lhs && i0 != 0) return cudaErrorInvalidValue;  // broadcast form is always short
    b.I = cnt;
    dim3 grid((unsigned)((a.N + 7) / 8), (unsigned)cnt, 1);
    if (a.rhs_dtype == QB200_INT64) gather_t_generic<BITS, XT, int64_t><<<grid, 256, 0, st>>>(b);
    else gather_t_generic<BITS, XT, uint32_t><<<grid, 256, 0, st>>>(b);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

template <int BITS>
cudaError_t gather_bits(const GatherArgs& a, cudaStream_t st) {
  switch (a.x_dtype) {
    case QB200_BFLOAT16: return gather_bits_x<BITS, __nv_bfloat16>(a, st);
    case QB200_FLOAT32: return gather_bits_x<BITS, float>(a, st);
    case QB200_FLOAT16: return gather_bits_x<BITS, __half>(a, st);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launch_qmm_generic(const QmmArgs& a, cudaStream_t st) {
  switch (a.bits) {
    case 2: return launch_bits<2>(a, st);
    case 4: return launch_bits<4>(a, st);
    case 8: return launch_bits<8>(a, st);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_gather_generic(const GatherArgs& a, cudaStream_t st) {
  switch (a.bits) {
    case 2: return gather_bits<2>(a, st);
    case 4: return gather_bits<4>(a, st);
    case 8: return gather_bits<8>(a, st);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace qb

// Sort of the routed-expert block's flattened index list by expert: the step moeMLP2 builds from
// argsort(flat_inds), argsort(order), take(flat_inds, order) and order // k
// (mlx-serve src/transformer.zig:14961-15006), as one stable counting sort in one launch.
//
// One CTA of 32 warps.  Warp w owns the contiguous slice [w * per, (w + 1) * per) of the list and walks
// it in order, 32 entries at a time, twice: once to count its entries per expert into its own row of a
// [32][E + 1] table in shared memory, once -- after a scan has turned the table into the first output
// position of every (warp, expert) pair -- to place them.  Inside a 32-entry step the lanes that hold the
// same expert find each other with match.any and take consecutive positions in lane order, so equal
// experts keep their original order (a stable sort, the order numpy's argsort(kind="stable") gives).
// Index values outside [0, E) go to an extra bin behind every expert.
#include "kernels.h"

namespace qb {
namespace {

constexpr int kSortWarps = 32;

__device__ __forceinline__ int load_key(const void* p, int is64, int64_t i, int E) {
  const long long v = is64 ? ((const long long*)p)[i] : (long long)((const int*)p)[i];
  return (v < 0 || v >= E) ? E : (int)v;
}

__global__ void __launch_bounds__(kSortWarps * 32) moe_sort_kernel(MoeSortArgs a) {
  extern __shared__ int cnt[];   // [kSortWarps][E + 1]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bins = a.E + 1;
  for (int i = tid; i < kSortWarps * bins; i += kSortWarps * 32) cnt[i] = 0;
  __syncthreads();
  const int64_t per = ((a.n + kSortWarps - 1) / kSortWarps + 31) / 32 * 32;   // slice length, whole 32-entry steps
  const int64_t lo = (int64_t)warp * per, hi = lo + per < a.n ? lo + per : a.n;
  int* mine = cnt + warp * bins;
  // (eight 32-entry steps of keys are loaded before any is used: the loop is bound by load latency otherwise)
  constexpr int kAhead = 8;
  for (int64_t c0 = lo; c0 < hi; c0 += 32 * kAhead) {
    int keys[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int64_t i = c0 + 32 * u + lane;
      keys[u] = i < hi ? load_key(a.inds, a.inds_i64, i, a.E) : -1 - lane;   // dead lanes match nobody
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (c0 + 32 * u >= hi) break;
      const int key = keys[u];
      const unsigned same = __match_any_sync(0xffffffffu, key);
      if (key >= 0 && (same & ((1u << lane) - 1u)) == 0) mine[key] += __popc(same);   // the group's first lane
      __syncwarp();
    }
  }
  __syncthreads();
  // first position of every (warp, expert): experts in ascending order, inside an expert the warps in order
  // (one thread per expert sums its column; then a scan over the experts)
  __shared__ int total[1024 + 1 + 1];
  for (int e = tid; e < bins; e += kSortWarps * 32) {
    int s = 0;
    for (int w = 0; w < kSortWarps; ++w) { const int c = cnt[w * bins + e]; cnt[w * bins + e] = s; s += c; }
    total[e] = s;
  }
  __syncthreads();
  if (warp == 0) {   // exclusive scan of total[0 .. bins) by one warp, 32 at a time
    int carry = 0;
    for (int e0 = 0; e0 < bins; e0 += 32) {
      const int e = e0 + lane;
      const int v = e < bins ? total[e] : 0;
      int inc = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
      }
      if (e < bins) total[e] = carry + inc - v;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) total[bins] = carry;
  }
  __syncthreads();
  if (a.offsets)
    for (int e = tid; e <= a.E; e += kSortWarps * 32) a.offsets[e] = total[e];   // rows of expert e: [offsets[e], offsets[e+1])
  for (int e = tid; e < bins; e += kSortWarps * 32) {
    const int base = total[e];
    for (int w = 0; w < kSortWarps; ++w) cnt[w * bins + e] += base;
  }
  __syncthreads();
  for (int64_t c0 = lo; c0 < hi; c0 += 32 * kAhead) {
    int keys[kAhead], raw[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int64_t i = c0 + 32 * u + lane;
      raw[u] = 0;
      keys[u] = -1 - lane;
      if (i < hi) {
        raw[u] = a.inds_i64 ? (int)((const long long*)a.inds)[i] : ((const int*)a.inds)[i];
        keys[u] = load_key(a.inds, a.inds_i64, i, a.E);
      }
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (c0 + 32 * u >= hi) break;
      const int64_t i = c0 + 32 * u + lane;
      const bool live = i < hi;
      const int key = keys[u];
      const unsigned same = __match_any_sync(0xffffffffu, key);
      const int rank = __popc(same & ((1u << lane) - 1u));
      int pos = 0;
      if (live) pos = mine[key] + rank;
      __syncwarp();
      if (live && rank == 0) mine[key] += __popc(same);
      __syncwarp();
      if (live) {
        if (a.order) a.order[pos] = (int)i;
        if (a.inv_order) a.inv_order[i] = pos;
        if (a.sorted_inds) a.sorted_inds[pos] = raw[u];
        if (a.token_rows) a.token_rows[pos] = (int)(i / a.topk);
      }
    }
  }
}

}  // namespace

cudaError_t launch_moe_sort(const MoeSortArgs& a, cudaStream_t st) {
  if (a.n <= 0) {
    if (a.offsets) return cudaMemsetAsync(a.offsets, 0, (size_t)(a.E + 1) * sizeof(int), st);
    return cudaSuccess;
  }
  const size_t smem = (size_t)kSortWarps * (a.E + 1) * sizeof(int);
  if (smem > 48 * 1024) {
    std::lock_guard<std::mutex> lk(setup_mutex());
    static bool done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !done[dev]) {
      cudaError_t e = cudaFuncSetAttribute(moe_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  moe_sort_kernel<<<1, kSortWarps * 32, smem, st>>>(a);
  return cudaGetLastError();
}

}  // namespace qb

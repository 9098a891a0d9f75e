// Sort of the routed-expert block's flattened index list by expert: the step moeMLP2 builds from
// argsort(flat_inds), argsort(order), take(flat_inds, order) and order // k
// (mlx-serve src/transformer.zig:14961-15006), as one stable counting sort: one launch up to 2048 entries (the
// decode widths), two launches (count per slice, then place) for the prefill widths.
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
constexpr int kMaxSortCtas = 64;
constexpr int kMaxSortExperts = 1024;
// per-CTA expert counts of the two-launch form: [kMaxSortCtas][kMaxSortExperts + 1]
static __device__ int g_sort_counts[kMaxSortCtas * (kMaxSortExperts + 1)];

__device__ __forceinline__ int load_key(const void* p, int is64, int64_t i, int E) {
  const long long v = is64 ? ((const long long*)p)[i] : (long long)((const int*)p)[i];
  return (v < 0 || v >= E) ? E : (int)v;
}

// PHASE 0: the whole sort in one CTA.  PHASE 1 / 2: the list is cut into one contiguous slice per CTA; phase 1
// writes each CTA's per-expert counts to `counts`, phase 2 (a second launch) recounts its slice, turns the table of
// all CTAs' counts into the first output position of its own (warp, expert) pairs and places its entries.
template <int PHASE>
__global__ void __launch_bounds__(kSortWarps * 32) moe_sort_kernel(MoeSortArgs a, int* counts) {
  extern __shared__ int cnt[];   // [kSortWarps][E + 1]
  __shared__ int total[kMaxSortExperts + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bins = a.E + 1, nct = (int)gridDim.x, cta = (int)blockIdx.x;
  for (int i = tid; i < kSortWarps * bins; i += kSortWarps * 32) cnt[i] = 0;
  __syncthreads();
  // this CTA's slice, then this warp's slice of it: whole 32-entry steps, in list order
  const int64_t per_cta = ((a.n + nct - 1) / nct + 31) / 32 * 32;
  const int64_t c_lo = (int64_t)cta * per_cta, c_hi = c_lo + per_cta < a.n ? c_lo + per_cta : a.n;
  const int64_t span = c_hi > c_lo ? c_hi - c_lo : 0;
  const int64_t per = ((span + kSortWarps - 1) / kSortWarps + 31) / 32 * 32;
  const int64_t lo = c_lo + (int64_t)warp * per, hi = lo + per < c_hi ? lo + per : c_hi;
  int* mine = cnt + warp * bins;
  for (int64_t i0 = lo; i0 < hi; i0 += 32) {
    const int64_t i = i0 + lane;
    const int key = i < hi ? load_key(a.inds, a.inds_i64, i, a.E) : -1 - lane;   // dead lanes match nobody
    const unsigned same = __match_any_sync(0xffffffffu, key);
    if (key >= 0 && (same & ((1u << lane) - 1u)) == 0) mine[key] += __popc(same);   // the group's first lane
    __syncwarp();
  }
  __syncthreads();
  // first position of every (warp, expert) inside the CTA: the warps in order (one thread per expert sums its column)
  for (int e = tid; e < bins; e += kSortWarps * 32) {
    int s = 0;
    for (int w = 0; w < kSortWarps; ++w) { const int c = cnt[w * bins + e]; cnt[w * bins + e] = s; s += c; }
    total[e] = s;
    if (PHASE == 1) counts[cta * (kMaxSortExperts + 1) + e] = s;
  }
  if (PHASE == 1) return;
  __syncthreads();
  if (PHASE == 2) {   // experts in ascending order, inside an expert the CTAs in order, inside a CTA the warps
    for (int e = tid; e < bins; e += kSortWarps * 32) {
      int before = 0, all = 0;
      for (int c = 0; c < nct; ++c) {
        const int v = counts[c * (kMaxSortExperts + 1) + e];
        if (c < cta) before += v;
        all += v;
      }
      total[e] = all;
      for (int w = 0; w < kSortWarps; ++w) cnt[w * bins + e] += before;
    }
    __syncthreads();
  }
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
  if (a.offsets && cta == 0)
    for (int e = tid; e <= a.E; e += kSortWarps * 32) a.offsets[e] = total[e];   // rows of expert e: [offsets[e], offsets[e+1])
  for (int e = tid; e < bins; e += kSortWarps * 32) {
    const int base = total[e];
    for (int w = 0; w < kSortWarps; ++w) cnt[w * bins + e] += base;
  }
  __syncthreads();
  for (int64_t i0 = lo; i0 < hi; i0 += 32) {
    const int64_t i = i0 + lane;
    const bool live = i < hi;
    int raw = 0, key = -1 - lane;
    if (live) {
      raw = a.inds_i64 ? (int)((const long long*)a.inds)[i] : ((const int*)a.inds)[i];
      key = load_key(a.inds, a.inds_i64, i, a.E);
    }
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
      if (a.sorted_inds) a.sorted_inds[pos] = raw;
      if (a.token_rows) a.token_rows[pos] = (int)(i / a.topk);
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
  int* counts = nullptr;
  {
    std::lock_guard<std::mutex> lk(setup_mutex());
    static bool done[64] = {};
    static int* addr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!done[dev]) {
      cudaError_t e = cudaFuncSetAttribute(moe_sort_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(moe_sort_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(moe_sort_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      void* p = nullptr;
      if (e == cudaSuccess) e = cudaGetSymbolAddress(&p, g_sort_counts);
      if (e != cudaSuccess) return e;
      addr[dev] = (int*)p;
      done[dev] = true;
    }
    counts = addr[dev];
  }
  // up to 2048 entries (the decode widths): one CTA, one launch.  Longer lists: a slice of ~1024 entries per CTA
  // (one match per warp and pass) and a second launch that places them.
  if (a.n <= 2048) {
    moe_sort_kernel<0><<<1, kSortWarps * 32, smem, st>>>(a, counts);
    return cudaGetLastError();
  }
  int ctas = (int)((a.n + 1023) / 1024);
  ctas = ctas > kMaxSortCtas ? kMaxSortCtas : ctas;
  moe_sort_kernel<1><<<ctas, kSortWarps * 32, smem, st>>>(a, counts);
  moe_sort_kernel<2><<<ctas, kSortWarps * 32, smem, st>>>(a, counts);
  return cudaGetLastError();
}

}  // namespace qb

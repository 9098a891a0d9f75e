// Expert-parallel routed-expert block: the exchange around the library's own MoE entries.
// See include/qb200_ep.h for the contract.  The block's arithmetic is the single-device one (moeMLP2,
// mlx-serve src/transformer.zig:14945-15140); only where a row is computed changes.
//
// Layout of the exchange buffers: [world][capacity] rows.  Slot j of peer r holds this rank's j-th row routed to
// an expert of rank r, in the order of the sort by expert (so a rank's rows for one peer are one contiguous run
// of the sorted list); slots past the run carry the expert id E/world, which the gather kernels treat as out of
// range: such rows are neither read nor written.
#include <nccl.h>

#include <cstdio>
#include <cstring>

#include "../../include/qb200_ep.h"
#include "common.cuh"

namespace {

int ep_fail(int status, const char* what) {
  fprintf(stderr, "qb200_ep: %s\n", what);
  return status;
}

struct PackArgs {
  const uint16_t* x;        // [T, H]
  const int* rows;          // [n]: token of sorted position p
  const int* sinds;         // [n]: expert of sorted position p
  const int* inv;           // [n]: sorted position of index entry i
  const int* offsets;       // [E + 1]
  uint16_t* send_x;         // [world][C][H]
  int* send_e;              // [world][C]
  int* back_row;            // [n]: row of the returned buffer that holds entry i, or -1
  int* overflow;            // may be null
  int n, E, El, world, C, H;
};

// One warp per send slot (copy of a row of x), then the same threads map the n index entries to their slot.
__global__ void __launch_bounds__(256) ep_pack_kernel(PackArgs a) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nslots = a.world * a.C;
  if (warp < nslots) {
    const int r = warp / a.C, slot = warp - r * a.C;
    const int p0 = a.offsets[r * a.El], p1 = a.offsets[(r + 1) * a.El];
    const int p = p0 + slot;
    if (p < p1) {
      const uint4* src = (const uint4*)(a.x + (int64_t)a.rows[p] * a.H);
      uint4* dst = (uint4*)(a.send_x + (int64_t)warp * a.H);
      for (int i = lane; i < a.H / 8; i += 32) dst[i] = src[i];
      if (lane == 0) a.send_e[warp] = a.sinds[p] - r * a.El;
    } else if (lane == 0) {
      a.send_e[warp] = a.El;   // padding: out of range for the local bank
    }
    if (slot == 0 && lane == 0 && p1 - p0 > a.C && a.overflow) atomicAdd(a.overflow, p1 - p0 - a.C);
  }
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < a.n) {
    const int p = a.inv[i], e = a.sinds[p];
    int row = -1;
    if (e >= 0 && e < a.E) {
      const int r = e / a.El, slot = p - a.offsets[r * a.El];
      if (slot < a.C) row = r * a.C + slot;
    }
    a.back_row[i] = row;
  }
}

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct Layout {
  size_t order, inv, sinds, rows, offsets, back_row, send_x, send_e, recv_x, recv_e, act, yd, back, total;
};
Layout layout(int64_t T, int topk, int64_t H, int64_t I, int E, int world, int64_t C) {
  Layout l;
  const size_t n = (size_t)T * topk, slots = (size_t)world * C;
  size_t o = 0;
  l.order = o; o += align256(n * 4);
  l.inv = o; o += align256(n * 4);
  l.sinds = o; o += align256(n * 4);
  l.rows = o; o += align256(n * 4);
  l.offsets = o; o += align256((size_t)(E + 1) * 4);
  l.back_row = o; o += align256(n * 4);
  l.send_x = o; o += align256(slots * H * 2);
  l.send_e = o; o += align256(slots * 4);
  l.recv_x = o; o += align256(slots * H * 2);
  l.recv_e = o; o += align256(slots * 4);
  l.act = o; o += align256(slots * I * 2);
  l.yd = o; o += align256(slots * H * 2);
  l.back = o; o += align256(slots * H * 2);
  l.total = o;
  return l;
}

qb200_tensor tensor(void* data, int dtype, int ndim, const int64_t* shape) {
  qb200_tensor t;
  std::memset(&t, 0, sizeof(t));
  t.data = data; t.dtype = dtype; t.ndim = ndim;
  int64_t st = 1;
  for (int d = ndim - 1; d >= 0; --d) { t.shape[d] = shape[d]; t.stride[d] = st; st *= shape[d]; }
  return t;
}

}  // namespace

extern "C" {

QB200_API int qb200_ep_unique_id(void* id_out) {
  static_assert(sizeof(ncclUniqueId) == QB200_EP_UNIQUE_ID_BYTES, "unique id size");
  if (!id_out) return QB200_ERR_BAD_ARG;
  return ncclGetUniqueId((ncclUniqueId*)id_out) == ncclSuccess ? QB200_OK : ep_fail(QB200_ERR_CUDA, "ncclGetUniqueId failed");
}

QB200_API int qb200_ep_comm_create(void** comm_out, int world, int rank, const void* id) {
  if (!comm_out || !id || world < 1 || rank < 0 || rank >= world) return QB200_ERR_BAD_ARG;
  ncclUniqueId uid;
  std::memcpy(&uid, id, sizeof(uid));
  ncclComm_t c = nullptr;
  if (ncclCommInitRank(&c, world, uid, rank) != ncclSuccess) return ep_fail(QB200_ERR_CUDA, "ncclCommInitRank failed");
  *comm_out = (void*)c;
  return QB200_OK;
}

QB200_API int qb200_ep_comm_destroy(void* comm) {
  if (!comm) return QB200_OK;
  return ncclCommDestroy((ncclComm_t)comm) == ncclSuccess ? QB200_OK : QB200_ERR_CUDA;
}

QB200_API int64_t qb200_moe_block_ep_capacity(int64_t T, int topk, int world) {
  if (T <= 0 || topk <= 0 || world <= 0) return 0;
  const int64_t cap = 2048 / world, all = T * topk;
  return all < cap ? all : cap;
}

QB200_API size_t qb200_moe_block_ep_workspace_size(int64_t T, int topk, int64_t H, int64_t I, int num_experts, int world,
                                                   int64_t capacity) {
  if (T <= 0 || topk <= 0 || H <= 0 || I <= 0 || num_experts <= 0 || world <= 0 || capacity <= 0) return 0;
  return layout(T, topk, H, I, num_experts, world, capacity).total;
}

QB200_API int qb200_moe_block_ep(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* inds,
                                 const qb200_tensor* scores, const qb200_tensor* w_gate, const qb200_tensor* s_gate,
                                 const qb200_tensor* b_gate, const qb200_tensor* w_up, const qb200_tensor* s_up,
                                 const qb200_tensor* b_up, const qb200_tensor* w_down, const qb200_tensor* s_down,
                                 const qb200_tensor* b_down, int num_experts, int world, int rank, void* comm,
                                 int64_t capacity, int group_size, int bits, int* overflow, void* workspace,
                                 size_t workspace_bytes, qb200_stream s) {
  if (!res || !x || !inds || !scores || !w_gate || !w_up || !w_down || !comm || !workspace)
    return ep_fail(QB200_ERR_BAD_ARG, "moe_block_ep: null argument");
  if (x->ndim != 2 || res->ndim != 2 || inds->ndim != 2 || scores->ndim != 2)
    return ep_fail(QB200_ERR_BAD_SHAPE, "moe_block_ep: x, res [T, H]; inds, scores [T, k]");
  if (x->dtype != QB200_BFLOAT16 || res->dtype != QB200_BFLOAT16 || scores->dtype != QB200_BFLOAT16 || inds->dtype != QB200_INT32)
    return ep_fail(QB200_ERR_BAD_DTYPE, "moe_block_ep: bf16 activations and scores, int32 indices");
  const int64_t T = x->shape[0], H = x->shape[1], topk = inds->shape[1];
  if (world < 1 || rank < 0 || rank >= world || num_experts % world != 0 || num_experts > 1024)
    return ep_fail(QB200_ERR_BAD_ARG, "moe_block_ep: the experts must divide evenly over the ranks (at most 1024)");
  const int El = num_experts / world;
  if (w_gate->ndim != 3 || w_down->ndim != 3 || w_gate->shape[0] != El || w_up->shape[0] != El || w_down->shape[0] != El)
    return ep_fail(QB200_ERR_BAD_SHAPE, "moe_block_ep: the banks must hold this rank's E/world experts");
  const int64_t I = w_gate->shape[1];
  if (inds->shape[0] != T || scores->shape[0] != T || scores->shape[1] != topk || res->shape[0] != T || res->shape[1] != H ||
      w_down->shape[1] != H || H % 8 != 0 || T <= 0 || topk <= 0)
    return ep_fail(QB200_ERR_BAD_SHAPE, "moe_block_ep: shapes disagree");
  if (x->stride[1] != 1 || x->stride[0] != H || res->stride[0] != H || inds->stride[0] != topk || scores->stride[0] != topk)
    return ep_fail(QB200_ERR_BAD_STRIDE, "moe_block_ep: x, res, inds and scores must be contiguous");
  if (capacity < 1 || (int64_t)world * capacity > 2048)
    return ep_fail(QB200_ERR_UNSUPPORTED, "moe_block_ep: world * capacity must be within 1..2048 rows");
  const Layout l = layout(T, (int)topk, H, I, num_experts, world, capacity);
  if (workspace_bytes < l.total) return ep_fail(QB200_ERR_WORKSPACE, "moe_block_ep: workspace too small");
  cudaStream_t st = (cudaStream_t)s;
  char* ws = (char*)workspace;
  const int64_t n = T * topk, slots = (int64_t)world * capacity;
  int rc;

  // 1. sort the index entries by expert
  const int64_t sh_n[1] = {n}, sh_off[1] = {num_experts + 1};
  qb200_tensor t_order = tensor(ws + l.order, QB200_INT32, 1, sh_n), t_inv = tensor(ws + l.inv, QB200_INT32, 1, sh_n);
  qb200_tensor t_sinds = tensor(ws + l.sinds, QB200_INT32, 1, sh_n), t_rows = tensor(ws + l.rows, QB200_INT32, 1, sh_n);
  qb200_tensor t_off = tensor(ws + l.offsets, QB200_INT32, 1, sh_off);
  if ((rc = qb200_moe_sort_by_expert(&t_order, &t_inv, &t_sinds, &t_rows, &t_off, inds, num_experts, s))) return rc;

  // 2. pack rows and local expert ids per destination rank
  if (overflow) cudaMemsetAsync(overflow, 0, sizeof(int), st);
  PackArgs pa;
  pa.x = (const uint16_t*)x->data; pa.rows = (const int*)(ws + l.rows); pa.sinds = (const int*)(ws + l.sinds);
  pa.inv = (const int*)(ws + l.inv); pa.offsets = (const int*)(ws + l.offsets);
  pa.send_x = (uint16_t*)(ws + l.send_x); pa.send_e = (int*)(ws + l.send_e); pa.back_row = (int*)(ws + l.back_row);
  pa.overflow = overflow;
  pa.n = (int)n; pa.E = num_experts; pa.El = El; pa.world = world; pa.C = (int)capacity; pa.H = (int)H;
  {
    const int64_t threads = slots * 32 > n ? slots * 32 : n;
    ep_pack_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(pa);
    if (cudaGetLastError() != cudaSuccess) return ep_fail(QB200_ERR_CUDA, "moe_block_ep: pack launch failed");
  }

  // 3. dispatch: rows and expert ids to their owners
  ncclComm_t nc = (ncclComm_t)comm;
  const size_t row_bytes = (size_t)capacity * H * 2, id_bytes = (size_t)capacity * 4;
  ncclGroupStart();
  for (int r = 0; r < world; ++r) {
    ncclSend(ws + l.send_x + r * row_bytes, row_bytes, ncclUint8, r, nc, st);
    ncclRecv(ws + l.recv_x + r * row_bytes, row_bytes, ncclUint8, r, nc, st);
    ncclSend(ws + l.send_e + r * id_bytes, id_bytes, ncclUint8, r, nc, st);
    ncclRecv(ws + l.recv_e + r * id_bytes, id_bytes, ncclUint8, r, nc, st);
  }
  if (ncclGroupEnd() != ncclSuccess) return ep_fail(QB200_ERR_CUDA, "moe_block_ep: dispatch exchange failed");

  // 4. the received rows through this rank's experts (rows of padding carry the id El: skipped)
  const int64_t sh_x[3] = {slots, 1, H}, sh_a[3] = {slots, 1, I}, sh_e[1] = {slots};
  qb200_tensor t_rx = tensor(ws + l.recv_x, QB200_BFLOAT16, 3, sh_x), t_act = tensor(ws + l.act, QB200_BFLOAT16, 3, sh_a);
  qb200_tensor t_yd = tensor(ws + l.yd, QB200_BFLOAT16, 3, sh_x), t_re = tensor(ws + l.recv_e, QB200_INT32, 1, sh_e);
  qb200_tensor none;
  std::memset(&none, 0, sizeof(none));
  const qb200_optional_int og = {group_size, true}, ob = {bits, true};
  if ((rc = qb200_gather_qmm_swiglu(&t_act, &t_rx, w_gate, s_gate, b_gate, w_up, s_up, b_up, &none, &t_re, og, ob, "affine", false, s)))
    return rc;
  if ((rc = qb200_gather_qmm(&t_yd, &t_act, w_down, s_down, b_down, &none, &t_re, true, og, ob, "affine", false, s))) return rc;

  // 5. combine: every row back to the rank that routed it
  ncclGroupStart();
  for (int r = 0; r < world; ++r) {
    ncclSend(ws + l.yd + r * row_bytes, row_bytes, ncclUint8, r, nc, st);
    ncclRecv(ws + l.back + r * row_bytes, row_bytes, ncclUint8, r, nc, st);
  }
  if (ncclGroupEnd() != ncclSuccess) return ep_fail(QB200_ERR_CUDA, "moe_block_ep: combine exchange failed");

  // 6. x scores, sum over top-k in token order
  const int64_t sh_back[2] = {slots, H};
  qb200_tensor t_back = tensor(ws + l.back, QB200_BFLOAT16, 2, sh_back), t_br = tensor(ws + l.back_row, QB200_INT32, 1, sh_n);
  return qb200_moe_weighted_sum(res, &t_back, scores, &t_br, s);
}

}  // extern "C"

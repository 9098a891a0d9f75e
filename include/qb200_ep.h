/*
 * qb200_ep.h -- expert-parallel form of the routed-expert block, for one process per GPU on one NVLink box.
 * Built as libqb200_ep.so, which links libqb200.so and NCCL (the core library stays free of dependencies).
 *
 * The reference runs the routed-expert block on one device (moeMLP2, src/transformer.zig:14945-15140).  Here the
 * experts are split over `world` ranks -- rank r owns experts [r*E/world, (r+1)*E/world) and holds only their
 * banks -- while the tokens stay data-parallel: every rank brings its own T tokens, their top-k expert indices
 * and router scores.  One call runs, on the given stream and without any host synchronisation:
 *   sort of the T*k index entries by expert (qb200_moe_sort_by_expert)
 *   -> rows packed per destination rank (one kernel) -> all-to-all of rows and local expert ids
 *      (ncclSend/ncclRecv inside one group, fixed `capacity` rows per peer)
 *   -> gate/up projections + SwiGLU and down projection of the received rows on the local banks
 *      (qb200_gather_qmm_swiglu, qb200_gather_qmm: rows of padding carry an out-of-range expert id and cost nothing)
 *   -> all-to-all back -> products with the router scores and the sum over top-k in the reference's order
 *      (qb200_moe_weighted_sum, src/transformer.zig:15127-15140).
 * Every rank of the communicator must make the call with the same T, k, H, I, capacity and dtype.
 */
#ifndef QB200_EP_H
#define QB200_EP_H

#include "qb200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Communicator helpers for hosts without an NCCL binding of their own: thin wrappers over ncclGetUniqueId,
 * ncclCommInitRank (on the current device) and ncclCommDestroy of the NCCL this library is linked with.  A host
 * that already has an ncclComm_t passes it to qb200_moe_block_ep directly. */
#define QB200_EP_UNIQUE_ID_BYTES 128
QB200_API int qb200_ep_unique_id(void* id_out /* QB200_EP_UNIQUE_ID_BYTES */);
QB200_API int qb200_ep_comm_create(void** comm_out, int world, int rank, const void* id);
QB200_API int qb200_ep_comm_destroy(void* comm);

/* Rows each rank can send to one peer: the largest capacity the local kernels serve, world * capacity <= 2048,
 * but never more than T*k (which can never overflow). */
QB200_API int64_t qb200_moe_block_ep_capacity(int64_t T, int topk, int world);
QB200_API size_t qb200_moe_block_ep_workspace_size(int64_t T, int topk, int64_t H, int64_t I, int num_experts,
                                                   int world, int64_t capacity);

/* res [T, H] = the routed-expert block over x [T, H] (bf16) with inds [T, k] (int32) and scores [T, k] (bf16).
 * gate/up banks [E/world, I, H*bits/32] and the down bank [E/world, H, I*bits/32] with their scales and biases are
 * this rank's experts.  `comm` is an ncclComm_t over `world` ranks in which this process is `rank`.
 * `capacity` rows can go to each peer; when more of this rank's rows are routed to one peer, the surplus rows
 * contribute nothing and *overflow (an int on the device, optional) is set to the number of surplus rows -- with
 * capacity >= T*k that cannot happen.  workspace: qb200_moe_block_ep_workspace_size bytes of device memory. */
QB200_API int qb200_moe_block_ep(qb200_tensor* res, const qb200_tensor* x, const qb200_tensor* inds,
                                 const qb200_tensor* scores, const qb200_tensor* w_gate, const qb200_tensor* s_gate,
                                 const qb200_tensor* b_gate, const qb200_tensor* w_up, const qb200_tensor* s_up,
                                 const qb200_tensor* b_up, const qb200_tensor* w_down, const qb200_tensor* s_down,
                                 const qb200_tensor* b_down, int num_experts, int world, int rank, void* comm,
                                 int64_t capacity, int group_size, int bits, int* overflow, void* workspace,
                                 size_t workspace_bytes, qb200_stream s);

#ifdef __cplusplus
}
#endif
#endif /* QB200_EP_H */

"""Expert-parallel routed-MoE block around gather_qmm (one process per GPU).

mlx-serve runs its MoE layer on one device: route, sort rows by expert, three ``gather_qmm`` calls with a
SwiGLU in between, un-permute, weight by the router scores and sum over the top-k
(``moeMLP2``, src/transformer.zig:14961-15043 and :15127-15140; routing ``moeRoutingChain`` :17022-17063).
Here the experts are partitioned over the ranks of a process group -- rank r owns experts
[r*E/G, (r+1)*E/G) -- and the token rows are exchanged once each way:

    route locally -> sort rows by expert (rows for one destination rank are then contiguous)
    -> all-to-all of per-destination row counts
    -> dispatch all-to-all of the rows (and their expert ids)
    -> local gather_qmm(gate), gather_qmm(up), SwiGLU, gather_qmm(down) on the owned experts
    -> combine all-to-all back to the row's owner
    -> owner applies the router weights and sums over the top-k.

Two exchange plans: ``moe_block_ep`` sends exactly the routed rows (the per-destination counts are exchanged
first, which costs a host synchronisation: right for prefill-sized inputs) and ``moe_block_ep_padded`` sends
fixed-size blocks (every rank may receive all of a peer's T*k rows; unused slots carry expert id -1, which
gather_qmm skips), so that nothing on the host waits for the device: right for decode-sized inputs.

``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests) is only the plumbing; the expert math is
``expert_fn``, by default the library's gather_qmm through the C ABI.  The rows a rank receives are a
concatenation of sorted runs, one per source rank, which gather_qmm accepts as is (it never relies on the
order of the indices).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def route(logits: torch.Tensor, k: int, dtype=torch.bfloat16):
    """softmax -> top-k -> renormalise (src/transformer.zig:17022-17063).  Returns (inds [T,k] int64, w [T,k])."""
    p = torch.softmax(logits.float(), dim=-1)
    topv, topi = torch.topk(p, k, dim=-1)
    w = (topv / topv.sum(dim=-1, keepdim=True)).to(dtype)
    return topi, w


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """silu(g) * u with each op's result in the activation dtype (src/transformer.zig:20157-20159)."""
    return (torch.nn.functional.silu(g.float()).to(g.dtype).float() * u.float()).to(g.dtype)


def default_expert_fn(banks, group_size=64, bits=4):
    """expert_fn over local banks {'gate','up','down': (q, scales, biases)} using the CUDA library."""
    import qb200

    def fn(name, rows, expert_ids):
        q, s, b = banks[name]
        out = qb200.gather_qmm(rows.unsqueeze(1).contiguous(), q, s, b, None, expert_ids.to(torch.int32).contiguous(),
                               True, group_size, bits, sorted_indices=False)
        return out.squeeze(1)
    return fn


def _a2a(t: torch.Tensor, out_splits, in_splits, group):
    out = t.new_empty((int(sum(out_splits)),) + tuple(t.shape[1:]))
    dist.all_to_all_single(out, t.contiguous(), output_split_sizes=list(out_splits), input_split_sizes=list(in_splits),
                           group=group)
    return out


def moe_block_ep(x: torch.Tensor, inds: torch.Tensor, weights: torch.Tensor, num_experts: int, expert_fn,
                 group=None) -> torch.Tensor:
    """One routed-MoE block for this rank's tokens x [T, H]; experts are spread over ``group``.

    ``expert_fn(name, rows [R, K], local_expert_ids [R]) -> [R, N]`` runs one projection on the owned experts.
    With a single rank (or no initialised process group) the exchange degenerates to the identity.
    """
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    T, k = inds.shape
    per_rank = (num_experts + world - 1) // world
    flat = inds.reshape(-1)
    order = torch.argsort(flat, stable=True)
    sorted_e = flat[order]
    src_tok = torch.div(order, k, rounding_mode="floor")
    rows = x[src_tok]
    if world > 1:
        dest = torch.div(sorted_e, per_rank, rounding_mode="floor")
        send_counts = torch.bincount(dest, minlength=world).to(torch.int64)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        send_l, recv_l = send_counts.tolist(), recv_counts.tolist()
        rows_in = _a2a(rows, recv_l, send_l, group)
        e_in = _a2a(sorted_e, recv_l, send_l, group)
    else:
        send_l = recv_l = None
        rows_in, e_in = rows, sorted_e
    local_e = e_in - rank * per_rank
    if rows_in.shape[0] > 0:
        g = expert_fn("gate", rows_in, local_e)
        u = expert_fn("up", rows_in, local_e)
        d = expert_fn("down", swiglu(g, u), local_e)
    else:
        d = rows_in.new_empty((0, x.shape[1]))
    d_back = _a2a(d, send_l, recv_l, group) if world > 1 else d
    # weight by the router score (product rounded to the activation dtype, src/transformer.zig:20567-20571)
    w_sorted = weights.reshape(-1)[order]
    contrib = (d_back.float() * w_sorted.float().unsqueeze(1)).to(x.dtype).float()
    out = torch.zeros((T, x.shape[1]), dtype=torch.float32, device=x.device)
    out.index_add_(0, src_tok, contrib)
    return out.to(x.dtype)


def moe_block_ep_padded(x: torch.Tensor, inds: torch.Tensor, weights: torch.Tensor, num_experts: int, expert_fn,
                        group=None) -> torch.Tensor:
    """The same block with fixed-size exchange buffers and no host synchronisation.

    Every rank sends each peer a block of T*k row slots (rows for that peer first, in expert order; the rest
    empty with expert id -1) and gets blocks of the same size back, so all collectives have static shapes and
    the whole block can be enqueued (or captured in a CUDA graph) without reading anything back.
    ``expert_fn`` must leave rows whose local expert id is negative alone (the library's gather_qmm does).
    """
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    T, k = inds.shape
    R, H = T * k, x.shape[1]
    per_rank = (num_experts + world - 1) // world
    dev = x.device
    flat = inds.reshape(-1)
    order = torch.argsort(flat, stable=True)
    sorted_e = flat[order]
    src_tok = torch.div(order, k, rounding_mode="floor")
    dest = torch.div(sorted_e, per_rank, rounding_mode="floor")           # ascending
    starts = torch.searchsorted(dest, torch.arange(world, device=dev, dtype=dest.dtype))
    pos = torch.arange(R, device=dev) - starts[dest]                      # slot inside the destination's block
    send_rows = x.new_zeros((world, R, H))
    send_rows[dest, pos] = x[src_tok]
    send_ids = torch.full((world, R), -1, dtype=torch.int64, device=dev)
    send_ids[dest, pos] = sorted_e - dest * per_rank
    if world > 1:
        rows_in = torch.empty_like(send_rows)
        ids_in = torch.empty_like(send_ids)
        dist.all_to_all_single(rows_in, send_rows, group=group)
        dist.all_to_all_single(ids_in, send_ids, group=group)
    else:
        rows_in, ids_in = send_rows, send_ids
    rows_in = rows_in.reshape(world * R, H)
    ids_in = ids_in.reshape(world * R)
    g = expert_fn("gate", rows_in, ids_in)
    u = expert_fn("up", rows_in, ids_in)
    d = expert_fn("down", swiglu(g, u), ids_in).reshape(world, R, H)
    if world > 1:
        d_back = torch.empty_like(d)
        dist.all_to_all_single(d_back, d.contiguous(), group=group)
    else:
        d_back = d
    picked = d_back[dest, pos]                                            # [R, H]: the routed rows, in sorted order
    w_sorted = weights.reshape(-1)[order]
    contrib = (picked.float() * w_sorted.float().unsqueeze(1)).to(x.dtype).float()
    out = torch.zeros((T, H), dtype=torch.float32, device=dev)
    out.index_add_(0, src_tok, contrib)
    return out.to(x.dtype)

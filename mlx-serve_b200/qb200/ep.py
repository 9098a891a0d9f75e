"""Expert-parallel routed-expert block: binding of libqb200_ep.so and a host mirror of its exchange plan.

The product is the C entry ``qb200_moe_block_ep`` (include/qb200_ep.h): sort by expert, pack per destination
rank, NCCL all-to-all of rows and expert ids, the library's fused gate/up + SwiGLU and down kernels on the local
experts, all-to-all back, score-weighted sum -- rank r owns experts [r*E/world, (r+1)*E/world).  It stands for
moeMLP2 (mlx-serve src/transformer.zig:14945-15140) run over several GPUs.

``plan_pack`` / ``moe_block_ep_host`` restate the same plan on the host with numpy index arithmetic and
``torch.distributed`` (any backend), the expert math supplied by the caller.  They exist for the CPU tests of the
exchange logic (gloo ranks, expert math by the CPU oracle) and are not on any GPU path.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch
import torch.distributed as dist

from . import Tensor, _packed, check, desc, lib as core_lib

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EP_LIB_PATH = os.path.join(_PKG, "libqb200_ep.so")
_ep = None


def ep_lib():
    """Load libqb200_ep.so (after the core library, which it links); fails loudly when it has not been built."""
    global _ep
    if _ep is None:
        core_lib()
        if not os.path.exists(EP_LIB_PATH):
            raise FileNotFoundError(f"{EP_LIB_PATH} is missing: build it with `make -C {_PKG}`")
        L = C.CDLL(EP_LIB_PATH)
        TP = C.POINTER(Tensor)
        L.qb200_ep_unique_id.argtypes = [C.c_void_p]
        L.qb200_ep_comm_create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p]
        L.qb200_ep_comm_destroy.argtypes = [C.c_void_p]
        L.qb200_moe_block_ep_capacity.restype = C.c_int64
        L.qb200_moe_block_ep_capacity.argtypes = [C.c_int64, C.c_int, C.c_int]
        L.qb200_moe_block_ep_workspace_size.restype = C.c_size_t
        L.qb200_moe_block_ep_workspace_size.argtypes = [C.c_int64, C.c_int, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int64]
        L.qb200_moe_block_ep.argtypes = [TP] * 13 + [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_int,
                                                     C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        for n in ("qb200_ep_unique_id", "qb200_ep_comm_create", "qb200_ep_comm_destroy", "qb200_moe_block_ep"):
            getattr(L, n).restype = C.c_int
        _ep = L
    return _ep


def make_comm(world: int, rank: int, device):
    """An NCCL communicator for the block, made with the NCCL the library links; the unique id travels over
    torch.distributed (plumbing only)."""
    L = ep_lib()
    buf = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        raw = (C.c_ubyte * 128)()
        check(L.qb200_ep_unique_id(raw))
        buf = torch.tensor(list(raw), dtype=torch.uint8)
    if world > 1:
        on = buf.to(device) if dist.get_backend() == "nccl" else buf
        dist.broadcast(on, 0)
        buf = on.cpu()
    raw = (C.c_ubyte * 128)(*buf.tolist())
    comm = C.c_void_p()
    check(L.qb200_ep_comm_create(C.byref(comm), world, rank, raw))
    return comm


def capacity(T: int, topk: int, world: int) -> int:
    return int(ep_lib().qb200_moe_block_ep_capacity(T, topk, world))


class Block:
    """Workspace, overflow counter and output of one expert-parallel block, allocated once and reused."""

    def __init__(self, T, topk, H, I, E, world, rank, comm, banks, cap=None, group_size=64, bits=4, device="cuda"):
        L = ep_lib()
        self.T, self.topk, self.H, self.I, self.E, self.world, self.rank, self.comm = T, topk, H, I, E, world, rank, comm
        self.cap = capacity(T, topk, world) if cap is None else cap
        self.gs, self.bits = group_size, bits
        need = int(L.qb200_moe_block_ep_workspace_size(T, topk, H, I, E, world, self.cap))
        self.ws = torch.empty(need, dtype=torch.uint8, device=device)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=device)
        self.out = torch.empty((T, H), dtype=torch.bfloat16, device=device)
        self.banks = banks   # {"gate": (q, s, b), "up": ..., "down": ...} of this rank's experts

    def run(self, x, inds, scores):
        L = ep_lib()
        ds = [desc(self.out), desc(x), desc(inds), desc(scores)]
        for name in ("gate", "up", "down"):
            q, s, b = self.banks[name]
            ds += [_packed(q), desc(s), desc(b)]
        check(L.qb200_moe_block_ep(*[C.byref(d) for d in ds], self.E, self.world, self.rank, self.comm, self.cap, self.gs,
                                   self.bits, C.c_void_p(self.overflow.data_ptr()), C.c_void_p(self.ws.data_ptr()),
                                   self.ws.numel(), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return self.out


# ---------------------------------------------------------------------------------------------------------------
# Host mirror of the exchange plan (index arithmetic only), for the CPU tests.

def plan_pack(inds: np.ndarray, E: int, world: int, cap: int):
    """inds [T, k] -> (send_src [world, cap] position in the flattened index list or -1, send_e [world, cap] local
    expert id or E/world for padding, back_row [T*k] row of the returned buffer or -1, overflow rows)."""
    flat = inds.reshape(-1)
    n, El = flat.size, E // world
    key = np.where((flat < 0) | (flat >= E), E, flat)
    order = np.argsort(key, kind="stable")
    inv = np.argsort(order, kind="stable")
    offs = np.concatenate([[0], np.cumsum(np.bincount(key, minlength=E + 1)[:E])])
    send_src = np.full((world, cap), -1, np.int64)
    send_e = np.full((world, cap), El, np.int32)
    overflow = 0
    for r in range(world):
        p0, p1 = offs[r * El], offs[(r + 1) * El]
        m = min(p1 - p0, cap)
        send_src[r, :m] = order[p0:p0 + m]
        send_e[r, :m] = flat[order[p0:p0 + m]] - r * El
        overflow += max(0, p1 - p0 - cap)
    back_row = np.full(n, -1, np.int64)
    for i in range(n):
        e = flat[i]
        if 0 <= e < E:
            r = e // El
            slot = inv[i] - offs[r * El]
            if slot < cap:
                back_row[i] = r * cap + slot
    return send_src, send_e, back_row, int(overflow)


def moe_block_ep_host(x: np.ndarray, inds: np.ndarray, scores: np.ndarray, E: int, cap: int, expert_fn, weighted_sum):
    """The block over torch.distributed with the plan above.  ``expert_fn(rows [R, H], local_ids [R]) -> [R, H]``
    computes gate/up + SwiGLU + down for rows whose id is in range and leaves the others alone;
    ``weighted_sum(y [R, H], scores [T, k], rows [T*k]) -> [T, H]``.  A peer that does not show up makes the
    all_to_all raise after the process group's timeout: the exchange has no other way to wait."""
    world, rank = dist.get_world_size(), dist.get_rank()
    T, k = inds.shape
    H = x.shape[1]
    src, send_e, back_row, overflow = plan_pack(inds, E, world, cap)
    send_x = np.zeros((world, cap, H), np.float32)
    live = src >= 0
    send_x[live] = x[src[live] // k]
    recv_x, recv_e = torch.empty((world, cap, H)), torch.empty((world, cap), dtype=torch.int32)
    dist.all_to_all_single(recv_x, torch.from_numpy(send_x))
    dist.all_to_all_single(recv_e, torch.from_numpy(send_e))
    y = expert_fn(recv_x.numpy().reshape(world * cap, H), recv_e.numpy().reshape(-1))
    back = torch.empty((world, cap, H))
    dist.all_to_all_single(back, torch.from_numpy(np.ascontiguousarray(y, np.float32).reshape(world, cap, H)))
    return weighted_sum(back.numpy().reshape(world * cap, H), scores, back_row), overflow


# ---------------------------------------------------------------------------------------------------------------

def bench_block(dev, g, world, rank, steps=20, T=64):
    """Benchmark configuration 3, decode: 128 experts top-8, hidden 2048, expert width 768, 4-bit g64, T tokens per
    GPU, experts sharded over the ranks.  Device time of the block (max over ranks), tokens/s of the whole job."""
    from . import moe_route, quantize
    E, H, I, topk = 128, 2048, 768, 8
    per = E // world
    banks = {}
    for name, (n, k) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
        w = (torch.randn((per, n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
        banks[name] = quantize(w, 64, 4)
        del w
    comm = make_comm(world, rank, dev)
    blk = Block(T, topk, H, I, E, world, rank, comm, banks, device=dev)
    x = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
    inds, scores = moe_route(torch.randn((T, E), device=dev, generator=g).to(torch.bfloat16), topk)
    for _ in range(5):
        out = blk.run(x, inds, scores)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = blk.run(x, inds, scores)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    res = {"n_gpus": world, "experts_per_gpu": per, "tokens_per_gpu": T, "capacity_rows_per_peer": blk.cap,
           "us_per_block": ms * 1e3, "tokens_per_s": world * T / (ms * 1e-3), "overflow_rows": int(blk.overflow.item()),
           "nan": bool(torch.isnan(out).any()),
           "nvlink_bytes_per_gpu_per_block": 2 * (world - 1) * blk.cap * H * 2 + (world - 1) * blk.cap * 4,
           "launches_per_block": "5 kernels (sort, pack, gate/up+SwiGLU, down, weighted sum) + 2 NCCL groups"}
    ep_lib().qb200_ep_comm_destroy(comm)
    return res

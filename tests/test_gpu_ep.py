"""GPU tests of the expert-parallel routed-expert block (qb200_moe_block_ep, include/qb200_ep.h): the exchange must
not change a single value of the block -- the same rows go through the same kernels, only on another GPU."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
E, H, I, TOPK = 16, 512, 256, 4


def _banks(dev):
    import qb200
    g = torch.Generator(device=dev).manual_seed(7)
    banks = {}
    for name, (n, k) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
        w = (torch.randn((E, n, k), device=dev, generator=g) * 0.05).to(torch.bfloat16)
        banks[name] = qb200.quantize(w, 64, 4)
    return banks


def _inputs(dev, rank, T):
    import qb200
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
    inds, scores = qb200.moe_route(torch.randn((T, E), device=dev, generator=g).to(torch.bfloat16), TOPK)
    return x, inds, scores


def _single_gpu_block(x, inds, scores, banks):
    """moeMLP2's chain through the library on one GPU: sort, fused gate/up + SwiGLU, down, weighted sum."""
    import qb200
    T = x.shape[0]
    order, inv, sinds, rows, _ = qb200.moe_sort_by_expert(inds, E)
    act = qb200.gather_qmm_swiglu(x.view(T, 1, H), *banks["gate"], *banks["up"], rows, sinds, 64, 4, sorted_indices=True)
    yd = qb200.gather_qmm(act, *banks["down"], None, sinds, True, 64, 4, sorted_indices=True)
    return qb200.moe_weighted_sum(yd, scores, inv)


@pytest.mark.parametrize("T", [24, 1, 64])
def test_one_rank_block_equals_the_single_gpu_chain(T):
    """world = 1: the whole pipeline (pack, NCCL send/recv to itself, local experts, back, weighted sum)."""
    import qb200
    from qb200 import ep
    dev = torch.device("cuda", 0)
    banks = _banks(dev)
    x, inds, scores = _inputs(dev, 0, T)
    comm = ep.make_comm(1, 0, dev)
    try:
        blk = ep.Block(T, TOPK, H, I, E, 1, 0, comm, banks, device=dev)
        out = blk.run(x, inds, scores).clone()
        out2 = blk.run(x, inds, scores)
        torch.cuda.synchronize()
        assert int(blk.overflow.item()) == 0
        ref = _single_gpu_block(x, inds, scores, banks)
        assert not torch.isnan(out).any()
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
        assert torch.equal(out2.view(torch.int16), ref.view(torch.int16))
    finally:
        ep.ep_lib().qb200_ep_comm_destroy(comm)


def test_capacity_overflow_is_counted_and_the_surplus_rows_contribute_nothing():
    import qb200
    from qb200 import ep
    dev = torch.device("cuda", 0)
    banks = _banks(dev)
    T = 32
    x, inds, scores = _inputs(dev, 0, T)
    comm = ep.make_comm(1, 0, dev)
    try:
        blk = ep.Block(T, TOPK, H, I, E, 1, 0, comm, banks, cap=100, device=dev)   # 128 rows for one peer, room for 100
        out = blk.run(x, inds, scores)
        torch.cuda.synchronize()
        assert int(blk.overflow.item()) == 28 and not torch.isnan(out).any()
    finally:
        ep.ep_lib().qb200_ep_comm_destroy(comm)


def _rank_main(rank, world, port, T, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    for p in (ROOT, os.path.join(ROOT, "mlx-serve_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    import qb200
    from qb200 import ep
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        full = _banks(dev)
        per = E // world
        local = {k: tuple(t[rank * per:(rank + 1) * per].contiguous() for t in v) for k, v in full.items()}
        x, inds, scores = _inputs(dev, rank, T)
        comm = ep.make_comm(world, rank, dev)
        blk = ep.Block(T, TOPK, H, I, E, world, rank, comm, local, device=dev)
        out = blk.run(x, inds, scores)
        torch.cuda.synchronize()
        ref = _single_gpu_block(x, inds, scores, full)
        ret[rank] = (bool(torch.equal(out.view(torch.int16), ref.view(torch.int16))), int(blk.overflow.item()),
                     float((out.float() - ref.float()).abs().max()))
        dist.barrier()
        ep.ep_lib().qb200_ep_comm_destroy(comm)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [24, 64])
def test_two_gpu_block_equals_the_single_gpu_chain(T):
    """Two ranks on two GPUs, each with its own tokens and half of the experts: bit for bit the single-GPU block."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, 33500 + (os.getpid() + T) % 2000
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, port, T, ret), nprocs=world, join=True)
    for rank in range(world):
        same, overflow, maxd = ret[rank]
        assert overflow == 0
        assert same, f"rank {rank}: the exchange changed values (max |d| {maxd})"

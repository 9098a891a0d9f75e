"""Expert-parallel MoE exchange on CPU: two gloo ranks, expert math by the CPU oracle.

Covers the host logic of the one real exchange step on the path (counts all-to-all, dispatch, local
gather_qmm on the owned experts, combine) against the single-process block on the same seeded inputs."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "mlx-serve_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

E, H, I, K_TOP, T = 8, 256, 256, 2, 12


def _banks():
    from oracle import qoracle as qo
    rng = np.random.default_rng(3)
    banks = {}
    for name, (n, k) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
        w = qo.bf16_round((rng.standard_normal((E, n, k)) * 0.05).astype(np.float32))
        banks[name] = qo.quantize(w, 64, 4)
    return banks


def _oracle_fn(banks, lo, hi):
    """expert_fn over experts [lo, hi) computed by the CPU oracle (bf16 outputs, like the CUDA kernels)."""
    from oracle import qoracle as qo

    def fn(name, rows, local_ids):
        q, s, b = (a[lo:hi] for a in banks[name])
        ids = local_ids.numpy()
        live = np.nonzero(ids >= 0)[0]          # empty slots of the padded exchange carry -1 and stay untouched
        x = rows.float().numpy().reshape(rows.shape[0], 1, rows.shape[1])
        y = np.full((rows.shape[0], q.shape[1]), np.nan, np.float32)
        if live.size:
            y[live] = qo.gather_qmm(x[live], q, s, b, np.arange(live.size), ids[live], 64, 4)[:, 0, :]
        return torch.from_numpy(y).to(torch.bfloat16)
    return fn


def _inputs(rank):
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn((T, H), generator=g).to(torch.bfloat16)
    logits = torch.randn((T, E), generator=g)
    return x, logits


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from qb200 import ep
        banks = _banks()
        per = E // world
        x, logits = _inputs(rank)
        inds, w = ep.route(logits, K_TOP)
        fn = _oracle_fn(banks, rank * per, (rank + 1) * per)
        out = ep.moe_block_ep(x, inds, w, E, fn)
        ret[rank] = out.float().numpy()
        ret[world + rank] = ep.moe_block_ep_padded(x, inds, w, E, fn).float().numpy()
    finally:
        dist.destroy_process_group()


def test_two_rank_exchange_matches_single_process():
    from qb200 import ep
    world, port = 2, 29500 + os.getpid() % 2000
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    banks = _banks()
    for rank in range(world):
        x, logits = _inputs(rank)
        inds, w = ep.route(logits, K_TOP)
        ref = ep.moe_block_ep(x, inds, w, E, _oracle_fn(banks, 0, E)).float().numpy()
        assert not np.isnan(ret[rank]).any()
        assert np.array_equal(ret[rank], ref), "the exchange must not change any value"
        assert not np.isnan(ret[world + rank]).any(), "an empty slot of the padded exchange leaked into the result"
        assert np.array_equal(ret[world + rank], ref), "the padded exchange must not change any value"
        assert np.array_equal(ep.moe_block_ep_padded(x, inds, w, E, _oracle_fn(banks, 0, E)).float().numpy(), ref)


def test_route_renormalises_and_orders():
    from qb200 import ep
    logits = torch.tensor([[0.0, 2.0, 1.0, -1.0]])
    inds, w = ep.route(logits, 2, dtype=torch.float32)
    assert inds.tolist() == [[1, 2]]
    assert abs(float(w.sum()) - 1.0) < 1e-6 and float(w[0, 0]) > float(w[0, 1])

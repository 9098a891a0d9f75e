"""Expert-parallel MoE exchange on CPU: two gloo ranks, expert math by the CPU oracle.

Covers the host logic of the one real exchange step on the path -- the plan the CUDA entry qb200_moe_block_ep follows
(sort by expert, fixed-capacity blocks per destination rank whose padding carries an out-of-range expert id,
all-to-all out and back, rows picked out of the returned buffer) -- against the single-process block on the same
seeded inputs, and what a rank sees when its peer never joins the exchange."""
import datetime
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


def _expert_fn(banks, lo, hi):
    """gate/up + SwiGLU + down over experts [lo, hi) by the CPU oracle, every op output rounded to bf16 like the CUDA
    kernels; rows whose id is out of range (the padding of the exchange) are left as NaN, so a leak would show."""
    from oracle import qoracle as qo

    def fn(rows, local_ids):
        live = np.nonzero((local_ids >= 0) & (local_ids < hi - lo))[0]
        y = np.full((rows.shape[0], H), np.nan, np.float32)
        if live.size:
            x = rows[live].reshape(live.size, 1, H)
            sel = np.arange(live.size)
            gq, gs, gb = (a[lo:hi] for a in banks["gate"])
            uq, us, ub = (a[lo:hi] for a in banks["up"])
            dq, ds, db = (a[lo:hi] for a in banks["down"])
            gate = qo.bf16_round(qo.gather_qmm(x, gq, gs, gb, sel, local_ids[live], 64, 4))
            up = qo.bf16_round(qo.gather_qmm(x, uq, us, ub, sel, local_ids[live], 64, 4))
            act = qo.bf16_to_f32(qo.swiglu_bf16(gate, up))
            y[live] = qo.bf16_round(qo.gather_qmm(act, dq, ds, db, sel, local_ids[live], 64, 4))[:, 0, :]
        return y
    return fn


def _weighted_sum(y, scores, rows):
    from oracle import qoracle as qo
    safe = np.where(rows >= 0, rows, 0)
    picked = np.where((rows >= 0)[:, None], y[safe], 0.0).astype(np.float32)   # rows that overflowed contribute nothing
    return qo.moe_weighted_sum(picked, scores, None)


def _inputs(rank):
    from oracle import qoracle as qo
    rng = np.random.default_rng(100 + rank)
    x = qo.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    inds, scores = qo.moe_route(qo.bf16_round(rng.standard_normal((T, E)).astype(np.float32)), K_TOP)
    return x, inds, scores


def _single_process(x, inds, scores, banks):
    """The block on one device: every entry through its own expert, then the weighted sum in token order."""
    fn = _expert_fn(banks, 0, E)
    rows = np.repeat(x, K_TOP, axis=0)
    y = fn(rows, inds.reshape(-1))
    return _weighted_sum(y, scores, np.arange(T * K_TOP))


def _worker(rank, world, port, cap, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from qb200 import ep
        banks = _banks()
        per = E // world
        x, inds, scores = _inputs(rank)
        out, overflow = ep.moe_block_ep_host(x, inds, scores, E, cap, _expert_fn(banks, rank * per, (rank + 1) * per), _weighted_sum)
        ret[rank] = (out, overflow)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cap", [T * K_TOP, 16])
def test_two_rank_exchange_matches_single_process(cap):
    world, port = 2, 29500 + (os.getpid() + cap) % 2000
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, cap, ret), nprocs=world, join=True)
    banks = _banks()
    for rank in range(world):
        x, inds, scores = _inputs(rank)
        ref = _single_process(x, inds, scores, banks)
        out, overflow = ret[rank]
        assert overflow == 0
        assert not np.isnan(out).any(), "a padding slot of the exchange leaked into the result"
        assert np.array_equal(out, ref), "the exchange must not change any value"


def test_plan_pack_capacity_and_overflow():
    from qb200 import ep
    inds = np.array([[0, 1], [0, 5], [0, 2], [7, 0], [9, 3]], np.int32)   # expert 0 four times; 9 is out of range
    src, send_e, back, overflow = ep.plan_pack(inds, 8, 2, 4)
    assert overflow == 3                      # rank 0 is sent 7 rows (experts 0,0,0,0,1,2,3), capacity 4
    assert send_e[0].tolist() == [0, 0, 0, 0] and send_e[1].tolist() == [1, 3, 4, 4]   # 4 = padding for rank 1
    assert (back >= 0).sum() == 6 and back[8] == -1          # the out-of-range entry has no row
    src, send_e, back, overflow = ep.plan_pack(inds, 8, 2, 10)
    assert overflow == 0 and (back >= 0).sum() == 9
    # every live entry finds its own row again
    flat = inds.reshape(-1)
    for i in np.nonzero(back >= 0)[0]:
        r, slot = divmod(back[i], 10)
        assert src[r, slot] == i and send_e[r, slot] == flat[i] - r * 4


def _absent_peer(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        if rank == 1:
            ret[rank] = "left before the exchange"    # between steps, with nothing in flight
            return
        from qb200 import ep
        x, inds, scores = _inputs(rank)
        try:
            ep.moe_block_ep_host(x, inds, scores, E, T * K_TOP, _expert_fn(_banks(), 0, E // world), _weighted_sum)
            ret[rank] = "returned"
        except Exception as ex:   # the collective's timeout is how the absence is learnt
            ret[rank] = "raised " + type(ex).__name__
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_a_rank_that_never_joins_the_exchange_surfaces_as_an_error():
    world, port = 2, 31500 + os.getpid() % 2000
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_absent_peer, args=(world, port, ret), nprocs=world, join=True)
    assert ret[1] == "left before the exchange"
    assert ret[0].startswith("raised"), ret[0]

"""GPU parity of qb200_moe_sort_by_expert against numpy's stable argsort (the sort step of moeMLP2,
src/transformer.zig:14961-15006): integer work, compared bit for bit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(inds_np, E, k, dtype=torch.int32):
    import qb200
    flat = inds_np.reshape(-1)
    d = torch.from_numpy(inds_np).to(dtype).cuda()
    order, inv, sinds, rows, offs = qb200.moe_sort_by_expert(d, E)
    torch.cuda.synchronize()
    key = np.where((flat < 0) | (flat >= E), E, flat)          # out-of-range entries sort behind every expert
    want = np.argsort(key, kind="stable").astype(np.int32)
    assert np.array_equal(order.cpu().numpy(), want)
    assert np.array_equal(inv.cpu().numpy(), np.argsort(want, kind="stable").astype(np.int32))
    assert np.array_equal(sinds.cpu().numpy(), flat[want].astype(np.int32))
    assert np.array_equal(rows.cpu().numpy(), want // k)
    cnt = np.bincount(key, minlength=E + 1)[:E]
    assert np.array_equal(offs.cpu().numpy(), np.concatenate([[0], np.cumsum(cnt)]).astype(np.int32))


@pytest.mark.parametrize("T,E,k", [(64, 128, 8), (4096, 128, 8), (1, 128, 8), (7, 4, 2), (333, 1024, 6), (5000, 60, 4)])
def test_sort_matches_stable_argsort(T, E, k):
    """Benchmark configuration 3's two token counts (64 and 4096 tokens, top-8 of 128 experts) and ragged others."""
    rng = np.random.default_rng(T + E + k)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    inds = np.argsort(-logits, axis=-1, kind="stable")[:, :k].astype(np.int32)
    _check(inds, E, k)


def test_int64_indices_out_of_range_entries_and_one_hot_expert():
    rng = np.random.default_rng(5)
    inds = rng.integers(-2, 20, size=(100, 4)).astype(np.int64)   # values -2, -1, 16..19 are outside [0, 16)
    _check(inds, 16, 4, torch.int64)
    _check(np.full((257, 8), 3, np.int32), 8, 8)                   # every entry the same expert: order = identity


def test_outputs_are_optional_and_empty_input_is_accepted():
    import ctypes as C
    import qb200
    L = qb200.lib()
    inds = torch.randint(0, 8, (33, 2), dtype=torch.int32, device="cuda")
    sinds = torch.empty((66,), dtype=torch.int32, device="cuda")
    e = qb200.desc(None)
    qb200.check(L.qb200_moe_sort_by_expert(C.byref(e), C.byref(e), C.byref(qb200.desc(sinds)), C.byref(e), C.byref(e),
                                           C.byref(qb200.desc(inds)), 8, None))
    torch.cuda.synchronize()
    assert np.array_equal(sinds.cpu().numpy(), np.sort(inds.cpu().numpy().reshape(-1), kind="stable"))
    offs = torch.full((9,), -1, dtype=torch.int32, device="cuda")
    none = torch.empty((0, 2), dtype=torch.int32, device="cuda")
    qb200.check(L.qb200_moe_sort_by_expert(C.byref(e), C.byref(e), C.byref(e), C.byref(e), C.byref(qb200.desc(offs)),
                                           C.byref(qb200.desc(none)), 8, None))
    torch.cuda.synchronize()
    assert int(offs.abs().sum()) == 0

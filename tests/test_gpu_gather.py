"""GPU parity of gather_qmm through the C ABI against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import qoracle as qo
from util import dev_triple, gate_bf16, gate_f32, make_weight, rand_bf16, to_dev_bf16

pytestmark = pytest.mark.gpu


def _route(rng, T, E, k):
    """softmax -> top-k (src/transformer.zig:17022-17063); returns expert ids [T, k]."""
    logits = rng.standard_normal((T, E)).astype(np.float32)
    return np.argsort(-logits, axis=1)[:, :k].astype(np.int32)


def test_reference_small_cases():
    """src/transformer.zig:24643-24835: E=4, IN=32, OUT=8, gs=32, 8-bit; decode 5-D + sorted [N,1,IN]; tol 2e-2."""
    import qb200
    E, IN, OUT = 4, 32, 8
    wh = ((np.arange(E * OUT * IN) % 13).astype(np.float32) - 6) * np.float32(0.05)
    q, s, b = qo.quantize(qo.bf16_round(wh.reshape(E, OUT, IN)), 32, 8)
    dq, ds, db = dev_triple(q, s, b)
    wd = qo.bf16_to_f32(qo.dequantize(q, s, b, 32, 8, out_bf16=True))
    x = qo.bf16_round((((np.arange(IN) % 5).astype(np.float32)) - 2) * np.float32(0.1))
    inds = np.array([[[1, 3]]], np.int32)
    y = qb200.gather_qmm(to_dev_bf16(qo.f32_to_bf16(x)).view(1, 1, 1, 1, IN), dq, ds, db, None,
                         torch.from_numpy(inds).cuda(), True, 32, 8, sorted_indices=False)
    assert tuple(y.shape) == (1, 1, 2, 1, OUT)
    gt = np.stack([wd[e] @ x for e in (1, 3)])
    assert np.abs(y.float().cpu().numpy().reshape(2, OUT) - gt).max() < 2e-2
    N = 5
    xs = qo.bf16_round((((np.arange(N * IN) % 7).astype(np.float32)) - 3) * np.float32(0.07)).reshape(N, 1, IN)
    srt = np.array([0, 0, 1, 2, 3], np.int32)
    y = qb200.gather_qmm(to_dev_bf16(qo.f32_to_bf16(xs)), dq, ds, db, None, torch.from_numpy(srt).cuda(), True, 32, 8,
                         sorted_indices=True)
    assert tuple(y.shape) == (N, 1, OUT)
    gt = np.stack([wd[e] @ xs[i, 0] for i, e in enumerate(srt)])
    assert np.abs(y.float().cpu().numpy().reshape(N, OUT) - gt).max() < 2e-2


@pytest.mark.parametrize("proj", ["gate", "down"])
def test_config3_decode_sorted(proj):
    """Benchmark configuration 3, decode: 64 tokens x top-8 of 128 experts, rows sorted by expert, x_rep = x[order // 8]."""
    import qb200
    E, H, I, T, k = 128, 2048, 768, 64, 8
    N, K = (I, H) if proj == "gate" else (H, I)
    rng = np.random.default_rng(0xC3)
    q, s, b = make_weight(rng, (E, N, K), 64, 4)
    dq, ds, db = dev_triple(q, s, b)
    flat = _route(rng, T, E, k).reshape(-1)
    order = np.argsort(flat, kind="stable")
    sorted_inds = flat[order]
    x = rand_bf16(rng, (T, K))
    x_rep = x[order // k].reshape(T * k, 1, K)
    ref = qo.gather_qmm(x_rep, q, s, b, np.arange(T * k), sorted_inds, 64, 4)
    idx = torch.from_numpy(sorted_inds).cuda()
    y32 = qb200.gather_qmm(torch.from_numpy(x_rep).cuda(), dq, ds, db, None, idx, True, 64, 4, sorted_indices=True)
    gate_f32(y32.cpu().numpy(), ref, "fp32")
    y16 = qb200.gather_qmm(to_dev_bf16(qo.f32_to_bf16(x_rep)), dq, ds, db, None, idx, True, 64, 4, sorted_indices=True)
    gate_bf16(y16.float().cpu().numpy(), ref, "bf16")
    # explicit lhs indices over the un-replicated x give the same rows
    lhs = torch.from_numpy((order // k).astype(np.int32)).cuda()
    y_l = qb200.gather_qmm(to_dev_bf16(qo.f32_to_bf16(x)).view(T, 1, K), dq, ds, db, lhs, idx, True, 64, 4,
                           sorted_indices=True)
    assert torch.equal(y_l.view(torch.int16), y16.view(torch.int16))


def test_decode_unsorted_5d_shape():
    """Stock decode shape (src/transformer.zig:15091-15119): x [B,S,1,1,D], rhs [B,S,K] -> [B,S,K,1,N]."""
    import qb200
    E, D, N, B, S, k = 16, 512, 256, 2, 3, 4
    rng = np.random.default_rng(31)
    q, s, b = make_weight(rng, (E, N, D), 64, 4)
    dq, ds, db = dev_triple(q, s, b)
    x = rand_bf16(rng, (B, S, 1, 1, D))
    inds = _route(rng, B * S, E, k).reshape(B, S, k)
    y = qb200.gather_qmm(to_dev_bf16(qo.f32_to_bf16(x)), dq, ds, db, None, torch.from_numpy(inds).cuda(), True, 64, 4)
    assert tuple(y.shape) == (B, S, k, 1, N)
    lhs = np.repeat(np.arange(B * S), k)
    ref = qo.gather_qmm(x.reshape(B * S, 1, D), q, s, b, lhs, inds.reshape(-1), 64, 4)
    gate_bf16(y.float().cpu().numpy().reshape(B * S * k, 1, N), ref, "5-D decode")
    y64 = qb200.gather_qmm(to_dev_bf16(qo.f32_to_bf16(x)), dq, ds, db, None,
                           torch.from_numpy(inds.astype(np.int64)).cuda(), True, 64, 4)
    assert torch.equal(y64.view(torch.int16), y.view(torch.int16))


@pytest.mark.parametrize("bits,gs,K", [(8, 64, 512), (4, 128, 1024), (4, 64, 64), (2, 64, 256)])
def test_other_geometries_and_ragged_tail(bits, gs, K):
    """Index counts that do not fill a token block, other widths, and K only the generic path serves."""
    import qb200
    E, N, I = 6, 72, 13
    rng = np.random.default_rng(bits + gs + K)
    q, s, b = make_weight(rng, (E, N, K), gs, bits)
    dq, ds, db = dev_triple(q, s, b)
    x = rand_bf16(rng, (I, 1, K))
    inds = np.sort(rng.integers(0, E, I)).astype(np.int32)
    ref = qo.gather_qmm(x, q, s, b, np.arange(I), inds, gs, bits)
    y = qb200.gather_qmm(to_dev_bf16(qo.f32_to_bf16(x)), dq, ds, db, None, torch.from_numpy(inds).cuda(), True, gs, bits,
                         sorted_indices=True)
    gate_bf16(y.float().cpu().numpy(), ref, "ragged")
    y32 = qb200.gather_qmm(torch.from_numpy(x).cuda(), dq, ds, db, None, torch.from_numpy(inds).cuda(), True, gs, bits)
    gate_f32(y32.cpu().numpy(), ref, "ragged fp32")


@pytest.mark.parametrize("bits,gs,N,K", [(4, 64, 256, 512), (8, 64, 200, 768), (4, 128, 768, 1024)])
def test_config3_prefill_sorted_grouped(bits, gs, N, K):
    """Benchmark configuration 3, prefill form: thousands of routed rows sorted by expert, x already gathered ([I, 1, K]),
    which the library serves as a grouped GEMM on the tensor-core kernel.  Uneven runs per expert, including an
    expert without rows, one with a single row and runs that are not multiples of the 256-row tile.  The weight
    term is rounded to bf16 once on that route (as in the dense prefill route), so the reference is built from
    the oracle's bf16 dequantisation."""
    import qb200
    E = 8
    counts = [0, 1, 300, 1000, 257, 2, 2000, 536]
    I = sum(counts)
    rng = np.random.default_rng(N + K + bits)
    q, s, b = make_weight(rng, (E, N, K), gs, bits)
    dq, ds, db = dev_triple(q, s, b)
    rhs = np.repeat(np.arange(E, dtype=np.int32), counts)
    x = rand_bf16(rng, (I, 1, K))
    wd = qo.bf16_to_f32(qo.dequantize(q, s, b, gs, bits, out_bf16=True)).astype(np.float64)
    ref = np.empty((I, 1, N), np.float32)
    pos = 0
    for e, c in enumerate(counts):
        if c:
            ref[pos:pos + c, 0] = (x[pos:pos + c, 0].astype(np.float64) @ wd[e].T).astype(np.float32)
        pos += c
    y = qb200.gather_qmm(to_dev_bf16(qo.f32_to_bf16(x)), dq, ds, db, None, torch.from_numpy(rhs).cuda(), True, gs, bits,
                         sorted_indices=True)
    assert qb200.lib().qb200_debug_tc_status() == 0
    assert tuple(y.shape) == (I, 1, N)
    gate_bf16(y.float().cpu().numpy(), ref, "grouped prefill gather", slack=2e-3)
    # int64 indices take the same route
    y64 = qb200.gather_qmm(to_dev_bf16(qo.f32_to_bf16(x)), dq, ds, db, None, torch.from_numpy(rhs.astype(np.int64)).cuda(),
                           True, gs, bits, sorted_indices=True)
    assert torch.equal(y64.view(torch.int16), y.view(torch.int16))


@pytest.mark.parametrize("proj", ["gate", "down"])
def test_config3_prefill_full_size_row_sample_against_the_oracle(proj):
    """Benchmark configuration 3 at its prefill size: 128 experts, 4096 tokens x top-8 = 32768 rows sorted by expert
    (the device sort entry produces the order), gate 2048->768 and down 768->2048, 4-bit g64.  The oracle is
    row-independent, so a row sample is checked: the first two and last two rows of every expert's run."""
    import qb200
    from util import from_dev_bf16, from_dev_u32, half_ulp_fraction, record
    E, T, k = 128, 4096, 8
    N, K = (768, 2048) if proj == "gate" else (2048, 768)
    g = torch.Generator(device="cuda").manual_seed(0xC3 + N)
    w = (torch.randn((E, N, K), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    dq, ds, db = qb200.quantize(w, 64, 4)
    del w
    logits = torch.randn((T, E), device="cuda", generator=g)
    inds, _ = qb200.moe_route(logits, k)
    order, inv, sinds, rows, offs = qb200.moe_sort_by_expert(inds, E)
    xtok = torch.randn((T, K), device="cuda", generator=g).to(torch.bfloat16)
    x_rep = xtok[rows.long()].reshape(T * k, 1, K).contiguous()
    y = qb200.gather_qmm(x_rep, dq, ds, db, None, sinds, True, 64, 4, sorted_indices=True)
    torch.cuda.synchronize()
    assert qb200.lib().qb200_debug_tc_status() == 0
    assert tuple(y.shape) == (T * k, 1, N) and not torch.isnan(y).any()
    o = offs.cpu().numpy()
    sample = sorted({int(r) for e in range(E) for r in (o[e], o[e] + 1, o[e + 1] - 2, o[e + 1] - 1) if o[e] <= r < o[e + 1]})
    sample = np.array(sample, np.int64)
    hq, hs, hb = from_dev_u32(dq), from_dev_bf16(ds), from_dev_bf16(db)
    xs = x_rep[torch.from_numpy(sample).cuda()].float().cpu().numpy()                 # [S, 1, K]
    es = sinds.cpu().numpy()[sample]
    ref_w16 = np.empty((len(sample), 1, N), np.float32)
    for e in np.unique(es):
        m = es == e
        ref_w16[m, 0] = qo.qmm(np.ascontiguousarray(xs[m, 0]), hq[e], hs[e], hb[e], 64, 4, True, bf16_weights=True)
    ref = qo.gather_qmm(xs, hq, hs, hb, np.arange(len(sample)), es, 64, 4)
    got = y[torch.from_numpy(sample).cuda()].float().cpu().numpy()
    # this many sorted rows per expert run on the grouped tensor-core form: weight term rounded to bf16 once
    gate_bf16(got, ref_w16, "full-size prefill gather, bf16 weight term", slack=2e-3)
    r16 = gate_bf16(got, ref, "full-size prefill gather vs fp32 weight term", slack=1e-2)
    record(f"C3 prefill {proj} 128 experts x 32768 rows (sample of {len(sample)} rows)",
           "bf16 activations vs oracle (unrounded fp32)", r16, half_ulp_fraction(got, ref), int(ref.size))
    # the same rows through explicit lhs indices (no x_rep copy) on the first 2048 sorted rows, bit for bit
    y_l = qb200.gather_qmm(xtok.view(T, 1, K), dq, ds, db, rows[:2048].contiguous(), sinds[:2048].contiguous(), True, 64, 4,
                           sorted_indices=True)
    y_r = qb200.gather_qmm(x_rep[:2048].contiguous(), dq, ds, db, None, sinds[:2048].contiguous(), True, 64, 4, sorted_indices=True)
    assert torch.equal(y_l.view(torch.int16), y_r.view(torch.int16))


def test_non_finite_activations_reach_the_output():
    """An Inf or a NaN activation must not come out as a finite number: every output that depends on the group
    holding it is non-finite, other tokens are untouched (MLX's quantized_matmul propagates them likewise)."""
    import qb200
    rng = np.random.default_rng(404)
    q, s, b = make_weight(rng, (512, 1024), 64, 4)
    dq, ds, db = dev_triple(q, s, b)
    for M in (1, 8, 20):
        x = rand_bf16(rng, (M, 1024))
        clean = qb200.quantized_matmul(to_dev_bf16(qo.f32_to_bf16(x)), dq, ds, db, True, 64, 4).float().cpu().numpy()
        x[0, 100] = np.inf
        if M > 1:
            x[M - 1, 700] = np.nan
        for dev_x in (to_dev_bf16(qo.f32_to_bf16(x)), torch.from_numpy(x).cuda()):
            y = qb200.quantized_matmul(dev_x, dq, ds, db, True, 64, 4).float().cpu().numpy()
            assert not np.isfinite(y[0]).any()
            if M > 1:
                assert not np.isfinite(y[M - 1]).any()
            if M > 2:
                assert np.isfinite(y[1:M - 1]).all()
        if M > 2:
            y16 = qb200.quantized_matmul(to_dev_bf16(qo.f32_to_bf16(x)), dq, ds, db, True, 64, 4).float().cpu().numpy()
            assert np.array_equal(y16[1:M - 1], clean[1:M - 1])
    # gather form
    E = 4
    bq, bs, bb = make_weight(rng, (E, 256, 512), 64, 4)
    inds = np.sort(rng.integers(0, E, 40)).astype(np.int32)
    xr = rand_bf16(rng, (40, 1, 512))
    xr[7, 0, 3] = np.nan
    y = qb200.gather_qmm(to_dev_bf16(qo.f32_to_bf16(xr)), *dev_triple(bq, bs, bb), None, torch.from_numpy(inds).cuda(), True, 64, 4,
                         sorted_indices=True).float().cpu().numpy()
    assert not np.isfinite(y[7]).any() and np.isfinite(np.delete(y, 7, axis=0)).all()


@pytest.mark.parametrize("T,bits,gs", [(64, 4, 64), (1, 4, 64), (5, 8, 64), (33, 4, 128)])
def test_fused_gate_up_swiglu_matches_the_unfused_chain(T, bits, gs):
    """qb200_gather_qmm_swiglu against (a) the library's own two gather_qmm results pushed through the oracle's
    SwiGLU restatement -- bit for bit, since the fused kernel forms the same fp32 sums -- and (b) the full oracle
    chain within the matmul gate.  T=1 takes the form in which several warps share a tile's K range."""
    import qb200
    E, H, I, k = 128, 2048, 768, 8
    rng = np.random.default_rng(0xF1 + T + bits)
    qg, sg, bg = make_weight(rng, (E, I, H), gs, bits)
    qu, su, bu = make_weight(rng, (E, I, H), gs, bits)
    dg, du = dev_triple(qg, sg, bg), dev_triple(qu, su, bu)
    flat = _route(rng, T, E, k).reshape(-1)
    order = np.argsort(flat, kind="stable")
    sorted_inds = flat[order]
    x = rand_bf16(rng, (T, H))
    x_rep = x[order // k].reshape(T * k, 1, H)
    idx = torch.from_numpy(sorted_inds).cuda()
    x16 = to_dev_bf16(qo.f32_to_bf16(x_rep))
    g16 = qb200.gather_qmm(x16, *dg, None, idx, True, gs, bits, sorted_indices=True)
    u16 = qb200.gather_qmm(x16, *du, None, idx, True, gs, bits, sorted_indices=True)
    want = qo.swiglu_bf16(g16.float().cpu().numpy(), u16.float().cpu().numpy())
    y16 = qb200.gather_qmm_swiglu(x16, *dg, *du, None, idx, gs, bits, sorted_indices=True)
    assert y16.dtype == torch.bfloat16 and tuple(y16.shape) == (T * k, 1, I)
    got = y16.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} elements differ from the unfused chain"
    # full oracle chain (fp32 activations): tolerance of the matmul gate on the product
    rg = qo.gather_qmm(x_rep, qg, sg, bg, np.arange(T * k), sorted_inds, gs, bits)
    ru = qo.gather_qmm(x_rep, qu, su, bu, np.arange(T * k), sorted_inds, gs, bits)
    ref = qo.swiglu_f32(rg, ru)
    y32 = qb200.gather_qmm_swiglu(torch.from_numpy(x_rep).cuda(), *dg, *du, None, idx, gs, bits, sorted_indices=True)
    gate_f32(y32.cpu().numpy(), ref, "fused fp32")
    # bf16 form against the fp32 chain: four bf16 roundings (gate, sigmoid, two products), 2^-9 relative each
    d = np.abs(y16.float().cpu().numpy().astype(np.float64) - ref)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    assert (d <= 2.0 ** -6 * np.abs(ref) + 1e-2 * rms).all()


def test_fused_gate_up_swiglu_decode_shape_and_declined_shapes():
    """The stock decode shape (x [B,S,1,1,D] broadcast against rhs [B,S,K], src/transformer.zig:15091-15119) and a
    shape the fused kernel declines (the caller keeps the unfused chain)."""
    import qb200
    E, H, I, k = 16, 1024, 512, 4
    rng = np.random.default_rng(0xF2)
    qg, sg, bg = make_weight(rng, (E, I, H), 64, 4)
    qu, su, bu = make_weight(rng, (E, I, H), 64, 4)
    dg, du = dev_triple(qg, sg, bg), dev_triple(qu, su, bu)
    inds = _route(rng, 3, E, k).reshape(1, 3, k)
    x = rand_bf16(rng, (1, 3, 1, 1, H))
    idx = torch.from_numpy(inds).cuda()
    x16 = to_dev_bf16(qo.f32_to_bf16(x))
    g16 = qb200.gather_qmm(x16, *dg, None, idx, True, 64, 4)
    u16 = qb200.gather_qmm(x16, *du, None, idx, True, 64, 4)
    want = qo.swiglu_bf16(g16.float().cpu().numpy(), u16.float().cpu().numpy())
    y16 = qb200.gather_qmm_swiglu(x16, *dg, *du, None, idx, 64, 4)
    assert tuple(y16.shape) == (1, 3, k, 1, I)
    assert np.array_equal(y16.view(torch.int16).cpu().numpy().view(np.uint16), want)
    # K = 320 is not a multiple of 256: declined, nothing written
    q2, s2, b2 = make_weight(rng, (4, 32, 320), 64, 4)
    d2 = dev_triple(q2, s2, b2)
    x2 = to_dev_bf16(qo.f32_to_bf16(rand_bf16(rng, (2, 1, 320))))
    with pytest.raises(qb200.Qb200Error) as ei:
        qb200.gather_qmm_swiglu(x2, *d2, *d2, None, torch.tensor([0, 3], dtype=torch.int32).cuda(), 64, 4)
    assert ei.value.status == 1


@pytest.mark.parametrize("T,k,H", [(64, 8, 2048), (1, 8, 2048), (7, 2, 264)])
def test_moe_weighted_sum_bit_exact(T, k, H):
    """qb200_moe_weighted_sum against the oracle restatement: bit-exact in both dtypes, with and without inv_order."""
    import qb200
    rng = np.random.default_rng(T * 31 + k + H)
    y = qo.bf16_round(rng.standard_normal((T * k, 1, H)).astype(np.float32))
    sc = qo.bf16_round(rng.random((T, k)).astype(np.float32))
    inv = rng.permutation(T * k).astype(np.int32)
    for use_inv in (True, False):
        want16 = qo.f32_to_bf16(qo.moe_weighted_sum(y.reshape(T * k, H), sc, inv if use_inv else None, as_bf16=True))
        got16 = qb200.moe_weighted_sum(to_dev_bf16(qo.f32_to_bf16(y)), to_dev_bf16(qo.f32_to_bf16(sc)),
                                       torch.from_numpy(inv).cuda() if use_inv else None)
        assert tuple(got16.shape) == (T, H)
        assert np.array_equal(got16.view(torch.int16).cpu().numpy().view(np.uint16), want16)
        want32 = qo.moe_weighted_sum(y.reshape(T * k, H), sc, inv if use_inv else None, as_bf16=False)
        got32 = qb200.moe_weighted_sum(torch.from_numpy(y).cuda(), torch.from_numpy(sc).cuda(),
                                       torch.from_numpy(inv.astype(np.int64)).cuda() if use_inv else None)
        assert np.array_equal(got32.cpu().numpy(), want32)


def test_moe_block_fused_path_end_to_end():
    """The routed-expert block of moeMLP2 (src/transformer.zig:14961-15043, :15127-15140) through the fused entries:
    sort by expert, gate/up + SwiGLU, down, rows back to token order times the scores; against the oracle chain."""
    import qb200
    E, H, I, T, k = 32, 1024, 512, 16, 4
    rng = np.random.default_rng(0xB10C)
    banks = {n: make_weight(rng, (E, I, H) if n != "down" else (E, H, I), 64, 4) for n in ("gate", "up", "down")}
    dev = {n: dev_triple(*banks[n]) for n in banks}
    inds = _route(rng, T, E, k)
    flat = inds.reshape(-1)
    order = np.argsort(flat, kind="stable")
    inv = np.argsort(order, kind="stable").astype(np.int32)
    sorted_inds = flat[order]
    scores = qo.bf16_round(rng.random((T, k)).astype(np.float32))
    scores = qo.bf16_round(scores / scores.sum(-1, keepdims=True))
    x = rand_bf16(rng, (T, H))
    x_rep = x[order // k].reshape(T * k, 1, H)
    # oracle chain with the same rounding points
    g = qo.gather_qmm(x_rep, *banks["gate"], np.arange(T * k), sorted_inds, 64, 4)
    u = qo.gather_qmm(x_rep, *banks["up"], np.arange(T * k), sorted_inds, 64, 4)
    act = qo.bf16_to_f32(qo.swiglu_bf16(g, u))
    d = qo.bf16_round(qo.gather_qmm(act.reshape(T * k, 1, I), *banks["down"], np.arange(T * k), sorted_inds, 64, 4))
    ref = qo.moe_weighted_sum(d.reshape(T * k, H), scores, inv, as_bf16=True)
    idx = torch.from_numpy(sorted_inds).cuda()
    a16 = qb200.gather_qmm_swiglu(to_dev_bf16(qo.f32_to_bf16(x_rep)), *dev["gate"], *dev["up"], None, idx, 64, 4,
                                  sorted_indices=True)
    d16 = qb200.gather_qmm(a16, *dev["down"], None, idx, True, 64, 4, sorted_indices=True)
    out = qb200.moe_weighted_sum(d16, to_dev_bf16(qo.f32_to_bf16(scores)), torch.from_numpy(inv).cuda())
    got = out.float().cpu().numpy()
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    # bf16 roundings of the intermediate tensors can flip by one ulp where the oracle's and the kernels' fp32 sums
    # differ in their last bits; the block's result stays within a few bf16 ulps
    assert np.abs(got - ref).max() <= 2.0 ** -6 * np.abs(ref).max() + 1e-2 * rms


def test_fused_gate_up_swiglu_long_k_explicit_lhs():
    """K = 4096 (one expert segment staged at a time), explicit lhs_indices into a shared activation batch, unsorted
    experts, an out-of-range expert id (its row is left untouched)."""
    import qb200
    E, H, I = 8, 4096, 72
    rng = np.random.default_rng(0xF3)
    qg, sg, bg = make_weight(rng, (E, I, H), 64, 4)
    qu, su, bu = make_weight(rng, (E, I, H), 64, 4)
    dg, du = dev_triple(qg, sg, bg), dev_triple(qu, su, bu)
    x = rand_bf16(rng, (5, 1, H))
    lhs = np.array([4, 0, 0, 3, 1, 2, 2, 4, 1], np.int32)
    rhs = np.array([7, 2, 5, 2, 0, 7, 9, 1, 3], np.int32)   # 9 is out of range
    x16 = to_dev_bf16(qo.f32_to_bf16(x))
    li, ri = torch.from_numpy(lhs).cuda(), torch.from_numpy(rhs).cuda()
    g16 = torch.full((9, 1, I), 3.0, dtype=torch.bfloat16, device="cuda")
    u16 = g16.clone()
    y16 = g16.clone()
    qb200.gather_qmm(x16, *dg, li, ri, True, 64, 4, out=g16)
    qb200.gather_qmm(x16, *du, li, ri, True, 64, 4, out=u16)
    qb200.gather_qmm_swiglu(x16, *dg, *du, li, ri, 64, 4, out=y16)
    want = qo.swiglu_bf16(g16.float().cpu().numpy(), u16.float().cpu().numpy())
    got = y16.view(torch.int16).cpu().numpy().view(np.uint16)
    keep = rhs < E
    assert np.array_equal(got[keep], want[keep])
    assert (y16[6].float() == 3.0).all()


@pytest.mark.parametrize("T,E,k", [(64, 128, 8), (1, 128, 8), (5, 1024, 6), (3, 40, 4)])
def test_moe_route_matches_the_oracle(T, E, k):
    """qb200_moe_route: the indices exactly (logits with ties included), the scores within one rounding step of the
    logits' dtype (the kernel's expf and sum order differ from the oracle's in the last fp32 bits)."""
    import qb200
    rng = np.random.default_rng(T + E + k)
    lg = qo.bf16_round(rng.standard_normal((T, E)).astype(np.float32) * 2)
    lg[0, 3] = lg[0, E - 1] = lg[0].max() + 1      # a tie at the top
    inds_ref, sc_ref = qo.moe_route(lg, k, as_bf16=True)
    inds, sc = qb200.moe_route(to_dev_bf16(qo.f32_to_bf16(lg)), k)
    assert inds.dtype == torch.int32 and tuple(inds.shape) == (T, k) and sc.dtype == torch.bfloat16
    assert np.array_equal(inds.cpu().numpy(), inds_ref)
    got = sc.float().cpu().numpy()
    assert np.abs(got - sc_ref).max() <= 2.0 ** -7 * np.abs(sc_ref).max()
    assert (got != sc_ref).mean() < 0.05
    i32, s32 = qb200.moe_route(torch.from_numpy(lg).cuda(), k)
    ir, sr = qo.moe_route(lg, k, as_bf16=False)
    assert np.array_equal(i32.cpu().numpy(), ir)
    assert np.allclose(s32.cpu().numpy(), sr, rtol=2e-6, atol=1e-9)
    assert np.allclose(s32.cpu().numpy().sum(-1), 1.0, atol=1e-5)


@pytest.mark.parametrize("T,bits,gs,H,I", [(1, 4, 64, 2048, 768), (3, 8, 64, 512, 512), (2, 4, 128, 1000, 1024)])
def test_moe_down_reduce_matches_the_unfused_tail(T, bits, gs, H, I):
    """qb200_moe_down_reduce (the reference's gatherQmvDownReduce, src/transformer.zig:20559-20623) against the
    library's own gather_qmm + moe_weighted_sum (same rounding points; the dot products may differ in their last fp32
    bits where the unfused kernel splits K over warps) and against the oracle chain."""
    import qb200
    E, k = 32, 8
    rng = np.random.default_rng(0xD0 + T + bits + H)
    q, s, b = make_weight(rng, (E, H, I), gs, bits)
    dw = dev_triple(q, s, b)
    inds = _route(rng, T, E, k)
    inds[0, 2] = E + 3 if T > 1 else inds[0, 2]          # an out-of-range expert contributes nothing
    scores = qo.bf16_round(rng.random((T, k)).astype(np.float32))
    act = rand_bf16(rng, (T, k, I))
    a16 = to_dev_bf16(qo.f32_to_bf16(act))
    s16 = to_dev_bf16(qo.f32_to_bf16(scores))
    idx = torch.from_numpy(inds).cuda()
    got = qb200.moe_down_reduce(a16, *dw, idx, s16, gs, bits)
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == (T, H)
    # the unfused tail on the GPU (rows of out-of-range experts are left untouched by gather_qmm: start from zeros)
    d16 = torch.zeros((T * k, 1, H), dtype=torch.bfloat16, device="cuda")
    qb200.gather_qmm(a16.view(T * k, 1, I), *dw, None, idx.view(-1), True, gs, bits, out=d16)
    want = qb200.moe_weighted_sum(d16, s16, None).float().cpu().numpy()
    g = got.float().cpu().numpy()
    assert (g != want).mean() < 0.02
    assert np.abs(g - want).max() <= 2.0 ** -6 * np.abs(want).max()
    # oracle chain
    keep = (inds.reshape(-1) < E)
    rows = qo.gather_qmm(act.reshape(T * k, 1, I), q, s, b, np.arange(T * k), np.where(keep, inds.reshape(-1), 0), gs, bits)
    rows = qo.bf16_round(rows.reshape(T * k, H)) * keep[:, None]
    ref = qo.moe_weighted_sum(rows, scores, None, as_bf16=True)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    assert np.abs(g - ref).max() <= 2.0 ** -6 * np.abs(ref).max() + 1e-2 * rms
    # fp32 form
    g32 = qb200.moe_down_reduce(torch.from_numpy(act).cuda(), *dw, idx, torch.from_numpy(scores).cuda(), gs, bits)
    rows32 = qo.gather_qmm(act.reshape(T * k, 1, I), q, s, b, np.arange(T * k), np.where(keep, inds.reshape(-1), 0), gs, bits)
    ref32 = qo.moe_weighted_sum(rows32.reshape(T * k, H) * keep[:, None], scores, None, as_bf16=False)
    gate_f32(g32.cpu().numpy(), ref32, "down+reduce fp32")


def test_moe_down_reduce_declines_wide_batches():
    import qb200
    rng = np.random.default_rng(3)
    q, s, b = make_weight(rng, (4, 64, 256), 64, 4)
    dw = dev_triple(q, s, b)
    act = to_dev_bf16(qo.f32_to_bf16(rand_bf16(rng, (8, 2, 256))))
    sc = to_dev_bf16(qo.f32_to_bf16(rand_bf16(rng, (8, 2))))
    with pytest.raises(qb200.Qb200Error) as ei:
        qb200.moe_down_reduce(act, *dw, torch.zeros((8, 2), dtype=torch.int32, device="cuda"), sc, 64, 4)
    assert ei.value.status == 1

"""The CPU oracle must reproduce, bit for bit, the golden vectors produced by the
reference's own numpy restatement of MLX's affine quantization
(tests/golden/make_golden.py imports tests/dsv4_imatrix.py of the mlx-serve tree).
"""
import os

import numpy as np
import pytest

from oracle import qoracle as qo

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_affine.npz"))
QUANT_KEYS = sorted({k.split("/")[0] for k in G.files if k.startswith("quant_")})
DEQ_KEYS = sorted({k.split("/")[0] for k in G.files if k.startswith("deq_rand_")})


def _parse(key):
    bits = int(key.split("_b")[-1].split("_")[0])
    gs = int(key.split("_g")[-1])
    return bits, gs


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_pack_layout(bits):
    q, packed = G[f"pack_b{bits}/q"], G[f"pack_b{bits}/packed"]
    assert np.array_equal(qo.pack(q, bits), packed)
    assert np.array_equal(qo.unpack(packed, bits), q)


def test_bf16_rounding():
    f, u = G["bf16/f32"], G["bf16/u16"]
    assert np.array_equal(qo.f32_to_bf16(f), u)
    assert np.array_equal(qo.bf16_to_f32(u).view(np.uint32), u.astype(np.uint32) << 16)


@pytest.mark.parametrize("key", QUANT_KEYS)
def test_quantize_matches_reference(key):
    bits, gs = _parse(key)
    name = key[len("quant_"):key.rindex("_b")]
    x = G[f"x_{name}"]
    q, s, b = qo.quantize(x, gs, bits)
    assert np.array_equal(q, G[key + "/packed"]), "codes"
    assert np.array_equal(s, G[key + "/scales"]), "scales"
    assert np.array_equal(b, G[key + "/biases"]), "biases"


@pytest.mark.parametrize("key", QUANT_KEYS + DEQ_KEYS)
def test_dequantize_matches_reference(key):
    bits, gs = _parse(key)
    w, s, b = G[key + "/packed"], G[key + "/scales"], G[key + "/biases"]
    f = qo.dequantize(w, s, b, gs, bits)
    assert not np.isnan(f).any()
    assert np.array_equal(f.view(np.uint32), G[key + "/deq_f32"].view(np.uint32))
    h = qo.dequantize(w, s, b, gs, bits, out_bf16=True)
    assert np.array_equal(h, G[key + "/deq_bf16"])


def test_round_trip_bounds_of_reference_tests():
    """src/kv_quant.zig:743-805: smooth ramp, D=256, gs=64: max err < 0.05 (4-bit), < 0.01 (8-bit)."""
    x = G["x_smooth_ramp"]
    for bits, bound in ((4, 0.05), (8, 0.01)):
        q, s, b = qo.quantize(x, 64, bits)
        assert q.shape[-1] == 256 * bits // 32 and s.shape[-1] == 4
        back = qo.bf16_to_f32(qo.dequantize(q, s, b, 64, bits, out_bf16=True))
        assert not np.isnan(back).any()
        assert np.abs(back - x).max() < bound


def _dense_ref(x, w, s, b, gs, bits, transpose):
    wd = qo.dequantize(w, s, b, gs, bits).astype(np.float64)
    return x.astype(np.float64) @ (wd.T if transpose else wd)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("transpose", [True, False])
def test_qmm_vs_dense_float64(bits, transpose):
    rng = np.random.default_rng(5)
    K, N, M = 256, 192, 5
    wf = qo.bf16_round(rng.standard_normal((N, K) if transpose else (K, N)).astype(np.float32) * 0.02)
    w, s, b = qo.quantize(wf, 64, bits)
    x = qo.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    y = qo.qmm(x, w, s, b, 64, bits, transpose)
    ref = _dense_ref(x, w, s, b, 64, bits, transpose)
    assert not np.isnan(y).any()
    assert np.abs(y - ref).max() <= 1e-5 * np.sqrt((ref ** 2).mean()) + 1e-6


def test_qmm_reference_4d_cases():
    """src/kv_quant.zig:968-1094: [1,2,3,64] x [1,2,5,64]^T and [1,2,3,5] x [1,2,5,64]."""
    wf = G["x_smooth_bhtd"][:, :64].reshape(1, 2, 5, 64)
    w, s, b = qo.quantize(wf, 64, 4)
    tot = 1 * 2 * 3 * 64
    bb, hh, tt, dd = np.meshgrid(np.arange(1), np.arange(2), np.arange(3), np.arange(64), indexing="ij")
    x = qo.bf16_round(((bb * 17 + hh * 5 + tt * 3 + dd).astype(np.float32) / np.float32(tot)) * 2 - 1)
    y = qo.qmm_batched(x, w, s, b, 64, 4, True)
    assert y.shape == (1, 2, 3, 5)
    wd = qo.bf16_to_f32(qo.dequantize(w, s, b, 64, 4, out_bf16=True))
    ref = np.einsum("bhtd,bhkd->bhtk", x, wd)
    assert np.abs(y - ref).max() / np.abs(ref).max() < 0.02
    tot = 1 * 2 * 3 * 5
    bb, hh, tt, dd = np.meshgrid(np.arange(1), np.arange(2), np.arange(3), np.arange(5), indexing="ij")
    x2 = qo.bf16_round(((bb * 17 + hh * 5 + tt * 3 + dd).astype(np.float32) / np.float32(tot)) * 2 - 1)
    y2 = qo.qmm_batched(x2, w, s, b, 64, 4, False)
    assert y2.shape == (1, 2, 3, 64)
    assert np.abs(y2 - np.einsum("bhtk,bhkd->bhtd", x2, wd)).max() < 0.05


def test_gather_qmm_reference_cases():
    """src/transformer.zig:24643-24835: E=4, IN=32, OUT=8, gs=32, 8-bit; decode inds [1,3], sorted [0,0,1,2,3]."""
    E, IN, OUT = 4, 32, 8
    wh = ((np.arange(E * OUT * IN) % 13).astype(np.float32) - 6) * np.float32(0.05)
    wf = qo.bf16_round(wh.reshape(E, OUT, IN))
    w, s, b = qo.quantize(wf, 32, 8)
    wd = qo.bf16_to_f32(qo.dequantize(w, s, b, 32, 8, out_bf16=True))
    x = qo.bf16_round((((np.arange(IN) % 5).astype(np.float32)) - 2) * np.float32(0.1)).reshape(1, 1, IN)
    inds = np.array([1, 3])
    y = qo.gather_qmm(x, w, s, b, np.zeros(2, np.int64), inds, 32, 8)
    gt = np.stack([wd[e] @ x[0, 0] for e in inds])
    assert np.abs(y[:, 0, :] - gt).max() < 2e-2
    N = 5
    xs = qo.bf16_round((((np.arange(N * IN) % 7).astype(np.float32)) - 3) * np.float32(0.07)).reshape(N, 1, IN)
    srt = np.array([0, 0, 1, 2, 3])
    y = qo.gather_qmm(xs, w, s, b, np.arange(N), srt, 32, 8)
    gt = np.stack([wd[e] @ xs[i, 0] for i, e in enumerate(srt)])
    assert np.abs(y[:, 0, :] - gt).max() < 2e-2


@pytest.mark.parametrize("bits", [4, 8])
def test_kv_decode_attention_vs_dense_float64(bits):
    """Composed definition of src/kv_quant.zig:478-687 with Tq=1, GQA 4:1, strided views, ragged lens."""
    rng = np.random.default_rng(9)
    B, Hq, Hkv, T, D, cap = 3, 8, 2, 77, 128, 256
    kf = qo.bf16_round(rng.standard_normal((B, Hkv, cap, D)).astype(np.float32))
    vf = qo.bf16_round(rng.standard_normal((B, Hkv, cap, D)).astype(np.float32))
    kq, ks, kb = qo.quantize(kf, 64, bits)
    vq, vs, vb = qo.quantize(vf, 64, bits)
    views = [a[:, :, :T, :] for a in (kq, ks, kb, vq, vs, vb)]
    q = qo.bf16_round(rng.standard_normal((B, Hq, D)).astype(np.float32))
    lens = np.array([T, 40, 1], np.int32)
    scale = 1.0 / np.sqrt(D)
    out = qo.kv_decode_attention(q, *views, 64, bits, scale, kv_lens=lens)
    assert not np.isnan(out).any()
    kd = qo.dequantize(kq, ks, kb, 64, bits).astype(np.float64)[:, :, :T]
    vd = qo.dequantize(vq, vs, vb, 64, bits).astype(np.float64)[:, :, :T]
    for bi in range(B):
        for h in range(Hq):
            L = lens[bi]
            sc = (kd[bi, h // 4, :L] @ q[bi, h].astype(np.float64)) * scale
            p = np.exp(sc - sc.max())
            ref = (p / p.sum()) @ vd[bi, h // 4, :L]
            assert np.abs(out[bi, h] - ref).max() < 1e-4


def test_swiglu_restatement_rounding_points():
    """bf16 form: sigmoid, g*sig and act*up are each rounded to bf16 (src/transformer.zig:19842-19851); checked
    against numpy in float64 with the same rounding points."""
    rng = np.random.default_rng(5)
    g = rng.standard_normal(4096).astype(np.float32) * 3
    u = rng.standard_normal(4096).astype(np.float32)
    got = qo.bf16_to_f32(qo.swiglu_bf16(g, u))
    g16, u16 = qo.bf16_round(g), qo.bf16_round(u)
    sig = qo.bf16_round((1.0 / (1.0 + np.exp(-g16.astype(np.float64)))).astype(np.float32))
    act = qo.bf16_round(g16 * sig)
    want = qo.bf16_round(act * u16)
    assert (got != want).mean() < 1e-3            # float64 vs fp32 exp may flip a rounding at a tie
    assert np.abs(got - want).max() <= np.abs(want).max() * 2.0 ** -7
    f = qo.swiglu_f32(g, u)
    assert np.allclose(f, g / (1 + np.exp(-g.astype(np.float64))) * u, rtol=1e-5, atol=1e-7)
    assert qo.bf16_to_f32(qo.swiglu_bf16(np.zeros(4, np.float32), np.ones(4, np.float32))).tolist() == [0.0] * 4


def test_moe_weighted_sum_restatement():
    """Inverse permutation + score-weighted sum over top-k against plain numpy (fp32 form) and with bf16 rounding
    of every product and of the running sum (bf16 form)."""
    rng = np.random.default_rng(6)
    T, k, H = 5, 4, 16
    y = qo.bf16_round(rng.standard_normal((T * k, H)).astype(np.float32))
    sc = qo.bf16_round(rng.random((T, k)).astype(np.float32))
    inv = rng.permutation(T * k).astype(np.int64)
    f = qo.moe_weighted_sum(y, sc, inv, as_bf16=False)
    want = np.zeros((T, H), np.float32)
    for j in range(k):   # same order of additions
        want = want + y[inv.reshape(T, k)[:, j]] * sc[:, j:j + 1]
    assert np.array_equal(f, want)
    b = qo.moe_weighted_sum(y, sc, inv, as_bf16=True)
    wb = np.zeros((T, H), np.float32)
    for j in range(k):   # bf16 accumulator: rounded after every add (src/transformer.zig:20566-20571)
        wb = qo.bf16_round(wb + qo.bf16_round(y[inv.reshape(T, k)[:, j]] * sc[:, j:j + 1]))
    assert np.array_equal(b, wb)
    assert np.array_equal(qo.moe_weighted_sum(y, sc, None, as_bf16=False), qo.moe_weighted_sum(y, sc, np.arange(T * k), as_bf16=False))


def test_moe_route_restatement():
    """Router: top-k by logit (ties by lower index), softmax, renormalised scores; against numpy."""
    rng = np.random.default_rng(7)
    T, E, k = 9, 128, 8
    lg = qo.bf16_round(rng.standard_normal((T, E)).astype(np.float32))
    lg[0, 5] = lg[0, 77] = 9.0            # a tie at the top: lower index first
    inds, sc = qo.moe_route(lg, k, as_bf16=False)
    assert inds[0, 0] == 5 and inds[0, 1] == 77
    p = np.exp(lg.astype(np.float64) - lg.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-lg[t, e], e))[:k]
        assert inds[t].tolist() == order
        w = p[t, order]
        assert np.allclose(sc[t], w / w.sum(), rtol=1e-5)
    _, sb = qo.moe_route(lg, k, as_bf16=True)
    assert np.array_equal(sb, qo.bf16_round(sb)) and np.abs(sb - sc).max() < 2.0 ** -8

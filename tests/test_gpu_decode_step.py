"""GPU parity of the small operators of the batched decode step (forwardBatchedDecode, src/transformer.zig:9562-9924)
and of a whole layer tick composed from the library's entries, against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import qoracle as qo
from util import bf16_ulp, dev_triple, from_dev_bf16, from_dev_u32, gate_bf16, make_weight, rand_bf16, record, to_dev_bf16

pytestmark = pytest.mark.gpu


def _dev(a):
    return to_dev_bf16(qo.f32_to_bf16(a))


def _within_one_ulp(got, ref, what, allow_frac=0.0, steps=1.0):
    """bf16 outputs of transcendental / reduced quantities: exact up to `steps` bf16 rounding steps of the reference where
    the last fp32 bits of rsqrt / sin / cos differ between device and host (the norm rounds twice: a flipped inner
    rounding times a weight above 2 moves the result by more than one step); `allow_frac` of the outputs may differ at all."""
    d = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    assert (d <= steps * bf16_ulp(ref) * (1 + 1e-6) + 1e-30).all(), f"{what}: more than {steps} rounding steps off"
    frac = float((d > 0).mean())
    assert frac <= allow_frac, f"{what}: {frac:.4f} of the outputs differ"
    return frac


@pytest.mark.parametrize("rows,d", [(8, 4096), (1, 4096), (32, 14336), (5, 128), (3, 2050)])
def test_rms_norm_and_fused_add(rows, d):
    import qb200
    rng = np.random.default_rng(rows + d)
    x, r, w = rand_bf16(rng, (rows, d)), rand_bf16(rng, (rows, d), 0.5), rand_bf16(rng, (d,), 1.0) + 1.0
    w = qo.bf16_round(w.astype(np.float32))
    y = qb200.rms_norm(_dev(x), _dev(w), 1e-5).float().cpu().numpy()
    _within_one_ulp(y, qo.rms_norm(x, w, 1e-5), "rms_norm", allow_frac=5e-3, steps=4.0)
    s, n = qb200.add_rms_norm(_dev(x), _dev(r), _dev(w), 1e-5)
    h = qo.bf16_round(x + r)
    assert np.array_equal(s.float().cpu().numpy(), h), "the residual sum is one exact rounding"
    _within_one_ulp(n.float().cpu().numpy(), qo.rms_norm(h, w, 1e-5), "add + rms_norm", allow_frac=5e-3, steps=4.0)
    s2, none = qb200.add_rms_norm(_dev(x), _dev(r), want_norm=False)
    assert none is None and np.array_equal(s2.float().cpu().numpy(), h)


@pytest.mark.parametrize("n,heads,d,dims,base", [(8, 40, 128, 128, 500000.0), (3, 8, 64, 32, 10000.0), (1, 32, 128, 128, 10000.0)])
def test_rope_with_one_position_per_sequence(n, heads, d, dims, base):
    import qb200
    rng = np.random.default_rng(n + heads)
    x = rand_bf16(rng, (n, heads, d))
    offs = rng.integers(0, 40000, n).astype(np.int32)
    offs[0] = 0
    if n > 1:
        offs[-1] = 37
    ref = qo.rope(x, dims, base, 1.0, offs)
    assert np.array_equal(ref[0], x[0]), "position 0 is the identity"
    dx = _dev(x).view(n, heads, 1, d)
    y = qb200.rope(dx, dims, base, 1.0, torch.from_numpy(offs).cuda()).float().cpu().numpy().reshape(n, heads, d)
    # The angle position * base^(-2i/dims) is an fp32 product: at positions of tens of thousands one last-bit difference
    # between the device's and the host's exp2 moves it by ~2e-3 rad, i.e. the rotated pair by ~2e-3 of its length.
    half = dims // 2
    mag = np.zeros_like(x)
    mag[..., :half] = mag[..., half:dims] = np.hypot(x[..., :half], x[..., half:dims])
    diff = np.abs(y.astype(np.float64) - ref)
    assert (diff <= bf16_ulp(ref) * (1 + 1e-6) + 5e-3 * mag).all(), "rope: beyond one rounding step + 5e-3 of the pair's length"
    assert np.array_equal(y[..., dims:], x[..., dims:]), "elements beyond dims pass through"
    small = offs < 64                                    # small angles: at most one rounding step
    if small.any():
        _within_one_ulp(y[small], ref[small], "rope at small positions", allow_frac=0.02)
    # in place over a strided view: the q and k heads of a wider fused-projection buffer
    wide = torch.zeros((n, heads + 3, d), dtype=torch.bfloat16, device="cuda")
    wide[:, :heads] = dx.view(n, heads, d)
    view = wide[:, :heads].unsqueeze(2)
    qb200.rope(view, dims, base, 1.0, torch.from_numpy(offs).cuda(), out=view)
    assert torch.equal(wide[:, :heads].float().cpu(), torch.from_numpy(y)) and float(wide[:, heads:].abs().sum()) == 0.0


def test_dense_swiglu_is_bit_exact():
    import qb200
    rng = np.random.default_rng(9)
    g, u = rand_bf16(rng, (8, 14336), 2.0), rand_bf16(rng, (8, 14336))
    y = qb200.swiglu(_dev(g), _dev(u))
    assert np.array_equal(from_dev_bf16(y), qo.swiglu_bf16(g, u))


@pytest.mark.parametrize("bits", [4, 8])
def test_kv_append_into_per_sequence_caches(bits):
    """Eight caches of different capacity and fill: the new token's triples land at each cache's own offset, bit for bit
    the oracle's quantize, and nothing else in the buffers changes."""
    import qb200
    rng = np.random.default_rng(bits)
    N, Hkv, D = 8, 8, 128
    k, v = rand_bf16(rng, (N, Hkv, 1, D)), rand_bf16(rng, (N, Hkv, 1, D))
    caps = [256 * int(c) for c in rng.integers(1, 4, N)]
    offs = [int(rng.integers(0, c)) for c in caps]
    offs[0], offs[1] = 0, caps[1] - 1
    kt, vt = [], []
    for n in range(N):
        mk = lambda last, dt: torch.full((1, Hkv, caps[n], last), 7, dtype=dt, device="cuda")
        kt.append([mk(D * bits // 32, torch.int32), mk(D // 64, torch.bfloat16), mk(D // 64, torch.bfloat16)])
        vt.append([mk(D * bits // 32, torch.int32), mk(D // 64, torch.bfloat16), mk(D // 64, torch.bfloat16)])
    qb200.kv_append_seqs(kt, vt, _dev(k), _dev(v), offs, bits, 64)
    torch.cuda.synchronize()
    for dense, triples in ((k, kt), (v, vt)):
        q, s, b = qo.quantize(dense, 64, bits)
        for n in range(N):
            assert np.array_equal(from_dev_u32(triples[n][0][0, :, offs[n]]), q[n, :, 0])
            assert np.array_equal(from_dev_bf16(triples[n][1][0, :, offs[n]]), s[n, :, 0])
            assert np.array_equal(from_dev_bf16(triples[n][2][0, :, offs[n]]), b[n, :, 0])
            untouched = triples[n][0].clone()
            untouched[0, :, offs[n]] = 7
            assert bool((untouched == 7).all())

@pytest.mark.parametrize("bits,D,dims", [(4, 128, 128), (8, 128, 128), (4, 128, 64), (8, 64, 64)])
def test_rope_fused_into_the_cache_update_equals_the_two_calls(bits, D, dims):
    """qb200_rope_kv_append_seqs: the queries rotated in place and the keys on their way into the cache, one launch --
    bit for bit what qb200_rope on q and k followed by qb200_kv_append_seqs writes (the dense k stays as it was)."""
    import qb200
    rng = np.random.default_rng(bits + D + dims)
    N, Hq, Hkv = 6, 8, 2
    qkv = _dev(rand_bf16(rng, (N, Hq + 2 * Hkv, D)))          # one fused-projection buffer, as the decode step has it
    q4, k4, v4 = qkv[:, :Hq].unsqueeze(2), qkv[:, Hq:Hq + Hkv].unsqueeze(2), qkv[:, Hq + Hkv:].unsqueeze(2)
    caps = [256 * int(c) for c in rng.integers(1, 3, N)]
    offs = [int(rng.integers(0, c)) for c in caps]
    offs[0], offs[1] = 0, caps[1] - 1

    def fresh():
        kt, vt = [], []
        for n in range(N):
            mk = lambda last, dt: torch.full((1, Hkv, caps[n], last), 7, dtype=dt, device="cuda")
            kt.append([mk(D * bits // 32, torch.int32), mk(D // 64, torch.bfloat16), mk(D // 64, torch.bfloat16)])
            vt.append([mk(D * bits // 32, torch.int32), mk(D // 64, torch.bfloat16), mk(D // 64, torch.bfloat16)])
        return kt, vt
    # the two calls
    two = qkv.clone()
    tq, tk, tv = two[:, :Hq].unsqueeze(2), two[:, Hq:Hq + Hkv].unsqueeze(2), two[:, Hq + Hkv:].unsqueeze(2)
    pos = torch.tensor(offs, dtype=torch.int32, device="cuda")
    qk = two[:, :Hq + Hkv].unsqueeze(2)
    qb200.rope(qk, dims, 500000.0, 1.0, pos, out=qk)
    kt2, vt2 = fresh()
    qb200.kv_append_seqs(kt2, vt2, tk, tv, offs, bits, 64)
    # one call
    one = qkv.clone()
    oq, ok_, ov = one[:, :Hq].unsqueeze(2), one[:, Hq:Hq + Hkv].unsqueeze(2), one[:, Hq + Hkv:].unsqueeze(2)
    kt1, vt1 = fresh()
    qb200.kv_append_seqs(kt1, vt1, ok_, ov, offs, bits, 64, rope_q=oq, rope_dims=dims, rope_base=500000.0)
    torch.cuda.synchronize()
    assert torch.equal(oq.view(torch.int16), tq.view(torch.int16)), "queries"
    assert torch.equal(ok_.view(torch.int16), qkv[:, Hq:Hq + Hkv].unsqueeze(2).view(torch.int16)), "the dense keys are read only"
    for a, b in zip(kt1 + vt1, kt2 + vt2):
        for x, y in zip(a, b):
            assert torch.equal(x.view(torch.int16) if x.dtype == torch.bfloat16 else x, y.view(torch.int16) if y.dtype == torch.bfloat16 else y)


def test_one_layer_tick_against_the_oracle_chain():
    """A Llama-shaped layer tick (hidden 1024, 8 query / 2 KV heads of 128, MLP 2816, 4-bit g64 weights, 4-bit packed
    cache) for five sequences of different length, every operator through the C ABI in the reference's order
    (src/transformer.zig:9656-9861), against the same chain computed by the oracle."""
    import qb200
    rng = np.random.default_rng(2024)
    N, Hd, Hq, Hkv, D, F, bits = 5, 1024, 8, 2, 128, 2816, 4
    lens = [17, 300, 1, 255, 64]                 # tokens already cached per sequence
    names = {"q": (Hq * D, Hd), "k": (Hkv * D, Hd), "v": (Hkv * D, Hd), "o": (Hd, Hq * D), "gate": (F, Hd), "up": (F, Hd), "down": (Hd, F)}
    W = {n_: make_weight(rng, shp, 64, 4) for n_, shp in names.items()}
    dW = {n_: dev_triple(*t) for n_, t in W.items()}
    w_in, w_post = qo.bf16_round(1.0 + 0.1 * rng.standard_normal(Hd).astype(np.float32)), qo.bf16_round(1.0 + 0.1 * rng.standard_normal(Hd).astype(np.float32))
    h = rand_bf16(rng, (N, Hd))
    caches = []
    for n in range(N):
        cap = (lens[n] + 256) // 256 * 256
        kc = qo.quantize(rand_bf16(rng, (1, Hkv, cap, D)), 64, bits)
        vc = qo.quantize(rand_bf16(rng, (1, Hkv, cap, D)), 64, bits)
        caches.append((kc, vc))
    offs = np.array(lens, np.int32)
    dk = [dev_triple(*c[0]) for c in caches]   # device copies made before the oracle writes the new token into its own
    dv = [dev_triple(*c[1]) for c in caches]

    # ---- oracle chain (every operator output rounded to bf16, like the reference's graph) ----
    r = qo.bf16_round
    normed = qo.rms_norm(h, w_in, 1e-5)
    q = r(qo.qmm(normed, *W["q"], 64, 4)); k = r(qo.qmm(normed, *W["k"], 64, 4)); v = r(qo.qmm(normed, *W["v"], 64, 4))
    q = qo.rope(q.reshape(N, Hq, D), D, 500000.0, 1.0, offs); k = qo.rope(k.reshape(N, Hkv, D), D, 500000.0, 1.0, offs)
    attn = np.empty((N, Hq, D), np.float32)
    for n in range(N):
        (kq, ks, kb), (vq, vs, vb) = caches[n]
        nk, nv = qo.quantize(k[n].reshape(1, Hkv, 1, D), 64, bits), qo.quantize(v[n].reshape(1, Hkv, 1, D), 64, bits)
        for buf, new in ((kq, nk[0]), (ks, nk[1]), (kb, nk[2]), (vq, nv[0]), (vs, nv[1]), (vb, nv[2])):
            buf[:, :, lens[n]] = new[:, :, 0]
        T = lens[n] + 1
        attn[n] = qo.kv_decode_attention(q[n:n + 1], kq[:, :, :T], ks[:, :, :T], kb[:, :, :T], vq[:, :, :T], vs[:, :, :T], vb[:, :, :T],
                                         64, bits, D ** -0.5)[0]
    attn = r(attn)
    o = r(qo.qmm(attn.reshape(N, Hq * D), *W["o"], 64, 4))
    h1 = r(h + o)
    ff = qo.rms_norm(h1, w_post, 1e-5)
    act = qo.bf16_to_f32(qo.swiglu_bf16(r(qo.qmm(ff, *W["gate"], 64, 4)), r(qo.qmm(ff, *W["up"], 64, 4))))
    ref = h1 + r(qo.qmm(act, *W["down"], 64, 4))          # compared before the final rounding

    # ---- the same tick through the library ----
    dh = _dev(h)
    n1 = qb200.rms_norm(dh, _dev(w_in), 1e-5)
    qkv = torch.empty((N, (Hq + 2 * Hkv) * D), dtype=torch.bfloat16, device="cuda")
    outs = [qkv[:, :Hq * D], qkv[:, Hq * D:(Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D:]]
    qb200.quantized_matmul_batch(n1, [dW["q"], dW["k"], dW["v"]], outs, True, 64, 4)
    doffs = torch.from_numpy(offs).cuda()
    qk = qkv[:, :(Hq + Hkv) * D].view(N, Hq + Hkv, 1, D)
    qb200.rope(qk, D, 500000.0, 1.0, doffs, out=qk)        # q and k heads in one launch, in place
    dq_ = qkv[:, :Hq * D].view(N, Hq, 1, D)
    dk_new = qkv[:, Hq * D:(Hq + Hkv) * D].view(N, Hkv, 1, D)
    dv_new = qkv[:, (Hq + Hkv) * D:].view(N, Hkv, 1, D)
    qb200.kv_append_seqs(dk, dv, dk_new, dv_new, lens, bits, 64)
    kviews = [[t[:, :, :lens[n] + 1] for t in dk[n]] for n in range(N)]
    vviews = [[t[:, :, :lens[n] + 1] for t in dv[n]] for n in range(N)]
    a = qb200.kv_decode_attention_ptrs(dq_, kviews, vviews, bits, 64, D ** -0.5)
    o_d = qb200.quantized_matmul(a.view(N, Hq * D), *dW["o"], True, 64, 4)
    h1_d, ff_d = qb200.add_rms_norm(dh, o_d, _dev(w_post), 1e-5)
    gu = [torch.empty((N, F), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    qb200.quantized_matmul_batch(ff_d, [dW["gate"], dW["up"]], gu, True, 64, 4)
    act_d = qb200.swiglu(gu[0], gu[1])
    down_d = qb200.quantized_matmul(act_d, *dW["down"], True, 64, 4)
    out, _ = qb200.add_rms_norm(h1_d, down_d, want_norm=False)
    got = out.float().cpu().numpy()
    # bf16 roundings along the chain may flip where device and host differ in the last fp32 bits (norm, rope, exp):
    # a flipped intermediate moves the output by about one rounding step of that intermediate
    rel = gate_bf16(got, ref, "layer tick", slack=2e-2)
    record("f3 one layer tick (5 sequences, hidden 1024)", "bf16 chain vs oracle chain", rel, None, int(ref.size))
    # the caches received exactly the oracle's new triples
    for n in range(N):
        assert np.array_equal(from_dev_u32(dk[n][0][0, :, lens[n]]), caches[n][0][0][0, :, lens[n]])

"""GPU parity, bit-exact: dequantize / quantize / kv_append through the C ABI against the golden
vectors of the reference's numpy restatement and against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import qoracle as qo
from util import from_dev_bf16, from_dev_u32, rand_bf16, to_dev_bf16, to_dev_u32

pytestmark = pytest.mark.gpu

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_affine.npz"))
QUANT_KEYS = sorted({k.split("/")[0] for k in G.files if k.startswith("quant_")})
DEQ_KEYS = sorted({k.split("/")[0] for k in G.files if k.startswith("deq_rand_")})


def _parse(key):
    return int(key.split("_b")[-1].split("_")[0]), int(key.split("_g")[-1])


@pytest.mark.parametrize("key", QUANT_KEYS + DEQ_KEYS)
def test_dequantize_golden(key):
    import qb200
    bits, gs = _parse(key)
    w, s, b = to_dev_u32(G[key + "/packed"]), to_dev_bf16(G[key + "/scales"]), to_dev_bf16(G[key + "/biases"])
    out = qb200.dequantize(w, s, b, gs, bits, dtype=torch.bfloat16)
    assert np.array_equal(from_dev_bf16(out), G[key + "/deq_bf16"])
    out32 = qb200.dequantize(w, s, b, gs, bits, dtype=torch.float32)
    assert np.array_equal(out32.cpu().numpy().view(np.uint32), G[key + "/deq_f32"].view(np.uint32))


@pytest.mark.parametrize("key", QUANT_KEYS)
def test_quantize_golden(key):
    import qb200
    bits, gs = _parse(key)
    name = key[len("quant_"):key.rindex("_b")]
    x = G[f"x_{name}"]
    xd = to_dev_bf16(qo.f32_to_bf16(x))
    q, s, b = qb200.quantize(xd, gs, bits)
    assert np.array_equal(from_dev_u32(q), G[key + "/packed"]), "codes"
    assert np.array_equal(from_dev_bf16(s), G[key + "/scales"]), "scales"
    assert np.array_equal(from_dev_bf16(b), G[key + "/biases"]), "biases"
    # fp32 input carrying the same values must give the same triple
    q2, s2, b2 = qb200.quantize(torch.from_numpy(x).cuda(), gs, bits)
    assert torch.equal(q, q2) and torch.equal(s.view(torch.int16), s2.view(torch.int16))
    assert torch.equal(b.view(torch.int16), b2.view(torch.int16))


@pytest.mark.parametrize("bits,gs", [(4, 64), (8, 64), (4, 32), (8, 128), (2, 64)])
def test_quantize_dequantize_vs_oracle_large(bits, gs):
    """C5-sized rows: [16, 8, 257, 128] ~N(0,1); every code, scale, bias and dequantised value identical."""
    import qb200
    rng = np.random.default_rng(1000 + bits + gs)
    x = rand_bf16(rng, (16, 8, 257, 128))
    q, s, b = qo.quantize(x, gs, bits)
    dq, ds, db = qb200.quantize(to_dev_bf16(qo.f32_to_bf16(x)), gs, bits)
    assert np.array_equal(from_dev_u32(dq), q)
    assert np.array_equal(from_dev_bf16(ds), s)
    assert np.array_equal(from_dev_bf16(db), b)
    out = qb200.dequantize(dq, ds, db, gs, bits, dtype=torch.bfloat16)
    assert np.array_equal(from_dev_bf16(out), qo.dequantize(q, s, b, gs, bits, out_bf16=True))


def test_round_trip_property_full_size():
    """Size-independent property at C5's full cache size (16 x 8 x 4096 x 128): re-quantising the
    dequantised values reproduces codes and dequantised values exactly wherever the group is non-degenerate,
    and the round-trip error is bounded by half a step."""
    import qb200
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((16, 8, 4096, 128), device="cuda", generator=g).to(torch.bfloat16)
    for bits in (4, 8):
        q, s, b = qb200.quantize(x, 64, bits)
        d = qb200.dequantize(q, s, b, 64, bits, dtype=torch.float32)
        assert not torch.isnan(d).any()
        step = s.float().abs().repeat_interleave(64, dim=-1)
        err = (d - x.float()).abs()
        # the snapped grid can clip the far end of the range by up to one step; plus the bf16 rounding of
        # scale/bias (relative 2^-8 of the value range)
        bound = 1.0 * step + (2.0 ** -8) * (x.float().abs() + step * (2 ** bits))
        assert bool((err <= bound).all())
        assert int(q.view(torch.int32).ne(0).sum()) > 0


def test_dequantize_strided_cache_view():
    """Views of capacity buffers: head stride = cap*last, not T*last (src/transformer.zig:3472-3495)."""
    import qb200
    rng = np.random.default_rng(3)
    B, H, cap, T, D = 2, 3, 256, 77, 128
    x = rand_bf16(rng, (B, H, cap, D))
    q, s, b = qo.quantize(x, 64, 4)
    dq, ds, db = to_dev_u32(q), to_dev_bf16(s), to_dev_bf16(b)
    out = qb200.dequantize(dq[:, :, 5:5 + T], ds[:, :, 5:5 + T], db[:, :, 5:5 + T], 64, 4, dtype=torch.bfloat16)
    ref = qo.dequantize(q, s, b, 64, 4, out_bf16=True)[:, :, 5:5 + T]
    assert out.shape == (B, H, T, D)
    assert np.array_equal(from_dev_bf16(out), ref)


@pytest.mark.parametrize("bits", [4, 8])
def test_kv_append_matches_oracle_and_leaves_neighbours(bits):
    """updateAffine steps 2+5 (src/transformer.zig:3224-3337): quantise S new tokens into the capacity buffers."""
    import qb200
    rng = np.random.default_rng(7)
    B, H, cap, D, off, S = 2, 4, 512, 128, 300, 3
    cq = torch.full((B, H, cap, D * bits // 32), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    cs = torch.full((B, H, cap, D // 64), 7.0, dtype=torch.bfloat16, device="cuda")
    cb = torch.full((B, H, cap, D // 64), -7.0, dtype=torch.bfloat16, device="cuda")
    x = rand_bf16(rng, (B, H, S, D))
    qb200.kv_append(cq, cs, cb, to_dev_bf16(qo.f32_to_bf16(x)), off, bits, 64)
    q, s, b = qo.quantize(x, 64, bits)
    assert np.array_equal(from_dev_u32(cq[:, :, off:off + S]), q)
    assert np.array_equal(from_dev_bf16(cs[:, :, off:off + S]), s)
    assert np.array_equal(from_dev_bf16(cb[:, :, off:off + S]), b)
    assert bool((cq[:, :, :off] == 0x5A5A5A5A).all()) and bool((cq[:, :, off + S:] == 0x5A5A5A5A).all())
    assert bool((cs[:, :, :off] == 7.0).all()) and bool((cb[:, :, off + S:] == -7.0).all())
    with pytest.raises(qb200.Qb200Error):
        qb200.kv_append(cq, cs, cb, to_dev_bf16(qo.f32_to_bf16(x)), cap - 1, bits, 64)

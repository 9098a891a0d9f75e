"""GPU parity of decode attention over the packed KV cache (C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import qoracle as qo
from util import dev_triple, gate_bf16, gate_f32, rand_bf16, to_dev_bf16

pytestmark = pytest.mark.gpu


def _cache(rng, B, Hkv, cap, D, bits, gs=64):
    k = rand_bf16(rng, (B, Hkv, cap, D))
    v = rand_bf16(rng, (B, Hkv, cap, D))
    return qo.quantize(k, gs, bits), qo.quantize(v, gs, bits)


def _run(rng, B, Hq, Hkv, T, D, bits, cap=None, lens=None, mask=None, start=0, gs=64):
    import qb200
    cap = cap or T
    kt, vt = _cache(rng, B, Hkv, cap, D, bits, gs)
    q = rand_bf16(rng, (B, Hq, D))
    scale = 1.0 / np.sqrt(D)
    sl = slice(start, start + T)
    kviews = [a[:, :, sl] for a in kt]
    vviews = [a[:, :, sl] for a in vt]
    ref = qo.kv_decode_attention(q, *kviews, *vviews, gs, bits, scale, kv_lens=lens, mask=mask)
    dk = [t[:, :, sl] for t in dev_triple(*kt)]
    dv = [t[:, :, sl] for t in dev_triple(*vt)]
    dl = None if lens is None else torch.from_numpy(np.asarray(lens, np.int32)).cuda()
    dm32 = None if mask is None else torch.from_numpy(mask.reshape(B, 1, 1, T)).cuda()
    o32 = qb200.kv_decode_attention(torch.from_numpy(q).cuda().view(B, Hq, 1, D), dk, dv, bits, gs, scale,
                                    "array" if mask is not None else "", dm32, dl)
    assert tuple(o32.shape) == (B, Hq, 1, D)
    r32 = gate_f32(o32.cpu().numpy().reshape(B, Hq, D), ref, "fp32 q")
    dm16 = None if mask is None else dm32.to(torch.bfloat16)
    ref16 = ref if mask is None else qo.kv_decode_attention(q, *kviews, *vviews, gs, bits, scale, kv_lens=lens,
                                                           mask=dm16.float().cpu().numpy().reshape(B, T))
    o16 = qb200.kv_decode_attention(to_dev_bf16(qo.f32_to_bf16(q)).view(B, Hq, 1, D), dk, dv, bits, gs, scale,
                                    "array" if mask is not None else "causal", dm16, dl)
    gate_bf16(o16.float().cpu().numpy().reshape(B, Hq, D), ref16, "bf16 q", slack=4e-3)
    return r32


@pytest.mark.parametrize("Hq,Hkv,D,bits,T", [(8, 2, 128, 4, 38), (12, 2, 64, 8, 22), (4, 4, 128, 8, 701),
                                              (6, 1, 256, 4, 701), (8, 2, 128, 8, 38), (32, 8, 128, 4, 1000)])
def test_reference_kernel_cases(Hq, Hkv, D, bits, T):
    """Shapes of the packed decode kernel's parity test (src/transformer.zig:21939-22101): GQA 4:1, 6:1, 1:1, 6:1;
    D 64/128/256; bits 4/8; T 38, 22, 701; over strided views of a larger capacity buffer."""
    rng = np.random.default_rng(Hq * 1000 + T + bits)
    cap = (T + 255) // 256 * 256 + 256
    _run(rng, 1, Hq, Hkv, T, D, bits, cap=cap, start=3)


@pytest.mark.parametrize("bits", [4, 8])
def test_additive_mask_row_and_ragged_lengths(bits):
    rng = np.random.default_rng(77 + bits)
    B, T = 3, 333
    mask = np.zeros((B, T), np.float32)
    mask[:, ::7] = -np.inf
    mask[1, :50] = -2.5
    _run(rng, B, 8, 2, T, 128, bits, cap=512, mask=mask)
    _run(rng, B, 8, 2, T, 128, bits, cap=512, lens=[T, 100, 1])
    _run(rng, B, 8, 2, T, 128, bits, cap=512, lens=[0, 64, 65])


@pytest.mark.parametrize("bits", [4, 8])
def test_config5_t4096(bits):
    """Benchmark configuration 5 at T=4096: B=16, Hq=32, Hkv=8, D=128, cap = next capacity so head stride != T*last."""
    rng = np.random.default_rng(0xC5 + bits)
    _run(rng, 16, 32, 8, 4096, 128, bits, cap=4352)


def test_config5_t32768_one_sequence_and_full_batch_property():
    """T=32768: one sequence against the oracle; the full 16-sequence batch through a size-independent property:
    the output for a cache made of two identical halves equals the output over one half (softmax weights pair up)."""
    import qb200
    rng = np.random.default_rng(0xC5)
    _run(rng, 1, 32, 8, 32768, 128, 4)
    g = torch.Generator(device="cuda").manual_seed(1)
    B, Hq, Hkv, Th, D = 16, 32, 8, 16384, 128
    k = torch.randn((B, Hkv, Th, D), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((B, Hkv, Th, D), device="cuda", generator=g).to(torch.bfloat16)
    kt = [torch.cat([t, t], dim=2) for t in qb200.quantize(k, 64, 4)]
    vt = [torch.cat([t, t], dim=2) for t in qb200.quantize(v, 64, 4)]
    q = torch.randn((B, Hq, 1, D), device="cuda", generator=g)
    full = qb200.kv_decode_attention(q, kt, vt, 4, 64, D ** -0.5)
    half = qb200.kv_decode_attention(q, [t[:, :, :Th] for t in kt], [t[:, :, :Th] for t in vt], 4, 64, D ** -0.5)
    assert not torch.isnan(full).any()
    r = float(half.pow(2).mean().sqrt())
    # p * v_scale enters the integer tensor cores as 15-bit fixed point per 128-token block
    assert float((full - half).abs().max()) <= 5e-3 * r
    lens = torch.full((B,), Th, dtype=torch.int32, device="cuda")
    masked = qb200.kv_decode_attention(q, kt, vt, 4, 64, D ** -0.5, kv_lens=lens)
    assert float((masked - half).abs().max()) <= 5e-3 * r

"""GPU parity of decode attention over the packed KV cache (C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import qoracle as qo
from util import dev_triple, from_dev_bf16, from_dev_u32, gate_bf16, gate_f32, half_ulp_fraction, rand_bf16, record, to_dev_bf16

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


def _device_cache(g, B, Hkv, cap, D, bits):
    """A packed cache made on the device with the library's quantize (bit-exact against the oracle's, see the
    elementwise tests); the host copy of chosen sequences feeds the oracle."""
    import qb200
    k = torch.randn((B, Hkv, cap, D), device="cuda", generator=g).to(torch.bfloat16)
    kt = qb200.quantize(k, 64, bits)
    k.normal_(generator=g)
    vt = qb200.quantize(k, 64, bits)
    del k
    return kt, vt


def _host_seq(triple, b, T):
    qd, sd, bd = (t[b:b + 1, :, :T].contiguous() for t in triple)
    return from_dev_u32(qd), from_dev_bf16(sd), from_dev_bf16(bd)


@pytest.mark.parametrize("bits", [4, 8])
def test_config5_t32768_full_batch_ragged_lengths_two_sequences_against_the_oracle(bits):
    """Benchmark configuration 5 at T=32768, both widths: the full batch of 16 sequences with ragged lengths runs on
    the GPU, a full-length sequence and a ragged one are checked against the oracle."""
    import qb200
    g = torch.Generator(device="cuda").manual_seed(0xC5 + bits)
    B, Hq, Hkv, T, D = 16, 32, 8, 32768, 128
    kt, vt = _device_cache(g, B, Hkv, T + 256, D, bits)
    kv, vv = [t[:, :, :T] for t in kt], [t[:, :, :T] for t in vt]
    q = torch.randn((B, Hq, 1, D), device="cuda", generator=g).to(torch.bfloat16)
    lens_np = np.full((B,), T, np.int32)
    lens_np[5], lens_np[9], lens_np[12] = 20001, 1, 32767
    lens = torch.from_numpy(lens_np).cuda()
    out = qb200.kv_decode_attention(q, kv, vv, bits, 64, D ** -0.5, kv_lens=lens)
    out32 = qb200.kv_decode_attention(q.float(), kv, vv, bits, 64, D ** -0.5, kv_lens=lens)
    torch.cuda.synchronize()
    assert not torch.isnan(out).any()
    for b in (0, 5):
        qh = q[b:b + 1, :, 0].float().cpu().numpy()
        ref = qo.kv_decode_attention(qh, *_host_seq(kt, b, T), *_host_seq(vt, b, T), 64, bits, D ** -0.5,
                                     kv_lens=lens_np[b:b + 1])
        r32 = gate_f32(out32[b:b + 1, :, 0].cpu().numpy(), ref, f"fp32 q, sequence {b}")
        got = out[b:b + 1, :, 0].float().cpu().numpy()
        r16 = gate_bf16(got, ref, f"bf16 q, sequence {b}", slack=4e-3)
        record(f"C5 T=32768 {bits}-bit, B=16 ragged, sequence {b}", "fp32 q vs oracle", r32, None, int(ref.size))
        record(f"C5 T=32768 {bits}-bit, B=16 ragged, sequence {b}", "bf16 q vs oracle (unrounded fp32)", r16,
               half_ulp_fraction(got, ref), int(ref.size))


@pytest.mark.parametrize("bits", [4, 8])
def test_sixteen_caches_of_different_capacity_through_the_pointer_form(bits):
    """forwardBatchedDecode's situation (src/transformer.zig:9742-9792): every slot owns a B=1 cache with its own
    capacity and offset.  Sixteen such caches through qb200_kv_decode_attention_ptrs against the oracle, sequence by
    sequence, and against the single-tensor entry on the same data."""
    import qb200
    rng = np.random.default_rng(0xA14 + bits)
    B, Hq, Hkv, D = 16, 32, 8, 128
    lens = [int(x) for x in rng.integers(1, 1500, B)]
    lens[0], lens[1], lens[2] = 1, 128, 1499
    q = rand_bf16(rng, (B, Hq, D))
    ktr, vtr, refs, hk, hv = [], [], [], [], []
    for b in range(B):
        cap = (lens[b] + 255) // 256 * 256 + 256 * int(rng.integers(0, 3))   # capacity grows in 256-token chunks
        kt, vt = _cache(rng, 1, Hkv, cap, D, bits)
        hk.append([a[:, :, :lens[b]] for a in kt])
        hv.append([a[:, :, :lens[b]] for a in vt])
        refs.append(qo.kv_decode_attention(q[b:b + 1], *hk[b], *hv[b], 64, bits, D ** -0.5))
        ktr.append([t[:, :, :lens[b]] for t in dev_triple(*kt)])
        vtr.append([t[:, :, :lens[b]] for t in dev_triple(*vt)])
    ref = np.concatenate(refs, 0)
    o32 = qb200.kv_decode_attention_ptrs(torch.from_numpy(q).cuda().view(B, Hq, 1, D), ktr, vtr, bits, 64, D ** -0.5)
    r32 = gate_f32(o32.cpu().numpy().reshape(B, Hq, D), ref, "fp32 q, pointer form")
    o16 = qb200.kv_decode_attention_ptrs(to_dev_bf16(qo.f32_to_bf16(q)).view(B, Hq, 1, D), ktr, vtr, bits, 64, D ** -0.5)
    got = o16.float().cpu().numpy().reshape(B, Hq, D)
    r16 = gate_bf16(got, ref, "bf16 q, pointer form", slack=4e-3)
    record(f"a14 16 caches of different capacity, {bits}-bit", "fp32 q vs oracle", r32, None, int(ref.size))
    record(f"a14 16 caches of different capacity, {bits}-bit", "bf16 q vs oracle (unrounded fp32)", r16,
           half_ulp_fraction(got, ref), int(ref.size))
    # kv_lens on top of the views' own lengths
    cut = np.array([max(1, n // 2) for n in lens], np.int32)
    o_cut = qb200.kv_decode_attention_ptrs(torch.from_numpy(q).cuda().view(B, Hq, 1, D), ktr, vtr, bits, 64, D ** -0.5,
                                           kv_lens=torch.from_numpy(cut).cuda())
    for b in (3, 7):
        rb = qo.kv_decode_attention(q[b:b + 1], *hk[b], *hv[b], 64, bits, D ** -0.5, kv_lens=cut[b:b + 1])
        gate_f32(o_cut[b:b + 1].cpu().numpy().reshape(1, Hq, D), rb, "pointer form with kv_lens")


def test_pointer_form_other_head_dims_and_more_than_32_sequences():
    """Geometries only the generic kernel serves (D=64, GQA 6:1) and a batch beyond one launch's table of 32 views."""
    import qb200
    rng = np.random.default_rng(0xA15)
    for (B, Hq, Hkv, D, bits) in ((3, 12, 2, 64, 8), (40, 8, 2, 128, 4)):
        lens = [int(x) for x in rng.integers(1, 300, B)]
        q = rand_bf16(rng, (B, Hq, D))
        ktr, vtr, refs = [], [], []
        for b in range(B):
            kt, vt = _cache(rng, 1, Hkv, lens[b] + 7, D, bits)
            refs.append(qo.kv_decode_attention(q[b:b + 1], *[a[:, :, :lens[b]] for a in kt], *[a[:, :, :lens[b]] for a in vt],
                                               64, bits, D ** -0.5))
            ktr.append([t[:, :, :lens[b]] for t in dev_triple(*kt)])
            vtr.append([t[:, :, :lens[b]] for t in dev_triple(*vt)])
        o = qb200.kv_decode_attention_ptrs(torch.from_numpy(q).cuda().view(B, Hq, 1, D), ktr, vtr, bits, 64, D ** -0.5)
        gate_f32(o.cpu().numpy().reshape(B, Hq, D), np.concatenate(refs, 0), f"pointer form D={D} B={B}")


@pytest.mark.parametrize("Tq,bits,B,Hq,Hkv,T", [(2, 4, 1, 32, 8, 300), (4, 8, 1, 8, 2, 129), (8, 4, 2, 16, 4, 1000), (3, 4, 1, 12, 2, 64)])
def test_verify_widths_with_the_causal_tail(Tq, bits, B, Hq, Hkv, T):
    """qkvAttnVerifyKernel's widths (src/transformer.zig:5464-5588): T_q = 2..8 queries over a cache that already holds
    them; query position tq sees the first T - T_q + 1 + tq positions (:5314-5318).  Against the oracle row by row."""
    import qb200
    rng = np.random.default_rng(Tq * 100 + T)
    D = 128 if Hq != 12 else 64
    kt, vt = _cache(rng, B, Hkv, T + 40, D, bits)
    q = rand_bf16(rng, (B, Hq, Tq, D))
    dk = [t[:, :, :T] for t in dev_triple(*kt)]
    dv = [t[:, :, :T] for t in dev_triple(*vt)]
    out = qb200.kv_decode_attention(torch.from_numpy(q).cuda(), dk, dv, bits, 64, D ** -0.5, mask_mode="causal")
    assert tuple(out.shape) == (B, Hq, Tq, D)
    got = out.cpu().numpy()
    for tq in range(Tq):
        lens = np.full((B,), T - Tq + 1 + tq, np.int32)
        ref = qo.kv_decode_attention(np.ascontiguousarray(q[:, :, tq]), *[a[:, :, :T] for a in kt], *[a[:, :, :T] for a in vt],
                                     64, bits, D ** -0.5, kv_lens=lens)
        gate_f32(got[:, :, tq], ref, f"verify width {Tq}, position {tq}")
    with pytest.raises(qb200.Qb200Error):
        qb200.kv_decode_attention(torch.from_numpy(q).cuda(), dk, dv, bits, 64, D ** -0.5)   # no mask mode: declined

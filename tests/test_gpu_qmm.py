"""GPU parity of quantized_matmul through the C ABI against the CPU oracle.

Gates (tests/util.py): fp32 activations -> max|d| <= 1e-2 * RMS(out) (the stated tolerance, with
orders of magnitude to spare); bf16 activations -> within half a bf16 ulp + 2e-3*RMS of the oracle's
unrounded fp32 result."""
import numpy as np
import pytest
import torch

from oracle import qoracle as qo
from util import dev_triple, gate_bf16, gate_f32, half_ulp_fraction, make_weight, rand_bf16, record, to_dev_bf16

pytestmark = pytest.mark.gpu


def _run(x32, q, s, b, gs, bits, transpose=True, tag=None):
    import qb200
    dq, ds, db = dev_triple(q, s, b)
    ref = qo.qmm_batched(x32, q, s, b, gs, bits, transpose) if x32.ndim > 2 or q.ndim > 2 else qo.qmm(x32, q, s, b, gs, bits, transpose)
    y32 = qb200.quantized_matmul(torch.from_numpy(x32).cuda(), dq, ds, db, transpose, gs, bits)
    r32 = gate_f32(y32.cpu().numpy(), ref, "fp32 activations")
    y16 = qb200.quantized_matmul(to_dev_bf16(qo.f32_to_bf16(x32)), dq, ds, db, transpose, gs, bits)
    assert y16.dtype == torch.bfloat16 and tuple(y16.shape) == ref.shape
    got16 = y16.float().cpu().numpy()
    if transpose and x32.ndim == 2 and q.ndim == 2 and _tensor_core_route(x32.shape[0], x32.shape[1], bits, gs):
        # Widths routed to the tensor-core prefill kernel take the dense route's semantics: the weight term is
        # rounded to bf16 once (src/transformer.zig:20987-21011).  Such a result must match that definition
        # tightly and the fp32-weight oracle within the stated 1e-2 * RMS (plus the output's own half ulp).
        ref_w16 = qo.qmm(x32, q, s, b, gs, bits, True, bf16_weights=True)
        r16 = gate_bf16(got16, ref_w16, "bf16 activations, bf16 weight term")
        gate_bf16(got16, ref, "bf16 activations vs fp32 weight term", slack=1e-2)
    else:
        r16 = gate_bf16(got16, ref, "bf16 activations")
    if tag:
        record(tag, "fp32 activations vs oracle", r32, None, int(ref.size))
        record(tag, "bf16 activations vs oracle (unrounded fp32)", r16, half_ulp_fraction(got16, ref), int(ref.size))
    return r32, r16


def _tensor_core_route(M, K, bits, gs):
    """The dispatch rule of qb200_quantized_matmul for bf16 activations: from 9 tokens a kernel that rounds the weight
    term to bf16 once, as the reference's dense route does -- the wide streaming kernel (4/8 bits at group 64, 4 bits
    at group 128, K a multiple of 256 up to 16384; 9..32 tokens) or the tcgen05 kernel (K a multiple of 256, 4/8 bits,
    group 64/128; from 33 tokens, and where the wide kernel does not serve); up to 8 tokens, and for other formats,
    the fp32 weight term."""
    tc_ok = K % 256 == 0 and bits in (4, 8) and gs in (64, 128)
    return tc_ok and M > 8 and (M > 32 or K <= 16384 or (bits, gs) == (8, 128))


def test_config1_qmv_4096x4096():
    """Benchmark configuration 1: x [1,4096] ~N(0,1), W [4096,4096] ~N(0,0.02), 4-bit g64."""
    rng = np.random.default_rng(0xC1)
    q, s, b = make_weight(rng, (4096, 4096), 64, 4)
    r32, _ = _run(rand_bf16(rng, (1, 4096)), q, s, b, 64, 4, tag="C1 qmv 1x4096->4096")
    assert r32 < 1e-4  # hi/lo-split fp32 activations: far inside the 1e-2 gate


LLAMA = {"q": (4096, 4096), "k": (1024, 4096), "gate": (14336, 4096), "down": (4096, 14336)}


@pytest.mark.parametrize("proj", list(LLAMA))
@pytest.mark.parametrize("M", [1, 8, 32])
def test_config2_llama_projections(proj, M):
    """Benchmark configuration 2: the Llama-3-8B layer shapes (v = k, o = q, up = gate) at decode widths."""
    N, K = LLAMA[proj]
    rng = np.random.default_rng(0xC2 + M + N)
    q, s, b = make_weight(rng, (N, K), 64, 4)
    _run(rand_bf16(rng, (M, K)), q, s, b, 64, 4, tag=f"C2 {proj} M={M}")


@pytest.mark.parametrize("bits,gs", [(4, 64), (8, 64), (4, 128)])
@pytest.mark.parametrize("M,N,K", [(16, 4096, 4096), (9, 1024, 4096), (13, 1000, 2048), (16, 512, 14336), (24, 2048, 1024),
                                   (31, 640, 4096), (16, 14336, 4096), (12, 256, 256), (40, 1000, 2048), (64, 640, 4096),
                                   (57, 4096, 1024), (33, 16, 512)])
def test_nine_to_sixty_four_tokens(bits, gs, M, N, K):
    """9..32 tokens: the wide streaming kernel reads the weights once per pass (16- and 32-token forms, ragged token
    counts and row counts, K from one ring stage to the longest projection, work cut over the CTAs inside tile blocks);
    33..64 tokens take the tensor-core kernel."""
    rng = np.random.default_rng(M * 7 + N + K + bits)
    q, s, b = make_weight(rng, (N, K), gs, bits)
    _run(rand_bf16(rng, (M, K)), q, s, b, gs, bits)


_WIDE64_CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2]); sys.path.insert(0, sys.argv[3])
from oracle import qoracle as qo
import qb200
from util import make_weight, rand_bf16, dev_triple, to_dev_bf16, gate_bf16
for (M, N, K, bits, gs) in [(64, 640, 4096, 4, 64), (40, 1000, 2048, 8, 64), (57, 4096, 1024, 4, 128), (33, 16, 512, 4, 64)]:
    rng = np.random.default_rng(M + N + K)
    q, s, b = make_weight(rng, (N, K), gs, bits)
    xh = qo.f32_to_bf16(rand_bf16(rng, (M, K)))
    y = qb200.quantized_matmul(to_dev_bf16(xh), *dev_triple(q, s, b), True, gs, bits)
    ref = qo.qmm(qo.bf16_to_f32(xh), q, s, b, gs, bits, True, bf16_weights=True)
    gate_bf16(y.float().cpu().numpy(), ref, f"64-token form {M}x{N}x{K}")
assert qb200.lib().qb200_debug_tc_status() == 0
print("ok")
"""


def test_wide_kernel_64_token_form_behind_the_environment_switch():
    """QB200_WIDE_MAX_TOKENS=64 (read once per process, hence a child process) sends 33..64 tokens to the wide streaming
    kernel's 64-token form, which the default routing no longer reaches."""
    import os, subprocess, sys
    here = os.path.dirname(os.path.abspath(__file__))
    root = os.path.dirname(here)
    env = dict(os.environ, QB200_WIDE_MAX_TOKENS="64")
    out = subprocess.run([sys.executable, "-c", _WIDE64_CHILD, root, os.path.join(root, "mlx-serve_b200"), here],
                         env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stdout[-2000:] + out.stderr[-2000:]


def test_config2_m128():
    rng = np.random.default_rng(0xC2 + 128)
    q, s, b = make_weight(rng, (4096, 4096), 64, 4)
    _run(rand_bf16(rng, (128, 4096)), q, s, b, 64, 4, tag="C2 q M=128 (tensor cores)")


@pytest.mark.parametrize("bits,gs", [(8, 64), (4, 128), (8, 128), (4, 32), (8, 32), (2, 64)])
@pytest.mark.parametrize("M", [1, 5])
def test_other_widths_and_group_sizes(bits, gs, M):
    rng = np.random.default_rng(bits * 100 + gs + M)
    q, s, b = make_weight(rng, (1536, 2048), gs, bits)
    _run(rand_bf16(rng, (M, 2048)), q, s, b, gs, bits)


@pytest.mark.parametrize("N,K,M", [(24, 256, 1), (1000, 512, 3), (16, 256, 9), (520, 768, 2), (8, 64, 4), (40, 320, 2)])
def test_ragged_shapes(N, K, M):
    """Row counts that are not a multiple of the 16-row tile, minimum K, K that only the generic path serves."""
    rng = np.random.default_rng(N + K + M)
    q, s, b = make_weight(rng, (N, K), 64, 4)
    _run(rand_bf16(rng, (M, K)), q, s, b, 64, 4)


def test_reference_4d_broadcast_cases():
    """src/kv_quant.zig:968-1094: [1,2,3,64] x [1,2,5,64]^T -> [1,2,3,5] and [1,2,3,5] x [1,2,5,64] -> [1,2,3,64]."""
    rng = np.random.default_rng(11)
    wf = rand_bf16(rng, (1, 2, 5, 64), 0.5)
    q, s, b = qo.quantize(wf, 64, 4)
    _run(rand_bf16(rng, (1, 2, 3, 64)), q, s, b, 64, 4, True)
    _run(rand_bf16(rng, (1, 2, 3, 5)), q, s, b, 64, 4, False)


@pytest.mark.parametrize("transpose", [True, False])
def test_batch_broadcast_and_transpose_false_attention_shapes(transpose):
    """quantAttention's two products (src/kv_quant.zig:528-533, :657-674): q [B,Hkv,g,D] . K^T and attn [B,Hkv,g,T] . V."""
    rng = np.random.default_rng(12)
    B, H, g, T, D = 2, 2, 4, 96, 128
    kv = rand_bf16(rng, (B, H, T, D))
    q, s, b = qo.quantize(kv, 64, 8)
    x = rand_bf16(rng, (B, H, g, D) if transpose else (B, H, g, T), 0.3)
    _run(x, q, s, b, 64, 8, transpose)
    # weights shared across the batch (broadcast of w's leading dims)
    _run(x, q[:1], s[:1], b[:1], 64, 8, transpose)


# attn @ V of the composed quantized attention (src/kv_quant.zig:657-674): x [B, Hkv, g*Tq, T], W the packed value cache
# [B, Hkv, T, D*bits/32] quantised along D.  The shapes below take the row-streaming tensor-core kernel (one or more 64- /
# 32-wide column blocks, 4 or 8 bits); the last two stay on the generic kernel (2 bits; a width the blocks do not tile).
@pytest.mark.parametrize("batch,M,T,D,bits,gs", [
    ((4, 8), 4, 4096, 128, 4, 64),      # decode over a 4K cache, GQA 4: K split over a cluster
    ((2, 8), 4, 4099, 128, 4, 64),      # an odd row pitch of the probabilities: scalar activation loads, partial last tile
    ((2, 2), 4, 1000, 128, 8, 64),      # T not a multiple of the 16-row tile
    ((3,), 1, 17, 64, 4, 64),           # one token, one column block, two tiles
    ((1,), 8, 1, 128, 4, 64),           # a single cached position
    ((2,), 12, 300, 128, 4, 128),       # two token tiles, group 128 = two column blocks per scale
    ((2,), 16, 333, 256, 8, 32),        # 8 column blocks of 32, one scale each
    ((1, 2), 32, 200, 64, 8, 64),       # four token tiles (verify widths), two blocks per scale
    ((2,), 5, 77, 512, 4, 64),          # the widest row the kernel takes
    ((1,), 4, 32768, 128, 4, 64),       # one long sequence: 8 CTAs of a cluster, 256 tiles each
    ((2,), 3, 50, 128, 2, 64),          # generic kernel
    ((2,), 3, 50, 192, 4, 64),          # generic kernel (three column blocks)
])
def test_transpose_false_value_cache_shapes(batch, M, T, D, bits, gs):
    rng = np.random.default_rng(T * 7 + D + bits + M)
    kv = rand_bf16(rng, batch + (T, D))
    q, s, b = qo.quantize(kv, gs, bits)
    x = rand_bf16(rng, batch + (M, T), 0.3)
    tag = "attn @ V, T=%d D=%d %d-bit" % (T, D, bits) if T in (4096, 32768) else None
    _run(x, q, s, b, gs, bits, False, tag=tag)


# q @ K^T of the composed quantized attention (src/kv_quant.zig:528-533): x [B, Hkv, g*Tq, D], W the packed key cache
# [B, Hkv, T, D*bits/32], one W per batch element, a contraction of one head dimension.  The shapes below take the
# batched short-contraction tensor-core kernel (up to 32 rows); the last two stay on the generic kernel (group 32; fp32
# activations of 20 rows at four groups, whose fragments would not fit the registers -- the bf16 half of the same case
# still takes the kernel).
@pytest.mark.parametrize("batch,M,T,D,bits,gs", [
    ((4, 8), 4, 4096, 128, 4, 64),      # decode over a 4K cache, GQA 4
    ((2, 2), 4, 1000, 128, 8, 64),      # T not a multiple of the 16-row tile: the partial last tile
    ((3,), 1, 17, 64, 4, 64),           # one query row, one group, two tiles
    ((2,), 8, 1, 128, 4, 64),           # a single cached position, eight rows
    ((2,), 5, 333, 256, 4, 64),         # four groups
    ((1, 2), 3, 200, 64, 8, 64),        # 8-bit, one group
    ((2,), 2, 77, 256, 8, 64),          # 8-bit, four groups
    ((2,), 4, 40000, 128, 4, 64),       # a long cache: many CTAs per batch element
    ((2,), 3, 50, 128, 8, 32),          # generic kernel (group 32)
    ((2,), 9, 50, 128, 4, 64),          # two token tiles
    ((2, 2), 16, 300, 128, 8, 64),      # two token tiles, 8-bit
    ((2,), 32, 130, 128, 4, 64),        # four token tiles (verify widths)
    ((2,), 20, 90, 256, 4, 64),         # four groups: bf16 activations take the kernel, fp32 the generic one
])
def test_transpose_true_key_cache_shapes(batch, M, T, D, bits, gs):
    rng = np.random.default_rng(T * 5 + D + bits + M)
    kv = rand_bf16(rng, batch + (T, D))
    q, s, b = qo.quantize(kv, gs, bits)
    x = rand_bf16(rng, batch + (M, D), 0.3)
    tag = "q @ K^T, T=%d D=%d %d-bit" % (T, D, bits) if T == 4096 else None
    _run(x, q, s, b, gs, bits, True, tag=tag)


def test_transpose_true_over_a_strided_cache_view():
    """The key cache as a slice [:, :, :T] of capacity buffers and the queries as a slice of a wider block."""
    import qb200
    rng = np.random.default_rng(78)
    B, H, cap, T, D, g = 2, 3, 160, 100, 128, 4
    kv = rand_bf16(rng, (B, H, cap, D))
    q, s, b = qo.quantize(kv, 64, 4)
    dq, ds, db = dev_triple(q, s, b)
    xw = rand_bf16(rng, (B, H, g, D + 8), 0.3)
    dx = to_dev_bf16(qo.f32_to_bf16(xw))
    y = qb200.quantized_matmul(dx[..., 3:D + 3], dq[:, :, :T], ds[:, :, :T], db[:, :, :T], True, 64, 4)
    ref = qo.qmm_batched(xw[..., 3:D + 3], q[:, :, :T], s[:, :, :T], b[:, :, :T], 64, 4, True)
    gate_bf16(y.float().cpu().numpy(), ref, "strided key cache")


def test_non_finite_activations_reach_the_output_of_the_attention_products():
    """An Inf or a NaN in a row of the activations makes that row's outputs non-finite and leaves the other rows
    bit for bit as they were, for both products of the composed attention (q @ K^T and attn @ V)."""
    import qb200
    rng = np.random.default_rng(405)
    B, T, D, M = 3, 200, 128, 6
    kv = rand_bf16(rng, (B, T, D))
    q, s, b = qo.quantize(kv, 64, 4)
    dq, ds, db = dev_triple(q, s, b)
    for transpose, width in ((True, D), (False, T)):
        x = rand_bf16(rng, (B, M, width), 0.3)
        clean = qb200.quantized_matmul(to_dev_bf16(qo.f32_to_bf16(x)), dq, ds, db, transpose, 64, 4).float().cpu().numpy()
        x[1, 0, 5] = np.inf
        x[1, M - 1, width - 3] = np.nan
        for dev_x in (to_dev_bf16(qo.f32_to_bf16(x)), torch.from_numpy(x).cuda()):
            y = qb200.quantized_matmul(dev_x, dq, ds, db, transpose, 64, 4).float().cpu().numpy()
            assert not np.isfinite(y[1, 0]).any() and not np.isfinite(y[1, M - 1]).any()
            assert np.isfinite(y[1, 1:M - 1]).all() and np.isfinite(y[0]).all() and np.isfinite(y[2]).all()
        y16 = qb200.quantized_matmul(to_dev_bf16(qo.f32_to_bf16(x)), dq, ds, db, transpose, 64, 4).float().cpu().numpy()
        assert np.array_equal(y16[1, 1:M - 1], clean[1, 1:M - 1]) and np.array_equal(y16[0], clean[0])


def test_transpose_false_over_a_strided_cache_view():
    """The value cache is a slice [:, :, :T] of capacity buffers, the probabilities a slice of a wider score block: batch
    strides that differ from the dense ones, and an activation pitch that rules the vector loads out."""
    import qb200
    rng = np.random.default_rng(77)
    B, H, cap, T, D, g = 2, 3, 160, 100, 128, 4
    kv = rand_bf16(rng, (B, H, cap, D))
    q, s, b = qo.quantize(kv, 64, 4)
    dq, ds, db = dev_triple(q, s, b)
    xw = rand_bf16(rng, (B, H, g, cap + 3), 0.3)
    dx = to_dev_bf16(qo.f32_to_bf16(xw))
    y = qb200.quantized_matmul(dx[..., 1:T + 1], dq[:, :, :T], ds[:, :, :T], db[:, :, :T], False, 64, 4)
    ref = qo.qmm_batched(xw[..., 1:T + 1], q[:, :, :T], s[:, :, :T], b[:, :, :T], 64, 4, False)
    gate_bf16(y.float().cpu().numpy(), ref, "strided value cache")


@pytest.mark.parametrize("M", [1, 8])
def test_fp32_activations_just_below_a_power_of_two(M):
    """fp32 activations whose group maximum rounds up to 2^14 on the 15-bit fixed-point grid (the staging clamps them
    to 16383), zeros, and a group of very small values next to a group of large ones."""
    rng = np.random.default_rng(77 + M)
    q, s, b = make_weight(rng, (512, 1024), 64, 4)
    x = rng.standard_normal((M, 1024)).astype(np.float32)
    x[:, 0:64] = np.nextafter(np.float32(2.0), np.float32(0.0))
    x[:, 64:128] = -np.nextafter(np.float32(0.5), np.float32(0.0))
    x[:, 128:192] = 0.0
    x[:, 192:256] *= 1e-20
    x[:, 256:320] *= 1e4
    ref = qo.qmm(x, q, s, b, 64, 4, True)
    import qb200
    dq, ds, db = dev_triple(q, s, b)
    y = qb200.quantized_matmul(torch.from_numpy(x).cuda(), dq, ds, db, True, 64, 4)
    gate_f32(y.cpu().numpy(), ref, "fp32 activations at the clamp")


def test_strided_operands_and_1d_x():
    import qb200
    rng = np.random.default_rng(13)
    N, K = 512, 1024
    q, s, b = make_weight(rng, (2 * N, K), 64, 4)
    dq, ds, db = dev_triple(q, s, b)
    xbig = rand_bf16(rng, (4, 2 * K))
    xd = to_dev_bf16(qo.f32_to_bf16(xbig))
    y = qb200.quantized_matmul(xd[:, K:], dq[::2], ds[::2], db[::2], True, 64, 4)
    ref = qo.qmm(np.ascontiguousarray(xbig[:, K:]), q[::2], s[::2], b[::2], 64, 4)
    gate_bf16(y.float().cpu().numpy(), ref, "strided")
    y1 = qb200.quantized_matmul(xd[0, :K], dq[:N], ds[:N], db[:N], True, 64, 4)
    assert tuple(y1.shape) == (N,)
    gate_bf16(y1.float().cpu().numpy(), qo.qmm(xbig[:1, :K], q[:N], s[:N], b[:N], 64, 4)[0], "1-D x")


def test_linearity_full_size_gate_proj():
    """Size-independent property at full size (14336 x 4096, M=8, fp32 activations):
    qmm(a*x1 + x2) == a*qmm(x1) + qmm(x2) up to accumulation noise, and scaling x by 2 doubles y exactly."""
    import qb200
    g = torch.Generator(device="cuda").manual_seed(99)
    w = (torch.randn((14336, 4096), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    q, s, b = qb200.quantize(w, 64, 4)
    x1 = torch.randn((8, 4096), device="cuda", generator=g).to(torch.bfloat16).float()
    x2 = torch.randn((8, 4096), device="cuda", generator=g).to(torch.bfloat16).float()
    y1 = qb200.quantized_matmul(x1, q, s, b, True, 64, 4)
    y2 = qb200.quantized_matmul(x2, q, s, b, True, 64, 4)
    y12 = qb200.quantized_matmul(0.5 * x1 + x2, q, s, b, True, 64, 4)
    r = float(y12.pow(2).mean().sqrt())
    # activations enter the integer tensor cores as 15-bit fixed point per 64-wide group: 2^-15 steps
    assert float((y12 - (0.5 * y1 + y2)).abs().max()) <= 1e-3 * r
    assert torch.equal(qb200.quantized_matmul(2 * x1, q, s, b, True, 64, 4), 2 * y1)
    # and against dequantize + fp32 matmul of the same triple
    wd = qb200.dequantize(q, s, b, 64, 4, dtype=torch.float32)
    yref = x1.double() @ wd.double().t()
    assert float((y1.double() - yref).abs().max()) <= 2e-4 * r


@pytest.mark.parametrize("M", [1, 8])
def test_batch_entry_matches_single_calls(M):
    """q, k, v on one input through qb200_quantized_matmul_batch: bit-identical to three single calls."""
    import qb200
    rng = np.random.default_rng(21 + M)
    K = 4096
    x = to_dev_bf16(qo.f32_to_bf16(rand_bf16(rng, (M, K))))
    triples = [dev_triple(*make_weight(rng, (n, K), 64, 4)) for n in (4096, 1024, 1000)]
    single = [qb200.quantized_matmul(x, *t, True, 64, 4) for t in triples]
    outs = [torch.empty_like(s) for s in single]
    qb200.quantized_matmul_batch(x, triples, outs, True, 64, 4)
    for a, b in zip(single, outs):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))

@pytest.mark.parametrize("bits,gs", [(4, 64), (8, 64), (4, 128)])
@pytest.mark.parametrize("M,K,Ns", [(128, 4096, (4096, 1024, 1024)), (200, 1024, (1000, 520)), (100, 768, (256, 48, 640, 1008)),
                                    (65, 14336, (512, 512)), (128, 2048, (7168, 7168))])
def test_batch_entry_beyond_64_tokens_one_tensor_core_launch(bits, gs, M, K, Ns):
    """Several matrices on one input above the streaming kernels' widths (q, k, v and gate, up at 65..256 tokens): one
    launch of the tensor-core kernel walks the tiles of all of them, with K split over a cluster where the tiles are
    few.  Every output against the oracle of that route (weight term rounded to bf16 once), and against the single
    calls within the order-of-summation noise of fp32 partial sums."""
    import qb200
    if K % gs:
        pytest.skip("K not a multiple of the group size")
    rng = np.random.default_rng(M + K + bits + gs + len(Ns))
    xh = qo.f32_to_bf16(rand_bf16(rng, (M, K)))
    x = to_dev_bf16(xh)
    host = [make_weight(rng, (n, K), gs, bits) for n in Ns]
    triples = [dev_triple(*t) for t in host]
    outs = [torch.full((M, n), float("nan"), dtype=torch.bfloat16, device="cuda") for n in Ns]
    qb200.quantized_matmul_batch(x, triples, outs, True, gs, bits)
    assert qb200.lib().qb200_debug_tc_status() == 0
    for (q, s, b), t, o in zip(host, triples, outs):
        assert not torch.isnan(o).any()
        ref = qo.qmm(qo.bf16_to_f32(xh), q, s, b, gs, bits, True, bf16_weights=True)
        gate_bf16(o.float().cpu().numpy(), ref, f"batched tensor-core launch N={q.shape[0]}")
        one = qb200.quantized_matmul(x, *t, True, gs, bits)
        d = (o.float() - one.float()).abs().max().item()
        assert d <= 2.0 ** -6 * max(1.0, one.float().abs().max().item()), d


@pytest.mark.parametrize("bits,gs", [(4, 64), (8, 64), (4, 128)])
@pytest.mark.parametrize("M,N,K", [(512, 1024, 4096), (300, 1000, 1024), (17, 128, 64), (2048, 256, 2048),
                                   (256, 640, 768), (1100, 208, 1536), (4096, 2560, 512)])
def test_config4_prefill_shapes(bits, gs, M, N, K):
    """Benchmark configuration 4 (dense prefill qmm) at oracle-sized shapes, incl. ragged M and N, the minimum K, K that is
    not a whole window of scales (768, 1536 at group size 128) and more tiles than SMs (several tiles per CTA)."""
    import qb200
    if K % gs:
        pytest.skip("K not a multiple of the group size")
    rng = np.random.default_rng(M + N + K + bits + gs)
    q, s, b = make_weight(rng, (N, K), gs, bits)
    _run(rand_bf16(rng, (M, K)), q, s, b, gs, bits)
    assert qb200.lib().qb200_debug_tc_status() == 0


@pytest.mark.parametrize("bits", [4, 8])
def test_config4_full_size_vs_dequantize_plus_fp32_matmul(bits):
    """Benchmark configuration 4 at full size (x [2048,4096], W [14336,4096]): the fused kernel against the route it replaces,
    dequantize to bf16 + a plain fp32 matmul (torch, TF32 off)."""
    import qb200
    g = torch.Generator(device="cuda").manual_seed(0xC4)
    w = (torch.randn((14336, 4096), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    q, s, b = qb200.quantize(w, 64, bits)
    x = torch.randn((2048, 4096), device="cuda", generator=g).to(torch.bfloat16)
    y = qb200.quantized_matmul(x, q, s, b, True, 64, bits)
    assert qb200.lib().qb200_debug_tc_status() == 0
    wd = qb200.dequantize(q, s, b, 64, bits, dtype=torch.bfloat16)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = x.float() @ wd.float().t()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    assert not torch.isnan(y).any()
    r = float(ref.pow(2).mean().sqrt())
    d = (y.float() - ref).abs()
    ulp = torch.pow(2.0, torch.floor(torch.log2(ref.abs().clamp_min(1e-30))) - 7)
    assert bool((d <= 0.5 * ulp * (1 + 1e-6) + 1e-3 * r).all())


@pytest.mark.parametrize("bits,gs", [(4, 64), (8, 64), (4, 128)])
@pytest.mark.parametrize("M,N,K", [(128, 4096, 4096), (64, 1024, 4096), (100, 1000, 2048), (128, 512, 14336),
                                   (256, 4096, 4096), (200, 1024, 2048)])
def test_few_token_split_k_shapes(bits, gs, M, N, K):
    """32..256 tokens against few weight rows: the tensor-core kernel cuts K over the CTAs of a cluster and adds
    the partial accumulators in rank 0 (C2's M = 128 projections: q/o 4096x4096, k/v 1024x4096, down K = 14336)."""
    import qb200
    rng = np.random.default_rng(M + N + K + bits + gs)
    q, s, b = make_weight(rng, (N, K), gs, bits)
    _run(rand_bf16(rng, (M, K)), q, s, b, gs, bits)
    assert qb200.lib().qb200_debug_tc_status() == 0

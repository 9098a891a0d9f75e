"""The allocation-free decode-attention entry point (qb200_kv_decode_attention_noalloc).

Some hosts cannot hand the library a workspace: their device heap is carved up at start-up, or the call
sits where cudaMalloc is not allowed.  For them the library carries its own scratch array.  This file runs
last (pytest collects test files alphabetically) so that a failure here cannot hide any other test; it
passes both alone in a fresh process and after the rest of the suite.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, B, Hq, Hkv, T, D, bits):
    import qb200
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn((B, Hkv, T + 64, D), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((B, Hkv, T + 64, D), device="cuda", generator=g).to(torch.bfloat16)
    kt = [t[:, :, :T] for t in qb200.quantize(k, 64, bits)]
    vt = [t[:, :, :T] for t in qb200.quantize(v, 64, bits)]
    q = torch.randn((B, Hq, 1, D), device="cuda", generator=g).to(torch.bfloat16)
    lens = torch.randint(1, T + 1, (B,), device="cuda", generator=g).to(torch.int32)
    return q, kt, vt, lens


def test_noalloc_matches_workspace_entry_on_two_calls_in_a_row():
    import qb200
    for seed, (B, Hq, Hkv, T, D, bits) in enumerate([(4, 32, 8, 3000, 128, 4), (2, 8, 2, 777, 128, 8)]):
        q, kt, vt, lens = _case(100 + seed, B, Hq, Hkv, T, D, bits)
        ref = qb200.kv_decode_attention(q, kt, vt, bits, 64, D ** -0.5, kv_lens=lens)
        out = torch.full_like(ref, float("nan"))
        qb200.kv_decode_attention_noalloc(q, kt, vt, bits, 64, D ** -0.5, out, kv_lens=lens)
        torch.cuda.synchronize()
        assert not torch.isnan(out).any()
        r = float(ref.float().pow(2).mean().sqrt())
        # same kernels, same split plan: the tolerance of the attention parity tests is far more than needed
        assert float((out.float() - ref.float()).abs().max()) <= 4e-3 * r + 1e-30
        # and against the CPU oracle on the same packed cache (copied back to the host)
        from oracle import qoracle as qo
        from util import from_dev_bf16, from_dev_u32, gate_bf16
        hk = [from_dev_u32(kt[0]), from_dev_bf16(kt[1]), from_dev_bf16(kt[2])]
        hv = [from_dev_u32(vt[0]), from_dev_bf16(vt[1]), from_dev_bf16(vt[2])]
        want = qo.kv_decode_attention(q[:, :, 0].float().cpu().numpy(), *hk, *hv, 64, bits, D ** -0.5,
                                      kv_lens=lens.cpu().numpy())
        gate_bf16(out[:, :, 0].float().cpu().numpy(), want, "no-allocation entry vs oracle", slack=4e-3)
        # second call in a row reuses the array that the first one left dirty
        out2 = torch.full_like(ref, float("nan"))
        qb200.kv_decode_attention_noalloc(q, kt, vt, bits, 64, D ** -0.5, out2, kv_lens=lens)
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


def test_size_gate_agrees_with_the_plan_the_launch_uses():
    """The refusal is decided from the same workspace query the launch plans with: for the shapes tested above it
    must report a non-zero need that fits the built-in array (no kernel is launched here)."""
    import qb200
    cap = qb200.lib().qb200_kv_decode_attention_noalloc_max_scratch()
    for (B, Hq, Hkv, T, D) in [(4, 32, 8, 3000, 128), (2, 8, 2, 777, 128), (1, 8, 2, 1, 128)]:
        need = qb200.kv_decode_attention_workspace_size(B, Hq, Hkv, T, D)
        assert 0 < need <= cap


def test_noalloc_rejects_shapes_beyond_the_built_in_scratch():
    import qb200
    cap = qb200.lib().qb200_kv_decode_attention_noalloc_max_scratch()
    B, Hq, Hkv, T, D = 512, 64, 16, 4096, 128
    assert qb200.kv_decode_attention_workspace_size(B, Hq, Hkv, T, D) > cap
    # descriptors only: the request is refused before any kernel or memory access
    q = torch.empty((B, Hq, 1, D), dtype=torch.bfloat16, device="cuda")
    kq = torch.empty((1, 1, 1, D // 8), dtype=torch.int32, device="cuda").expand(B, Hkv, T, D // 8)
    ks = torch.empty((1, 1, 1, 2), dtype=torch.bfloat16, device="cuda").expand(B, Hkv, T, 2)
    with pytest.raises(qb200.Qb200Error) as ei:
        qb200.kv_decode_attention_noalloc(q, [kq, ks, ks], [kq, ks, ks], 4, 64, 0.1, torch.empty_like(q))
    assert ei.value.status == 7 and "built-in" in str(ei.value)

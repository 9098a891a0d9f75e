#!/usr/bin/env python3
"""Generate the golden vectors in this folder from the reference's own code.

Run in a checkout that has the mlx-serve tree available (its path is the first
argument, default: the checkout next to this build).  It imports the reference's numpy
restatement of MLX's affine quantization, ``tests/dsv4_imatrix.py``
(pack_bits / unpack_bits / dequant_np / _mlx_minmax_sb, and the code
derivation ``clip(rint((X - b) / s), 0, n)`` at :264) together with the bf16
helpers of ``tests/convert_dsv4_weights.py`` and records their outputs on
seeded inputs.  Nothing here calls the oracle or the CUDA library: these files
are what both are checked against.

    python tests/golden/make_golden.py [/path/to/mlx-serve]

Outputs (all small, compressed):
    golden_affine.npz   one entry set per case, keys ``<case>/<field>``; the
                        quantizer inputs are stored once per distribution as
                        ``x_<name>``
"""
import os
import sys
import warnings

import numpy as np

REF = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference")
sys.path.insert(0, os.path.join(REF, "tests"))
with warnings.catch_warnings():
    warnings.simplefilter("ignore")
    import dsv4_imatrix as ref  # noqa: E402
    from convert_dsv4_weights import bf16_to_f32, f32_to_bf16_u16  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_affine.npz")


def bf16_exact(x):
    """fp32 values that are exactly representable in bf16 (the path's input dtype)."""
    return bf16_to_f32(f32_to_bf16_u16(np.asarray(x, np.float32)))


def smooth_bf16(head_dim):
    """The ramp of src/kv_quant.zig:695-715 (buildSmoothBf16): [1,1,8,D] in [-1,1)."""
    T = 8
    i = np.arange(T * head_dim, dtype=np.float32)
    v = (i / np.float32(T * head_dim)) * np.float32(2.0) - np.float32(1.0)
    return bf16_exact(v.reshape(T, head_dim))


def smooth_bhtd(B, H, T, D):
    """src/kv_quant.zig:943-966 (buildSmoothBHTD)."""
    total = B * H * T * D
    b, h, t, d = np.meshgrid(np.arange(B), np.arange(H), np.arange(T), np.arange(D), indexing="ij")
    f = (b * 17 + h * 5 + t * 3 + d).astype(np.float32)
    v = (f / np.float32(total)) * np.float32(2.0) - np.float32(1.0)
    return bf16_exact(v.reshape(B * H * T, D))


def input_cases(rng):
    D = 256
    cases = {
        "normal": rng.standard_normal((8, D)).astype(np.float32),
        "weights_0p02": (rng.standard_normal((8, D)) * 0.02).astype(np.float32),
        "positive": np.abs(rng.standard_normal((8, D))).astype(np.float32) + 0.25,
        "negative": -np.abs(rng.standard_normal((8, D))).astype(np.float32) - 0.25,
        "wide": (rng.standard_normal((8, D)) * 300.0).astype(np.float32),
        "tiny": (rng.standard_normal((8, D)) * 1e-6).astype(np.float32),
        "smooth_ramp": smooth_bf16(D),
        "smooth_bhtd": np.concatenate([smooth_bhtd(1, 2, 5, 64)] * 4, axis=1),
    }
    # degenerate rows: all zero, constant, one outlier, mixed constant groups
    deg = np.zeros((6, D), np.float32)
    deg[1, :] = 0.75
    deg[2, :] = -3.0
    deg[3, 7] = 5.0
    deg[4, :128] = 1.0
    deg[4, 128:] = -1.0
    deg[5, ::2] = 1e-3
    cases["degenerate"] = deg
    return {k: bf16_exact(v) for k, v in cases.items()}


def main():
    rng = np.random.default_rng(20260801)
    store = {}

    # 1. packing layout
    for bits in (2, 4, 8):
        q = rng.integers(0, 1 << bits, size=(8, 256), dtype=np.uint8)
        packed = ref.pack_bits(q, bits)
        assert np.array_equal(ref.unpack_bits(packed, bits, 256), q)
        store[f"pack_b{bits}/q"] = q
        store[f"pack_b{bits}/packed"] = packed

    # 2. bf16 rounding
    f = np.concatenate([
        rng.standard_normal(512).astype(np.float32),
        (rng.standard_normal(256) * 1e-20).astype(np.float32),
        (rng.standard_normal(256) * 1e20).astype(np.float32),
        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, 65504.0], np.float32),
    ])
    store["bf16/f32"] = f
    store["bf16/u16"] = f32_to_bf16_u16(f)

    # 3. quantize + dequantize
    for name, x in input_cases(rng).items():
        for bits in (4, 8):
            for gs in (32, 64, 128):
                n_bins = (1 << bits) - 1
                X = x.reshape(x.shape[0], -1, gs)
                s0, b0 = ref._mlx_minmax_sb(X, n_bins)
                with np.errstate(all="ignore"):
                    q = np.clip(np.rint((X - b0[..., None]) / s0[..., None]), 0, n_bins)
                q = q.astype(np.uint8).reshape(x.shape)
                packed = ref.pack_bits(q, bits)
                s_u16, b_u16 = f32_to_bf16_u16(s0), f32_to_bf16_u16(b0)
                deq = ref.dequant_np(packed, s_u16, b_u16, bits, gs).reshape(x.shape).astype(np.float32)
                key = f"quant_{name}_b{bits}_g{gs}"
                store[f"x_{name}"] = x
                store[key + "/packed"] = packed
                store[key + "/scales"] = s_u16
                store[key + "/biases"] = b_u16
                store[key + "/deq_f32"] = deq
                store[key + "/deq_bf16"] = f32_to_bf16_u16(deq)

    # 4. dequantize with arbitrary (not quantizer-produced) scales and biases
    for bits in (2, 4, 8):
        for gs in (32, 64, 128):
            q = rng.integers(0, 1 << bits, size=(8, 256), dtype=np.uint8)
            packed = ref.pack_bits(q, bits)
            sc = f32_to_bf16_u16((rng.standard_normal((8, 256 // gs)) * 0.1).astype(np.float32))
            bi = f32_to_bf16_u16((rng.standard_normal((8, 256 // gs)) * 0.05).astype(np.float32))
            deq = ref.dequant_np(packed, sc, bi, bits, gs).reshape(8, 256).astype(np.float32)
            key = f"deq_rand_b{bits}_g{gs}"
            store[key + "/packed"] = packed
            store[key + "/scales"] = sc
            store[key + "/biases"] = bi
            store[key + "/deq_f32"] = deq
            store[key + "/deq_bf16"] = f32_to_bf16_u16(deq)

    np.savez_compressed(OUT, **store)
    print(f"wrote {OUT}: {len(store)} arrays, {os.path.getsize(OUT)} bytes")


if __name__ == "__main__":
    main()

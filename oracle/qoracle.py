"""ctypes front end of the CPU oracle (``oracle/qoracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark.  The shipped
library never imports this module.

All functions take and return numpy arrays.  bf16 values travel as ``uint16``
bit patterns; ``bf16_to_f32`` / ``f32_to_bf16`` convert (round to nearest even,
as tests/convert_dsv4_weights.py:154-162 in the reference tree does).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libqoracle.so")


def build(force: bool = False) -> str:
    """Compile ``libqoracle.so`` with the Makefile next to this file."""
    src = os.path.join(_HERE, "qoracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libqoracle.so"], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
    return _lib


def _p(a, ty):
    return a.ctypes.data_as(C.POINTER(ty)) if a is not None else None


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def num_threads() -> int:
    return int(lib().qo_num_threads())


def set_num_threads(n: int) -> None:
    """Threads the OpenMP loops use from now on (launchers like torchrun export OMP_NUM_THREADS=1)."""
    lib().qo_set_num_threads(int(n))


def f32_to_bf16(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().qo_f32_to_bf16(_p(x, C.c_float), _p(out, C.c_uint16), C.c_int64(x.size))
    return out


def bf16_to_f32(h) -> np.ndarray:
    h = _c(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().qo_bf16_to_f32(_p(h, C.c_uint16), _p(out, C.c_float), C.c_int64(h.size))
    return out


def bf16_round(x) -> np.ndarray:
    """fp32 -> nearest bf16 -> fp32."""
    return bf16_to_f32(f32_to_bf16(x))


def pack(q, bits: int) -> np.ndarray:
    q = _c(q, np.uint8)
    d = q.shape[-1]
    rows = q.size // d
    out = np.empty(q.shape[:-1] + (d * bits // 32,), np.uint32)
    lib().qo_pack(_p(q, C.c_uint8), C.c_int64(rows), C.c_int64(d), C.c_int(bits), _p(out, C.c_uint32))
    return out


def unpack(w, bits: int) -> np.ndarray:
    w = _c(w, np.uint32)
    d = w.shape[-1] * 32 // bits
    rows = w.size // w.shape[-1]
    out = np.empty(w.shape[:-1] + (d,), np.uint8)
    lib().qo_unpack(_p(w, C.c_uint32), C.c_int64(rows), C.c_int64(d), C.c_int(bits), _p(out, C.c_uint8))
    return out


def dequantize(w, s, b, gs: int, bits: int, out_bf16: bool = False) -> np.ndarray:
    """Packed triple -> dense.  fp32 by default, bf16 bit patterns if asked."""
    w, s, b = _c(w, np.uint32), _c(s, np.uint16), _c(b, np.uint16)
    d = w.shape[-1] * 32 // bits
    rows = w.size // w.shape[-1]
    if out_bf16:
        out = np.empty(w.shape[:-1] + (d,), np.uint16)
        lib().qo_dequantize_bf16(_p(w, C.c_uint32), _p(s, C.c_uint16), _p(b, C.c_uint16), C.c_int64(rows),
                                 C.c_int64(d), C.c_int(gs), C.c_int(bits), _p(out, C.c_uint16))
    else:
        out = np.empty(w.shape[:-1] + (d,), np.float32)
        lib().qo_dequantize_f32(_p(w, C.c_uint32), _p(s, C.c_uint16), _p(b, C.c_uint16), C.c_int64(rows),
                                C.c_int64(d), C.c_int(gs), C.c_int(bits), _p(out, C.c_float))
    return out


def quantize(x, gs: int, bits: int):
    """fp32 ``[..., D]`` -> (packed u32, scales bf16 bits, biases bf16 bits)."""
    x = _c(x, np.float32)
    d = x.shape[-1]
    rows = x.size // d
    q = np.empty(x.shape[:-1] + (d * bits // 32,), np.uint32)
    s = np.empty(x.shape[:-1] + (d // gs,), np.uint16)
    b = np.empty_like(s)
    lib().qo_quantize(_p(x, C.c_float), C.c_int64(rows), C.c_int64(d), C.c_int(gs), C.c_int(bits),
                      _p(q, C.c_uint32), _p(s, C.c_uint16), _p(b, C.c_uint16))
    return q, s, b


def qmm(x, w, s, b, gs: int, bits: int, transpose: bool = True, bf16_weights: bool = False) -> np.ndarray:
    """2-D quantized matmul in fp32.  transpose=True: w is [N, K*bits/32].

    ``bf16_weights`` rounds the dequantised weight to bf16 before the dot, as the reference's dense
    prefill route does (src/transformer.zig:20987-21011)."""
    x, w, s, b = _c(x, np.float32), _c(w, np.uint32), _c(s, np.uint16), _c(b, np.uint16)
    M, K = x.shape
    if transpose:
        N = w.shape[0]
        assert w.shape[1] * 32 // bits == K
        fn = lib().qo_qmm_t_bf16w if bf16_weights else lib().qo_qmm_t
    else:
        N = w.shape[1] * 32 // bits
        assert w.shape[0] == K
        fn = lib().qo_qmm_n
    y = np.empty((M, N), np.float32)
    fn(_p(x, C.c_float), _p(w, C.c_uint32), _p(s, C.c_uint16), _p(b, C.c_uint16), C.c_int64(M), C.c_int64(N),
       C.c_int64(K), C.c_int(gs), C.c_int(bits), _p(y, C.c_float))
    return y


def qmm_batched(x, w, s, b, gs: int, bits: int, transpose: bool = True) -> np.ndarray:
    """Leading dims of x and of (w, s, b) broadcast NumPy-style (src/kv_quant.zig:968-975)."""
    x = np.asarray(x, np.float32)
    w = np.asarray(w, np.uint32)
    xb, wb = x.shape[:-2], w.shape[:-2]
    bshape = np.broadcast_shapes(xb, wb)
    xs = np.broadcast_to(x, bshape + x.shape[-2:])
    ws = np.broadcast_to(w, bshape + w.shape[-2:])
    ss = np.broadcast_to(s, bshape + s.shape[-2:])
    bs = np.broadcast_to(b, bshape + b.shape[-2:])
    M = x.shape[-2]
    N = w.shape[-2] if transpose else w.shape[-1] * 32 // bits
    out = np.empty(bshape + (M, N), np.float32)
    for idx in np.ndindex(*bshape):
        out[idx] = qmm(xs[idx], ws[idx], ss[idx], bs[idx], gs, bits, transpose)
    return out


def swiglu_bf16(gate, up) -> np.ndarray:
    """silu(gate) * up with the fused kernel's rounding points (bf16 inputs, sigmoid, product, product); bf16 bits."""
    gate, up = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty(gate.shape, np.uint16)
    lib().qo_swiglu_bf16(_p(gate, C.c_float), _p(up, C.c_float), _p(out, C.c_uint16), C.c_int64(gate.size))
    return out


def swiglu_f32(gate, up) -> np.ndarray:
    gate, up = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty(gate.shape, np.float32)
    lib().qo_swiglu_f32(_p(gate, C.c_float), _p(up, C.c_float), _p(out, C.c_float), C.c_int64(gate.size))
    return out


def moe_route(logits, k: int, as_bf16: bool = True):
    """Router restatement: (inds [T, k] int32, norm_scores [T, k] fp32 carriers) for logits [T, E]."""
    logits = _c(logits, np.float32)
    T, E = logits.shape
    inds = np.empty((T, k), np.int32)
    scores = np.empty((T, k), np.float32)
    lib().qo_moe_route(_p(logits, C.c_float), C.c_int64(T), C.c_int64(E), C.c_int64(k), C.c_int(1 if as_bf16 else 0),
                       _p(inds, C.c_int32), _p(scores, C.c_float))
    return inds, scores


def moe_weighted_sum(y, scores, inv=None, as_bf16: bool = True) -> np.ndarray:
    """out[t, h] = sum_j y[inv[t*k + j], h] * scores[t, j]; y [T*k, H], scores [T, k] (fp32 carriers of bf16 values when
    as_bf16: products and the final sum are rounded to bf16)."""
    y, scores = _c(y, np.float32), _c(scores, np.float32)
    T, k = scores.shape
    H = y.shape[-1]
    out = np.empty((T, H), np.float32)
    invp = None if inv is None else _p(_c(inv, np.int64), C.c_int64)
    lib().qo_moe_weighted_sum(_p(y, C.c_float), _p(scores, C.c_float), invp, C.c_int64(T), C.c_int64(k), C.c_int64(H),
                              C.c_int(1 if as_bf16 else 0), _p(out, C.c_float))
    return out


def gather_qmm(x, w, s, b, lhs, rhs, gs: int, bits: int) -> np.ndarray:
    """x [XB, M, K] fp32, bank [E, N, K*bits/32]; y[i] = x[lhs[i]] . What[rhs[i]]^T -> [I, M, N]."""
    x, w, s, b = _c(x, np.float32), _c(w, np.uint32), _c(s, np.uint16), _c(b, np.uint16)
    lhs, rhs = _c(lhs, np.int64), _c(rhs, np.int64)
    _, M, K = x.shape
    _, N, _ = w.shape
    I = rhs.size
    y = np.empty((I, M, N), np.float32)
    lib().qo_gather_qmm_t(_p(x, C.c_float), _p(w, C.c_uint32), _p(s, C.c_uint16), _p(b, C.c_uint16),
                          _p(lhs, C.c_int64), _p(rhs, C.c_int64), C.c_int64(I), C.c_int64(M), C.c_int64(N),
                          C.c_int64(K), C.c_int(gs), C.c_int(bits), _p(y, C.c_float))
    return y


def _elem_strides(a):
    return np.array([st // a.itemsize for st in a.strides[:3]], np.int64)


def kv_decode_attention(q, kq, ks, kb, vq, vs, vb, gs: int, bits: int, scale: float, kv_lens=None, mask=None):
    """q [B,Hq,D] fp32; K/V triples [B,Hkv,T,*] (strided views allowed, last dim contiguous).

    Returns [B,Hq,Dv] fp32.  ``kv_lens`` int32 [B] masks t >= len; ``mask`` fp32 [B,T] is additive.
    """
    q = _c(q, np.float32)
    B, Hq, D = q.shape
    Hkv, T = kq.shape[1], kq.shape[2]
    Dv = vq.shape[3] * 32 // bits
    for a in (kq, ks, kb, vq, vs, vb):
        assert a.strides[3] == a.itemsize, "last dim must be contiguous"
    assert ks.strides == kb.strides and vs.strides == vb.strides
    out = np.empty((B, Hq, Dv), np.float32)
    kqs, ksbs, vqs, vsbs = _elem_strides(kq), _elem_strides(ks), _elem_strides(vq), _elem_strides(vs)
    lens = None if kv_lens is None else _c(kv_lens, np.int32)
    m = None if mask is None else _c(mask, np.float32)
    lib().qo_kv_decode_attention(
        _p(q, C.c_float), _p(kq, C.c_uint32), _p(ks, C.c_uint16), _p(kb, C.c_uint16), _p(vq, C.c_uint32),
        _p(vs, C.c_uint16), _p(vb, C.c_uint16), C.c_int64(B), C.c_int64(Hq), C.c_int64(Hkv), C.c_int64(T),
        C.c_int64(D), C.c_int64(Dv), C.c_int(gs), C.c_int(bits), _p(kqs, C.c_int64), _p(ksbs, C.c_int64),
        _p(vqs, C.c_int64), _p(vsbs, C.c_int64), C.c_float(scale), _p(lens, C.c_int32), _p(m, C.c_float),
        _p(out, C.c_float))
    return out


def rms_norm(x, w, eps: float, as_bf16: bool = True) -> np.ndarray:
    """mlx_fast_rms_norm restatement: x [..., d], w [d] (fp32 carriers of bf16 values when as_bf16)."""
    x, w = _c(x, np.float32), _c(w, np.float32)
    d = x.shape[-1]
    out = np.empty(x.shape, np.float32)
    lib().qo_rms_norm(_p(x, C.c_float), _p(w, C.c_float), C.c_int64(x.size // d), C.c_int64(d), C.c_float(eps),
                      C.c_int(1 if as_bf16 else 0), _p(out, C.c_float))
    return out


def rope(x, dims: int, base: float, scale: float, offsets, as_bf16: bool = True) -> np.ndarray:
    """mlx_fast_rope_dynamic (non-traditional) at sequence length 1: x [n, heads, d], offsets int32 [n]."""
    x = _c(x, np.float32)
    n, heads, d = x.shape
    out = np.empty(x.shape, np.float32)
    lib().qo_rope(_p(x, C.c_float), C.c_int64(n), C.c_int64(heads), C.c_int64(d), C.c_int(dims), C.c_float(base),
                  C.c_float(scale), _p(_c(offsets, np.int32), C.c_int32), C.c_int(1 if as_bf16 else 0), _p(out, C.c_float))
    return out


def turbo_rotate(x, seed: int, want_signs: bool = False):
    """x @ R along the last axis with TurboState's rotation R (src/kv_quant.zig:164-360); fp32 carriers of bf16 values."""
    x = _c(x, np.float32)
    n = x.shape[-1]
    out = np.empty(x.shape, np.float32)
    signs = np.zeros(n, np.uint8)
    lib().qo_turbo_rotate(_p(x, C.c_float), C.c_int64(x.size // n), C.c_int(n), C.c_uint64(seed), _p(out, C.c_float),
                          signs.ctypes.data_as(C.POINTER(C.c_ubyte)))
    return (out, signs) if want_signs else out

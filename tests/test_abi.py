"""CPU-side checks of the C ABI: libqb200.so loads, exports every symbol include/qb200.h declares,
and rejects bad input with the documented status before touching the GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def q():
    import qb200
    return qb200


def declared_symbols(header="qb200.h"):
    src = open(os.path.join(ROOT, "include", header)).read()
    return sorted(set(re.findall(r"QB200_API[^;(]*?\b(qb200_\w+)\s*\(", src)))


def test_header_declares_the_operator_set():
    syms = declared_symbols()
    for want in ("qb200_quantized_matmul", "qb200_gather_qmm", "qb200_dequantize", "qb200_quantize",
                 "qb200_kv_decode_attention", "qb200_kv_append", "qb200_set_error_handler", "qb200_last_error"):
        assert want in syms


def test_library_exports_every_declared_symbol(q):
    L = q.lib()
    for s in declared_symbols():
        assert hasattr(L, s), f"{s} declared in qb200.h but not exported"
    assert b"sm_100a" in L.qb200_version()


def test_expert_parallel_library_exports_every_declared_symbol(q):
    from qb200 import ep
    L = ep.ep_lib()
    syms = declared_symbols("qb200_ep.h")
    assert "qb200_moe_block_ep" in syms and "qb200_ep_comm_create" in syms
    for s in syms:
        assert hasattr(L, s), f"{s} declared in qb200_ep.h but not exported"
    # capacity rule: never more than T*k rows per peer, and world * capacity within the 2048 rows the local kernels serve
    assert L.qb200_moe_block_ep_capacity(64, 8, 8) == 256 and L.qb200_moe_block_ep_capacity(64, 8, 2) == 512
    assert L.qb200_moe_block_ep_capacity(4, 8, 2) == 32
    assert L.qb200_moe_block_ep_workspace_size(64, 8, 2048, 768, 128, 8, 256) > 3 * 2048 * 2048 * 2


def _t(q, dtype, shape, ptr=0x1000):
    stride, acc = [], 1
    for s in reversed(shape):
        stride.append(acc)
        acc *= s
    return q.raw_desc(ptr, dtype, shape, list(reversed(stride)))


def _qmm(q, x, w, s, b, res, transpose=True, gs=64, bits=4, mode=b"affine"):
    return q.lib().qb200_quantized_matmul(C.byref(res), C.byref(x), C.byref(w), C.byref(s), C.byref(b), transpose,
                                          q.OptInt(gs, True), q.OptInt(bits, True), mode, None)


def test_validation_statuses_without_a_gpu(q):
    x = _t(q, q.BFLOAT16, [1, 4096])
    w = _t(q, q.UINT32, [4096, 512])
    s = _t(q, q.BFLOAT16, [4096, 64])
    b = _t(q, q.BFLOAT16, [4096, 64])
    res = _t(q, q.BFLOAT16, [1, 4096])
    assert _qmm(q, x, w, s, b, res, mode=b"nvfp4") == 1  # UNSUPPORTED mode
    assert b"affine" in q.lib().qb200_last_error()
    assert _qmm(q, x, w, s, b, res, bits=3) == 1  # byte-stream packed widths are declined
    assert _qmm(q, x, w, s, b, res, gs=48) == 1
    assert _qmm(q, x, _t(q, q.UINT32, [4096, 256]), s, b, res) == 2  # K mismatch
    assert _qmm(q, x, w, _t(q, q.BFLOAT16, [4096, 32]), b, res) == 2
    assert _qmm(q, x, w, s, b, _t(q, q.BFLOAT16, [1, 4095])) == 2
    assert _qmm(q, x, w, s, b, _t(q, q.FLOAT32, [1, 4096])) == 4  # res dtype != x dtype
    assert _qmm(q, x, _t(q, q.INT32, [4096, 512]), s, b, res) == 4
    xs = _t(q, q.BFLOAT16, [1, 4096])
    xs.stride[1] = 2
    assert _qmm(q, xs, w, s, b, res) == 3  # last axis must be contiguous
    empty = q.desc(None)
    assert _qmm(q, x, w, s, empty, res) == 1  # no biases = non-affine mode


def test_error_handler_receives_the_message(q):
    seen = []
    CB = C.CFUNCTYPE(None, C.c_char_p, C.c_void_p)
    cb = CB(lambda msg, data: seen.append(msg))
    q.lib().qb200_set_error_handler.argtypes = [CB, C.c_void_p, C.c_void_p]
    q.lib().qb200_set_error_handler(cb, None, None)
    x = _t(q, q.BFLOAT16, [1, 64])
    w = _t(q, q.UINT32, [8, 8])
    s = _t(q, q.BFLOAT16, [8, 1])
    assert _qmm(q, x, w, s, s, _t(q, q.BFLOAT16, [1, 9])) == 2
    q.lib().qb200_set_error_handler(CB(0), None, None)
    assert seen and b"res dim" in seen[0]


def test_shape_inference_matches_reference_cases(q):
    """src/kv_quant.zig:968-1094: [1,2,3,64] x [1,2,5,64/8]^T -> [1,2,3,5]; [1,2,3,5] x [1,2,5,8] -> [1,2,3,64]."""
    shp = (C.c_int64 * 8)()
    nd = C.c_int32()
    x = _t(q, q.BFLOAT16, [1, 2, 3, 64])
    w = _t(q, q.UINT32, [1, 2, 5, 8])
    s = _t(q, q.BFLOAT16, [1, 2, 5, 1])
    st = q.lib().qb200_quantized_matmul_shape(C.byref(x), C.byref(w), C.byref(s), True, q.OptInt(64, True),
                                              q.OptInt(4, True), shp, C.byref(nd))
    assert st == 0 and [shp[i] for i in range(nd.value)] == [1, 2, 3, 5]
    x2 = _t(q, q.BFLOAT16, [1, 2, 3, 5])
    st = q.lib().qb200_quantized_matmul_shape(C.byref(x2), C.byref(w), C.byref(s), False, q.OptInt(64, True),
                                              q.OptInt(4, True), shp, C.byref(nd))
    assert st == 0 and [shp[i] for i in range(nd.value)] == [1, 2, 3, 64]


def test_gather_rejects_noncontiguous_bank(q):
    x = _t(q, q.BFLOAT16, [5, 1, 256])
    w = _t(q, q.UINT32, [4, 16, 32])
    w.stride[1] = 64  # a sliced view of a wider bank
    s = _t(q, q.BFLOAT16, [4, 16, 4])
    idx = _t(q, q.INT32, [5])
    res = _t(q, q.BFLOAT16, [5, 1, 16])
    st = q.lib().qb200_gather_qmm(C.byref(res), C.byref(x), C.byref(w), C.byref(s), C.byref(s), C.byref(q.desc(None)),
                                  C.byref(idx), True, q.OptInt(64, True), q.OptInt(4, True), b"affine", True, None)
    assert st == 3


def test_kv_attention_declines_wide_queries_and_checks_workspace(q):
    B, Hq, Hkv, T, D = 2, 8, 2, 300, 128
    qq = _t(q, q.BFLOAT16, [B, Hq, 2, D])
    kq = _t(q, q.UINT32, [B, Hkv, T, 16])
    ks = _t(q, q.BFLOAT16, [B, Hkv, T, 2])
    res = _t(q, q.BFLOAT16, [B, Hq, 2, D])
    e = q.desc(None)
    fn = q.lib().qb200_kv_decode_attention
    args = lambda r, qq_: [C.byref(r), C.byref(qq_), C.byref(kq), C.byref(ks), C.byref(ks), C.byref(kq), C.byref(ks),
                           C.byref(ks), 4, 64, 0.088, b"", C.byref(e), C.byref(e), None, 0, None]
    assert fn(*args(res, qq)) == 1  # T_q = 2 without the causal mask mode is declined
    q9 = _t(q, q.BFLOAT16, [B, Hq, 9, D])
    a9 = args(_t(q, q.BFLOAT16, [B, Hq, 9, D]), q9)
    a9[11] = b"causal"
    assert fn(*a9) == 1              # beyond the verify widths
    q1 = _t(q, q.BFLOAT16, [B, Hq, 1, D])
    r1 = _t(q, q.BFLOAT16, [B, Hq, 1, D])
    assert q.kv_decode_attention_workspace_size(B, Hq, Hkv, T, D) > 0
    assert fn(*args(r1, q1)) == 7  # workspace missing


def test_kv_attention_refuses_an_empty_cache_view_before_any_launch(q):
    """A cache view without tokens (offset 0) must not reach a kernel: both entries answer BAD_SHAPE on the host."""
    B, Hq, Hkv, D = 2, 8, 2, 128
    q1 = _t(q, q.BFLOAT16, [B, Hq, 1, D])
    r1 = _t(q, q.BFLOAT16, [B, Hq, 1, D])
    kq = _t(q, q.UINT32, [B, Hkv, 0, 16])
    ks = _t(q, q.BFLOAT16, [B, Hkv, 0, 2])
    e = q.desc(None)
    common = [C.byref(r1), C.byref(q1), C.byref(kq), C.byref(ks), C.byref(ks), C.byref(kq), C.byref(ks), C.byref(ks),
              4, 64, 0.088, b"", C.byref(e), C.byref(e)]
    assert q.kv_decode_attention_workspace_size(B, Hq, Hkv, 0, D) == 0
    assert q.lib().qb200_kv_decode_attention(*common, None, 0, None) == 2
    assert q.lib().qb200_kv_decode_attention(*common, C.c_void_p(0x1000), 1 << 20, None) == 2
    assert q.lib().qb200_kv_decode_attention_noalloc(*common, None) == 2
    assert b"no tokens" in q.lib().qb200_last_error()


def test_kv_chunk_entries_validate_before_any_copy(q, tmp_path):
    """Argument checks of the chunk save / restore entries run on the host: no path, an empty position range, a
    buffer that is not [1, Hkv, cap, cols], positions beyond the capacity, a file that does not exist."""
    L = q.lib()
    layers = (q.KvLayer * 1)()
    for name, dt, cols in (("k_q", q.UINT32, 16), ("k_scales", q.BFLOAT16, 2), ("k_biases", q.BFLOAT16, 2),
                           ("v_q", q.UINT32, 16), ("v_scales", q.BFLOAT16, 2), ("v_biases", q.BFLOAT16, 2)):
        setattr(layers[0], name, _t(q, dt, [1, 2, 64, cols]))
    path = str(tmp_path / "c.safetensors").encode()
    assert L.qb200_kv_chunk_save(None, layers, 1, 0, 8, None) == 5
    assert L.qb200_kv_chunk_save(path, layers, 1, 8, 8, None) == 2
    assert L.qb200_kv_chunk_save(path, layers, 1, 0, 65, None) == 2      # beyond the capacity
    layers[0].k_scales = _t(q, q.BFLOAT16, [2, 64, 2])
    assert L.qb200_kv_chunk_save(path, layers, 1, 0, 8, None) == 2      # not a 4-D capacity buffer
    assert L.qb200_kv_chunk_restore(path, layers, 1, 0, 0, None) == 2
    assert L.qb200_kv_chunk_restore(path, layers, 1, 0, 8, None) != 0                 # no such file
    assert not os.path.exists(path.decode())

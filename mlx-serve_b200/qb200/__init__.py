"""ctypes binding of libqb200's C ABI (``include/qb200.h``).

The functions keep the names, argument order and meaning of the mlx-c operators
mlx-serve calls (src/mlx.zig:262, :265, :271, :275) and of the two KV-cache
helpers built from them (src/kv_quant.zig:478-488, src/transformer.zig:3224-3337).
Tensors are ``torch`` CUDA tensors used purely as device buffers: this module
builds a ``qb200_tensor`` descriptor (pointer, dtype, shape, element strides)
for each and calls the library on torch's current stream.  Outputs are
allocated here with ``torch.empty`` because the library never allocates.

There is no CPU or PyTorch fallback: if ``libqb200.so`` is missing or a call is
declined, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libqb200.so")

MAX_DIMS = 8

# mlx_dtype values (src/mlx.zig:20-35)
UINT32, INT32, INT64, FLOAT16, FLOAT32, BFLOAT16 = 3, 7, 8, 9, 10, 12
_TORCH2Q = {
    torch.uint8: 1, torch.int8: 5, torch.int16: 6, torch.int32: 7, torch.int64: 8,
    torch.float16: 9, torch.float32: 10, torch.float64: 11, torch.bfloat16: 12, torch.bool: 0,
}
if hasattr(torch, "uint32"):
    _TORCH2Q[torch.uint32] = 3
if hasattr(torch, "uint16"):
    _TORCH2Q[torch.uint16] = 2

STATUS = {0: "OK", 1: "UNSUPPORTED", 2: "BAD_SHAPE", 3: "BAD_STRIDE", 4: "BAD_DTYPE", 5: "BAD_ARG", 6: "CUDA",
          7: "WORKSPACE", 8: "TIMEOUT"}


class Tensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("shape", C.c_int64 * MAX_DIMS), ("stride", C.c_int64 * MAX_DIMS)]


class OptInt(C.Structure):
    _fields_ = [("value", C.c_int), ("has_value", C.c_bool)]


class OptDtype(C.Structure):
    _fields_ = [("value", C.c_int), ("has_value", C.c_bool)]


class OptFloat(C.Structure):
    _fields_ = [("value", C.c_float), ("has_value", C.c_bool)]


class Qb200Error(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"qb200 status {status} ({STATUS.get(status, '?')}): {msg}")
        self.status = status


_lib = None


def lib():
    """Load libqb200.so; fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} is missing: build it with `make -C {_PKG}`")
        L = C.CDLL(LIB_PATH)
        TP = C.POINTER(Tensor)
        L.qb200_last_error.restype = C.c_char_p
        L.qb200_version.restype = C.c_char_p
        L.qb200_quantized_matmul.argtypes = [TP, TP, TP, TP, TP, C.c_bool, OptInt, OptInt, C.c_char_p, C.c_void_p]
        L.qb200_quantized_matmul_shape.argtypes = [TP, TP, TP, C.c_bool, OptInt, OptInt, C.POINTER(C.c_int64),
                                                   C.POINTER(C.c_int32)]
        L.qb200_quantized_matmul_batch.argtypes = [C.POINTER(TP), TP, C.POINTER(TP), C.POINTER(TP), C.POINTER(TP),
                                                   C.c_int, C.c_bool, OptInt, OptInt, C.c_char_p, C.c_void_p]
        L.qb200_gather_qmm.argtypes = [TP, TP, TP, TP, TP, TP, TP, C.c_bool, OptInt, OptInt, C.c_char_p, C.c_bool,
                                       C.c_void_p]
        L.qb200_gather_qmm_swiglu.argtypes = [TP] * 10 + [OptInt, OptInt, C.c_char_p, C.c_bool, C.c_void_p]
        L.qb200_moe_weighted_sum.argtypes = [TP, TP, TP, TP, C.c_void_p]
        L.qb200_moe_route.argtypes = [TP, TP, TP, C.c_int, C.c_void_p]
        L.qb200_moe_down_reduce.argtypes = [TP] * 7 + [OptInt, OptInt, C.c_char_p, C.c_void_p]
        L.qb200_dequantize.argtypes = [TP, TP, TP, TP, OptInt, OptInt, C.c_char_p, TP, OptDtype, C.c_void_p]
        L.qb200_quantize.argtypes = [TP, TP, TP, TP, OptInt, OptInt, C.c_char_p, TP, C.c_void_p]
        L.qb200_kv_append.argtypes = [TP, TP, TP, TP, C.c_int64, C.c_int, C.c_int, C.c_void_p]
        L.qb200_kv_decode_attention.argtypes = [TP, TP, TP, TP, TP, TP, TP, TP, C.c_int, C.c_int, C.c_float,
                                                C.c_char_p, TP, TP, C.c_void_p, C.c_size_t, C.c_void_p]
        L.qb200_kv_decode_attention_ptrs.argtypes = [TP, TP] + [C.POINTER(TP)] * 6 + [C.c_int, C.c_int, C.c_int, C.c_float,
                                                     C.c_char_p, TP, TP, C.c_void_p, C.c_size_t, C.c_void_p]
        L.qb200_kv_decode_attention_ptrs.restype = C.c_int
        L.qb200_kv_decode_attention_ptrs_workspace_size.restype = C.c_size_t
        L.qb200_kv_decode_attention_ptrs_workspace_size.argtypes = [C.c_int64] * 5
        L.qb200_moe_sort_by_expert.argtypes = [TP] * 6 + [C.c_int, C.c_void_p]
        L.qb200_moe_sort_by_expert.restype = C.c_int
        L.qb200_debug_tc_reset.restype = None
        L.qb200_kv_chunk_save.argtypes = [C.c_char_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p]
        L.qb200_kv_chunk_restore.argtypes = [C.c_char_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p]
        L.qb200_checkpoint_open.argtypes = [C.POINTER(C.c_void_p), C.c_char_p]
        L.qb200_checkpoint_close.argtypes = [C.c_void_p]
        L.qb200_checkpoint_close.restype = None
        L.qb200_checkpoint_num_tensors.argtypes = [C.c_void_p]
        L.qb200_checkpoint_tensor_name.argtypes = [C.c_void_p, C.c_int]
        L.qb200_checkpoint_tensor_name.restype = C.c_char_p
        L.qb200_checkpoint_tensor_info.argtypes = [C.c_void_p, C.c_char_p, TP, C.POINTER(C.c_size_t)]
        L.qb200_checkpoint_load_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_size_t]
        L.qb200_checkpoint_read_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]
        L.qb200_narrows_loaded_f16.argtypes = [C.c_char_p, C.c_int, C.c_int]
        L.qb200_narrows_loaded_f16.restype = C.c_bool
        L.qb200_affine_params_from_geometry.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.qb200_config_quantization.argtypes = [C.c_char_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_char_p, C.c_size_t]
        for name in ("qb200_checkpoint_open", "qb200_checkpoint_num_tensors", "qb200_checkpoint_tensor_info", "qb200_checkpoint_load_tensor",
                     "qb200_checkpoint_read_tensor", "qb200_affine_params_from_geometry", "qb200_config_quantization"):
            getattr(L, name).restype = C.c_int
        L.qb200_rms_norm.argtypes = [TP, TP, TP, C.c_float, C.c_void_p]
        L.qb200_add_rms_norm.argtypes = [TP, TP, TP, TP, TP, C.c_float, C.c_void_p]
        L.qb200_rope.argtypes = [TP, TP, C.c_int, C.c_bool, OptFloat, C.c_float, TP, TP, C.c_void_p]
        L.qb200_swiglu.argtypes = [TP, TP, TP, C.c_void_p]
        L.qb200_turbo_rotate.argtypes = [TP, TP, C.c_uint64, C.c_void_p]
        L.qb200_turbo_rotate.restype = C.c_int
        L.qb200_turbo_signs.argtypes = [C.c_uint64, C.c_int, C.POINTER(C.c_uint32)]
        L.qb200_turbo_signs.restype = C.c_int
        L.qb200_kv_append_seqs.argtypes = [C.POINTER(TP)] * 6 + [TP, TP, C.POINTER(C.c_int64), C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.qb200_rope_kv_append_seqs.argtypes = [TP, C.c_int, C.c_float, C.c_float] + L.qb200_kv_append_seqs.argtypes
        L.qb200_rope_kv_append_seqs.restype = C.c_int
        for name in ("qb200_rms_norm", "qb200_add_rms_norm", "qb200_rope", "qb200_swiglu", "qb200_kv_append_seqs"):
            getattr(L, name).restype = C.c_int
        L.qb200_kv_decode_attention_noalloc.argtypes = [TP, TP, TP, TP, TP, TP, TP, TP, C.c_int, C.c_int, C.c_float,
                                                        C.c_char_p, TP, TP, C.c_void_p]
        L.qb200_kv_decode_attention_noalloc.restype = C.c_int
        L.qb200_kv_decode_attention_noalloc_max_scratch.restype = C.c_size_t
        L.qb200_kv_decode_attention_workspace_size.restype = C.c_size_t
        L.qb200_kv_decode_attention_workspace_size.argtypes = [C.c_int64] * 5
        for name in ("qb200_quantized_matmul", "qb200_quantized_matmul_batch", "qb200_quantized_matmul_shape", "qb200_gather_qmm", "qb200_gather_qmm_swiglu", "qb200_moe_weighted_sum", "qb200_moe_route", "qb200_moe_down_reduce", "qb200_dequantize",
                     "qb200_quantize", "qb200_kv_append", "qb200_kv_decode_attention"):
            getattr(L, name).restype = C.c_int
        _lib = L
    return _lib


def desc(t, dtype_override=None) -> Tensor:
    """Descriptor of a torch tensor (or an empty handle for None)."""
    d = Tensor()
    if t is None:
        d.data, d.dtype, d.ndim = None, 0, 0
        return d
    d.data = t.data_ptr() if t.numel() > 0 else None
    d.dtype = dtype_override if dtype_override is not None else _TORCH2Q[t.dtype]
    d.ndim = t.dim()
    for i in range(t.dim()):
        d.shape[i] = t.shape[i]
        d.stride[i] = t.stride(i)
    return d


def raw_desc(ptr, dtype, shape, stride) -> Tensor:
    d = Tensor()
    d.data, d.dtype, d.ndim = ptr, dtype, len(shape)
    for i, (s, st) in enumerate(zip(shape, stride)):
        d.shape[i], d.stride[i] = s, st
    return d


def _packed(t):
    """uint32 payloads are carried in int32 torch tensors."""
    return desc(t, UINT32)


def _opt(v):
    return OptInt(0, False) if v is None else OptInt(int(v), True)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(status: int):
    if status != 0:
        raise Qb200Error(status, lib().qb200_last_error().decode())


def quantized_matmul(x, w, scales, biases, transpose=True, group_size=None, bits=None, mode="affine", out=None):
    """mlx_quantized_matmul (src/mlx.zig:262).  Returns x's dtype, shape broadcast(batch) + [M, N]."""
    L = lib()
    dx, dw, ds, db = desc(x), _packed(w), desc(scales), desc(biases)
    if out is None:
        shp = (C.c_int64 * MAX_DIMS)()
        nd = C.c_int32(0)
        check(L.qb200_quantized_matmul_shape(C.byref(dx), C.byref(dw), C.byref(ds), transpose, _opt(group_size),
                                             _opt(bits), shp, C.byref(nd)))
        out = torch.empty([shp[i] for i in range(nd.value)], dtype=x.dtype, device=x.device)
    do = desc(out)
    check(L.qb200_quantized_matmul(C.byref(do), C.byref(dx), C.byref(dw), C.byref(ds), C.byref(db), transpose,
                                   _opt(group_size), _opt(bits), mode.encode(), _stream()))
    return out


def quantized_matmul_batch(x, triples, outs, transpose=True, group_size=None, bits=None, mode="affine"):
    """Several (w, scales, biases) triples applied to the same x in one call; ``outs`` are preallocated."""
    L = lib()
    n = len(triples)
    TP = C.POINTER(Tensor)
    keep = [desc(x)] + [desc(o) for o in outs] + [_packed(t[0]) for t in triples] + \
           [desc(t[1]) for t in triples] + [desc(t[2]) for t in triples]
    arr = lambda lst: (TP * n)(*[C.pointer(d) for d in lst])
    check(L.qb200_quantized_matmul_batch(arr(keep[1:1 + n]), C.byref(keep[0]), arr(keep[1 + n:1 + 2 * n]),
                                         arr(keep[1 + 2 * n:1 + 3 * n]), arr(keep[1 + 3 * n:1 + 4 * n]), n, transpose,
                                         _opt(group_size), _opt(bits), mode.encode(), _stream()))
    return outs


def gather_qmm(x, w, scales, biases, lhs_indices=None, rhs_indices=None, transpose=True, group_size=None, bits=None,
               mode="affine", sorted_indices=False, out=None):
    """mlx_gather_qmm (src/mlx.zig:265).  Output [*rhs_indices.shape, M, N]."""
    L = lib()
    if out is None:
        M, N = x.shape[-2], w.shape[-2]
        out = torch.empty(list(rhs_indices.shape) + [M, N], dtype=x.dtype, device=x.device)
    do, dx, dw, ds, db = desc(out), desc(x), _packed(w), desc(scales), desc(biases)
    dl, dr = desc(lhs_indices), desc(rhs_indices)
    check(L.qb200_gather_qmm(C.byref(do), C.byref(dx), C.byref(dw), C.byref(ds), C.byref(db), C.byref(dl),
                             C.byref(dr), transpose, _opt(group_size), _opt(bits), mode.encode(), sorted_indices,
                             _stream()))
    return out


def gather_qmm_swiglu(x, w_gate, scales_gate, biases_gate, w_up, scales_up, biases_up, lhs_indices=None, rhs_indices=None,
                      group_size=None, bits=None, mode="affine", sorted_indices=False, out=None):
    """Fused gate/up projection + SwiGLU of the routed-expert block: silu(x . Wgate^T) * (x . Wup^T) per index entry
    (moeMLP2's two gatherExpertMm calls and fusedSwiGLU, src/transformer.zig:15007-15035, :19925-19931).
    Raises Qb200Error (status QB200_ERR_UNSUPPORTED) for shapes the fused kernel does not serve."""
    L = lib()
    if out is None:
        M, N = x.shape[-2], w_gate.shape[-2]
        out = torch.empty(list(rhs_indices.shape) + [M, N], dtype=x.dtype, device=x.device)
    do, dx = desc(out), desc(x)
    dg, dgs, dgb = _packed(w_gate), desc(scales_gate), desc(biases_gate)
    du, dus, dub = _packed(w_up), desc(scales_up), desc(biases_up)
    dl, dr = desc(lhs_indices), desc(rhs_indices)
    check(L.qb200_gather_qmm_swiglu(C.byref(do), C.byref(dx), C.byref(dg), C.byref(dgs), C.byref(dgb), C.byref(du),
                                    C.byref(dus), C.byref(dub), C.byref(dl), C.byref(dr), _opt(group_size), _opt(bits),
                                    mode.encode(), sorted_indices, _stream()))
    return out


def moe_down_reduce(act, w, scales, biases, inds, scores, group_size=None, bits=None, mode="affine", out=None):
    """gatherQmvDownReduce (src/transformer.zig:20559-20623): down projection of every slot, times its score, summed
    over top-k.  act [T, k, K], inds/scores [T, k] -> [T, N]."""
    L = lib()
    if out is None:
        out = torch.empty(list(scores.shape[:-1]) + [w.shape[-2]], dtype=act.dtype, device=act.device)
    check(L.qb200_moe_down_reduce(C.byref(desc(out)), C.byref(desc(act)), C.byref(_packed(w)), C.byref(desc(scales)),
                                  C.byref(desc(biases)), C.byref(desc(inds)), C.byref(desc(scores)), _opt(group_size),
                                  _opt(bits), mode.encode(), _stream()))
    return out


def moe_route(logits, k):
    """moeRoutingChain (src/transformer.zig:17022-17063): (inds int32 [..., T, k], norm_scores [..., T, k])."""
    L = lib()
    inds = torch.empty(list(logits.shape[:-1]) + [k], dtype=torch.int32, device=logits.device)
    scores = torch.empty(list(logits.shape[:-1]) + [k], dtype=logits.dtype, device=logits.device)
    check(L.qb200_moe_route(C.byref(desc(inds)), C.byref(desc(scores)), C.byref(desc(logits)), int(k), _stream()))
    return inds, scores


def moe_weighted_sum(y, scores, inv_order=None, out=None):
    """Rows back to token order, times the scores, summed over top-k (moeMLP2's take(inv_order) + multiply + sum,
    src/transformer.zig:15036-15042, :15127-15140).  y [T*k, H] or [T*k, 1, H], scores [..., T, k] -> [..., T, H]."""
    L = lib()
    if out is None:
        out = torch.empty(list(scores.shape[:-1]) + [y.shape[-1]], dtype=y.dtype, device=y.device)
    check(L.qb200_moe_weighted_sum(C.byref(desc(out)), C.byref(desc(y)), C.byref(desc(scores)), C.byref(desc(inv_order)),
                                   _stream()))
    return out


def dequantize(w, scales, biases, group_size=None, bits=None, mode="affine", dtype=None, out=None):
    """mlx_dequantize (src/mlx.zig:271)."""
    L = lib()
    b = 4 if bits is None else bits
    odt = scales.dtype if dtype is None else dtype
    if out is None:
        out = torch.empty(list(w.shape[:-1]) + [w.shape[-1] * 32 // b], dtype=odt, device=w.device)
    do, dw, ds, db, dg = desc(out), _packed(w), desc(scales), desc(biases), desc(None)
    od = OptDtype(0, False) if dtype is None else OptDtype(_TORCH2Q[dtype], True)
    check(L.qb200_dequantize(C.byref(do), C.byref(dw), C.byref(ds), C.byref(db), _opt(group_size), _opt(bits),
                             mode.encode(), C.byref(dg), od, _stream()))
    return out


def quantize(w, group_size=None, bits=None, mode="affine"):
    """mlx_quantize (src/mlx.zig:275): returns (q, scales, biases); q is uint32 carried as int32."""
    L = lib()
    gs = 64 if group_size is None else group_size
    b = 4 if bits is None else bits
    q = torch.empty(list(w.shape[:-1]) + [w.shape[-1] * b // 32], dtype=torch.int32, device=w.device)
    sdt = torch.bfloat16
    s = torch.empty(list(w.shape[:-1]) + [w.shape[-1] // gs], dtype=sdt, device=w.device)
    bi = torch.empty_like(s)
    dq, ds, db, dw, dg = _packed(q), desc(s), desc(bi), desc(w), desc(None)
    check(L.qb200_quantize(C.byref(dq), C.byref(ds), C.byref(db), C.byref(dw), _opt(group_size), _opt(bits),
                           mode.encode(), C.byref(dg), _stream()))
    return q, s, bi


def kv_append(cache_q, cache_scales, cache_biases, dense, offset, bits, group_size):
    """Quantise dense [B,Hkv,S,D] into the capacity buffers at token ``offset`` (updateAffine steps 2+5)."""
    L = lib()
    dq, ds, db, dd = _packed(cache_q), desc(cache_scales), desc(cache_biases), desc(dense)
    check(L.qb200_kv_append(C.byref(dq), C.byref(ds), C.byref(db), C.byref(dd), int(offset), int(bits),
                            int(group_size), _stream()))


def kv_decode_attention_workspace_size(B, Hq, Hkv, T, Dv) -> int:
    return int(lib().qb200_kv_decode_attention_workspace_size(B, Hq, Hkv, T, Dv))


def kv_decode_attention(q, k_triple, v_triple, bits, group_size, scale, mask_mode="", mask=None, kv_lens=None,
                        workspace=None, out=None):
    """Decode attention over packed K/V views; q [B,Hq,T_q,D] -> [B,Hq,T_q,Dv] (quantAttention at T_q = 1; the verify
    widths T_q = 2..8 with mask_mode "causal")."""
    L = lib()
    kq, ks, kb = k_triple
    vq, vs, vb = v_triple
    B, Hq = q.shape[0], q.shape[1]
    Hkv, T = kq.shape[1], kq.shape[2]
    Dv = vq.shape[3] * 32 // bits
    Tq = q.shape[2]
    if out is None:
        out = torch.empty((B, Hq, Tq, Dv), dtype=q.dtype, device=q.device)
    need = kv_decode_attention_workspace_size(Tq if Tq > 1 else B, Hq, Hkv, T, Dv)
    if workspace is None:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    args = [desc(out), desc(q), _packed(kq), desc(ks), desc(kb), _packed(vq), desc(vs), desc(vb)]
    dm, dl = desc(mask), desc(kv_lens)
    check(L.qb200_kv_decode_attention(*[C.byref(a) for a in args], int(bits), int(group_size), float(scale),
                                      mask_mode.encode(), C.byref(dm), C.byref(dl),
                                      C.c_void_p(workspace.data_ptr()), workspace.numel(), _stream()))
    return out


def kv_decode_attention_noalloc(q, k_triple, v_triple, bits, group_size, scale, out, mask_mode="", mask=None,
                                kv_lens=None):
    """kv_decode_attention for callers that cannot allocate: scratch comes from the array built into the library.
    ``out`` must be preallocated; nothing is allocated on the device by this call."""
    L = lib()
    args = [desc(out), desc(q), _packed(k_triple[0]), desc(k_triple[1]), desc(k_triple[2]), _packed(v_triple[0]),
            desc(v_triple[1]), desc(v_triple[2])]
    dm, dl = desc(mask), desc(kv_lens)
    check(L.qb200_kv_decode_attention_noalloc(*[C.byref(a) for a in args], int(bits), int(group_size), float(scale),
                                              mask_mode.encode(), C.byref(dm), C.byref(dl), _stream()))
    return out


def kv_decode_attention_ptrs(q, k_triples, v_triples, bits, group_size, scale, mask_mode="", mask=None, kv_lens=None,
                             workspace=None, out=None):
    """Decode attention over a batch whose sequences own separate caches: ``k_triples[b]`` / ``v_triples[b]`` are the
    (codes, scales, biases) views [1, Hkv, T_b, .] of sequence b (forwardBatchedDecode's per-slot caches,
    src/transformer.zig:9742-9792).  q [B,Hq,1,D] -> [B,Hq,1,Dv]."""
    L = lib()
    B, Hq = q.shape[0], q.shape[1]
    Hkv = k_triples[0][0].shape[1]
    tmax = max(t[0].shape[2] for t in k_triples)
    Dv = v_triples[0][0].shape[3] * 32 // bits
    if out is None:
        out = torch.empty((B, Hq, 1, Dv), dtype=q.dtype, device=q.device)
    need = int(L.qb200_kv_decode_attention_ptrs_workspace_size(B, Hq, Hkv, tmax, Dv))
    if workspace is None:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    TP = C.POINTER(Tensor)
    keep = []

    def arr(items, packed):
        ds = [(_packed(t) if packed else desc(t)) for t in items]
        keep.append(ds)
        return (TP * B)(*[C.pointer(d) for d in ds])
    lists = [arr([t[0] for t in k_triples], True), arr([t[1] for t in k_triples], False), arr([t[2] for t in k_triples], False),
             arr([t[0] for t in v_triples], True), arr([t[1] for t in v_triples], False), arr([t[2] for t in v_triples], False)]
    do, dq, dm, dl = desc(out), desc(q), desc(mask), desc(kv_lens)
    check(L.qb200_kv_decode_attention_ptrs(C.byref(do), C.byref(dq), *lists, int(B), int(bits), int(group_size),
                                           float(scale), mask_mode.encode(), C.byref(dm), C.byref(dl),
                                           C.c_void_p(workspace.data_ptr()), workspace.numel(), _stream()))
    return out


def moe_sort_by_expert(inds, num_experts, want_offsets=True):
    """Stable sort of the flattened top-k index list by expert (moeMLP2, src/transformer.zig:14961-15006).
    Returns (order, inv_order, sorted_inds, token_rows, expert_offsets), all int32."""
    L = lib()
    n = inds.numel()
    mk = lambda m: torch.empty((m,), dtype=torch.int32, device=inds.device)
    order, inv, sinds, rows = mk(n), mk(n), mk(n), mk(n)
    offs = mk(num_experts + 1) if want_offsets else None
    check(L.qb200_moe_sort_by_expert(C.byref(desc(order)), C.byref(desc(inv)), C.byref(desc(sinds)), C.byref(desc(rows)),
                                     C.byref(desc(offs)), C.byref(desc(inds)), int(num_experts), _stream()))
    return order, inv, sinds, rows, offs


def rms_norm(x, weight, eps, out=None):
    """mlx_fast_rms_norm (src/mlx.zig:319)."""
    if out is None:
        out = torch.empty_like(x)
    check(lib().qb200_rms_norm(C.byref(desc(out)), C.byref(desc(x)), C.byref(desc(weight)), float(eps), _stream()))
    return out


def add_rms_norm(a, b, weight=None, eps=1e-5, sum_out=None, norm_out=None, want_norm=True):
    """round(a + b) and its RMS norm in one launch (mlx_add + rmsNorm of the decode step).  Returns (sum, norm)."""
    if sum_out is None:
        sum_out = torch.empty_like(a)
    if norm_out is None and want_norm:
        norm_out = torch.empty_like(a)
    check(lib().qb200_add_rms_norm(C.byref(desc(sum_out)), C.byref(desc(norm_out)), C.byref(desc(a)), C.byref(desc(b)),
                                   C.byref(desc(weight if want_norm else None)), float(eps), _stream()))
    return sum_out, norm_out


def rope(x, dims, base, scale, offsets, out=None):
    """mlx_fast_rope_dynamic, non-traditional (src/mlx.zig:324): x [N, heads, 1, D], offsets int32 [N]; in place when
    out is x."""
    if out is None:
        out = torch.empty_like(x)
    check(lib().qb200_rope(C.byref(desc(out)), C.byref(desc(x)), int(dims), False, OptFloat(float(base), True), float(scale),
                           C.byref(desc(offsets)), C.byref(desc(None)), _stream()))
    return out


def turbo_rotate(x, seed, out=None):
    """x @ R along the last axis, R the Hadamard rotation of the TurboQuant schemes (src/kv_quant.zig:164-403;
    seed 0x9E37 ^ layer for K, 0x85EB ^ layer for V).  R is its own inverse."""
    if out is None:
        out = torch.empty_like(x)
    check(lib().qb200_turbo_rotate(C.byref(desc(out)), C.byref(desc(x)), int(seed), _stream()))
    return out


def turbo_signs(seed, n):
    """The rotation's sign vector as a 0/1 array (1 = -1)."""
    bits = (C.c_uint32 * ((n + 31) // 32))()
    check(lib().qb200_turbo_signs(int(seed), int(n), bits))
    return [(bits[e >> 5] >> (e & 31)) & 1 for e in range(n)]


def swiglu(gate, up, out=None):
    """fusedSwiGLU of the dense MLP (src/transformer.zig:8220-8243)."""
    if out is None:
        out = torch.empty_like(gate)
    check(lib().qb200_swiglu(C.byref(desc(out)), C.byref(desc(gate)), C.byref(desc(up)), _stream()))
    return out


def kv_append_seqs(k_triples, v_triples, dense_k, dense_v, offsets, bits, group_size, rope_q=None, rope_dims=0, rope_base=10000.0,
                   rope_scale=1.0):
    """One new token per sequence into per-sequence packed caches (the per-slot cache update of the batched decode,
    src/transformer.zig:9738-9756): k_triples[n] / v_triples[n] are the capacity buffers [1, Hkv, cap_n, .].
    With ``rope_q`` the same launch rotates the queries in place and the keys on their way into the cache."""
    n = len(k_triples)
    TP = C.POINTER(Tensor)
    keep = []

    def arr(items, packed):
        ds = [(_packed(t) if packed else desc(t)) for t in items]
        keep.append(ds)
        return (TP * n)(*[C.pointer(d) for d in ds])
    lists = [arr([t[0] for t in k_triples], True), arr([t[1] for t in k_triples], False), arr([t[2] for t in k_triples], False),
             arr([t[0] for t in v_triples], True), arr([t[1] for t in v_triples], False), arr([t[2] for t in v_triples], False)]
    offs = (C.c_int64 * n)(*[int(o) for o in offsets])
    if rope_q is not None:
        check(lib().qb200_rope_kv_append_seqs(C.byref(desc(rope_q)), int(rope_dims), C.c_float(rope_base), C.c_float(rope_scale), *lists,
                                              C.byref(desc(dense_k)), C.byref(desc(dense_v)), offs, n, int(bits), int(group_size),
                                              _stream()))
        return
    check(lib().qb200_kv_append_seqs(*lists, C.byref(desc(dense_k)), C.byref(desc(dense_v)), offs, n, int(bits), int(group_size),
                                     _stream()))


_Q2TORCH = {v: k for k, v in _TORCH2Q.items()}
_Q2TORCH[UINT32] = torch.int32   # packed codes are carried in int32 tensors

class KvLayer(C.Structure):
    _fields_ = [(n, Tensor) for n in ("k_q", "k_scales", "k_biases", "v_q", "v_scales", "v_biases")]


def _kv_layers(layers):
    """layers: per layer either None (no KV cache) or (k_triple, v_triple) of capacity buffers [1, Hkv, cap, cols]."""
    arr = (KvLayer * len(layers))()
    for i, l in enumerate(layers):
        if l is None:
            continue
        (kq, ks, kb), (vq, vs, vb) = l
        arr[i].k_q, arr[i].k_scales, arr[i].k_biases = _packed(kq), desc(ks), desc(kb)
        arr[i].v_q, arr[i].v_scales, arr[i].v_biases = _packed(vq), desc(vs), desc(vb)
    return arr


def kv_chunk_save(path, layers, pos0, pos1):
    """Positions [pos0, pos1) of every layer's six buffers as one chunk file of the prefix cache's SSD tier
    (src/kv_disk_cache.zig:1062-1074)."""
    arr = _kv_layers(layers)
    check(lib().qb200_kv_chunk_save(str(path).encode(), arr, len(layers), int(pos0), int(pos1), _stream()))


def kv_chunk_restore(path, layers, pos0, need):
    """The first ``need`` positions stored in a chunk file into positions [pos0, pos0 + need) of the cache
    (restoreKvInto, src/kv_disk_cache.zig:320-440)."""
    arr = _kv_layers(layers)
    check(lib().qb200_kv_chunk_restore(str(path).encode(), arr, len(layers), int(pos0), int(need), _stream()))


class Checkpoint:
    """One MLX-format .safetensors file: names, shapes, and tensors copied to the device in the layout the operators
    take (loadWeights' role, src/model.zig; f16 quant scales/biases and 1-D tables arrive as bf16)."""

    def __init__(self, path):
        self._h = C.c_void_p()
        check(lib().qb200_checkpoint_open(C.byref(self._h), os.fsencode(path)))

    def close(self):
        if self._h:
            lib().qb200_checkpoint_close(self._h)
            self._h = C.c_void_p()

    def names(self):
        L = lib()
        return [L.qb200_checkpoint_tensor_name(self._h, i).decode() for i in range(L.qb200_checkpoint_num_tensors(self._h))]

    def info(self, name):
        d, n = Tensor(), C.c_size_t()
        check(lib().qb200_checkpoint_tensor_info(self._h, name.encode(), C.byref(d), C.byref(n)))
        return d.dtype, [d.shape[i] for i in range(d.ndim)], n.value

    def read(self, name):
        """Host bytes as they would be uploaded (numpy uint8)."""
        import numpy as np
        _, _, n = self.info(name)
        buf = np.empty(n, np.uint8)
        check(lib().qb200_checkpoint_read_tensor(self._h, name.encode(), buf.ctypes.data_as(C.c_void_p), n, None))
        return buf

    def load(self, name, device="cuda"):
        dt, shape, n = self.info(name)
        out = torch.empty(shape, dtype=_Q2TORCH[dt], device=device)
        check(lib().qb200_checkpoint_load_tensor(self._h, name.encode(), C.c_void_p(out.data_ptr()), n))
        return out

    def load_triple(self, prefix, in_dim, device="cuda"):
        """(codes, scales, biases) of the quantized linear `prefix` and its (bits, group_size) solved from the geometry
        and the layer's input width (affineParamsFromGeometry, src/transformer.zig:16763-16790)."""
        q, s, b = (self.load(f"{prefix}.{k}", device) for k in ("weight", "scales", "biases"))
        bits, gs = C.c_int(), C.c_int()
        check(lib().qb200_affine_params_from_geometry(q.shape[-1], s.shape[-1], int(in_dim), C.byref(bits), C.byref(gs)))
        return (q, s, b), bits.value, gs.value

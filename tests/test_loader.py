"""The checkpoint loader: safetensors container, the f16 -> bf16 narrowing rule (src/model.zig:3030-3061, test cases
:5590-5617), geometry solving (src/transformer.zig:16763-16790) and config.json's quantization object
(src/model.zig:1480-1505).  Host-side checks run without a GPU; the upload and a matmul on loaded weights need one."""
import ctypes as C
import json
import struct

import numpy as np
import pytest

from oracle import qoracle as qo

F16, BF16, U32, F32 = 9, 12, 3, 10


def write_safetensors(path, tensors, metadata=None):
    """tensors: {name: (dtype string, numpy array)} -> an MLX-style .safetensors file."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, (dt, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def make_checkpoint(tmp_path, rng, f16_side=True):
    w = qo.bf16_round((rng.standard_normal((96, 256)) * 0.05).astype(np.float32))
    q, s, b = qo.quantize(w, 64, 4)
    sf, bf = qo.bf16_to_f32(s), qo.bf16_to_f32(b)
    side = (lambda a: ("F16", a.astype(np.float16))) if f16_side else (lambda a: ("BF16", qo.f32_to_bf16(a)))
    tensors = {
        "model.layers.0.mlp.gate_proj.weight": ("U32", q),
        "model.layers.0.mlp.gate_proj.scales": side(sf),
        "model.layers.0.mlp.gate_proj.biases": side(bf),
        "model.layers.0.input_layernorm.weight": ("F16", (1 + 0.1 * rng.standard_normal(256)).astype(np.float16)),
        "model.embed.dense": ("F16", rng.standard_normal((4, 8)).astype(np.float16)),
    }
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors, {"format": "mlx"})
    return path, tensors, (q, s, b)


def test_reference_cases_of_the_narrowing_rule():
    import qb200
    f = qb200.lib().qb200_narrows_loaded_f16
    assert f(b"model.layers.0.mlp.down_proj.scales", 2, F16) and f(b"model.layers.0.mlp.down_proj.biases", 2, F16)
    for name in (b"language_model.model.layers.0.input_layernorm.weight", b"language_model.model.layers.0.linear_attn.A_log",
                 b"language_model.model.layers.0.linear_attn.dt_bias", b"language_model.model.norm.weight"):
        assert f(name, 1, F16)
    assert not f(b"vision_tower.blocks.0.attn.qkv.weight", 2, F16)
    assert not f(b"language_model.model.layers.0.linear_attn.conv1d.weight", 3, F16)
    assert not f(b"model.layers.0.input_layernorm.weight", 1, BF16)
    assert not f(b"model.layers.0.mlp.down_proj.weight", 2, U32)
    assert not f(b"model.layers.0.mlp.down_proj.scales", 2, BF16)


def test_geometry_and_config_quantization():
    import qb200
    L = qb200.lib()
    bits, gs = C.c_int(), C.c_int()
    assert L.qb200_affine_params_from_geometry(512, 64, 4096, C.byref(bits), C.byref(gs)) == 0 and (bits.value, gs.value) == (4, 64)
    assert L.qb200_affine_params_from_geometry(1024, 32, 4096, C.byref(bits), C.byref(gs)) == 0 and (bits.value, gs.value) == (8, 128)
    assert L.qb200_affine_params_from_geometry(96, 24, 768, C.byref(bits), C.byref(gs)) == 0 and (bits.value, gs.value) == (4, 32)
    assert L.qb200_affine_params_from_geometry(500, 64, 4096, C.byref(bits), C.byref(gs)) != 0      # 32*500 does not divide
    assert L.qb200_affine_params_from_geometry(896, 64, 4096, C.byref(bits), C.byref(gs)) == 1      # 7 bits: no such MLX mode
    mode = C.create_string_buffer(16)
    cfg = json.dumps({"model_type": "llama", "hidden_size": 4096, "rope_scaling": {"factor": 8.0, "type": "x"},
                      "quantization": {"group_size": 64, "bits": 4, "model.layers.0.mlp": {"bits": 8}}, "eos_token_id": [1, 2]})
    assert L.qb200_config_quantization(cfg.encode(), C.byref(bits), C.byref(gs), mode, 16) == 0
    assert (bits.value, gs.value, mode.value) == (4, 64, b"affine")
    cfg2 = json.dumps({"quantization": {"group_size": 32, "bits": 4, "mode": "mxfp4"}})
    assert L.qb200_config_quantization(cfg2.encode(), C.byref(bits), C.byref(gs), mode, 16) == 0 and mode.value == b"mxfp4"
    assert L.qb200_config_quantization(json.dumps({"quantization": {"bits": 7, "group_size": 64}}).encode(), C.byref(bits), C.byref(gs), mode, 16) == 1
    assert L.qb200_config_quantization(json.dumps({"hidden_size": 8}).encode(), C.byref(bits), C.byref(gs), mode, 16) == 1   # dense checkpoint
    assert L.qb200_config_quantization(b'{"quantization": {', C.byref(bits), C.byref(gs), mode, 16) == 5


def test_open_info_and_host_bytes(tmp_path):
    import qb200
    rng = np.random.default_rng(0)
    path, tensors, (q, s, b) = make_checkpoint(tmp_path, rng)
    ck = qb200.Checkpoint(path)
    try:
        assert sorted(ck.names()) == sorted(tensors)
        dt, shape, n = ck.info("model.layers.0.mlp.gate_proj.weight")
        assert (dt, shape, n) == (U32, [96, 32], 96 * 32 * 4)
        assert np.array_equal(ck.read("model.layers.0.mlp.gate_proj.weight").view(np.uint32).reshape(96, 32), q)
        # f16 scales / biases and the 1-D norm weight arrive as bf16: f16 -> f32 exactly, then round to nearest even
        for name in ("model.layers.0.mlp.gate_proj.scales", "model.layers.0.mlp.gate_proj.biases", "model.layers.0.input_layernorm.weight"):
            dt, shape, n = ck.info(name)
            assert dt == BF16
            want = qo.f32_to_bf16(tensors[name][1].astype(np.float32))
            assert np.array_equal(ck.read(name).view(np.uint16).reshape(want.shape), want)
        # a dense 2-D f16 weight keeps its dtype and bytes
        dt, _, _ = ck.info("model.embed.dense")
        assert dt == F16 and np.array_equal(ck.read("model.embed.dense").view(np.float16).reshape(4, 8), tensors["model.embed.dense"][1])
        with pytest.raises(qb200.Qb200Error):
            ck.info("model.layers.9.missing")
    finally:
        ck.close()


def test_broken_files_are_refused(tmp_path):
    import qb200
    rng = np.random.default_rng(1)
    path, _, _ = make_checkpoint(tmp_path, rng)
    raw = open(path, "rb").read()
    cut = str(tmp_path / "cut.safetensors")
    open(cut, "wb").write(raw[:len(raw) - 100])            # an interrupted download: data shorter than the header says
    with pytest.raises(qb200.Qb200Error):
        qb200.Checkpoint(cut)
    short = str(tmp_path / "short.safetensors")
    open(short, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(qb200.Qb200Error):
        qb200.Checkpoint(short)
    with pytest.raises(qb200.Qb200Error):
        qb200.Checkpoint(str(tmp_path / "absent.safetensors"))
    empty = str(tmp_path / "empty.safetensors")
    hj = json.dumps({"__metadata__": {"format": "mlx"}}).encode()
    open(empty, "wb").write(struct.pack("<Q", len(hj)) + hj)
    with pytest.raises(qb200.Qb200Error):
        qb200.Checkpoint(empty)                            # a weightless file is an error, not an empty map


@pytest.mark.gpu
def test_loaded_triple_feeds_the_operators(tmp_path):
    """Upload a quantized linear (f16 side tensors) and run it: same result as the oracle on the bf16-narrowed triple."""
    import torch
    import qb200
    from util import gate_bf16, rand_bf16, to_dev_bf16
    rng = np.random.default_rng(2)
    path, tensors, (q, s, b) = make_checkpoint(tmp_path, rng)
    ck = qb200.Checkpoint(path)
    try:
        (dq, ds, db), bits, gs = ck.load_triple("model.layers.0.mlp.gate_proj", 256)
        assert (bits, gs) == (4, 64) and ds.dtype == torch.bfloat16
        x = rand_bf16(rng, (3, 256))
        y = qb200.quantized_matmul(to_dev_bf16(qo.f32_to_bf16(x)), dq, ds, db, True, gs, bits)
        # the file's f16 side tensors were made from bf16 values, so narrowing gives the original triple back
        gate_bf16(y.float().cpu().numpy(), qo.qmm(x, q, s, b, 64, 4), "matmul on loaded weights")
        nw = ck.load("model.layers.0.input_layernorm.weight")
        assert nw.dtype == torch.bfloat16 and tuple(nw.shape) == (256,)
    finally:
        ck.close()

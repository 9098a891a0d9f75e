"""Chunk files of the quantized KV cache (the SSD tier of the reference's prefix cache, src/kv_disk_cache.zig): save,
restore into a cache of another capacity, slicing down an over-long chunk, refusing a corrupt one."""
import os

import numpy as np
import pytest
import torch

from oracle import qoracle as qo
from util import rand_bf16

pytestmark = pytest.mark.gpu


def _cache(rng, Hkv, cap, D, bits, filled):
    """Capacity buffers [1, Hkv, cap, .] whose first `filled` positions hold quantized rows, the rest a sentinel."""
    cols = D * bits // 32
    bq = np.full((1, Hkv, cap, cols), 0x7EADBEEF, np.uint32)
    bs = np.full((1, Hkv, cap, D // 64), 0x7FC0, np.uint16)
    bb = np.full((1, Hkv, cap, D // 64), 0x7FC0, np.uint16)
    if filled:
        q, s, b = qo.quantize(rand_bf16(rng, (1, Hkv, filled, D)), 64, bits)
        bq[:, :, :filled], bs[:, :, :filled], bb[:, :, :filled] = q, s, b
    dev = lambda a, dt: torch.from_numpy(a.view(np.int32 if a.dtype == np.uint32 else np.int16)).cuda().view(dt)
    return (dev(bq, torch.int32), dev(bs, torch.bfloat16), dev(bb, torch.bfloat16)), (bq, bs, bb)


def _host(t):
    return t.cpu().contiguous().view(torch.int32 if t.dtype == torch.int32 else torch.int16).numpy()


@pytest.mark.parametrize("bits", [4, 8])
def test_chunks_round_trip_into_a_cache_of_another_capacity(tmp_path, bits):
    import qb200
    rng = np.random.default_rng(bits)
    Hkv, D, T = 2, 128, 300
    src = [None if li == 1 else (_cache(rng, Hkv, 512, D, bits, T), _cache(rng, Hkv, 512, D, bits, T)) for li in range(3)]
    layers = [None if l is None else (l[0][0], l[1][0]) for l in src]
    c0, c1 = tmp_path / "c000000.safetensors", tmp_path / "c000001.safetensors"
    qb200.kv_chunk_save(c0, layers, 0, 256)
    qb200.kv_chunk_save(c1, layers, 256, T)
    # the files name their tensors and shapes as the reference's chunks do; the layer without a cache is absent
    ck = qb200.Checkpoint(str(c1))
    names = set(ck.names())
    assert names == {f"l{li}.{k}" for li in (0, 2) for k in ("k", "v", "ks", "kb", "vs", "vb")}
    assert tuple(ck.info("l0.k")[1]) == (1, Hkv, T - 256, D * bits // 32) and tuple(ck.info("l2.vs")[1]) == (1, Hkv, T - 256, D // 64)
    ck.close()
    # restore into fresh buffers of a different capacity
    dst = [None if li == 1 else (_cache(rng, Hkv, 384, D, bits, 0), _cache(rng, Hkv, 384, D, bits, 0)) for li in range(3)]
    dl = [None if l is None else (l[0][0], l[1][0]) for l in dst]
    qb200.kv_chunk_restore(c0, dl, 0, 256)
    qb200.kv_chunk_restore(c1, dl, 256, T - 256)
    for li in (0, 2):
        for kv in (0, 1):
            for j in range(3):
                got, want = _host(dl[li][kv][j]), _host(layers[li][kv][j])
                assert np.array_equal(got[:, :, :T], want[:, :, :T]), (li, kv, j)
                sentinel = dst[li][kv][1][j][:, :, T:]
                assert np.array_equal(got[:, :, T:], sentinel.view(got.dtype)), "positions beyond the restored range were touched"
    # a chunk that holds more positions than asked for is sliced down
    d2 = [None if li == 1 else (_cache(rng, Hkv, 384, D, bits, 0), _cache(rng, Hkv, 384, D, bits, 0)) for li in range(3)]
    d2l = [None if l is None else (l[0][0], l[1][0]) for l in d2]
    qb200.kv_chunk_restore(c0, d2l, 0, 100)
    got = _host(d2l[0][0][0])
    assert np.array_equal(got[:, :, :100], _host(layers[0][0][0])[:, :, :100])
    assert np.array_equal(got[:, :, 100:], d2[0][0][1][0][:, :, 100:].view(got.dtype))
    # fewer stored positions than asked for, or another geometry: a corrupt chunk
    with pytest.raises(qb200.Qb200Error):
        qb200.kv_chunk_restore(c1, dl, 256, T - 256 + 1)
    other = [None if li == 1 else (_cache(rng, 4, 384, D, bits, 0), _cache(rng, 4, 384, D, bits, 0)) for li in range(3)]
    with pytest.raises(qb200.Qb200Error):
        qb200.kv_chunk_restore(c0, [None if l is None else (l[0][0], l[1][0]) for l in other], 0, 256)
    # a file in which a present layer misses one of its six tensors
    raw = bytearray(open(c0, "rb").read())
    hl = int.from_bytes(raw[:8], "little")
    hdr = raw[8:8 + hl].decode().replace('"l2.vb"', '"l2.xx"')
    open(tmp_path / "bad.safetensors", "wb").write(raw[:8] + hdr.encode() + raw[8 + hl:])
    with pytest.raises(qb200.Qb200Error):
        qb200.kv_chunk_restore(tmp_path / "bad.safetensors", dl, 0, 256)
    assert not os.path.exists(str(c0) + ".tmp")

"""The rotation of the TurboQuant cache schemes (src/kv_quant.zig:164-403): the sign generator on the host (CPU), the
rotation kernel against the oracle's explicit matrix product and the rotate -> quantize -> dequantize -> rotate chain (GPU)."""
import numpy as np
import pytest
import torch

from oracle import qoracle as qo
from util import rand_bf16


def test_sign_vector_matches_the_oracles_generator():
    import qb200
    for seed, n in ((0x9E37, 128), (0x9E37 ^ 5, 64), (0x85EB ^ 31, 256), (7, 1024)):
        _, sg = qo.turbo_rotate(np.zeros((1, n), np.float32), seed, want_signs=True)
        assert qb200.turbo_signs(seed, n) == sg.tolist()
    assert sum(qb200.turbo_signs(0x9E37, 128)) not in (0, 128)


def test_oracle_rotation_is_orthogonal_and_its_own_inverse():
    rng = np.random.default_rng(1)
    x = rand_bf16(rng, (16, 128))
    y = qo.turbo_rotate(x, 0x85EB ^ 2)
    assert abs(np.linalg.norm(y) / np.linalg.norm(x) - 1.0) < 2e-3        # |entries| are bf16(1/sqrt(128)), two roundings
    back = qo.turbo_rotate(y, 0x85EB ^ 2)
    assert np.abs(back - x).max() <= 2.0 ** -6 * np.abs(x).max()


def test_bad_arguments_are_refused_on_the_host():
    import ctypes as C
    import qb200
    L = qb200.lib()
    x = qb200.raw_desc(0x1000, qb200.BFLOAT16, [4, 96], [96, 1])
    assert L.qb200_turbo_rotate(C.byref(x), C.byref(x), 1, None) == 1            # not a power of two: declined
    y = qb200.raw_desc(0x1000, qb200.BFLOAT16, [4, 2048], [2048, 1])
    assert L.qb200_turbo_rotate(C.byref(y), C.byref(y), 1, None) == 1
    assert L.qb200_turbo_signs(1, 0, None) == 5


@pytest.mark.gpu
@pytest.mark.parametrize("D", [32, 64, 128, 256, 1024])
def test_rotation_against_the_explicit_matrix_product(D):
    import qb200
    rng = np.random.default_rng(D)
    x = rand_bf16(rng, (3, 5, 7, D))
    seed = 0x9E37 ^ (D % 13)
    ref = qo.turbo_rotate(x, seed)
    dx = torch.from_numpy(qo.f32_to_bf16(x).view(np.int16)).view(torch.bfloat16).cuda()
    y = qb200.turbo_rotate(dx, seed).float().cpu().numpy()
    # the butterfly sums the same +-x_j in another order than the matrix product: equal up to the last fp32 bits before
    # the rounding to bf16, so nearly all outputs are identical and the rest one rounding step apart
    ulp = np.maximum(np.abs(ref), 2.0 ** -126) * 2.0 ** -7
    assert (np.abs(y - ref) <= ulp).all()
    assert (y == ref).mean() > 0.98
    # a strided view, in place; R is its own inverse
    wide = torch.zeros((8, 2 * D), dtype=torch.bfloat16, device="cuda")
    wide[:, :D] = dx.reshape(-1, D)[:8]
    view = wide[:, :D]
    qb200.turbo_rotate(view, seed, out=view)
    assert torch.equal(view.float().cpu(), torch.from_numpy(y.reshape(-1, D)[:8])) and float(wide[:, D:].abs().sum()) == 0.0
    back = qb200.turbo_rotate(view, seed).float().cpu().numpy()
    assert np.abs(back - x.reshape(-1, D)[:8]).max() <= 2.0 ** -6 * np.abs(x).max()


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [2, 4])
def test_quantize_turbo_round_trip(bits):
    """quantizeTurbo / dequantizeTurbo (src/kv_quant.zig:374-403): rotate, affine-quantize, dequantize, rotate back.  The codes
    equal the oracle's quantiser applied to the library's rotated rows, and the reconstruction error is the affine
    quantiser's (the rotation is orthogonal)."""
    import qb200
    rng = np.random.default_rng(bits)
    x = rand_bf16(rng, (2, 4, 33, 128))
    seed = 0x85EB ^ 1
    dx = torch.from_numpy(qo.f32_to_bf16(x).view(np.int16)).view(torch.bfloat16).cuda()
    rot = qb200.turbo_rotate(dx, seed)
    q, s, b = qb200.quantize(rot, 64, bits)
    rq, rs, rb = qo.quantize(rot.float().cpu().numpy(), 64, bits)
    assert np.array_equal(q.cpu().numpy().view(np.uint32), rq)
    assert np.array_equal(s.view(torch.int16).cpu().numpy().view(np.uint16), rs)
    deq = qb200.dequantize(q, s, b, 64, bits)
    back = qb200.turbo_rotate(deq, seed).float().cpu().numpy()
    err = np.sqrt(((back - x) ** 2).mean()) / np.sqrt((x ** 2).mean())
    plain = qb200.dequantize(*qb200.quantize(dx, 64, bits), 64, bits).float().cpu().numpy()
    err_plain = np.sqrt(((plain - x) ** 2).mean()) / np.sqrt((x ** 2).mean())
    assert err < 1.25 * err_plain + 5e-3, (err, err_plain)

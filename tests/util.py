"""Helpers shared by the GPU parity tests: seeded inputs, host<->device moves, comparison gates."""
import json
import os

import numpy as np
import torch

from oracle import qoracle as qo


def to_dev_bf16(u16: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).view(torch.bfloat16).cuda()


def to_dev_u32(w: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(w).view(np.int32)).cuda()


def from_dev_bf16(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit patterns."""
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def from_dev_u32(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().cpu().numpy().view(np.uint32)


def rand_bf16(rng, shape, std=1.0) -> np.ndarray:
    """fp32 array whose values are exactly representable in bf16."""
    return qo.bf16_round((rng.standard_normal(shape) * std).astype(np.float32))


def make_weight(rng, shape, gs, bits, std=0.02):
    """~N(0, std) weights -> bf16 -> affine quantize with the oracle.  Returns (q u32, s u16, b u16)."""
    return qo.quantize(rand_bf16(rng, shape, std), gs, bits)


def dev_triple(q, s, b):
    return to_dev_u32(q), to_dev_bf16(s), to_dev_bf16(b)


def rms(a):
    return float(np.sqrt(np.mean(np.square(a.astype(np.float64)))))


def bf16_ulp(v):
    a = np.maximum(np.abs(v.astype(np.float64)), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(a)) - 7)


_TABLE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gpurun_out", "parity_table.jsonl")


def record(config: str, what: str, max_over_rms: float, frac_half_ulp=None, n=None):
    """Append one row of the measured-tolerance table (literal max|delta|/RMS and, for bf16 outputs, the fraction of
    outputs within half a bf16 ulp of the oracle's unrounded value).  Written only where the scratch folder exists."""
    try:
        os.makedirs(os.path.dirname(_TABLE), exist_ok=True)
        with open(_TABLE, "a") as f:
            f.write(json.dumps({"config": config, "what": what, "max_abs_delta_over_rms": max_over_rms,
                                "frac_within_half_ulp": frac_half_ulp, "outputs": n}) + "\n")
    except OSError:
        pass


def half_ulp_fraction(got_f32: np.ndarray, ref_f32: np.ndarray) -> float:
    """Fraction of bf16 outputs that are the correctly rounded value of the oracle's fp32 result (or within half an ulp)."""
    d = np.abs(got_f32.astype(np.float64) - ref_f32.astype(np.float64))
    return float((d <= 0.5 * bf16_ulp(ref_f32) * (1 + 1e-6)).mean())


def gate_f32(got: np.ndarray, ref: np.ndarray, what=""):
    """fp32 outputs: max |delta| <= 1e-2 * RMS(ref) (the stated tolerance); NaN checked first."""
    assert not np.isnan(got).any(), f"{what}: NaN in output"
    r = rms(ref)
    d = float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max())
    assert d <= 1e-2 * r + 1e-30, f"{what}: max|d|={d:.3e} > 1e-2*rms={1e-2 * r:.3e}"
    return d / max(r, 1e-30)


def gate_bf16(got_f32: np.ndarray, ref_f32: np.ndarray, what="", slack=2e-3):
    """bf16 outputs against the oracle's UNROUNDED fp32 value: half a bf16 ulp of rounding plus
    ``slack`` * RMS of accumulation-order noise.  (A bf16 ulp at |y| >= 2 RMS already exceeds
    1e-2 * RMS, so the fp32 gate is applied in fp32-output mode and this one to bf16 outputs.)"""
    assert not np.isnan(got_f32).any(), f"{what}: NaN in output"
    r = rms(ref_f32)
    d = np.abs(got_f32.astype(np.float64) - ref_f32.astype(np.float64))
    allowed = 0.5 * bf16_ulp(ref_f32) * (1 + 1e-6) + slack * r
    bad = d > allowed
    assert not bad.any(), f"{what}: {int(bad.sum())} elements beyond half-ulp + {slack}*rms; worst {float((d - allowed).max()):.3e}, rms {r:.3e}"
    return float(d.max() / max(r, 1e-30))

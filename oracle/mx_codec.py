"""MX8 / MX4 block codec of the Mamba2 recurrent state (test oracle, numpy).

A row of ``N`` fp32 values is cut into blocks of 16.  Each block stores one biased 8-bit
exponent, each pair of values one "micro-exponent" bit, each value one signed mantissa in
[-M, M] (M = 63 for MX8, 7 for MX4):  value ~= q * 2**(shared_exp - 127 + micro).

Reference lines restated here (``hybrid_quant/mamba_state_8b_kernel.py``):
  * exponent / micro-exponent / mantissa of the in-kernel requantisers: :168-203 (fused MX8
    row kernel), :463-484 (``_requantize_mx8_kernel``), :511-534 (``_requantize_mx4_kernel``);
  * the torch quantiser applied once after prefill: ``_quantize_initial_state_mx`` :547-572
    (same formulas, but ``torch.round`` = round-half-even instead of ``floor(x + 0.5)``);
  * dequantisation: :132 and :322.

Canonical float semantics (what the reference's CPU/interpreter execution does): IEEE-754
fp32 division, a correctly rounded fp32 ``log2`` and ``ceil``.  ``ceil(fl32(log2 t))`` is
NOT the exact ceiling of log2: for t a few ulps above 2**k the rounded logarithm equals k.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def ceil_log2_f32(t: np.ndarray) -> np.ndarray:
    """``ceil(fl32(log2(t)))`` with the logarithm correctly rounded to fp32 (computed in
    float64 and rounded once).  ``t`` must be positive fp32."""
    t = np.asarray(t, dtype=F32)
    return np.ceil(np.log2(t.astype(np.float64)).astype(F32))


def _exp2_int(e: np.ndarray) -> np.ndarray:
    """Exact 2**e in fp32 for integer-valued e in [-149, 128] (ldexp, no libm rounding)."""
    return np.ldexp(F32(1.0), np.asarray(e).astype(np.int32)).astype(F32)


def mx_block_scales(vals: np.ndarray, mantissa_max: int):
    """Shared exponent, base scale and per-pair micro-exponent of every 16-value block.

    mamba_state_8b_kernel.py:170-174 / :188-191 (MX8), :513-520 (MX4), :559-566 (torch).
    Returns (biased_exp uint8 [..., N/16], micro uint8 [..., N/2], pair_scale f32 [..., N/2]).
    """
    vals = np.asarray(vals, dtype=F32)
    n = vals.shape[-1]
    if n % 16:
        raise ValueError(f"state dim must be divisible by 16, got {n}")
    m = F32(mantissa_max)
    blocks = vals.reshape(*vals.shape[:-1], n // 16, 16)
    amax = np.abs(blocks).max(axis=-1)
    t = np.maximum(amax / F32(2.0 * mantissa_max), F32(1.0e-30))
    raw = ceil_log2_f32(t)
    biased = np.minimum(np.maximum(raw + F32(127.0), F32(1.0)), F32(254.0))
    base = np.where(amax == 0, F32(1.0), _exp2_int(biased - F32(127.0))).astype(F32)
    pairs = blocks.reshape(*blocks.shape[:-1], 8, 2)
    pair_amax = np.abs(pairs).max(axis=-1)
    micro = (pair_amax > m * base[..., None]).astype(np.uint8)
    pair_scale = (base[..., None] * _exp2_int(micro)).astype(F32)
    lead = vals.shape[:-1]
    return biased.astype(np.uint8), micro.reshape(*lead, n // 2), pair_scale.reshape(*lead, n // 2)


def mx_encode(vals: np.ndarray, mantissa_max: int = 63, rounding: str = "half_up", rnd: np.ndarray | None = None):
    """Quantise fp32 ``vals[..., N]`` -> (q int8 [..., N], shared_exp uint8 [..., N/16],
    micro_exp uint8 [..., N/2]) in the reference's unpacked storage layout.

    rounding:
      'half_up'     ``floor(|v|/s + 0.5)`` in fp32, in-kernel deterministic mode (:201, :482, :532)
      'half_even'   ``round(clamp(|v|/s, 0, M))``, the torch initial quantiser (:568)
      'stochastic'  ``floor(a) + (rnd < a - floor(a))`` with ``rnd`` fp32 in [0,1) per value
                    (:196-199, :478-480, :528-530)
    """
    vals = np.asarray(vals, dtype=F32)
    m = F32(mantissa_max)
    biased, micro, pair_scale = mx_block_scales(vals, mantissa_max)
    scale = np.repeat(pair_scale, 2, axis=-1)
    q_abs = np.minimum(np.abs(vals) / scale, m)
    if rounding == "half_up":
        level = np.floor(q_abs + F32(0.5))
    elif rounding == "half_even":
        level = np.rint(q_abs)
    elif rounding == "stochastic":
        if rnd is None:
            raise ValueError("stochastic rounding needs rnd")
        fl = np.floor(q_abs)
        level = fl + (np.asarray(rnd, dtype=F32) < (q_abs - fl)).astype(F32)
    else:
        raise ValueError(rounding)
    level = np.minimum(level, m)
    q = np.where(vals < 0, -level, level).astype(np.int8)
    return q, biased, micro


def mx_decode(q: np.ndarray, shared_exp: np.ndarray, micro_exp: np.ndarray) -> np.ndarray:
    """``q * 2**(shared_exp - 127 + micro)`` in fp32 (mamba_state_8b_kernel.py:132)."""
    e = np.repeat(shared_exp.astype(np.int32), 16, axis=-1) - 127 + np.repeat(micro_exp.astype(np.int32), 2, axis=-1)
    return (q.astype(F32) * _exp2_int(e)).astype(F32)


# ---- bit-packed storage used natively by the CUDA library (18 B / 10 B per block) -------------

def mx_pack_micro_bits(micro: np.ndarray) -> np.ndarray:
    """[..., N/2] 0/1 bytes -> [..., N/16] bytes; bit i of byte g = pair i of block g."""
    m = micro.reshape(*micro.shape[:-1], micro.shape[-1] // 8, 8).astype(np.uint8)
    w = (m << np.arange(8, dtype=np.uint8)).sum(axis=-1)
    return w.astype(np.uint8)


def mx_unpack_micro_bits(bits: np.ndarray) -> np.ndarray:
    b = (bits[..., None] >> np.arange(8, dtype=np.uint8)) & 1
    return b.reshape(*bits.shape[:-1], bits.shape[-1] * 8).astype(np.uint8)


def mx4_pack_nibbles(q: np.ndarray) -> np.ndarray:
    """int8 codes in [-8, 7] -> two's-complement nibbles, element 2j low, 2j+1 high."""
    u = (q.astype(np.int16) & 15).astype(np.uint8)
    return (u[..., 0::2] | (u[..., 1::2] << 4)).astype(np.uint8)


def mx4_unpack_nibbles(p: np.ndarray) -> np.ndarray:
    lo = (p & 15).astype(np.int16)
    hi = (p >> 4).astype(np.int16)
    both = np.stack([lo, hi], axis=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)
    return np.where(both >= 8, both - 16, both).astype(np.int8)


# ---- the library's own fixed-point stochastic rounding ("layered" Philox stream) --------------

def native_sr_encode(vals: np.ndarray, mantissa_max: int, r8: np.ndarray):
    """Exponents exactly as :func:`mx_encode`; mantissa by fixed-point stochastic rounding with an
    8-bit uniform draw: ``t = fl32(v/s + 49152 + r8/256)`` (one rounding, as an FMA computes it),
    ``q = floor(t) - 49152`` with ``r8`` in [0, 255].  This has no counterpart in the reference
    (its rule is ``floor(a) + (u < frac)`` on a 31-bit uniform ``u``); it defines the library's
    ``LQ_ROUND_PHILOX_LAYERED`` / ``LQ_ROUND_SUPPLIED_FIXED`` modes."""
    vals = np.asarray(vals, dtype=F32)
    biased, micro, pair_scale = mx_block_scales(vals, mantissa_max)
    scale = np.repeat(pair_scale, 2, axis=-1).astype(np.float64)
    c = 49152.0 + np.asarray(r8, dtype=np.float64) / 256.0
    t = (vals.astype(np.float64) / scale + c).astype(F32)  # exact sum in float64, rounded once
    q = np.floor(t.astype(np.float64)) - 49152.0
    return q.astype(np.int8), biased, micro

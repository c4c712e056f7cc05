"""Fused Mamba2 selective-state update on an MX8/MX4-held state (test oracle, numpy fp32).

Restates ``_state_update_requant_mx8_row_kernel`` (``hybrid_quant/mamba_state_8b_kernel.py``
:97-222) and, for MX4, ``_state_update_mx8_kernel`` FORMAT_BITS=4 (:289-368, :429-443) followed by
``_requantize_mx4_kernel`` (:494-544), as driven by ``mx_state_selective_update`` (:601-721).
Operation order matches the kernels' fp32 expressions one numpy op per Triton op, so a run of
the reference under ``TRITON_INTERPRET=1`` (which also evaluates in numpy) is reproduced bit
for bit; see tests/golden/make_golden.py.
"""
from __future__ import annotations

import numpy as np

from .mx_codec import mx_decode, mx_encode, native_sr_encode
from .philox import philox4x32_10, tl_rand

F32 = np.float32


def _softplus(x):
    # mamba_state_8b_kernel.py:28-30
    with np.errstate(over="ignore"):
        return np.where(x <= F32(20.0), np.log(F32(1.0) + np.exp(x)), x).astype(F32)


def reference_rng_offsets(step: int, shape) -> np.ndarray:
    """Philox counters the reference draws for a state of ``shape`` = (B, H, P, N) at ``step``.

    offset = RNG_OFFSET + row_id * dstate + n with RNG_OFFSET = step*B*H*P*N (:197-198, :659).
    In-kernel arithmetic is 32-bit while RNG_OFFSET < 2**32 (a constexpr below 2**31 is int32,
    one in [2**31, 2**32) is uint32; both wrap to the low word with a zero high word); beyond that
    Triton promotes the sum to int64 and both counter words are used."""
    b, h, p, n = shape
    total = b * h * p * n
    idx = np.arange(total, dtype=np.uint64).reshape(shape)
    base = int(step) * total
    if base < (1 << 32):
        return (np.uint64(base) + idx) & np.uint64(0xFFFFFFFF)
    return np.uint64(base) + idx


def layered_r8(seed: int, layer: int, step: int, shape) -> np.ndarray:
    """8 random bits per state value for the library's own stream: one Philox4x32-10 block per
    16-value MX block, counter = (block_lo, block_hi, step, layer), key = seed; value i of a block
    takes byte i & 3 of word i >> 2."""
    total = int(np.prod(shape))
    blocks = np.arange((total + 15) // 16, dtype=np.uint64)
    s = int(seed) & 0xFFFFFFFFFFFFFFFF
    w = philox4x32_10(s & 0xFFFFFFFF, s >> 32, blocks & np.uint64(0xFFFFFFFF), blocks >> np.uint64(32),
                      int(step) & 0xFFFFFFFF, int(layer) & 0xFFFFFFFF)
    words = np.stack(w, axis=-1).astype(np.uint32)  # [blocks, 4]
    bytes_ = (words[..., None] >> (np.arange(4, dtype=np.uint32) * 8)) & np.uint32(0xFF)  # [blocks, 4, 4]
    return bytes_.reshape(-1)[:total].reshape(shape).astype(np.int64)


def layered4_words(seed: int, layer: int, step: int, shape) -> np.ndarray:
    """One 32-bit word per state value for LQ_ROUND_PHILOX_LAYERED4: one Philox4x32-10 block per four values,
    counter = (quad_lo, quad_hi, step, layer), key = seed; value i of a quad takes word i.  The reference's rounding
    rule is then fed ``words_to_uniform`` of these words."""
    total = int(np.prod(shape))
    quads = np.arange((total + 3) // 4, dtype=np.uint64)
    s = int(seed) & 0xFFFFFFFFFFFFFFFF
    w = philox4x32_10(s & 0xFFFFFFFF, s >> 32, quads & np.uint64(0xFFFFFFFF), quads >> np.uint64(32),
                      int(step) & 0xFFFFFFFF, int(layer) & 0xFFFFFFFF)
    return np.stack(w, axis=-1).astype(np.uint32).reshape(-1)[:total].reshape(shape)


def mx_state_update(q_state, shared_exp, micro_exp, x, dt, A, B, C, D=None, z=None, dt_bias=None,
                    dt_softplus=False, format_bits=8, rounding="stochastic", seed=1234, step=0,
                    layer=0, rnd=None, r8=None, return_state=False):
    """One decode step.  All array arguments are numpy, already broadcast to the shapes the
    reference indexes: q_state int8 [B,H,P,N]; shared_exp uint8 [B,H,P,N/16]; micro_exp uint8
    [B,H,P,N/2]; x, dt, z [B,H,P]; A [H,P,N]; B, C [B,G,N]; D, dt_bias [H,P].

    rounding: 'stochastic' (reference Philox stream from seed/step, or ``rnd`` if supplied),
    'half_up' (reference deterministic), 'layered' (library stream from seed/layer/step, or
    ``r8`` if supplied), 'layered4' (the reference's rule on the library's keying).
    Returns (y fp32 [B,H,P], q', shared_exp', micro_exp') and the fp32 state h' if asked."""
    mmax = 63 if format_bits == 8 else 7
    bsz, nh, dim, dstate = q_state.shape
    ratio = nh // B.shape[1]
    state = mx_decode(q_state, shared_exp, micro_exp)  # :132
    x = np.asarray(x, dtype=F32)
    dt = np.asarray(dt, dtype=F32).copy()
    if dt_bias is not None:
        dt = dt + np.asarray(dt_bias, dtype=F32)[None]  # :136-137
    if dt_softplus:
        dt = _softplus(dt)  # :138-139
    Bh = np.repeat(np.asarray(B, dtype=F32), ratio, axis=1)[:, :, None, :]  # group = head // ratio (:141)
    Ch = np.repeat(np.asarray(C, dtype=F32), ratio, axis=1)[:, :, None, :]
    A = np.asarray(A, dtype=F32)[None]
    with np.errstate(over="ignore", under="ignore"):
        dA = np.exp(A * dt[..., None])
        state = state * dA + Bh * dt[..., None] * x[..., None]  # :158
    y = (state * Ch).sum(axis=-1, dtype=F32)  # :159
    if D is not None:
        y = y + x * np.asarray(D, dtype=F32)[None]  # :160-162
    if z is not None:
        y = y * np.asarray(z, dtype=F32)  # :163-165
    state = state.astype(F32)
    if rounding == "layered4":
        from .philox import words_to_uniform
        q, e, m = mx_encode(state, mmax, "stochastic", words_to_uniform(layered4_words(seed, layer, step, state.shape)))
    elif rounding == "layered":
        if r8 is None:
            r8 = layered_r8(seed, layer, step, state.shape)
        q, e, m = native_sr_encode(state, mmax, r8)
    elif rounding == "stochastic":
        if rnd is None:
            rnd = tl_rand(seed, reference_rng_offsets(step, state.shape))  # :197-198
        q, e, m = mx_encode(state, mmax, "stochastic", rnd)
    else:
        q, e, m = mx_encode(state, mmax, rounding)
    if return_state:
        return y.astype(F32), q, e, m, state
    return y.astype(F32), q, e, m

"""Philox4x32-10 exactly as Triton's ``tl.rand`` / ``tl.randint`` use it (test oracle).

Follows ``triton/language/random.py``: ``philox_impl`` (:12-43), ``philox`` (:46-69),
``randint4x`` (:88-110), ``uint_to_uniform_float`` (:126-144), ``rand`` (:147-156).
Call sites in the reference: ``hybrid_quant/mamba_state_8b_kernel.py:198,405,479,529``.
"""
from __future__ import annotations

import numpy as np

PHILOX_KEY_A = np.uint64(0x9E3779B9)
PHILOX_KEY_B = np.uint64(0xBB67AE85)
PHILOX_ROUND_A = np.uint64(0xD2511F53)
PHILOX_ROUND_B = np.uint64(0xCD9E8D57)
_M32 = np.uint64(0xFFFFFFFF)
_S32 = np.uint64(32)


def philox4x32_10(k0, k1, c0, c1, c2, c3, n_rounds: int = 10):
    """Ten rounds of Philox-4x32 on uint32 counters (arrays or scalars, held as uint64)."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) & _M32 for c in (c0, c1, c2, c3))
    k0 = np.uint64(int(k0) & 0xFFFFFFFF)
    k1 = np.uint64(int(k1) & 0xFFFFFFFF)
    for _ in range(n_rounds):
        pb = PHILOX_ROUND_B * c2  # < 2**64: exact in uint64
        pa = PHILOX_ROUND_A * c0
        c0, c2 = ((pb >> _S32) ^ c1 ^ k0) & _M32, ((pa >> _S32) ^ c3 ^ k1) & _M32
        c1, c3 = pb & _M32, pa & _M32
        k0 = (k0 + PHILOX_KEY_A) & _M32
        k1 = (k1 + PHILOX_KEY_B) & _M32
    return c0.astype(np.uint32), c1.astype(np.uint32), c2.astype(np.uint32), c3.astype(np.uint32)


def _seed_key(seed: int):
    s = int(seed) & 0xFFFFFFFFFFFFFFFF  # tl.to_tensor(seed).to(uint64): two's complement
    return s & 0xFFFFFFFF, s >> 32


def tl_randint(seed: int, offset) -> np.ndarray:
    """Word 0 of ``tl.randint4x(seed, offset)``; ``offset`` is the full (64-bit) counter:
    low word -> c0, high word -> c1, c2 = c3 = 0 (random.py:100-110)."""
    off = np.asarray(offset, dtype=np.uint64)
    k0, k1 = _seed_key(seed)
    w0, _, _, _ = philox4x32_10(k0, k1, off & _M32, off >> _S32, 0, 0)
    return w0


def words_to_uniform(words) -> np.ndarray:
    """uint32 word -> float32 in [0, 1): bitcast to int32, ``x<0 ? -x-1 : x``, convert to
    fp32 (round to nearest) and multiply by fp32(4.6566127342e-10) (random.py:126-144)."""
    x = np.asarray(words, dtype=np.uint32).view(np.int32).astype(np.int64)
    x = np.where(x < 0, -x - 1, x)
    return x.astype(np.float32) * np.float32(4.6566127342e-10)


def tl_rand(seed: int, offset) -> np.ndarray:
    return words_to_uniform(tl_randint(seed, offset))

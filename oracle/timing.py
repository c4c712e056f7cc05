"""Timed CPU runs of the oracle port, for bench.py's ``cpu_baseline`` and ``--impl reference`` legs
only.  The reference has no CPU implementation of the fused state update (its torch code covers
only the one-off initial quantiser), so the baseline is this numpy restatement of its kernel
(mamba_state_8b_kernel.py:97-222), one batch slice per worker thread (numpy releases the GIL)."""
from __future__ import annotations

import os
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from .mx_codec import mx_encode
from .mx_state import mx_state_update

MX8_STATE_BYTES_PER_SEQ_LAYER = 8192 * 8 * 18 * 2  # 128 heads x 64 rows x 8 blocks x 18 B, read + written
MX4_STATE_BYTES_PER_SEQ_LAYER = 8192 * 8 * 10 * 2


def make_config1_inputs(batch: int, seed: int = 0, heads: int = 128, dim: int = 64, dstate: int = 128, groups: int = 8):
    """benchmark configuration 1 operands (numpy fp32 holding bf16-representable values where the model
    uses bf16): state ~ N(0, 0.5), x, B, C ~ N(0, 1), dt ~ N(0, 1) per head, dt_bias ~ U(-4, -2),
    A = -exp(U(0, ln 16)), D ~ U(0, 1)."""
    rng = np.random.default_rng(seed)

    def bf16(a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        u = a.view(np.uint32)
        u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
        return u.view(np.float32)

    return dict(
        state=(rng.standard_normal((batch, heads, dim, dstate)) * 0.5).astype(np.float32),
        x=bf16(rng.standard_normal((batch, heads, dim))), dt=bf16(rng.standard_normal((batch, heads))),
        A=(-np.exp(rng.random(heads) * np.log(16.0))).astype(np.float32),
        B=bf16(rng.standard_normal((batch, groups, dstate))), C=bf16(rng.standard_normal((batch, groups, dstate))),
        D=rng.random(heads).astype(np.float32), dt_bias=(rng.random(heads) * 2.0 - 4.0).astype(np.float32))


def time_mx_update(batch: int = 8, format_bits: int = 8, threads: int | None = None, repeats: int = 1, seed: int = 0):
    """Seconds per one-layer state update of ``batch`` sequences (stochastic rounding, reference
    Philox stream), best of ``repeats``.  Returns (seconds, threads_used, algorithmic_bytes)."""
    threads = threads or min(batch, os.cpu_count() or 1)
    d = make_config1_inputs(batch, seed)
    b, h, p, n = d["state"].shape
    mmax = 63 if format_bits == 8 else 7
    q, e, m = mx_encode(d["state"], mmax, "half_even")
    per_seq = MX8_STATE_BYTES_PER_SEQ_LAYER if format_bits == 8 else MX4_STATE_BYTES_PER_SEQ_LAYER
    bounds = np.linspace(0, b, threads + 1).astype(int)

    def work(i):
        lo, hi = bounds[i], bounds[i + 1]
        if lo == hi:
            return
        # each slice draws the counters the full-batch kernel would give its rows
        from .philox import tl_rand
        idx = np.arange(lo * h * p * n, hi * h * p * n, dtype=np.uint64).reshape(hi - lo, h, p, n)
        rnd = tl_rand(seed, idx & np.uint64(0xFFFFFFFF))
        mx_state_update(q[lo:hi], e[lo:hi], m[lo:hi], d["x"][lo:hi], np.broadcast_to(d["dt"][lo:hi, :, None], (hi - lo, h, p)),
                        np.broadcast_to(d["A"][:, None, None], (h, p, n)), d["B"][lo:hi], d["C"][lo:hi],
                        D=np.broadcast_to(d["D"][:, None], (h, p)), dt_bias=np.broadcast_to(d["dt_bias"][:, None], (h, p)),
                        dt_softplus=True, format_bits=format_bits, rounding="stochastic", rnd=rnd)

    best = float("inf")
    with ThreadPoolExecutor(max_workers=threads) as pool:
        for _ in range(repeats):
            t0 = time.perf_counter()
            list(pool.map(work, range(threads)))
            best = min(best, time.perf_counter() - t0)
    return best, threads, per_seq * batch

"""Timed CPU runs of the oracle port, for bench.py's ``cpu_baseline`` and ``--impl reference`` legs
only.  The reference has no CPU implementation of the fused state update (its torch code covers
only the one-off initial quantiser), so the baseline is this numpy restatement of its kernel
(mamba_state_8b_kernel.py:97-222), cut into (sequence, B/C group) pieces over the worker threads
(numpy releases the GIL).  kind = "port": this is NOT the reference's own code."""
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


def time_mx_update(batch: int = 8, format_bits: int = 8, threads: int | None = None, repeats: int = 1, seed: int = 0,
                   heads: int = 128, layers: int = 1):
    """Seconds per state update of ``layers`` layers (the same one-layer problem done ``layers`` times) of ``batch``
    sequences x ``heads`` heads (stochastic rounding, reference Philox stream), best of ``repeats``.  The work is
    cut into (sequence, B/C group) pieces dealt round-robin to ``threads`` workers, so every worker has work whenever batch x groups >= threads.
    Returns (seconds, threads that had work, algorithmic bytes, seconds of that spent drawing the
    Philox numbers): the draw is part of the reference kernel, so it is inside the timed region; it is
    reported separately because numpy evaluates Philox far less efficiently than the update."""
    threads = threads or (os.cpu_count() or 1)
    groups = 8
    d = make_config1_inputs(batch, seed, heads=heads, groups=groups)
    b, h, p, n = d["state"].shape
    hpg = h // groups
    mmax = 63 if format_bits == 8 else 7
    q, e, m = mx_encode(d["state"], mmax, "half_even")
    per_seq = (MX8_STATE_BYTES_PER_SEQ_LAYER if format_bits == 8 else MX4_STATE_BYTES_PER_SEQ_LAYER) * h // 128
    pieces = [(bi, g) for bi in range(b) for g in range(groups)]
    threads = min(threads, len(pieces))
    draw_seconds = [0.0] * threads
    from .philox import tl_rand

    def work(w):
        for bi, g in pieces[w::threads] * layers:
            h0, h1 = g * hpg, (g + 1) * hpg
            # the counters the full-batch kernel gives these rows (:197-198)
            t0 = time.perf_counter()
            first = (bi * h + h0) * p * n
            idx = np.arange(first, first + hpg * p * n, dtype=np.uint64).reshape(1, hpg, p, n)
            rnd = tl_rand(seed, idx & np.uint64(0xFFFFFFFF))
            draw_seconds[w] += time.perf_counter() - t0
            mx_state_update(q[bi:bi + 1, h0:h1], e[bi:bi + 1, h0:h1], m[bi:bi + 1, h0:h1], d["x"][bi:bi + 1, h0:h1],
                            np.broadcast_to(d["dt"][bi:bi + 1, h0:h1, None], (1, hpg, p)),
                            np.broadcast_to(d["A"][h0:h1, None, None], (hpg, p, n)), d["B"][bi:bi + 1, g:g + 1], d["C"][bi:bi + 1, g:g + 1],
                            D=np.broadcast_to(d["D"][h0:h1, None], (hpg, p)), dt_bias=np.broadcast_to(d["dt_bias"][h0:h1, None], (hpg, p)),
                            dt_softplus=True, format_bits=format_bits, rounding="stochastic", rnd=rnd)

    best, best_draw = float("inf"), 0.0
    with ThreadPoolExecutor(max_workers=threads) as pool:
        for _ in range(repeats):
            for w in range(threads):
                draw_seconds[w] = 0.0
            t0 = time.perf_counter()
            list(pool.map(work, range(threads)))
            sec = time.perf_counter() - t0
            if sec < best:
                best, best_draw = sec, max(draw_seconds)
    return best, threads, per_seq * batch * layers, best_draw

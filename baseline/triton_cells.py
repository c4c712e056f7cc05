"""The reference's own Triton kernels timed on the GPU this library runs on (``bench.py``'s
``triton_ref_*`` cells).  The kernels come unmodified from ``baseline/_ref`` (see
``baseline/reference.py``); this file only builds inputs of the benchmark shapes, calls the
reference's wrappers and times them with CUDA events.  Throughput uses the same algorithmic byte
counts as the library's own cells (160 / 144 B per token row for the INT4 cache, 18 / 10 B per
16-value MX block read and written), whatever the reference's storage layout moves.

The reference bakes the Philox offset (``step * numel``) into its MX kernels as a compile-time
constant, so every decode step re-compiles them.  The timed loops here hold ``cache.step`` fixed,
which excludes that cost; ``mx8_rejit_ms`` reports it separately (wall clock of one call at a step
not seen before, minus a warm call).
"""
from __future__ import annotations

import math
import time

import torch

L2_BYTES = 126e6


def _events(fn, iters: int, warmup: int = 2) -> float:
    """Mean seconds per call of ``fn`` over ``iters`` calls, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / iters


def attn_bytes(batch: int, ctx: int, gs: int, hkv: int = 8, hq: int = 32, d: int = 128) -> int:
    row = d // 2 * 2 + 2 * 4 * (d // gs)
    return batch * (hkv * ctx * row + hkv * row + 2 * hkv * d * 2 + 2 * hq * d * 2)


def decode_attention_cell(ia, batch: int, ctx: int, gs: int, dev, iters: int = 3) -> dict:
    """``_pack_kv_into_cache`` (one new token) + ``_decode_attention`` of the reference at
    (batch, context), rotating over enough distinct caches to defeat the L2."""
    hq, hkv, d = 32, 8, 128
    gen = torch.Generator(device=dev).manual_seed(7)
    nbytes = attn_bytes(batch, ctx, gs)
    reps = max(1, min(16, math.ceil(4 * L2_BYTES / nbytes)))
    caches = []
    for _ in range(reps):
        c = ia._allocate_layer_cache(batch, hkv, ctx, d, d // gs, dev)
        for t in (c.k_packed, c.v_packed):
            t.copy_(torch.randint(0, 256, t.shape, generator=gen, device=dev, dtype=torch.int16).to(torch.uint8))
        for t in (c.k_scale, c.v_scale):
            t.copy_(torch.rand(t.shape, generator=gen, device=dev) * 0.4 + 0.1)
        caches.append(c)
    q = torch.randn((batch, hq, 1, d), generator=gen, device=dev).to(torch.bfloat16)
    kn = torch.randn((batch, hkv, 1, d), generator=gen, device=dev).to(torch.bfloat16)
    vn = torch.randn((batch, hkv, 1, d), generator=gen, device=dev).to(torch.bfloat16)
    pos = torch.tensor([ctx - 1], device=dev)

    def attn_only():
        for c in caches:
            ia._decode_attention(q, c, ctx, hq // hkv, gs)

    def pack_only():
        for c in caches:
            ia._pack_kv_into_cache(c, kn, vn, pos, gs)  # two launches and a host sync, as shipped

    s_attn = _events(attn_only, iters) / reps
    s_pack = _events(pack_only, iters) / reps
    gbs = nbytes / (s_attn + s_pack) / 1e9
    return {"attn_us": round(s_attn * 1e6, 1), "pack_us": round(s_pack * 1e6, 1), "GBps": round(gbs, 2), "caches": reps,
            "group_size": gs}


def _update_operands(batch: int, dev, gen):
    h, p, n, g = 128, 64, 128, 8
    bf = torch.bfloat16
    return dict(
        x=torch.randn((batch, h, p), generator=gen, device=dev).to(bf),
        dt=torch.randn((batch, h), generator=gen, device=dev).to(bf)[:, :, None].expand(batch, h, p),
        A=(-torch.exp(torch.rand(h, generator=gen, device=dev) * math.log(16.0)))[:, None, None].expand(h, p, n),
        B=torch.randn((batch, g, n), generator=gen, device=dev).to(bf),
        C=torch.randn((batch, g, n), generator=gen, device=dev).to(bf),
        D=torch.rand(h, generator=gen, device=dev)[:, None].expand(h, p),
        dt_bias=(torch.rand(h, generator=gen, device=dev) * 2.0 - 4.0)[:, None].expand(h, p))


def mx8_update_cell(mk, batch: int, n_states: int, dev, iters: int = 3, rejit: bool = False) -> dict:
    """``mx_state_selective_update`` of the reference (fused MX8 row kernel) over ``n_states`` distinct
    layer states, ``cache.step`` held at 0 so that no call recompiles."""
    h, p, n = 128, 64, 128
    gen = torch.Generator(device=dev).manual_seed(11)
    o = _update_operands(batch, dev, gen)
    caches = [mk.allocate_state_kernel_cache(torch.randn((batch, h, p, n), generator=gen, device=dev) * 0.5, 16, 8)
              for _ in range(n_states)]

    def step():
        for c in caches:
            c.step = 0
            mk.mx_state_selective_update(c, o["x"], o["dt"], o["A"], o["B"], o["C"], D=o["D"], dt_bias=o["dt_bias"],
                                         dt_softplus=True, stochastic=True, seed=0)

    sec = _events(step, iters) / n_states
    nbytes = batch * h * p * (n // 16) * 18 * 2
    out = {"us_per_launch": round(sec * 1e6, 1), "GBps": round(nbytes / sec / 1e9, 2), "states": n_states}
    if rejit:
        c = caches[0]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        c.step = 0
        mk.mx_state_selective_update(c, o["x"], o["dt"], o["A"], o["B"], o["C"], D=o["D"], dt_bias=o["dt_bias"],
                                     dt_softplus=True, stochastic=True, seed=0)
        torch.cuda.synchronize()
        warm = time.perf_counter() - t0
        t0 = time.perf_counter()
        c.step = 7  # an offset no earlier call used: the reference compiles a new kernel for it
        mk.mx_state_selective_update(c, o["x"], o["dt"], o["A"], o["B"], o["C"], D=o["D"], dt_bias=o["dt_bias"],
                                     dt_softplus=True, stochastic=True, seed=0)
        torch.cuda.synchronize()
        out["mx8_rejit_ms"] = round((time.perf_counter() - t0 - warm) * 1e3, 1)
    return out


def mx4_update_cell(mk, batch: int, n_states: int, dev, iters: int = 3) -> dict:
    """The reference's MX4 pair (tiled update into an fp32 temporary + ``_requantize_mx4_kernel``).  Its
    wrapper raises TypeError for MX4 as shipped (the tiled kernel is not given its HAS_* flags), so the
    two kernels are launched directly with those flags, everything else as the wrapper passes it."""
    h, p, n, g = 128, 64, 128, 8
    gen = torch.Generator(device=dev).manual_seed(13)
    o = _update_operands(batch, dev, gen)
    caches = [mk.allocate_state_kernel_cache(torch.randn((batch, h, p, n), generator=gen, device=dev) * 0.5, 16, 4)
              for _ in range(n_states)]
    y = torch.empty_like(o["x"])
    tmp = torch.empty((batch, h, p, n), dtype=torch.float32, device=dev)
    rows = batch * h * p

    def step():
        for c in caches:
            mk._state_update_mx8_kernel[((p + 15) // 16, batch, h)](
                c.q_state, c.shared_exp, c.micro_exp, o["x"], o["dt"], o["dt_bias"], o["A"], o["B"], o["C"], o["D"], None, y, tmp,
                h // g, *c.q_state.stride(), *c.shared_exp.stride(), *c.micro_exp.stride(), *o["x"].stride(), *o["dt"].stride(),
                *o["A"].stride(), *o["B"].stride(), *o["C"].stride(), *o["D"].stride(), 0, 0, 0, *y.stride(), p, n, True,
                HAS_DT_BIAS=True, HAS_D=True, HAS_Z=False, FORMAT_BITS=4, STOCHASTIC=True, RNG_SEED=0, RNG_OFFSET=0,
                BLOCK_SIZE_M=16, BLOCK_SIZE_N=n)
            mk._requantize_mx4_kernel[(rows * (n // 16),)](tmp, c.q_state, c.shared_exp, c.micro_exp, rows, n, True, 0, 0)

    sec = _events(step, iters) / n_states
    nbytes = batch * h * p * (n // 16) * 10 * 2
    return {"us_per_step": round(sec * 1e6, 1), "GBps": round(nbytes / sec / 1e9, 2), "states": n_states}

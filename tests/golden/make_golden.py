"""Generate tests/golden/*.npz by running the UNMODIFIED reference (phcool/Layer_Quant) on CPU.

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference /path/to/Layer_Quant
    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference /path/to/Layer_Quant --check

``--check`` regenerates every fixture into a temporary directory and compares it array by array
with the committed files (exit status 1 on any difference); nothing in the tree is written.

The reference's Triton kernels are executed by Triton's interpreter (numpy on CPU); its torch
helpers run as they are.  Every file stores the inputs and the reference's outputs, so the
tests need neither the reference nor Triton.  ``_pack_int4_kv_kernel`` contains inline PTX and
cannot be interpreted; its arithmetic is pinned through ``int4_quant_dequant`` (same scale,
rounding and clamp expressions) instead.  ``mx_state_selective_update`` raises TypeError for
MX4 as shipped (the tiled kernel lacks the HAS_* heuristics), so the two MX4 kernels are
launched directly with those flags passed explicitly.
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bf16_round(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).bfloat16()


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def codec_edge_rows() -> np.ndarray:
    """fp32 rows of 128 that hit the codec's float corner cases."""
    rng = np.random.default_rng(7)
    rows = []
    # block maxima straddling 2M * 2**k by a few ulps, both formats (126 and 14)
    for two_m in (126.0, 14.0):
        for k in list(range(-30, 31, 3)) + [-100, -99, -98, 100, 120]:
            for j in (0, 1, 2, 3, 5, 6, 9):
                top = np.float32(two_m) * np.ldexp(np.float32(1), k)
                top = np.nextafter(top, np.float32(np.inf), dtype=np.float32) if j else top
                for _ in range(max(j - 1, 0)):
                    top = np.nextafter(top, np.float32(np.inf), dtype=np.float32)
                row = (rng.standard_normal(128).astype(np.float32) * top * np.float32(0.3))
                row = np.clip(row, -top, top)
                row[::16] = top * np.where(rng.random(8) < 0.5, -1, 1).astype(np.float32)
                rows.append(row.astype(np.float32))
    # exact ties (x.5 levels), pair maxima exactly at M*base, zeros, signed zeros, tiny, huge
    base = np.float32(2.0 ** -3)
    tie = (np.arange(128, dtype=np.float32) % 63 + np.float32(0.5)) * base
    tie[0] = np.float32(126.0) * base * np.float32(0.99)
    rows.append(tie)
    rows.append(-tie)
    edge = np.zeros(128, np.float32)
    edge[0] = 100.0
    edge[2:4] = [63.0, -63.0]
    edge[4:6] = [63.0000038, 1.0]
    edge[6:8] = [7.0, -7.0000005]
    edge[16] = -0.0
    rows.append(edge)
    rows.append(np.zeros(128, np.float32))
    rows.append(np.full(128, -0.0, np.float32))
    rows.append((rng.standard_normal(128) * 1e-36).astype(np.float32))
    rows.append((rng.standard_normal(128) * 1e-41).astype(np.float32))
    rows.append((rng.standard_normal(128) * 1e37).astype(np.float32))
    big = (rng.standard_normal(128)).astype(np.float32)
    big[5] = np.float32(3.0e38)
    rows.append(big)
    for s in (1e-3, 0.5, 40.0):
        rows.append((rng.standard_normal(128) * s).astype(np.float32))
    return np.stack(rows).astype(np.float32)


def gen_philox(out: Path):
    import triton
    import triton.language as tl

    @triton.jit
    def k32(out_i, out_f, off_ptr, seed, n: tl.constexpr):
        i = tl.arange(0, n)
        off = tl.load(off_ptr + i)
        tl.store(out_i + i, tl.randint(seed, off))
        tl.store(out_f + i, tl.rand(seed, off))

    res = {}
    off32 = np.array([0, 1, 2, 3, 12345, 2**31 - 1, -1, -2**31, 65536, 99999999, 7, 8, 9, 10, 11, 12], dtype=np.int32)
    off64 = np.array([0, 1, 2**31, 2**32 + 5, 2**40, 2**32 - 1, 2**32, 2**33 + 17], dtype=np.int64)
    for seed in (0, 1234, 2**31 - 1, 2**40 + 3):
        for name, off in (("i32", off32), ("i64", off64)):
            oi = torch.zeros(len(off), dtype=torch.int32)
            of = torch.zeros(len(off), dtype=torch.float32)
            k32[(1,)](oi, of, torch.from_numpy(off), seed, len(off))
            res[f"seed{seed}_{name}_off"] = off
            res[f"seed{seed}_{name}_word"] = oi.numpy().view(np.uint32)
            res[f"seed{seed}_{name}_rand"] = of.numpy()
    np.savez_compressed(out / "philox_kat.npz", **res)


def gen_codec(out: Path, mk):
    rows = codec_edge_rows()
    n_rows, n = rows.shape
    res = {"vals": rows}
    st = torch.from_numpy(rows)
    for bits, kern, mmax in ((8, mk._requantize_mx8_kernel, 63.0), (4, mk._requantize_mx4_kernel, 7.0)):
        q0, e0, m0 = mk._quantize_initial_state_mx(st, format_bits=bits, block_size=16, pair_size=2, mantissa_max=mmax)
        res[f"init{bits}_q"], res[f"init{bits}_e"], res[f"init{bits}_m"] = q0.numpy(), e0.numpy(), m0.numpy()
        for tag, stoch, seed, off in (("det", False, 0, 0), ("sr", True, 1234, 0), ("sr2", True, 0, 3 * n_rows * n)):
            q = torch.zeros(n_rows, n, dtype=torch.int8)
            e = torch.zeros(n_rows, n // 16, dtype=torch.uint8)
            m = torch.zeros(n_rows, n // 2, dtype=torch.uint8)
            kern[(n_rows * (n // 16),)](st, q, e, m, n_rows, n, stoch, seed, off)
            res[f"mx{bits}_{tag}_q"], res[f"mx{bits}_{tag}_e"], res[f"mx{bits}_{tag}_m"] = q.numpy(), e.numpy(), m.numpy()
            res[f"mx{bits}_{tag}_seed_off"] = np.array([seed, off], dtype=np.int64)
    np.savez_compressed(out / "mx_codec.npz", **res)


def make_update_inputs(seed, b, h, p, n, g, with_d=True, with_z=False, with_bias=True, state_sigma=0.5):
    gen = torch.Generator().manual_seed(seed)
    state = torch.randn(b, h, p, n, generator=gen) * state_sigma
    # bf16-representable values held in fp32: outputs then come back as exact fp32 (the
    # interpreter truncates instead of rounding when it stores fp32 into a bf16 tensor)
    x = torch.randn(b, h, p, generator=gen).bfloat16().float()
    dt = torch.randn(b, h, generator=gen).bfloat16().float()
    a = -torch.exp(torch.rand(h, generator=gen) * float(np.log(16.0)))
    bm = torch.randn(b, g, n, generator=gen).bfloat16().float()
    cm = torch.randn(b, g, n, generator=gen).bfloat16().float()
    d = torch.rand(h, generator=gen) if with_d else None
    z = torch.randn(b, h, p, generator=gen).bfloat16().float() if with_z else None
    bias = (torch.rand(h, generator=gen) * 2.0 - 4.0) if with_bias else None
    return state, x, dt, a, bm, cm, d, z, bias


def gen_update(out: Path, mk):
    cases = [
        # name, bits, (B,H,P,N,G), D, z, bias, softplus, stochastic, seed, steps
        ("mx8_sr", 8, (2, 4, 4, 128, 2), True, False, True, True, True, 0, 2),
        ("mx8_det_z", 8, (1, 2, 3, 128, 1), True, True, False, False, False, 0, 1),
        ("mx8_sr_nod", 8, (1, 2, 4, 64, 2), False, False, True, True, True, 1234, 1),
        ("mx4_sr", 4, (2, 2, 16, 128, 1), True, False, True, True, True, 0, 2),
        ("mx4_det", 4, (1, 2, 16, 128, 2), True, True, True, True, False, 0, 1),
    ]
    for name, bits, (b, h, p, n, g), wd, wz, wb, sp, stoch, seed, steps in cases:
        state, x, dt, a, bm, cm, d, z, bias = make_update_inputs(11 + len(name), b, h, p, n, g, wd, wz, wb)
        cache = mk.allocate_state_kernel_cache(state, 16, bits)
        res = dict(state0=state.numpy(), x=f32(x), dt=f32(dt), A=a.numpy(), B=f32(bm), C=f32(cm),
                   q_init=cache.q_state.numpy().copy(), e_init=cache.shared_exp.numpy().copy(), m_init=cache.micro_exp.numpy().copy(),
                   meta=np.array([bits, int(sp), int(stoch), seed, steps], dtype=np.int64))
        if d is not None:
            res["D"] = d.numpy()
        if z is not None:
            res["z"] = f32(z)
        if bias is not None:
            res["dt_bias"] = bias.numpy()
        dt_e = dt[:, :, None].expand(b, h, p)
        a_e = a[:, None, None].expand(h, p, n)
        d_e = d[:, None].expand(h, p) if d is not None else None
        bias_e = bias[:, None].expand(h, p) if bias is not None else None
        for s in range(steps):
            if bits == 8:
                y = mk.mx_state_selective_update(cache, x, dt_e, a_e, bm, cm, D=d_e, z=z, dt_bias=bias_e,
                                                 dt_softplus=sp, stochastic=stoch, seed=seed)
            else:
                y = torch.empty_like(x)
                tmp = torch.empty(cache.q_state.shape, dtype=torch.float32)
                ds = d_e.stride() if d_e is not None else (0, 0)
                zs = z.stride() if z is not None else (0, 0, 0)
                mk._state_update_mx8_kernel[((p + 15) // 16, b, h)](
                    cache.q_state, cache.shared_exp, cache.micro_exp, x, dt_e, bias_e, a_e, bm, cm, d_e, z, y, tmp,
                    h // g, *cache.q_state.stride(), *cache.shared_exp.stride(), *cache.micro_exp.stride(),
                    *x.stride(), *dt_e.stride(), *a_e.stride(), *bm.stride(), *cm.stride(), *ds, *zs, *y.stride(),
                    p, n, sp, HAS_DT_BIAS=bias_e is not None, HAS_D=d_e is not None, HAS_Z=z is not None,
                    FORMAT_BITS=4, STOCHASTIC=stoch, RNG_SEED=seed, RNG_OFFSET=cache.step * b * h * p * n,
                    BLOCK_SIZE_M=16, BLOCK_SIZE_N=n)
                rows = b * h * p
                mk._requantize_mx4_kernel[(rows * (n // 16),)](tmp, cache.q_state, cache.shared_exp, cache.micro_exp,
                                                               rows, n, stoch, seed, cache.step * rows * n)
                cache.step += 1
                res[f"h{s}"] = tmp.numpy().copy()
            res[f"y{s}"] = f32(y)
            res[f"q{s}"] = cache.q_state.numpy().copy()
            res[f"e{s}"] = cache.shared_exp.numpy().copy()
            res[f"m{s}"] = cache.micro_exp.numpy().copy()
        np.savez_compressed(out / f"update_{name}.npz", **res)
        print("update", name, flush=True)


def gen_attention(out: Path, ia):
    gen = torch.Generator().manual_seed(0)
    # codec pin through the reference's fake-quant
    x = torch.randn(3, 2, 5, 128, generator=gen)
    x[0, 0, 0, :32] = 0.0
    x[0, 0, 1, 3] = 8.0 * 5
    x[1, 1, 2] *= 1e-9
    x[2, 0, 3, ::2] = x[2, 0, 3, 0]  # many identical magnitudes -> ties after division
    tie = torch.arange(-8, 8, dtype=torch.float32).repeat(8) * 0.5 + 0.25
    x[2, 1, 4] = tie
    res = {"codec_x": x.numpy()}
    for gs in (16, 32, 64, 128):
        res[f"codec_qdq_gs{gs}"] = ia.int4_quant_dequant(x, gs).numpy()
    np.savez_compressed(out / "int4_codec.npz", **res)

    from oracle import int4_encode, int4_pack_nibbles  # layout :86-97; arithmetic pinned above
    cases = [("t1", 1, 8, 2, 1, 32, None), ("t63", 2, 8, 2, 63, 32, None), ("t64", 1, 4, 1, 64, 64, None),
             ("t65", 1, 8, 2, 65, 32, None), ("t200_mask", 2, 8, 2, 200, 64, "add4d"), ("t130_bool", 2, 4, 4, 130, 32, "bool2d")]
    for name, b, hq, hkv, t, gs, mk_ in cases:
        q = torch.randn(b, hq, 1, 128, generator=gen).bfloat16().float()  # fp32 carrier -> fp32 output
        k = torch.randn(b, hkv, t, 128, generator=gen).bfloat16()
        v = torch.randn(b, hkv, t, 128, generator=gen).bfloat16()
        sel = torch.rand(b, hkv, t, 128, generator=gen) < 0.01
        k = torch.where(sel, torch.full_like(k, 8.0), k)
        cap = max(16, 1 << int(np.ceil(np.log2(max(t, 1)))))
        cache = ia._allocate_layer_cache(b, hkv, cap, 128, 128 // gs, torch.device("cpu"))
        for t_ in (cache.k_packed, cache.v_packed):
            t_.fill_(0x77)
        for t_ in (cache.k_scale, cache.v_scale):
            t_.fill_(1.0e3)
        kq, ks = int4_encode(f32(k), gs)
        vq, vs = int4_encode(f32(v), gs)
        cache.k_packed[:, :, :t] = torch.from_numpy(int4_pack_nibbles(kq))
        cache.v_packed[:, :, :t] = torch.from_numpy(int4_pack_nibbles(vq))
        cache.k_scale[:, :, :t] = torch.from_numpy(ks)
        cache.v_scale[:, :, :t] = torch.from_numpy(vs)
        mask = None
        if mk_ == "add4d":
            mask = torch.zeros(b, 1, 1, t)
            mask[:, :, :, 70:90] = -float("inf")
            mask[1, :, :, 5] = -2.5
        elif mk_ == "bool2d":
            mask = torch.ones(b, t, dtype=torch.bool)
            mask[0, 64:100] = False
            mask[1, 3] = False
        o = ia._decode_attention(q, cache, t, hq // hkv, gs, attention_mask=mask)
        d = dict(q=f32(q), k=f32(k), v=f32(v), k_packed=cache.k_packed.numpy(), v_packed=cache.v_packed.numpy(),
                 k_scale=cache.k_scale.numpy(), v_scale=cache.v_scale.numpy(), out=f32(o),
                 meta=np.array([b, hq, hkv, t, gs], dtype=np.int64))
        if mask is not None:
            d["mask"] = mask.numpy()
        np.savez_compressed(out / f"attn_{name}.npz", **d)
        print("attn", name, flush=True)


def gen_prefill(out: Path, ia):
    """The reference's own causal kernel over the packed cache (_int4_prefill_attention_kernel,
    launched through _prefill_attention): a kernel the reference defines but never calls."""
    from oracle import int4_encode, int4_pack_nibbles
    gen = torch.Generator().manual_seed(5)
    cases = [("p70_gs32", 1, 4, 2, 70, 32), ("p33_gs64", 2, 8, 2, 33, 64), ("p17_g1", 1, 2, 2, 17, 128)]
    for name, b, hq, hkv, t, gs in cases:
        q = torch.randn(b, hq, t, 128, generator=gen).bfloat16().float()  # fp32 carrier -> fp32 output
        k = torch.randn(b, hkv, t, 128, generator=gen).bfloat16()
        v = torch.randn(b, hkv, t, 128, generator=gen).bfloat16()
        sel = torch.rand(b, hkv, t, 128, generator=gen) < 0.01
        k = torch.where(sel, torch.full_like(k, 8.0), k)
        cap = max(16, 1 << int(np.ceil(np.log2(max(t, 1)))))
        cache = ia._allocate_layer_cache(b, hkv, cap, 128, 128 // gs, torch.device("cpu"))
        for t_ in (cache.k_packed, cache.v_packed):
            t_.fill_(0x77)
        for t_ in (cache.k_scale, cache.v_scale):
            t_.fill_(1.0e3)
        kq, ks = int4_encode(f32(k), gs)
        vq, vs = int4_encode(f32(v), gs)
        cache.k_packed[:, :, :t] = torch.from_numpy(int4_pack_nibbles(kq))
        cache.v_packed[:, :, :t] = torch.from_numpy(int4_pack_nibbles(vq))
        cache.k_scale[:, :, :t] = torch.from_numpy(ks)
        cache.v_scale[:, :, :t] = torch.from_numpy(vs)
        o = ia._prefill_attention(q, cache, hq // hkv, gs)
        np.savez_compressed(out / f"prefill_{name}.npz", q=f32(q), k_packed=cache.k_packed.numpy(), v_packed=cache.v_packed.numpy(),
                            k_scale=cache.k_scale.numpy(), v_scale=cache.v_scale.numpy(), out=f32(o),
                            meta=np.array([b, hq, hkv, t, gs], dtype=np.int64))
        print("prefill", name, flush=True)


def compare_dirs(fresh: Path, committed: Path) -> int:
    """Array-by-array comparison of two fixture directories; returns the number of differences."""
    bad = 0
    names = sorted(p.name for p in fresh.glob("*.npz"))
    for name in names:
        if not (committed / name).exists():
            print(f"MISSING  {name}: not committed")
            bad += 1
            continue
        a, b = np.load(fresh / name), np.load(committed / name)
        if sorted(a.files) != sorted(b.files):
            print(f"DIFFERENT {name}: array names differ")
            bad += 1
            continue
        diff = [k for k in a.files if a[k].dtype != b[k].dtype or a[k].shape != b[k].shape
                or a[k].tobytes() != b[k].tobytes()]
        if diff:
            print(f"DIFFERENT {name}: {diff}")
            bad += 1
        else:
            print(f"identical {name} ({len(a.files)} arrays)")
    return bad


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a phcool/Layer_Quant checkout (imported, never copied)")
    ap.add_argument("--only", default="", help="comma-separated subset of philox,codec,update,attn,prefill")
    ap.add_argument("--check", action="store_true", help="regenerate into a temporary directory and compare with the committed files")
    args = ap.parse_args()
    ref = Path(args.reference).resolve()
    root = HERE.parents[1]
    # The reference checkout comes FIRST on the path: this repository has a package called hybrid_quant
    # too (its drop-in aliases), which must not shadow the reference's.  The repository root goes last and
    # only supplies `oracle` (the nibble layout used to fill the attention fixtures' caches).
    sys.path[:] = [p for p in sys.path if Path(p or ".").resolve() != root]
    sys.path.insert(0, str(ref))
    sys.path.append(str(root))
    from hybrid_quant import int4_8b_attention as ia
    from hybrid_quant import mamba_state_8b_kernel as mk
    for mod in (ia, mk):
        assert Path(mod.__file__).resolve().is_relative_to(ref), f"{mod.__name__} came from {mod.__file__}, not from the reference"
    todo = args.only.split(",") if args.only else ["philox", "codec", "update", "attn", "prefill"]
    out = HERE
    tmp = None
    if args.check:
        import tempfile
        tmp = tempfile.TemporaryDirectory()
        out = Path(tmp.name)
    if "philox" in todo:
        gen_philox(out)
    if "codec" in todo:
        gen_codec(out, mk)
    if "update" in todo:
        gen_update(out, mk)
    if "attn" in todo:
        gen_attention(out, ia)
    if "prefill" in todo:
        gen_prefill(out, ia)
    if args.check:
        bad = compare_dirs(out, HERE)
        tmp.cleanup()
        print("check:", "FAILED" if bad else "all regenerated fixtures are bit-identical to the committed ones")
        sys.exit(1 if bad else 0)


if __name__ == "__main__":
    main()

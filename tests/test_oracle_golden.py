"""The CPU oracle against fixtures produced by the reference itself (tests/golden/make_golden.py:
the reference's Triton kernels under TRITON_INTERPRET=1 and its torch helpers).  Bit-exact for
the codecs and the Philox words; the fused update reproduces the interpreter run bit for bit."""
import glob

import numpy as np
import pytest

import oracle


def test_philox_known_answers(golden_dir):
    k = np.load(golden_dir / "philox_kat.npz")
    checked = 0
    for name in k.files:
        if not name.endswith("_off"):
            continue
        seed = int(name.split("_")[0][4:])
        kind = name.split("_")[1]
        off = k[name]
        off64 = off.astype(np.int64).astype(np.uint64) if kind == "i64" else off.view(np.uint32).astype(np.uint64)
        assert np.array_equal(oracle.tl_randint(seed, off64), k[name[:-3] + "word"]), name
        assert np.array_equal(oracle.tl_rand(seed, off64), k[name[:-3] + "rand"]), name
        checked += 1
    assert checked == 8
    # the words quoted for triton 3.6.0's tl.randint(seed, offset)
    assert [int(v) for v in oracle.tl_randint(1234, [0, 1, 2, 3])] == [0x2090B348, 0x9EEEDE35, 0x3FC9C8D8, 0xB6269A3E]
    assert [int(v) for v in oracle.tl_randint(0, [2**31, 2**32 + 5, 2**40])] == [0xBF9C529B, 0xAC2FBCCA, 0x1EE5E208]


@pytest.mark.parametrize("bits", [8, 4])
def test_mx_codec_matches_reference_kernels(golden_dir, bits):
    g = np.load(golden_dir / "mx_codec.npz")
    vals = g["vals"]
    mmax = 63 if bits == 8 else 7
    q, e, m = oracle.mx_encode(vals, mmax, "half_even")
    assert np.array_equal(q, g[f"init{bits}_q"]) and np.array_equal(e, g[f"init{bits}_e"]) and np.array_equal(m, g[f"init{bits}_m"])
    q, e, m = oracle.mx_encode(vals, mmax, "half_up")
    assert np.array_equal(q, g[f"mx{bits}_det_q"]) and np.array_equal(e, g[f"mx{bits}_det_e"]) and np.array_equal(m, g[f"mx{bits}_det_m"])
    for tag in ("sr", "sr2"):
        seed, off = (int(v) for v in g[f"mx{bits}_{tag}_seed_off"])
        offs = (np.uint64(off) + np.arange(vals.size, dtype=np.uint64)).reshape(vals.shape)
        q, e, m = oracle.mx_encode(vals, mmax, "stochastic", oracle.tl_rand(seed, offs))
        assert np.array_equal(q, g[f"mx{bits}_{tag}_q"]), tag
        assert np.array_equal(e, g[f"mx{bits}_{tag}_e"]) and np.array_equal(m, g[f"mx{bits}_{tag}_m"])


def test_mx_decode_roundtrip_and_packing():
    rng = np.random.default_rng(3)
    vals = (rng.standard_normal((5, 7, 128)) * 3).astype(np.float32)
    for mmax in (63, 7):
        q, e, m = oracle.mx_encode(vals, mmax, "half_up")
        dec = oracle.mx_decode(q, e, m)
        # re-encoding a decoded state is the identity (values are exactly representable)
        q2, e2, m2 = oracle.mx_encode(dec, mmax, "half_up")
        assert np.array_equal(oracle.mx_decode(q2, e2, m2), dec)
        assert np.abs(q).max() <= mmax
        bits = oracle.mx_pack_micro_bits(m)
        assert bits.shape == (5, 7, 8) and np.array_equal(oracle.mx_unpack_micro_bits(bits), m)
    q4, _, _ = oracle.mx_encode(vals, 7, "half_up")
    assert np.array_equal(oracle.mx4_unpack_nibbles(oracle.mx4_pack_nibbles(q4)), q4)


def _load_update(path):
    g = np.load(path)
    bits, sp, stoch, seed, steps = (int(v) for v in g["meta"])
    q = g["q_init"]
    b, h, p, n = q.shape
    bias = None
    if "dt_bias" in g:
        # the reference kernel addresses dt_bias with D's strides (mamba_state_8b_kernel.py:137), which
        # are (0, 0) when D is None: every head then reads dt_bias[0]
        bias = np.broadcast_to(g["dt_bias"][:, None], (h, p)) if "D" in g else np.full((h, p), g["dt_bias"][0], np.float32)
    args = dict(
        x=g["x"], dt=np.broadcast_to(g["dt"][:, :, None], (b, h, p)), A=np.broadcast_to(g["A"][:, None, None], (h, p, n)),
        B=g["B"], C=g["C"], D=np.broadcast_to(g["D"][:, None], (h, p)) if "D" in g else None,
        z=g["z"] if "z" in g else None, dt_bias=bias,
        dt_softplus=bool(sp), format_bits=bits, rounding="stochastic" if stoch else "half_up", seed=seed)
    return g, args, steps


@pytest.mark.parametrize("path", sorted(glob.glob(str(__import__("pathlib").Path(__file__).parent / "golden" / "update_*.npz"))))
def test_fused_update_matches_reference_interpreter(path):
    g, args, steps = _load_update(path)
    mmax = 63 if args["format_bits"] == 8 else 7
    q0, e0, m0 = oracle.mx_encode(g["state0"], mmax, "half_even")
    assert np.array_equal(q0, g["q_init"]) and np.array_equal(e0, g["e_init"]) and np.array_equal(m0, g["m_init"])
    q, e, m = g["q_init"], g["e_init"], g["m_init"]
    for s in range(steps):
        y, q, e, m, h = oracle.mx_state_update(q, e, m, step=s, return_state=True, **args)
        assert np.array_equal(q, g[f"q{s}"]), f"step {s}: {(q != g[f'q{s}']).sum()} codes differ"
        assert np.array_equal(e, g[f"e{s}"]) and np.array_equal(m, g[f"m{s}"])
        if f"h{s}" in g:
            assert np.array_equal(h, g[f"h{s}"])
        np.testing.assert_allclose(y, g[f"y{s}"], rtol=2e-5, atol=2e-5 * np.abs(g[f"y{s}"]).max())


def test_int4_codec_matches_reference_fake_quant(golden_dir):
    g = np.load(golden_dir / "int4_codec.npz")
    x = g["codec_x"]
    for gs in (16, 32, 64, 128):
        assert np.array_equal(oracle.int4_quant_dequant(x, gs), g[f"codec_qdq_gs{gs}"]), gs
        q, s = oracle.int4_encode(x, gs)
        assert q.min() >= -8 and q.max() <= 7
        assert np.array_equal(oracle.int4_unpack_nibbles(oracle.int4_pack_nibbles(q)), q)


@pytest.mark.parametrize("name", ["t1", "t63", "t64", "t65", "t200_mask", "t130_bool"])
def test_decode_attention_matches_reference_kernel(golden_dir, name):
    g = np.load(golden_dir / f"attn_{name}.npz")
    b, hq, hkv, t, gs = (int(v) for v in g["meta"])
    # the fixture's cache rows are what the oracle codec produces from the stored K/V
    kq, ks = oracle.int4_encode(g["k"], gs)
    assert np.array_equal(oracle.int4_pack_nibbles(kq), g["k_packed"][:, :, :t]) and np.array_equal(ks, g["k_scale"][:, :, :t])
    bias = oracle.decode_attention_mask(g["mask"], b, t) if "mask" in g else None
    o = oracle.int4_decode_attention(g["q"][:, :, 0], g["k_packed"], g["v_packed"], g["k_scale"], g["v_scale"], t, gs, bias)
    ref = g["out"]  # fp32 output of the reference kernel (fp32 accumulation)
    assert np.abs(o - ref).max() <= 2e-5 * np.abs(ref).max()


@pytest.mark.parametrize("name", ["p70_gs32", "p33_gs64", "p17_g1"])
def test_prefill_attention_matches_reference_kernel(golden_dir, name):
    """The reference's own causal kernel over the packed cache (_int4_prefill_attention_kernel, run under the
    interpreter through _prefill_attention) against the prefill restatement."""
    g = np.load(golden_dir / f"prefill_{name}.npz")
    b, hq, hkv, t, gs = (int(v) for v in g["meta"])
    o = oracle.int4_prefill_attention(g["q"], g["k_packed"], g["v_packed"], g["k_scale"], g["v_scale"], 1, gs)
    ref = g["out"]  # fp32 output of the reference kernel
    assert ref.shape == (b, hq, t, 128)
    assert np.abs(o - ref).max() <= 2e-5 * np.abs(ref).max()


def test_ceil_log2_is_not_exact_ceiling():
    # a few ulps above a power of two the rounded fp32 logarithm is still the integer
    t = np.nextafter(np.float32(2.0 ** -10), np.float32(1.0))
    assert oracle.ceil_log2_f32(np.array([t]))[0] == -10.0
    assert oracle.ceil_log2_f32(np.array([np.float32(2.0 ** -10 * 1.001)]))[0] == -9.0
    assert oracle.ceil_log2_f32(np.array([np.nextafter(np.float32(1.0), np.float32(2.0))]))[0] == 1.0


def test_prefill_oracle_is_the_decode_oracle_per_position():
    """The causal prefill restatement must equal the decode restatement (pinned by the reference fixtures) run
    on every query position alone."""
    import numpy as np
    import oracle
    rng = np.random.default_rng(3)
    b, hkv, ratio, tq, first, gs = 2, 2, 4, 9, 5, 32
    total = first + tq - 1
    k = rng.standard_normal((b, hkv, total, 128)).astype(np.float32)
    v = rng.standard_normal((b, hkv, total, 128)).astype(np.float32)
    kc, ks = oracle.int4_encode(k, gs)
    vc, vs = oracle.int4_encode(v, gs)
    kp, vp = oracle.int4_pack_nibbles(kc), oracle.int4_pack_nibbles(vc)
    q = rng.standard_normal((b, hkv * ratio, tq, 128)).astype(np.float32)
    whole = oracle.int4_prefill_attention(q, kp, vp, ks, vs, first, gs)
    for i in range(tq):
        one = oracle.int4_decode_attention(q[:, :, i], kp, vp, ks, vs, first + i, gs)
        np.testing.assert_allclose(whole[:, :, i], one, rtol=1e-12, atol=1e-12)


def _dense_from_fixture(g):
    """Operands of the un-quantised update for a reference-run MX fixture: the decoded initial state as a dense fp32
    state, everything else as the reference kernel was given it."""
    bits, sp, stoch, seed, steps = (int(v) for v in g["meta"])
    b, h, p, n = g["q_init"].shape
    bias = None
    if "dt_bias" in g:  # the MX kernel addresses dt_bias with D's strides: without D every head reads element 0
        bias = np.broadcast_to(g["dt_bias"][:, None], (h, p)) if "D" in g else np.full((h, p), g["dt_bias"][0], np.float32)
    state = oracle.mx_decode(g["q_init"], g["e_init"], g["m_init"])
    ops = dict(x=g["x"], dt=np.broadcast_to(g["dt"][:, :, None], (b, h, p)), A=np.broadcast_to(g["A"][:, None, None], (h, p, n)),
               B=g["B"], C=g["C"], D=np.broadcast_to(g["D"][:, None], (h, p)) if "D" in g else None, dt_bias=bias,
               dt_softplus=bool(sp))
    return state, ops


@pytest.mark.parametrize("name", ["mx8_sr", "mx8_sr_nod", "mx4_sr"])
def test_dense_update_oracle_is_pinned_by_the_reference_mx_kernels(golden_dir, name):
    """The reference's MX kernels compute h' = h exp(A dt) + (B dt) x and y = <h', C> + D x in fp32 on the decoded state
    before they requantise it: the same expression the un-quantised update evaluates.  Their y (and the MX4 pair's fp32
    h', which the fixture keeps) therefore pin the dense-state restatement for the un-gated case."""
    g = np.load(golden_dir / f"update_{name}.npz")
    state, ops = _dense_from_fixture(g)
    h, y = oracle.dense_state_update(state, **ops)
    assert np.abs(y - g["y0"]).max() <= 2e-6 * np.abs(g["y0"]).max()
    if "h0" in g:
        assert np.array_equal(h, g["h0"])

"""Host-side mirror of the reference interface that needs no GPU: cache bookkeeping, masks,
positions, the torch fake-quantiser, error behaviour and the drop-in import path."""
import numpy as np
import pytest
import torch

import oracle


def test_drop_in_import_path_and_names():
    import hybrid_quant.int4_8b_attention as a
    import hybrid_quant.mamba_state_8b_kernel as m
    for name in ("Int4KVLayerCache", "int4_quant_dequant", "patch_nemotron_h_attention_int4_kv", "_allocate_layer_cache",
                 "_ensure_layer_cache", "_pack_kv_into_cache", "_decode_attention", "_forward_fused_int4_kv"):
        assert hasattr(a, name), name
    for name in ("MX8_BLOCK_SIZE", "MX8_PAIR_SIZE", "MX8_MANTISSA_MAX", "MX4_BLOCK_SIZE", "MX4_PAIR_SIZE", "MX4_MANTISSA_MAX",
                 "MambaStateKernelCache", "allocate_state_kernel_cache", "mx_state_selective_update", "mx8_state_selective_update",
                 "mx4_state_selective_update", "patch_nemotron_h_mamba_decode_state_kernel", "register_mamba_state_kernel_caches"):
        assert hasattr(m, name), name
    assert (m.MX8_BLOCK_SIZE, m.MX8_MANTISSA_MAX, m.MX4_MANTISSA_MAX) == (16, 63.0, 7.0)
    import inspect
    sig = inspect.signature(m.mx_state_selective_update)
    assert list(sig.parameters)[:12] == ["cache", "x", "dt", "A", "B", "C", "D", "z", "dt_bias", "dt_softplus", "stochastic", "seed"]
    assert sig.parameters["seed"].default == 1234 and sig.parameters["stochastic"].default is True
    assert inspect.signature(a.patch_nemotron_h_attention_int4_kv).parameters["group_size"].default == 64
    c = m.MambaStateKernelCache(torch.zeros(1), torch.zeros(1), torch.zeros(1))
    assert (c.format_bits, c.step) == (8, 0)


def test_fake_quant_matches_oracle_and_golden(golden_dir):
    from layer_quant_b200.int4_8b_attention import int4_quant_dequant
    g = np.load(golden_dir / "int4_codec.npz")
    x = torch.from_numpy(g["codec_x"])
    for gs in (16, 32, 64, 128):
        assert np.array_equal(int4_quant_dequant(x, gs).numpy(), g[f"codec_qdq_gs{gs}"])
    assert int4_quant_dequant(x.bfloat16(), 32).dtype == torch.bfloat16
    with pytest.raises(ValueError, match="must be divisible by group_size=48"):
        int4_quant_dequant(x, 48)


def test_cache_allocation_growth_on_cpu_tensors():
    from layer_quant_b200 import int4_8b_attention as a

    class Holder:
        pass

    pkv = Holder()
    cpu = torch.device("cpu")
    c = a._ensure_layer_cache(pkv, 3, 2, 8, 1, 128, 64, cpu)
    assert c.k_packed.shape == (2, 8, 16, 64) and c.k_packed.dtype == torch.uint8
    assert c.v_scale.shape == (2, 8, 16, 2) and c.v_scale.dtype == torch.float32
    assert a._cache_dict(pkv)[3] is c
    c.k_packed.fill_(7); c.k_scale.fill_(1.5); c.length = 16
    g = a._ensure_layer_cache(pkv, 3, 2, 8, 100, 128, 64, cpu)
    assert g.k_packed.shape[2] == 128 and g.length == 16
    assert (g.k_packed[:, :, :16] == 7).all() and (g.k_scale[:, :, :16] == 1.5).all()
    assert a._ensure_layer_cache(pkv, 5, 1, 2, 1025, 128, 64, cpu).k_packed.shape[2] == 2048
    with pytest.raises(ValueError, match="does not match batch/kv_heads"):
        a._ensure_layer_cache(pkv, 3, 4, 8, 1, 128, 64, cpu)


def test_positions_and_masks():
    from layer_quant_b200 import int4_8b_attention as a
    cpu = torch.device("cpu")
    assert a._positions(None, 4, cpu).tolist() == [0, 1, 2, 3]
    assert a._positions(torch.tensor([9]), 1, cpu).dtype == torch.long
    with pytest.raises(ValueError, match="cache_position has 2 entries for q_len=3"):
        a._positions(torch.tensor([1, 2]), 3, cpu)
    assert a._decode_attention_mask(None, 2, 5, cpu) is None
    m4 = torch.zeros(2, 1, 3, 9)
    m4[:, :, -1, 2] = -1.5
    out = a._decode_attention_mask(m4, 2, 5, cpu)
    assert out.shape == (2, 1, 1, 5) and out.dtype == torch.float32 and out[0, 0, 0, 2] == -1.5
    b4 = torch.ones(2, 1, 1, 5, dtype=torch.bool)
    b4[1, 0, 0, 4] = False
    out = a._decode_attention_mask(b4, 2, 5, cpu)
    assert out[1, 0, 0, 4] == -float("inf") and out[0].abs().sum() == 0
    k2 = torch.ones(2, 8)
    k2[0, -1] = 0
    out = a._decode_attention_mask(k2, 2, 5, cpu)
    assert out.shape == (2, 1, 1, 5) and out[0, 0, 0, 4] == -float("inf")
    for mask in (m4, b4, k2):
        got = a._decode_attention_mask(mask, 2, 5, cpu)[:, 0, 0].numpy()
        assert np.array_equal(got, oracle.decode_attention_mask(mask.numpy(), 2, 5))
    with pytest.raises(ValueError, match="only supports 2D or 4D"):
        a._decode_attention_mask(torch.zeros(2, 3, 4), 2, 5, cpu)


def test_kernels_refuse_cpu_tensors():
    from layer_quant_b200 import int4_8b_attention as a, mamba_state_8b_kernel as m
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        m.allocate_state_kernel_cache(torch.zeros(1, 2, 4, 128))
    cache = a._allocate_layer_cache(1, 2, 16, 128, 4, torch.device("cpu"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        a._decode_attention(torch.zeros(1, 8, 1, 128), cache, 4, 4, 32)
    with pytest.raises(ValueError, match="expects q_len=1"):
        a._decode_attention(torch.zeros(1, 8, 2, 128), cache, 4, 4, 32)


def test_state_cache_validation_without_device():
    from layer_quant_b200 import mamba_state_8b_kernel as m
    st = torch.zeros(1, 2, 4, 128)
    with pytest.raises(ValueError, match="fixed 16-value block"):
        m.allocate_state_kernel_cache(st, group_size=8)
    with pytest.raises(ValueError, match="Only MX8 and MX4"):
        m.allocate_state_kernel_cache(st, format_bits=16)
    with pytest.raises(ValueError, match="must be divisible by 16, got 24"):
        m.allocate_state_kernel_cache(torch.zeros(1, 2, 4, 24))
    c = m.MambaStateKernelCache(torch.zeros(1, 2, 4, 64, dtype=torch.uint8), torch.zeros(1, 2, 4, 8, dtype=torch.uint8),
                                torch.zeros(1, 2, 4, 8, dtype=torch.uint8), format_bits=4, layout="packed")
    assert c.state_shape == (1, 2, 4, 128)
    with pytest.raises(ValueError, match="Expected x shape"):
        m.mx_state_selective_update(c, torch.zeros(1, 2, 5), None, None, torch.zeros(1, 1, 128), torch.zeros(1, 1, 128))


class _FakeRemote:
    """Stands in for the HF remote modeling module the patch functions reach through
    ``model.__class__.__module__``."""


def test_patch_functions_route_by_state_identity(monkeypatch):
    import sys
    import types
    from layer_quant_b200 import mamba_state_8b_kernel as m
    mod = types.ModuleType("fake_nemotron_remote")
    calls = []
    mod.selective_state_update = lambda ssm_state, *a, **k: calls.append("original") or "orig"
    mod.repeat_kv = lambda x, n: x
    sys.modules["fake_nemotron_remote"] = mod
    Model = type("Model", (), {})
    Model.__module__ = "fake_nemotron_remote"
    model = Model()
    m.patch_nemotron_h_mamba_decode_state_kernel(model, stochastic=False, seed=7)
    assert mod._mx_state_kernel_patched and mod._mx_state_kernel_seed == 7 and mod._mx_state_kernel_stochastic is False
    assert model._mx_state_kernel_group_size == 16
    patched = mod.selective_state_update
    m.patch_nemotron_h_mamba_decode_state_kernel(model, stochastic=True, seed=9)  # second call: no double wrap
    assert mod.selective_state_update is patched and mod._mx_state_kernel_seed == 9
    state = torch.zeros(2, 3)
    assert mod.selective_state_update(state, 1, 2, 3, 4, 5) == "orig" and calls == ["original"]
    seen = {}
    monkeypatch.setattr(m, "mx_state_selective_update", lambda cache, *a, **k: seen.update(cache=cache, **k) or "mx")
    mod._mamba_decode_state_kernel_caches = {id(state): "the-cache"}
    assert mod.selective_state_update(state, 1, 2, 3, 4, 5, dt_softplus=True) == "mx"
    assert seen["cache"] == "the-cache" and seen["seed"] == 9 and seen["stochastic"] is True and seen["dt_softplus"] is True
    with pytest.raises(ValueError, match="Only MX8 and MX4 state caches"):
        m.register_mamba_state_kernel_caches(model, None, {0: "int8"})
    # attention patch: only attention blocks, once
    from layer_quant_b200 import int4_8b_attention as a
    mixers = [types.SimpleNamespace(forward=lambda **k: "orig") for _ in range(3)]
    model.backbone = types.SimpleNamespace(layers=[types.SimpleNamespace(block_type=bt, mixer=mx)
                                                   for bt, mx in zip(("mamba", "attention", "mlp"), mixers)])
    a.patch_nemotron_h_attention_int4_kv(model, group_size=32)
    assert getattr(mixers[1], "_int4_kv_patched", False) and mixers[1]._int4_kv_group_size == 32
    assert not hasattr(mixers[0], "_int4_kv_patched") and not hasattr(mixers[2], "_int4_kv_patched")
    fwd = mixers[1].forward
    a.patch_nemotron_h_attention_int4_kv(model, group_size=64)
    assert mixers[1].forward is fwd and mixers[1]._int4_kv_group_size == 32
    # non-CUDA input falls through to the original forward, as in the reference
    assert mixers[1].forward(torch.zeros(1, 1, 8), past_key_value=object()) == "orig"


def test_exponent_table_matches_oracle_formula():
    """The device look-up table (lq_exp_table.h) against ceil(log2()) evaluated by the oracle."""
    import re
    from pathlib import Path
    src = (Path(__file__).resolve().parents[1] / "layer_quant_b200" / "csrc" / "lq_exp_table.h").read_text()
    rng = np.random.default_rng(0)
    for name, mmax, shift in (("LQ_MX8_EXP_CUT", 63, 6), ("LQ_MX4_EXP_CUT", 7, 3)):
        body = src.split(name + "[256] = {")[1].split("};")[0]
        cut = np.array([int(x, 16) for x in re.findall(r"0x([0-9A-F]+)u", body)], dtype=np.uint32)
        assert cut.shape == (256,)
        bits = rng.integers(0, 0x7F800000, size=400_000, dtype=np.uint32)
        near = [(np.uint32(f) << np.uint32(23)) | np.clip(np.arange(int(cut[f]) - 40, int(cut[f]) + 40), 0, 0x7FFFFF).astype(np.uint32)
                for f in range(1, 255)]
        bits = np.concatenate([bits] + near)
        amax = bits.view(np.float32)
        vals = np.zeros((len(amax), 16), np.float32)
        vals[:, 3] = amax
        _, e, _ = oracle.mx_encode(vals, mmax, "half_up")
        f = (bits >> 23).astype(np.int64)
        mine = np.maximum(f - shift + ((bits & 0x7FFFFF) > cut[f]).astype(np.int64), 28)
        assert np.array_equal(mine, e[:, 0].astype(np.int64)), name


def test_required_len_without_device_round_trip():
    from layer_quant_b200 import int4_8b_attention as a
    cpu = torch.device("cpu")
    assert a._required_len(a._positions(None, 7, cpu), None, 7) == 7
    cp = torch.tensor([40, 41, 42])
    assert a._required_len(a._positions(cp, 3, cpu), cp, 3) == 43
    with pytest.raises(ValueError, match="prepare_graph_decode needs the caches"):
        a.prepare_graph_decode(object.__new__(type("Cache", (), {})), 64)


def test_recorded_launch_helpers_validate_on_the_host():
    from layer_quant_b200 import int4_8b_attention as a
    cache = a._allocate_layer_cache(1, 2, 16, 128, 4, torch.device("cpu"))
    with pytest.raises(ValueError, match="expects q_len=1"):
        a.Int4DecodePlan(torch.zeros(1, 8, 2, 128), cache, 4, 32)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        a.Int4DecodePlan(torch.zeros(1, 8, 1, 128), cache, 4, 32)


def test_unquantised_baselines_validate_on_the_host():
    from layer_quant_b200 import dense_state as d
    state = torch.zeros(2, 4, 8, 32)
    x = torch.zeros(2, 4, 8)
    A = torch.zeros(4, 8, 32)
    B = torch.zeros(2, 2, 32)
    with pytest.raises(ValueError, match="do not match state"):
        d.selective_state_update(state, x[:, :, :4], x, A, B, B)
    with pytest.raises(ValueError, match="A .* does not match"):
        d.selective_state_update(state, x, x, A[:, :, :16], B, B)
    with pytest.raises(ValueError, match="not a multiple"):
        d.selective_state_update(state, x, x, A, torch.zeros(2, 3, 32), torch.zeros(2, 3, 32))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        d.selective_state_update(state, x, x, A, B, B)
    conv = torch.zeros(2, 6, 4)
    with pytest.raises(NotImplementedError):
        d.causal_conv1d_update(torch.zeros(2, 6), conv, torch.zeros(6, 4), activation="relu")
    with pytest.raises(ValueError, match="weight"):
        d.causal_conv1d_update(torch.zeros(2, 6), conv, torch.zeros(6, 3))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        d.causal_conv1d_update(torch.zeros(2, 6), conv, torch.zeros(6, 4))


def test_dense_oracle_against_plain_torch():
    """The CPU restatement of the unquantised step against an independent torch formulation (fp64)."""
    rng = np.random.default_rng(0)
    b, h, p, n, g = 2, 4, 3, 16, 2
    state = rng.standard_normal((b, h, p, n)).astype(np.float32)
    x, dt = rng.standard_normal((b, h, p)).astype(np.float32), rng.standard_normal((b, h, p)).astype(np.float32)
    A = -np.exp(rng.standard_normal((h, p, n))).astype(np.float32)
    B, C = rng.standard_normal((b, g, n)).astype(np.float32), rng.standard_normal((b, g, n)).astype(np.float32)
    D, z, bias = rng.random((h, p)).astype(np.float32), rng.standard_normal((b, h, p)).astype(np.float32), rng.random((h, p)).astype(np.float32)
    hq, y = oracle.dense_state_update(state, x, dt, A, B, C, D, z, bias, True)
    T = lambda v: torch.from_numpy(v).double()
    dts = torch.nn.functional.softplus(T(dt) + T(bias))
    Bh, Ch = T(B).repeat_interleave(h // g, 1)[:, :, None], T(C).repeat_interleave(h // g, 1)[:, :, None]
    want_h = T(state) * torch.exp(T(A) * dts[..., None]) + Bh * (dts * T(x))[..., None]
    want_y = ((want_h * Ch).sum(-1) + T(x) * T(D)) * torch.nn.functional.silu(T(z))
    np.testing.assert_allclose(hq, want_h.numpy(), rtol=2e-5, atol=1e-6)
    np.testing.assert_allclose(y, want_y.numpy(), rtol=2e-5, atol=2e-5)
    conv = rng.standard_normal((2, 5, 4)).astype(np.float32)
    xc, w, bc = rng.standard_normal((2, 5)).astype(np.float32), rng.standard_normal((5, 4)).astype(np.float32), rng.standard_normal(5).astype(np.float32)
    win, out = oracle.causal_conv1d_update(conv, xc, w, bc, silu=True)
    seq = torch.cat([T(conv), T(xc)[:, :, None]], -1)  # [B, C, W + 1]
    want = torch.nn.functional.conv1d(seq, T(w)[:, None], T(bc), groups=5)[:, :, -1]
    np.testing.assert_allclose(out, torch.nn.functional.silu(want).numpy(), rtol=1e-5, atol=1e-6)
    assert np.array_equal(win, seq[:, :, 1:].float().numpy())


def test_prepare_graph_decode_counters_on_the_host():
    """prepare_graph_decode's bookkeeping needs no GPU: caches of one model share one step counter, advanced by the
    highest-numbered layer only; shared=False gives every cache a counter of its own; caches already in graph mode are
    left alone; graph_decode_steps adds the host-side step to the counter."""
    from types import SimpleNamespace
    from hybrid_quant import mamba_state_8b_kernel as mk

    def caches():
        out = []
        for layer, step in ((7, 3), (2, 3), (11, 3)):
            c = mk.MambaStateKernelCache(torch.zeros(1, 2, 16, 128, dtype=torch.int8), torch.zeros(1, 2, 16, 8, dtype=torch.uint8),
                                         torch.zeros(1, 2, 16, 64, dtype=torch.uint8), 8, step)
            c.layer = layer
            out.append(c)
        return out

    cs = caches()
    model = SimpleNamespace(_mamba_decode_state_kernel_caches={id(c): c for c in cs})
    mk.prepare_graph_decode(model)
    assert len({c.step_counter.data_ptr() for c in cs}) == 1 and cs[0].step_counter.dtype == torch.int64
    assert [c.advances_counter for c in cs] == [False, False, True]  # layer 11 is the last a forward pass reaches
    assert [c.step for c in cs] == [3, 3, 3]
    cs[0].step_counter += 4  # what four replayed decode steps leave behind
    assert mk.graph_decode_steps(model) == {7: 7, 2: 7, 11: 7}
    counter = cs[0].step_counter
    mk.prepare_graph_decode(model)  # a second call changes nothing
    assert all(c.step_counter is counter for c in cs)

    cs = caches()
    model = SimpleNamespace(_mamba_decode_state_kernel_caches={id(c): c for c in cs})
    mk.prepare_graph_decode(model, shared=False)
    assert len({c.step_counter.data_ptr() for c in cs}) == 3 and all(c.advances_counter for c in cs)
    assert mk.graph_decode_steps(model) == {7: 3, 2: 3, 11: 3}
    mk.prepare_graph_decode(SimpleNamespace())  # a model without registered caches: nothing to do

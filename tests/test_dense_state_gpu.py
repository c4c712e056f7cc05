"""GPU checks of the unquantised baselines (dense-state selective update, causal-conv1d update)
against their CPU restatement, through the C ABI.  Bar: the stored state equals the correctly rounded
fp32 value up to one ulp of the state's type (fp32 state: 1e-5 relative), outputs as
tests.util.assert_out_close; the conv window is moved bit-exactly."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import assert_out_close, bf16r, dev, expand_update_operands, make_update_case, t

pytestmark = pytest.mark.gpu


def ds():
    from layer_quant_b200 import dense_state as m
    return m


def dense_oracle_operands(d):
    b, h, p, n = d["state"].shape
    bc = lambda v, shape: None if v is None else np.broadcast_to(v, shape)
    return dict(x=d["x"], dt=np.broadcast_to(d["dt"][:, :, None], (b, h, p)), A=np.broadcast_to(d["A"][:, None, None], (h, p, n)),
                B=d["B"], C=d["C"], D=None if d["D"] is None else bc(d["D"][:, None], (h, p)), z=d["z"],
                dt_bias=None if d["dt_bias"] is None else bc(d["dt_bias"][:, None], (h, p)))


@pytest.mark.parametrize("state_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 16, 64, 128, 4), (3, 6, 24, 64, 2), (1, 4, 7, 16, 1), (2, 8, 64, 256, 8)])
def test_dense_update_matches_oracle(state_dtype, shape):
    b, h, p, n, g = shape
    d = make_update_case(11, b, h, p, n, g, with_z=(n == 64))
    state = t(d["state"], state_dtype)
    start = state.float().cpu().numpy()
    x, dt, A, B, C, D, z, bias = expand_update_operands(d)
    for step in range(2):
        want_h, want_y = oracle.dense_state_update(start, dt_softplus=True, **dense_oracle_operands(d))
        y = ds().selective_state_update(state, x, dt, A, B, C, D=D, z=z, dt_bias=bias, dt_softplus=True)
        assert y.dtype == x.dtype and tuple(y.shape) == (b, h, p)
        assert_out_close(y, want_y)
        got = state.float().cpu().numpy()
        if state_dtype == torch.float32:
            np.testing.assert_allclose(got, want_h, rtol=1e-5, atol=1e-6)
        else:
            ulp = 2.0 ** -7 if state_dtype == torch.bfloat16 else 2.0 ** -10
            # h' = h exp(A dt) + B dt x can cancel, and dt = log(1 + exp(.)) in fp32 moves by 2**-23 / dt when exp()
            # differs in its last bit; through exp(A dt) with |A| <= 16 that is a few 2**-19 of the operands
            ratio = np.abs(got - want_h) / (ulp * np.abs(want_h) + 2.0 ** -17 * (np.abs(start) + np.abs(want_h)) + 1e-7)
            worst = np.unravel_index(np.argmax(ratio), ratio.shape)
            assert ratio.max() <= 1.0, f"step {step}: state {got[worst]!r} vs {want_h[worst]!r} at {worst}, was {start[worst]!r}"
            # and almost everywhere exactly the rounded value
            rounded = torch.from_numpy(want_h).to(state_dtype).float().numpy()
            assert (got == rounded).mean() > 0.995
        start = got


def test_dense_update_general_operands_and_views():
    """Per-row dt / dt_bias, a full A tensor, fp32 activations, a state that is a strided view."""
    b, h, p, n, g = 2, 4, 8, 32, 2
    rng = np.random.default_rng(5)
    backing = t(bf16r(rng.standard_normal((b, h, p + 3, n)) * 0.5), torch.bfloat16)
    state = backing[:, :, 1:p + 1]
    before = backing.clone()
    start = state.float().cpu().numpy()
    x = rng.standard_normal((b, h, p)).astype(np.float32)
    dt = rng.standard_normal((b, h, p)).astype(np.float32)
    bias = (rng.random((h, p)) * 2 - 4).astype(np.float32)
    A = (-np.exp(rng.random((h, p, n)) * np.log(16.0))).astype(np.float32)
    B, C = rng.standard_normal((b, g, n)).astype(np.float32), rng.standard_normal((b, g, n)).astype(np.float32)
    want_h, want_y = oracle.dense_state_update(start, x, dt, A, B, C, None, None, bias, True)
    y = ds().selective_state_update(state, t(x), t(dt), t(A), t(B), t(C), dt_bias=t(bias), dt_softplus=True)
    assert_out_close(y, want_y)
    got = state.float().cpu().numpy()
    assert (np.abs(got - want_h) <= 2.0 ** -7 * np.abs(want_h) + 1e-7).all()
    assert torch.equal(backing[:, :, 0], before[:, :, 0]) and torch.equal(backing[:, :, p + 1:], before[:, :, p + 1:])  # rows outside the view


def test_dense_update_single_head_form_and_errors():
    m = ds()
    b, p, n = 3, 16, 64
    rng = np.random.default_rng(9)
    state = t(rng.standard_normal((b, p, n)).astype(np.float32))
    start = state.cpu().numpy()
    x, dt = rng.standard_normal((b, p)).astype(np.float32), rng.standard_normal((b, p)).astype(np.float32)
    A = -np.exp(rng.random((p, n))).astype(np.float32)
    B, C = rng.standard_normal((b, n)).astype(np.float32), rng.standard_normal((b, n)).astype(np.float32)
    want_h, want_y = oracle.dense_state_update(start[:, None], x[:, None], dt[:, None], A[None], B[:, None], C[:, None])
    y = m.selective_state_update(state, t(x), t(dt), t(A), t(B), t(C))
    assert tuple(y.shape) == (b, p)
    assert_out_close(y, want_y[:, 0])
    np.testing.assert_allclose(state.cpu().numpy(), want_h[:, 0], rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        m.selective_state_update(state, t(x)[:, :4], t(dt), t(A), t(B), t(C))
    with pytest.raises(NotImplementedError):
        s48 = t(rng.standard_normal((1, 1, 4, 48)).astype(np.float32))
        m.selective_state_update(s48, s48[..., 0], s48[..., 0], s48[0], s48[:, :, 0], s48[:, :, 0])
    with pytest.raises(RuntimeError):
        m.selective_state_update(state.cpu(), t(x), t(dt), t(A), t(B), t(C))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("width,act", [(4, "silu"), (2, None), (8, "swish")])
def test_conv1d_update(dtype, width, act):
    m = ds()
    b, c = 3, 10240 // 8 + 5
    rng = np.random.default_rng(width)
    state0 = bf16r(rng.standard_normal((b, c, width)))
    weight = bf16r(rng.standard_normal((c, width)) * 0.5)
    bias = bf16r(rng.standard_normal(c)) if width != 2 else None
    conv_state = t(state0, dtype)
    cur = state0
    for step in range(3):
        x = bf16r(rng.standard_normal((b, c)))
        win, want = oracle.causal_conv1d_update(cur, x, weight, bias, silu=act is not None)
        out = m.causal_conv1d_update(t(x, dtype), conv_state, t(weight, dtype), None if bias is None else t(bias, dtype), act)
        np.testing.assert_array_equal(conv_state.float().cpu().numpy(), win)
        assert_out_close(out, want)
        cur = win
    out3 = m.causal_conv1d_update(t(x, dtype)[:, :, None], conv_state, t(weight, dtype), None, None)
    assert tuple(out3.shape) == (b, c, 1)
    with pytest.raises(NotImplementedError):
        m.causal_conv1d_update(t(x, dtype), conv_state, t(weight, dtype), None, "gelu")
    with pytest.raises(ValueError):
        m.causal_conv1d_update(t(x, dtype)[:, :7], conv_state, t(weight, dtype))


@pytest.mark.parametrize("name", ["mx8_sr", "mx8_sr_nod", "mx4_sr"])
def test_dense_update_against_reference_mx_fixtures(golden_dir, name):
    """lq_dense_state_update on the decoded initial state of a reference-run MX fixture (an fp32 state, so the store
    does not round): y within the fp32 bar of the reference kernel's y, h' within a few ulps of the MX4 pair's fp32 h'."""
    from tests.test_oracle_golden import _dense_from_fixture
    g = np.load(golden_dir / f"update_{name}.npz")
    state_np, ops = _dense_from_fixture(g)
    b, h, p, n = state_np.shape
    state = t(state_np)
    dt = t(np.ascontiguousarray(ops["dt"][:, :, 0]))[:, :, None].expand(b, h, p)
    A = t(np.ascontiguousarray(ops["A"][:, 0, 0]))[:, None, None].expand(h, p, n)
    D = None if ops["D"] is None else t(np.ascontiguousarray(ops["D"][:, 0]))[:, None].expand(h, p)
    bias = None if ops["dt_bias"] is None else t(np.ascontiguousarray(ops["dt_bias"][:, 0]))[:, None].expand(h, p)
    y = ds().selective_state_update(state, t(ops["x"]), dt, A, t(ops["B"]), t(ops["C"]), D=D, dt_bias=bias,
                                    dt_softplus=ops["dt_softplus"])
    assert_out_close(y, g["y0"])
    if "h0" in g:
        np.testing.assert_allclose(state.cpu().numpy(), g["h0"], rtol=3e-6, atol=1e-7)

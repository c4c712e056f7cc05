"""CPU restatement of the unquantised Mamba2 decode step (TEST INFRASTRUCTURE ONLY): the dense-state
selective update and the causal-conv1d update.

The algorithms live in third-party dependencies that are absent from the reference tree and from this
machine: mamba-ssm==2.3.2.post1 (``mamba_ssm/ops/triton/selective_state_update.py``) and
causal-conv1d==1.6.2.post1 (``causal_conv1d_update``), both pinned in the reference's
``requirements.txt:7-8``.  What is restated here is their published behaviour for one decode token.

``dense_state_update`` is pinned for the un-gated case (z = None) through the reference's own MX
kernels: the reference hands the same ten arguments to either update
(``hybrid_quant/mamba_state_8b_kernel.py:743-761``), and its MX kernels evaluate the same fp32 expression
(``:135-166``) on the decoded state before they requantise it.  Fed the decoded initial state of the
reference-run fixtures (``tests/golden/update_*.npz``), this function must reproduce their y and, where the
fixture keeps it, their fp32 h' (``tests/test_oracle_golden.py``).  PARITY UNPINNED for the rest: the gate
``y * z * sigmoid(z)`` of the third-party update and the whole of ``causal_conv1d_update`` have no
execution of their own code to be checked against here.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def _softplus(x):
    # fp32 log(1 + exp(x)), the form the reference's kernels use (mamba_state_8b_kernel.py:28-30)
    x = np.asarray(x, dtype=F32)
    with np.errstate(over="ignore"):
        return np.where(x <= F32(20.0), np.log(F32(1.0) + np.exp(x)), x).astype(F32)


def dense_state_update(state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False):
    """state fp32 values of the stored type [B,H,P,N]; x, dt, z [B,H,P]; A [H,P,N]; B, C [B,G,N]; D,
    dt_bias [H,P].  Returns (h' fp32 before the store's rounding, y fp32 [B,H,P])."""
    state = np.asarray(state, dtype=F32)
    x = np.asarray(x, dtype=F32)
    dt = np.asarray(dt, dtype=F32).copy()
    if dt_bias is not None:
        dt = dt + np.asarray(dt_bias, dtype=F32)[None]
    if dt_softplus:
        dt = _softplus(dt)
    ratio = state.shape[1] // B.shape[1]
    Bh = np.repeat(np.asarray(B, dtype=F32), ratio, axis=1)[:, :, None, :]
    Ch = np.repeat(np.asarray(C, dtype=F32), ratio, axis=1)[:, :, None, :]
    with np.errstate(over="ignore", under="ignore"):
        dA = np.exp(np.asarray(A, dtype=F32)[None] * dt[..., None])
        h = (state * dA + (Bh * dt[..., None]) * x[..., None]).astype(F32)  # dB = B * dt, then dB * x
    y = (h.astype(np.float64) * Ch).sum(axis=-1)
    if D is not None:
        y = y + x * np.asarray(D, dtype=F32)[None]
    if z is not None:
        zz = np.asarray(z, dtype=np.float64)
        y = y * zz / (1.0 + np.exp(-zz))
    return h, y.astype(F32)


def causal_conv1d_update(conv_state, x, weight, bias=None, silu=False):
    """conv_state [B,C,W], x [B,C], weight [C,W], bias [C].  Returns (new window fp32, out fp32 [B,C])."""
    win = np.concatenate([np.asarray(conv_state, dtype=F32)[:, :, 1:], np.asarray(x, dtype=F32)[:, :, None]], axis=2)
    out = (win.astype(np.float64) * np.asarray(weight, dtype=np.float64)[None]).sum(axis=-1)
    if bias is not None:
        out = out + np.asarray(bias, dtype=np.float64)[None]
    if silu:
        out = out / (1.0 + np.exp(-out))
    return win, out.astype(F32)

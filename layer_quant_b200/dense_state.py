"""Unquantised baselines of the Mamba2 decode step on the same C ABI as the MX kernels.

The reference does not ship these: the global ``selective_state_update`` that its patch falls back
to (``hybrid_quant/mamba_state_8b_kernel.py:743-761``) is
``mamba_ssm.ops.triton.selective_state_update.selective_state_update`` and the step before it in
the mixer is ``causal_conv1d.causal_conv1d_update``, both third-party packages.  The two functions
here keep those packages' call signatures for the decode case (one token, no variable-length
batching) so that the MX state formats can be compared with the BF16 state on the same GPU and
through the same kind of kernel, and so that a model without those packages can still step.

No CPU or Triton fallback: CUDA tensors only.
"""
from __future__ import annotations

import ctypes as ct

import torch

from . import _lib


def selective_state_update(state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False, *, out=None):
    """One decode step on a dense state, in place.

    state [B,H,P,N] (bf16 / f16 / f32, last dim contiguous); x, dt, z [B,H,P]; A [H,P,N]; B, C [B,G,N];
    D, dt_bias [H,P] (expanded stride-0 views welcome); the 2-D forms of the third-party function
    (state [B,P,N], x [B,P], ...) are taken as one head.  Returns y like x:
    ``dt = softplus(dt + dt_bias)``, ``state = state * exp(A dt) + B dt x``, ``y = <state, C> + D x``
    and, with z, ``y * z * sigmoid(z)``.
    """
    squeeze = state.dim() == 3
    if squeeze:
        state, x, dt, A = state.unsqueeze(1), x.unsqueeze(1), dt.unsqueeze(1), A.unsqueeze(0)
        B, C = B.unsqueeze(1), C.unsqueeze(1)
        D = None if D is None else D.unsqueeze(0)
        z = None if z is None else z.unsqueeze(1)
        dt_bias = None if dt_bias is None else dt_bias.unsqueeze(0)
    if state.dim() != 4:
        raise ValueError(f"Expected state [B,H,P,N], got {tuple(state.shape)}")
    batch, heads, dim, dstate = state.shape
    if tuple(x.shape) != (batch, heads, dim) or tuple(dt.shape) != (batch, heads, dim):
        raise ValueError(f"x {tuple(x.shape)} / dt {tuple(dt.shape)} do not match state {tuple(state.shape)}")
    if tuple(A.shape) != (heads, dim, dstate):
        raise ValueError(f"A {tuple(A.shape)} does not match state {tuple(state.shape)}")
    if B.dim() != 3 or B.shape[0] != batch or B.shape[2] != dstate or tuple(C.shape) != tuple(B.shape):
        raise ValueError(f"B {tuple(B.shape)} / C {tuple(C.shape)} do not match state {tuple(state.shape)}")
    if heads % B.shape[1] != 0:
        raise ValueError(f"{heads} heads are not a multiple of {B.shape[1]} groups")
    for name, t in (("D", D), ("dt_bias", dt_bias)):
        if t is not None and tuple(t.shape) != (heads, dim):
            raise ValueError(f"{name} {tuple(t.shape)} does not match [H,P] = [{heads},{dim}]")
    if z is not None and tuple(z.shape) != tuple(x.shape):
        raise ValueError(f"z {tuple(z.shape)} does not match x {tuple(x.shape)}")
    dev = _lib.require_cuda(state, x, dt, A, B, C, D, z, dt_bias, out)
    if out is None:
        out = torch.empty_like(x)
    a = _lib.DenseUpdateArgs()
    a.state = state.data_ptr()
    for i in range(4):
        a.state_stride[i] = state.stride(i)
    a.state_dtype = _lib.dtype_code(state)
    a.batch, a.heads, a.dim, a.dstate = batch, heads, dim, dstate
    for name, t, n in (("x", x, 3), ("dt", dt, 3), ("dt_bias", dt_bias, 2), ("A", A, 3), ("B", B, 3), ("C", C, 3),
                       ("D", D, 2), ("z", z, 3), ("out", out, 3)):
        _lib.set_ptr_strides(a, name, t, n)
    a.ngroups, a.dt_softplus = B.shape[1], int(bool(dt_softplus))
    _lib.check(_lib.lib().lq_dense_state_update(ct.byref(a), _lib.stream_ptr(dev)))
    return out.squeeze(1) if squeeze else out


def causal_conv1d_update(x, conv_state, weight, bias=None, activation=None, *, out=None):
    """One decode step of the depthwise causal convolution, conv_state [B,C,W] updated in place.

    x [B,C] (or [B,C,1]); weight [C,W]; bias [C] or None; activation None, "silu" or "swish".
    The window moves one place to the left, x enters at the end, and the output is the window's dot
    product with the channel's weights (+ bias), through SiLU when asked."""
    if activation not in (None, "silu", "swish"):
        raise NotImplementedError("activation must be None, silu, or swish")
    unsqueeze = x.dim() == 3
    if unsqueeze:
        if x.shape[2] != 1:
            raise ValueError(f"causal_conv1d_update takes one token per call, got x {tuple(x.shape)}")
        x = x.squeeze(2)
    batch, channels = x.shape
    if conv_state.dim() != 3 or tuple(conv_state.shape[:2]) != (batch, channels):
        raise ValueError(f"conv_state {tuple(conv_state.shape)} does not match x {tuple(x.shape)}")
    width = conv_state.shape[2]
    if tuple(weight.shape) != (channels, width):
        raise ValueError(f"weight {tuple(weight.shape)} does not match [C,W] = [{channels},{width}]")
    if bias is not None and tuple(bias.shape) != (channels,):
        raise ValueError(f"bias {tuple(bias.shape)} does not match [C] = [{channels}]")
    dev = _lib.require_cuda(x, conv_state, weight, bias, out)
    if out is None:
        out = torch.empty_like(x)
    a = _lib.Conv1dUpdateArgs()
    a.conv_state = conv_state.data_ptr()
    for i in range(3):
        a.state_stride[i] = conv_state.stride(i)
    a.state_dtype = _lib.dtype_code(conv_state)
    for name, t, n in (("x", x, 2), ("weight", weight, 2), ("bias", bias, 1), ("out", out, 2)):
        _lib.set_ptr_strides(a, name, t, n)
    a.batch, a.channels, a.width, a.silu = batch, channels, width, int(activation is not None)
    _lib.check(_lib.lib().lq_causal_conv1d_update(ct.byref(a), _lib.stream_ptr(dev)))
    return out.unsqueeze(2) if unsqueeze else out

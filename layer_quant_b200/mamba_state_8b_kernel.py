"""Mamba2 decode state held in MX8 / MX4 blocks: host-side mirror of the reference module
``hybrid_quant/mamba_state_8b_kernel.py`` (phcool/Layer_Quant) over the sm_100a library.

Same public names, argument meaning and errors as the reference:

=====================================================  ======================================
here                                                   reference (mamba_state_8b_kernel.py)
=====================================================  ======================================
``MX8_BLOCK_SIZE`` ... ``MX4_MANTISSA_MAX``            :11-16
``MambaStateKernelCache``                              :19-25
``_quantize_initial_state_mx``                         :547-572
``allocate_state_kernel_cache``                        :575-598
``mx_state_selective_update`` (+ mx8_/mx4_ aliases)    :601-729
``patch_nemotron_h_mamba_decode_state_kernel``         :732-767
``register_mamba_state_kernel_caches``                 :770-796
=====================================================  ======================================

Differences a caller can see, all opt-out:

* ``allocate_state_kernel_cache`` stores the state bit-packed (18 / 10 bytes per 16-value block
  instead of 25): ``micro_exp`` holds one bit per pair and MX4 mantissas are nibbles.  Pass
  ``layout="reference"`` (or set ``DEFAULT_STATE_LAYOUT``) for the reference's tensors;
  ``cache.to_layout("reference")`` converts.  The decoded values are identical.
* MX4 works through ``mx_state_selective_update`` (the reference's wrapper raises TypeError for it)
  and needs no fp32 temporary.
* Stochastic rounding draws the library's own Philox stream, keyed on (seed, layer, step, block
  index), unless ``rng_stream="reference"`` is passed to the call or to
  ``patch_nemotron_h_mamba_decode_state_kernel`` (or ``RNG_STREAM`` is set): that reproduces the
  reference's ``tl.rand(seed, step * numel + index)`` numbers and rounding rule bit for bit at
  about a quarter of the speed (one Philox block per value instead of one per 16 values).
* Repeated calls with the same operand tensors (the decode loop) reuse the argument block prepared
  by the first call; only the output pointer and the step change.
* A decode step never recompiles anything (the reference re-JITs each step because its RNG offset
  is a compile-time constant).
"""
from __future__ import annotations

import ctypes as ct
from dataclasses import dataclass, field
from types import SimpleNamespace

import torch

from . import _lib

MX8_BLOCK_SIZE = 16
MX8_PAIR_SIZE = 2
MX8_MANTISSA_MAX = 63.0
MX4_BLOCK_SIZE = 16
MX4_PAIR_SIZE = 2
MX4_MANTISSA_MAX = 7.0

#: storage layout new caches get: "packed" (native) or "reference" (the reference's tensors)
DEFAULT_STATE_LAYOUT = "packed"
#: Random stream of stochastic rounding when neither the call nor the patch function names one:
#: "layered"   one Philox4x32-10 block per 16-value MX block keyed on (seed, layer, step, block index), 8 random bits per
#:             value, fixed-point rounding rule (LQ_ROUND_PHILOX_LAYERED): the fast stream, different layers draw
#:             different numbers;
#: "layered4"  the reference's rounding rule (floor(a) + (u < frac), 24-bit u) on the library's keying, one Philox block per
#:             four values (LQ_ROUND_PHILOX_LAYERED4): between the two in cost, isolates the keying from the rule;
#: "reference" exactly the reference's numbers and rule, ``tl.rand(seed, step * numel + index)`` with one Philox block per
#:             value and no layer term (LQ_ROUND_PHILOX_REF): bit-for-bit the reference's codes, about four times slower.
RNG_STREAM = "layered"

_LAYOUTS = {"reference": _lib.LQ_MX_LAYOUT_REFERENCE, "packed": _lib.LQ_MX_LAYOUT_PACKED}


@dataclass
class MambaStateKernelCache:
    q_state: torch.Tensor
    shared_exp: torch.Tensor
    micro_exp: torch.Tensor
    format_bits: int = 8
    step: int = 0
    layout: str = "reference"
    layer: int = 0
    # Not in the reference: the step count kept on the device (one int64) once prepare_graph_decode has
    # run; the kernel adds it to ``step`` when it runs, so a recorded launch draws fresh numbers on replay.
    step_counter: torch.Tensor | None = None
    # Whether this cache's update advances ``step_counter`` afterwards.  When the caches of one model share a counter
    # (prepare_graph_decode), only the last layer's update does, once per decode step.
    advances_counter: bool = True
    # Not in the reference: the argument block prepared by the last mx_state_selective_update call on this cache
    # and the operand signature it was prepared for.
    _plan: object = field(default=None, repr=False, compare=False)
    _plan_key: object = field(default=None, repr=False, compare=False)

    @property
    def state_shape(self) -> tuple[int, int, int, int]:
        """Logical [batch, heads, dim, dstate] of the state, whatever the storage layout."""
        b, h, p, n = self.q_state.shape
        if self.layout == "packed" and self.format_bits == 4:
            n *= 2
        return b, h, p, n

    def to_layout(self, layout: str) -> "MambaStateKernelCache":
        """A copy of this cache in the other storage layout (same values, same step)."""
        if layout not in _LAYOUTS:
            raise ValueError(f"unknown layout {layout!r}")
        out = _empty_cache(self.state_shape, self.format_bits, layout, self.q_state.device)
        out.step, out.layer = self.step, self.layer
        src, dst = _state_struct(self), _state_struct(out)
        _lib.check(_lib.lib().lq_mx_convert_layout(ct.byref(src), ct.byref(dst), _lib.stream_ptr(self.q_state.device)))
        return out

    def dequantize(self) -> torch.Tensor:
        """fp32 [batch, heads, dim, dstate]: q * 2**(shared_exp - 127 + micro)."""
        b, h, p, n = self.state_shape
        out = torch.empty((b, h, p, n), dtype=torch.float32, device=self.q_state.device)
        st = _state_struct(self)
        _lib.check(_lib.lib().lq_mx_dequantize(ct.byref(st), out.data_ptr(), n, _lib.stream_ptr(out.device)))
        return out


def _empty_cache(shape, format_bits: int, layout: str, device) -> MambaStateKernelCache:
    b, h, p, n = shape
    if layout == "packed":
        q = (torch.empty((b, h, p, n // 2), dtype=torch.uint8, device=device) if format_bits == 4
             else torch.empty((b, h, p, n), dtype=torch.int8, device=device))
        micro = torch.empty((b, h, p, n // 16), dtype=torch.uint8, device=device)
    else:
        q = torch.empty((b, h, p, n), dtype=torch.int8, device=device)
        micro = torch.empty((b, h, p, n // 2), dtype=torch.uint8, device=device)
    exp = torch.empty((b, h, p, n // 16), dtype=torch.uint8, device=device)
    return MambaStateKernelCache(q_state=q, shared_exp=exp, micro_exp=micro, format_bits=format_bits, layout=layout)


def _state_struct(cache: MambaStateKernelCache) -> _lib.MxState:
    if cache.layout not in _LAYOUTS:
        raise ValueError(f"unknown layout {cache.layout!r}")
    _lib.require_cuda(cache.q_state, cache.shared_exp, cache.micro_exp)
    for name in ("q_state", "shared_exp", "micro_exp"):
        t = getattr(cache, name)
        if t.ndim != 4:
            raise ValueError(f"Expected {name} [B,H,P,*], got {tuple(t.shape)}")
        if t.stride(-1) != 1:
            raise ValueError(f"{name} must be contiguous along its last dimension")
    s = _lib.MxState()
    s.q_state, s.shared_exp, s.micro_exp = cache.q_state.data_ptr(), cache.shared_exp.data_ptr(), cache.micro_exp.data_ptr()
    for i in range(3):
        s.q_stride[i] = cache.q_state.stride(i)
        s.exp_stride[i] = cache.shared_exp.stride(i)
        s.micro_stride[i] = cache.micro_exp.stride(i)
    s.batch, s.heads, s.dim, s.dstate = cache.state_shape
    s.format_bits = cache.format_bits
    s.layout = _LAYOUTS[cache.layout]
    return s


def _seed_u64(seed: int) -> int:
    return int(seed) & 0xFFFFFFFFFFFFFFFF


def _quantize_into(cache: MambaStateKernelCache, src: torch.Tensor, rounding: _lib.Rounding) -> None:
    n = src.shape[-1]
    src2 = src.reshape(-1, n)
    if src2.stride(-1) != 1:
        src2 = src2.contiguous()
    st = _state_struct(cache)
    _lib.check(_lib.lib().lq_mx_quantize(ct.byref(st), src2.data_ptr(), _lib.dtype_code(src2), src2.stride(0),
                                         ct.byref(rounding), _lib.stream_ptr(src.device)))


def _quantize_initial_state_mx(
    state: torch.Tensor,
    *,
    format_bits: int,
    block_size: int,
    pair_size: int,
    mantissa_max: float,
    layout: str = "reference",
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One-off quantisation of the post-prefill state, round-half-even (reference :547-572)."""
    if state.shape[-1] % block_size != 0:
        raise ValueError(f"MX{format_bits} state dim must be divisible by {block_size}, got {state.shape[-1]}")
    if block_size != 16 or pair_size != 2 or float(mantissa_max) != (63.0 if format_bits == 8 else 7.0):
        raise ValueError("the MX codec is fixed: 16-value blocks, pairs of 2, mantissa max 63 (MX8) / 7 (MX4)")
    _lib.require_cuda(state)
    lead = state.shape[:-1]
    flat = state.reshape(1, 1, -1, state.shape[-1])
    cache = _empty_cache(flat.shape, format_bits, layout, state.device)
    rounding = _lib.Rounding(mode=_lib.LQ_ROUND_HALF_EVEN)
    src = flat if flat.dtype in (torch.float32, torch.bfloat16, torch.float16) else flat.float()
    _quantize_into(cache, src, rounding)
    return (cache.q_state.reshape(*lead, -1), cache.shared_exp.reshape(*lead, -1), cache.micro_exp.reshape(*lead, -1))


def allocate_state_kernel_cache(ssm_state_4d: torch.Tensor, group_size: int = MX8_BLOCK_SIZE, format_bits: int = 8,
                                layout: str | None = None) -> MambaStateKernelCache:
    """Quantise a [B, H, P, N] state into a fresh cache (reference :575-598)."""
    if format_bits == 8:
        if group_size != MX8_BLOCK_SIZE:
            raise ValueError(f"MX8 uses a fixed {MX8_BLOCK_SIZE}-value block, got group_size={group_size}")
        mmax = MX8_MANTISSA_MAX
    elif format_bits == 4:
        if group_size != MX4_BLOCK_SIZE:
            raise ValueError(f"MX4 uses a fixed {MX4_BLOCK_SIZE}-value block, got group_size={group_size}")
        mmax = MX4_MANTISSA_MAX
    else:
        raise ValueError(f"Only MX8 and MX4 state quantization are supported, got format_bits={format_bits}")
    if ssm_state_4d.ndim != 4:
        raise ValueError(f"Expected ssm_state [B,H,P,N], got {tuple(ssm_state_4d.shape)}")
    layout = layout or DEFAULT_STATE_LAYOUT
    q, e, m = _quantize_initial_state_mx(ssm_state_4d, format_bits=format_bits, block_size=16, pair_size=2,
                                         mantissa_max=mmax, layout=layout)
    return MambaStateKernelCache(q_state=q, shared_exp=e, micro_exp=m, format_bits=format_bits, layout=layout)


class MxUpdatePlan:
    """A prepared ``mx_state_selective_update`` call: shapes are checked and the argument block of
    the C entry point is filled once, so that repeating the step costs one ctypes call.  The
    tensors handed in must stay alive and in place (the plan keeps references).

    ``step_counter`` (a 1-element int64 CUDA tensor) makes the launch replayable from a CUDA
    graph: the kernel adds its current value to the step when it runs; advance it with
    :func:`advance_step_counter` at the end of the captured step.  Without it the host-side
    ``cache.step`` is used and advanced on every :meth:`run`."""

    def __init__(self, cache, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False, stochastic=True,
                 seed=1234, *, rng_stream=None, rand_words=None, h_out=None, out=None, step_counter=None):
        if cache.q_state.ndim != 4:
            raise ValueError(f"Expected q_state [B,H,P,N], got {tuple(cache.q_state.shape)}")
        batch, nheads, dim, dstate = cache.state_shape
        if x.shape != (batch, nheads, dim):
            raise ValueError(f"Expected x shape {(batch, nheads, dim)}, got {tuple(x.shape)}")
        if B.ndim != 3 or C.ndim != 3:
            raise ValueError("Expected B and C with shape [batch, ngroups, dstate] for decode update.")
        if cache.format_bits not in (8, 4):
            raise ValueError(f"Unsupported MX state format_bits={cache.format_bits}")
        if dt.ndim != 3 or A.ndim != 3:
            raise ValueError("Expected dt [batch, heads, dim] and A [heads, dim, dstate] (expanded views are fine).")
        if D is not None and D.ndim != 2:
            raise ValueError("Expected D [heads, dim].")
        if z is not None and z.ndim != 3:
            raise ValueError("Expected z [batch, heads, dim].")
        self.device = _lib.require_cuda(cache.q_state, x, dt, A, B, C, D, z, dt_bias, rand_words, h_out, out, step_counter)
        self.cache = cache
        self.out = torch.empty_like(x) if out is None else out
        self._keep = (x, dt, A, B, C, D, z, dt_bias, rand_words, h_out, step_counter)
        self.numel = batch * nheads * dim * dstate
        a = self.args = _lib.MxUpdateArgs()
        a.state = _state_struct(cache)
        _lib.set_ptr_strides(a, "x", x, 3)
        _lib.set_ptr_strides(a, "dt", dt, 3)
        _lib.set_ptr_strides(a, "A", A, 3)
        _lib.set_ptr_strides(a, "B", B, 3)
        _lib.set_ptr_strides(a, "C", C, 3)
        _lib.set_ptr_strides(a, "D", D, 2)
        _lib.set_ptr_strides(a, "z", z, 3)
        _lib.set_ptr_strides(a, "out", self.out, 3)
        if dt_bias is not None:
            a.dt_bias = dt_bias.data_ptr()
            a.dt_bias_dtype = _lib.dtype_code(dt_bias)
            d_strides = D.stride() if D is not None else (0, 0)  # the reference indexes dt_bias with D's strides
            a.dt_bias_stride[0], a.dt_bias_stride[1] = d_strides[0], d_strides[1]
        a.ngroups = B.shape[1]
        a.dt_softplus = 1 if dt_softplus else 0
        stream = rng_stream or RNG_STREAM
        r = a.rounding
        r.seed = _seed_u64(seed)
        r.layer = int(cache.layer) & 0xFFFFFFFF
        if rand_words is not None:
            if (tuple(rand_words.shape) != (batch, nheads, dim, dstate) or rand_words.element_size() != 4
                    or not rand_words.is_contiguous()):
                raise ValueError(f"rand_words must be a contiguous 32-bit tensor of shape {(batch, nheads, dim, dstate)}")
            r.words = rand_words.data_ptr()
            r.mode = _lib.LQ_ROUND_SUPPLIED_FIXED if stream == "layered" else _lib.LQ_ROUND_SUPPLIED
        elif not stochastic:
            r.mode = _lib.LQ_ROUND_HALF_UP
        elif stream == "reference":
            r.mode = _lib.LQ_ROUND_PHILOX_REF
        elif stream == "layered":
            r.mode = _lib.LQ_ROUND_PHILOX_LAYERED
        elif stream == "layered4":
            r.mode = _lib.LQ_ROUND_PHILOX_LAYERED4
        else:
            raise ValueError(f"unknown rng_stream {stream!r}")
        if h_out is not None:
            if tuple(h_out.shape) != (batch, nheads, dim, dstate) or h_out.dtype != torch.float32 or not h_out.is_contiguous():
                raise ValueError(f"h_out must be contiguous float32 of shape {(batch, nheads, dim, dstate)}")
            a.h_out = h_out.data_ptr()
        if step_counter is not None:
            if step_counter.dtype != torch.int64 or step_counter.numel() != 1:
                raise ValueError("step_counter must be a 1-element int64 CUDA tensor")
            r.step_counter = step_counter.data_ptr()
        self._fn = _lib.lib().lq_mx_state_update
        self._ref = ct.byref(a)
        self._out_sig = (self.out.data_ptr(), self.out.stride(), self.out.dtype)

    def rebind_out(self, out: torch.Tensor) -> None:
        """Point the prepared call at another output tensor (shape and dtype of ``x``)."""
        sig = (out.data_ptr(), out.stride(), out.dtype)
        self.out = out
        if sig == self._out_sig:
            return
        self._out_sig = sig
        a = self.args
        a.out = sig[0]
        a.out_stride[0], a.out_stride[1], a.out_stride[2] = sig[1]
        a.out_dtype = _lib.dtype_code(out)

    def run(self) -> torch.Tensor:
        r = self.args.rounding
        step = int(self.cache.step)
        r.step = step
        r.rng_offset = (step * self.numel) & 0xFFFFFFFFFFFFFFFF
        rc = self._fn(self._ref, _lib.stream_ptr(self.device))
        if rc:
            _lib.check(rc)
        if not r.step_counter:
            self.cache.step = step + 1
        return self.out


def advance_step_counter(step_counter: torch.Tensor, inc: int = 1) -> None:
    """``step_counter += inc`` on the current stream with the library's own one-thread kernel
    (capturable in a CUDA graph together with the update launches that read the counter)."""
    dev = _lib.require_cuda(step_counter)
    _lib.check(_lib.lib().lq_counter_add(step_counter.data_ptr(), int(inc), _lib.stream_ptr(dev)))


def mx_state_selective_update(
    cache: MambaStateKernelCache,
    x: torch.Tensor,
    dt: torch.Tensor,
    A: torch.Tensor,
    B: torch.Tensor,
    C: torch.Tensor,
    D: torch.Tensor | None = None,
    z: torch.Tensor | None = None,
    dt_bias: torch.Tensor | None = None,
    dt_softplus: bool = False,
    stochastic: bool = True,
    seed: int = 1234,
    *,
    rng_stream: str | None = None,
    rand_words: torch.Tensor | None = None,
    h_out: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """One decode step on an MX-held state; returns y shaped and typed like ``x`` (reference
    :601-721).  ``cache`` is updated in place and ``cache.step`` advances by one.

    Operands may be expanded (stride-0) views exactly as the Nemotron-H decode path passes them:
    x, dt, z [B,H,P]; A [H,P,N]; B, C [B,G,N]; D, dt_bias [H,P].  As in the reference kernel,
    dt_bias is addressed with D's strides (with zeros when D is None).

    Extras (keyword-only, not in the reference): ``rng_stream`` overrides ``RNG_STREAM``;
    ``rand_words`` (uint32/int32 [B,H,P,N]) supplies the random bits instead of Philox;
    ``h_out`` (fp32 [B,H,P,N]) receives the updated state before requantisation; ``out`` is
    written instead of a fresh tensor.  :class:`MxUpdatePlan` prepares the same call once for
    loops that repeat it."""
    # the reference's own checks, in its order (:615-621)
    if cache.q_state.ndim != 4:
        raise ValueError(f"Expected q_state [B,H,P,N], got {tuple(cache.q_state.shape)}")
    if x.shape != cache.state_shape[:3]:
        raise ValueError(f"Expected x shape {cache.state_shape[:3]}, got {tuple(x.shape)}")
    if B.ndim != 3 or C.ndim != 3:
        raise ValueError("Expected B and C with shape [batch, ngroups, dstate] for decode update.")
    # The decode loop calls this with the same tensors every step: the prepared argument block of the previous call is
    # reused when every operand still has the same address and strides (and x / B the same shape and type: with the
    # state's shape they fix every other operand's shape).
    key = (x.data_ptr(), x.stride(), x.shape, x.dtype, dt.data_ptr(), dt.stride(), dt.dtype, A.data_ptr(), A.stride(), A.dtype,
           B.data_ptr(), B.stride(), B.shape, B.dtype, C.data_ptr(), C.stride(), C.dtype, _sig(D), _sig(z), _sig(dt_bias),
           _sig(rand_words), _sig(h_out), cache.q_state.data_ptr(), cache.shared_exp.data_ptr(), cache.micro_exp.data_ptr(),
           None if cache.step_counter is None else cache.step_counter.data_ptr(),
           dt_softplus, stochastic, seed, rng_stream or RNG_STREAM, cache.layout, cache.format_bits, cache.layer)
    plan = cache._plan if cache._plan_key == key else None
    if out is None:
        out = torch.empty_like(x)
    if plan is None:
        plan = MxUpdatePlan(cache, x, dt, A, B, C, D=D, z=z, dt_bias=dt_bias, dt_softplus=dt_softplus, stochastic=stochastic,
                            seed=seed, rng_stream=rng_stream, rand_words=rand_words, h_out=h_out, out=out,
                            step_counter=cache.step_counter)
        cache._plan, cache._plan_key = plan, key
    else:
        if out.shape != x.shape:
            raise ValueError(f"Expected out shape {tuple(x.shape)}, got {tuple(out.shape)}")
        plan.rebind_out(out)
    y = plan.run()
    if cache.step_counter is not None and cache.advances_counter:
        advance_step_counter(cache.step_counter)
    return y


def _sig(t):
    """What a prepared argument block depends on in an optional operand: address, strides, type."""
    return None if t is None else (t.data_ptr(), t.stride(), t.dtype)


def prepare_graph_decode(model, shared: bool = True) -> None:
    """Make the state updates of the registered caches replayable from a CUDA graph (not in the
    reference, whose launch bakes the step in as a compile-time constant, :659): the step count moves
    into a device counter that the kernel reads when it runs (it uses ``cache.step + counter``) and that
    is advanced on the stream.  ``graph_decode_steps`` reads the counters back.

    ``shared`` (default): the caches on one device share ONE counter, advanced once per decode step by
    the update of the highest-numbered layer, the last one a forward pass reaches, so a step costs one
    counter bump instead of one per layer.  This is for loops that run every registered layer once per
    step in layer order, which is what a model forward does; a loop that updates caches in another order,
    or only some of them, passes ``shared=False`` and every cache gets and advances its own counter."""
    caches = [c for c in getattr(model, "_mamba_decode_state_kernel_caches", {}).values() if c.step_counter is None]
    if not shared:
        for cache in caches:
            cache.step_counter = torch.zeros((1,), dtype=torch.int64, device=cache.q_state.device)
            cache.advances_counter = True
        return
    by_device: dict = {}
    for cache in caches:
        by_device.setdefault(cache.q_state.device, []).append(cache)
    for device, group in by_device.items():
        counter = torch.zeros((1,), dtype=torch.int64, device=device)
        last = max(group, key=lambda c: c.layer)
        for cache in group:
            cache.step_counter = counter
            cache.advances_counter = cache is last


def graph_decode_steps(model) -> dict[int, int]:
    """{layer: steps taken so far} of the caches in graph mode: the host-side step plus the device counter."""
    return {cache.layer: int(cache.step) + int(cache.step_counter.item())
            for cache in getattr(model, "_mamba_decode_state_kernel_caches", {}).values() if cache.step_counter is not None}


def mx8_state_selective_update(*args, **kwargs) -> torch.Tensor:
    return mx_state_selective_update(*args, **kwargs)


def mx4_state_selective_update(*args, **kwargs) -> torch.Tensor:
    return mx_state_selective_update(*args, **kwargs)


def _remote_module(model):
    return __import__(model.__class__.__module__, fromlist=["selective_state_update"])


def patch_nemotron_h_mamba_decode_state_kernel(
    model,
    group_size: int = MX8_BLOCK_SIZE,
    stochastic: bool = True,
    seed: int = 1234,
    *,
    rng_stream: str | None = None,
) -> None:
    """Route the remote modeling module's global ``selective_state_update`` through the MX kernels
    for every state tensor registered by :func:`register_mamba_state_kernel_caches`; any other
    state falls through to the original function (reference :732-767).  ``rng_stream`` (keyword-only,
    not in the reference) fixes the random stream of the patched calls: "layered" or "reference";
    None leaves it to ``RNG_STREAM`` at call time."""
    if rng_stream not in (None, "layered", "layered4", "reference"):
        raise ValueError(f"unknown rng_stream {rng_stream!r}")
    module = _remote_module(model)
    original = getattr(module, "_mx_state_kernel_original", module.selective_state_update)
    module._mx_state_kernel_stochastic = stochastic
    module._mx_state_kernel_seed = seed
    module._mx_state_kernel_rng_stream = rng_stream

    def selective_state_update_mx(ssm_state, x, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=False):
        kernel_cache = getattr(module, "_mamba_decode_state_kernel_caches", {}).get(id(ssm_state))
        if kernel_cache is None:
            return original(ssm_state, x, dt, A, B, C, D=D, z=z, dt_bias=dt_bias, dt_softplus=dt_softplus)
        return mx_state_selective_update(
            kernel_cache, x, dt, A, B, C, D=D, z=z, dt_bias=dt_bias, dt_softplus=dt_softplus,
            stochastic=getattr(module, "_mx_state_kernel_stochastic", True),
            seed=getattr(module, "_mx_state_kernel_seed", 1234),
            rng_stream=getattr(module, "_mx_state_kernel_rng_stream", None),
        )

    if not getattr(module, "_mx_state_kernel_patched", False):
        module._mx_state_kernel_original = original
        module.selective_state_update = selective_state_update_mx
        module._mx_state_kernel_patched = True
    model._mx_state_kernel_group_size = group_size


def register_mamba_state_kernel_caches(model, cache_params, mode_by_layer: dict[int, str]) -> None:
    """Quantise the post-prefill SSM state of the listed layers ('mx8' | 'mx4') and register the
    caches under ``id(ssm_state)`` on the model and on its remote module (reference :770-796)."""
    caches = {}
    meta = {}
    for layer_idx, mode in mode_by_layer.items():
        if mode not in {"mx8", "mx4"}:
            raise ValueError(f"Only MX8 and MX4 state caches are supported, got mode={mode!r}")
        mixer = model.backbone.layers[layer_idx].mixer
        ssm_state = cache_params.ssm_states[layer_idx]
        bits = 8 if mode == "mx8" else 4
        state_4d = ssm_state.view(ssm_state.shape[0], mixer.num_heads, mixer.head_dim, mixer.ssm_state_size)
        cache = allocate_state_kernel_cache(state_4d, group_size=16, format_bits=bits)
        cache.layer = int(layer_idx)
        caches[id(ssm_state)] = cache
        meta[layer_idx] = SimpleNamespace(mode=mode, block_size=16, format_bits=bits)
    model._mamba_decode_state_kernel_caches = caches
    _remote_module(model)._mamba_decode_state_kernel_caches = dict(caches)
    model._mamba_decode_state_kernel_meta = meta

"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import oracle


def dev():
    return torch.device("cuda", torch.cuda.current_device())


def t(a, dtype=None, device=None):
    x = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        x = x.to(dtype)
    return x.to(device or dev())


def bf16r(a):
    """Round a float array to bf16-representable fp32 values."""
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).bfloat16().float().numpy()


def cache_to_numpy(cache):
    """Reference-layout numpy (q int8, shared_exp u8, micro u8 [..., N/2]) of a state cache."""
    c = cache if cache.layout == "reference" else cache.to_layout("reference")
    return c.q_state.cpu().numpy(), c.shared_exp.cpu().numpy(), c.micro_exp.cpu().numpy()


def make_update_case(seed, b, h, p, n, g, with_d=True, with_z=False, with_bias=True, sigma=0.5):
    """Synthetic operands of one state-update step with Nemotron-H's value distributions:
    state ~ N(0, sigma), x, B, C ~ N(0, 1) in bf16, dt ~ N(0, 1) bf16 per head, dt_bias ~ U(-4, -2),
    A = -exp(U(0, ln 16)), D ~ U(0, 1).  Returned as numpy fp32 holding bf16-representable values."""
    rng = np.random.default_rng(seed)
    d = dict(
        state=(rng.standard_normal((b, h, p, n)) * sigma).astype(np.float32),
        x=bf16r(rng.standard_normal((b, h, p))), dt=bf16r(rng.standard_normal((b, h))),
        A=(-np.exp(rng.random(h) * np.log(16.0))).astype(np.float32),
        B=bf16r(rng.standard_normal((b, g, n))), C=bf16r(rng.standard_normal((b, g, n))),
        D=rng.random(h).astype(np.float32) if with_d else None,
        z=bf16r(rng.standard_normal((b, h, p))) if with_z else None,
        dt_bias=(rng.random(h) * 2.0 - 4.0).astype(np.float32) if with_bias else None,
    )
    return d


def expand_update_operands(d, io_dtype=torch.bfloat16):
    """Device tensors shaped and strided (stride-0 expands) the way the Nemotron-H decode path
    passes them to selective_state_update."""
    b, h, p, n = d["state"].shape
    x = t(d["x"], io_dtype)
    dt = t(d["dt"], io_dtype)[:, :, None].expand(b, h, p)
    A = t(d["A"])[:, None, None].expand(h, p, n)
    B = t(d["B"], io_dtype)
    C = t(d["C"], io_dtype)
    D = t(d["D"])[:, None].expand(h, p) if d["D"] is not None else None
    z = t(d["z"], io_dtype) if d["z"] is not None else None
    bias = t(d["dt_bias"])[:, None].expand(h, p) if d["dt_bias"] is not None else None
    return x, dt, A, B, C, D, z, bias


def oracle_update_operands(d):
    b, h, p, n = d["state"].shape
    bias = None
    if d["dt_bias"] is not None:
        # dt_bias is addressed with D's strides by the reference kernel: all heads read element 0 without D
        bias = np.broadcast_to(d["dt_bias"][:, None], (h, p)) if d["D"] is not None else np.full((h, p), d["dt_bias"][0], np.float32)
    return dict(x=d["x"], dt=np.broadcast_to(d["dt"][:, :, None], (b, h, p)), A=np.broadcast_to(d["A"][:, None, None], (h, p, n)),
                B=d["B"], C=d["C"], D=np.broadcast_to(d["D"][:, None], (h, p)) if d["D"] is not None else None, z=d["z"], dt_bias=bias)


def rel_err(a, ref):
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30))


def assert_out_close(out, ref, fp32_tol=1e-4):
    """Kernel output (torch tensor) against the float64 oracle.  fp32 outputs: within ``fp32_tol`` of
    the largest magnitude (the 2e-3 bar with a 20x margin).  bf16 / fp16 outputs carry the
    rounding of the store itself (half an ulp = 2**-8 / 2**-11 relative, already above 2e-3 for
    bf16), so they must equal the correctly rounded oracle value up to one ulp of the output type."""
    ref = np.asarray(ref, dtype=np.float64)
    got = out.float().cpu().numpy().astype(np.float64)
    scale = max(np.abs(ref).max(), 1e-30)
    if out.dtype == torch.float32:
        assert np.abs(got - ref).max() <= fp32_tol * scale, f"rel err {np.abs(got - ref).max() / scale:.3e}"
        return
    ulp = 2.0 ** -7 if out.dtype == torch.bfloat16 else 2.0 ** -10
    bad = np.abs(got - ref) > ulp * np.abs(ref) + fp32_tol * scale
    assert not bad.any(), f"{bad.sum()} outputs off by more than one ulp of {out.dtype}; worst {np.abs(got - ref).max() / scale:.3e} of max"

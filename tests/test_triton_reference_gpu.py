"""The reference's own Triton kernels, compiled for and run on this GPU, fed the same inputs as the
library (second oracle beside the CPU restatement).  The reference is imported unmodified from
``baseline/_ref`` (``baseline/reference.py`` is the recipe that puts it there); without that copy, or
without Triton, these tests skip: the reference is the yardstick here, not the product.

Real Triton evaluates ``x / scale`` and ``log2`` with approximate instructions and contracts
``state * dA + dB * x`` into one FMA, so its codes can differ from the canonical IEEE semantics (CPU
torch, the Triton interpreter, this library) where a value sits on a rounding boundary.  The tests
bound the rate of such differences (never more than one code step) and hold the outputs to the
2e-3 bar.  Set ``LQ_PARITY_REPORT=<file>`` to have the measured rates written as JSON lines."""
import json
import os

import numpy as np
import pytest
import torch

from tests.util import dev, expand_update_operands, make_update_case, t

pytestmark = pytest.mark.gpu


def _report(**kw):
    path = os.environ.get("LQ_PARITY_REPORT")
    print("parity:", json.dumps(kw))
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(kw) + "\n")


@pytest.fixture(scope="module")
def ref():
    from baseline import reference
    if not reference.available():
        pytest.skip("baseline/_ref is empty (python baseline/reference.py --from <Layer_Quant checkout>)")
    try:
        import triton  # noqa: F401
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"Triton is not importable: {exc}")
    return reference.load()


def test_pack_and_decode_attention_against_triton(ref):
    ria, _ = ref
    from layer_quant_b200 import int4_8b_attention as ia
    rng = np.random.default_rng(21)
    b, hq, hkv, tlen, d = 2, 32, 8, 777, 128
    for gs in (32, 64):
        k = rng.standard_normal((b, hkv, tlen, d)).astype(np.float32)
        v = rng.standard_normal((b, hkv, tlen, d)).astype(np.float32)
        k = np.where(rng.random(k.shape) < 0.01, 8.0 * np.sign(k), k)
        kt, vt = t(k, torch.bfloat16), t(v, torch.bfloat16)
        q = t(rng.standard_normal((b, hq, 1, d)), torch.bfloat16)
        pos = torch.arange(tlen, device=dev())
        ours = ia._allocate_layer_cache(b, hkv, 1024, d, d // gs, dev())
        theirs = ria._allocate_layer_cache(b, hkv, 1024, d, d // gs, dev())
        ia._pack_kv_into_cache(ours, kt, vt, pos, gs)
        ria._pack_kv_into_cache(theirs, kt, vt, pos, gs)
        torch.cuda.synchronize()
        assert ours.length == theirs.length == tlen
        # Triton's `/` is an approximate division: a scale may be an ulp off the IEEE quotient this library
        # computes, and a code may differ where x / scale is a tie or lands on the other side of one
        ks_o, ks_r = ours.k_scale[:, :, :tlen], theirs.k_scale[:, :, :tlen]
        scale_rel = ((ks_o - ks_r).abs() / ks_r).max().item()
        scale_diff = (ks_o != ks_r).float().mean().item()
        diff = (ours.k_packed[:, :, :tlen] != theirs.k_packed[:, :, :tlen]).float().mean().item()
        diff_v = (ours.v_packed[:, :, :tlen] != theirs.v_packed[:, :, :tlen]).float().mean().item()
        _report(test="int4_pack", group_size=gs, k_bytes_differ=diff, v_bytes_differ=diff_v, k_scales_differ=scale_diff,
                k_scale_max_rel_diff=scale_rel)
        assert scale_rel <= 2.5e-7 and diff < 1e-2 and diff_v < 1e-2
        # the two attention kernels on the SAME cache bytes
        o_ref = ria._decode_attention(q, ours_as(ria, ours), tlen, hq // hkv, gs).float()
        o_lq = ia._decode_attention(q, ours, tlen, hq // hkv, gs).float()
        torch.cuda.synchronize()
        err = ((o_lq - o_ref).abs().max() / o_ref.abs().max()).item()
        _report(test="int4_decode_attention", group_size=gs, rel_err_vs_triton=err)
        # both are bf16 outputs of fp32 accumulations: one bf16 ulp of the largest magnitude
        assert err <= 2.0 ** -7


def ours_as(ria, cache):
    """The library's cache object as the reference's dataclass (same four tensors)."""
    return ria.Int4KVLayerCache(k_packed=cache.k_packed, v_packed=cache.v_packed, k_scale=cache.k_scale, v_scale=cache.v_scale,
                                length=cache.length)


@pytest.mark.parametrize("bits", [8, 4])
def test_fused_state_update_against_triton(ref, bits):
    _, rmk = ref
    from layer_quant_b200 import mamba_state_8b_kernel as mk
    b, h, p, n, g = 2, 16, 64, 128, 2
    d = make_update_case(5, b, h, p, n, g)
    x, dt, A, B, C, D, z, bias = expand_update_operands(d, torch.bfloat16)
    state = t(d["state"])
    theirs = rmk.allocate_state_kernel_cache(state, 16, bits)  # torch ops on the GPU
    ours = mk.allocate_state_kernel_cache(state, 16, bits, layout="reference")
    torch.cuda.synchronize()
    init_diff = (ours.q_state != theirs.q_state).float().mean().item()
    _report(test="mx_initial_quantiser", bits=bits, codes_differ=init_diff,
            exps_differ=(ours.shared_exp != theirs.shared_exp).float().mean().item())
    assert init_diff < 1e-4
    # start both from the library's initial codes so that the step itself is what is compared
    for name in ("q_state", "shared_exp", "micro_exp"):
        getattr(theirs, name).copy_(getattr(ours, name))
    steps = 3
    for s in range(steps):
        y_lq = mk.mx_state_selective_update(ours, x, dt, A, B, C, D=D, dt_bias=bias, dt_softplus=True, stochastic=True, seed=0,
                                            rng_stream="reference")
        if bits == 8:
            y_ref = rmk.mx_state_selective_update(theirs, x, dt, A, B, C, D=D, dt_bias=bias, dt_softplus=True, stochastic=True, seed=0)
        else:  # the reference's wrapper raises TypeError for MX4 as shipped: launch its two kernels directly
            y_ref = torch.empty_like(x)
            tmp = torch.empty((b, h, p, n), dtype=torch.float32, device=dev())
            off = theirs.step * b * h * p * n
            rmk._state_update_mx8_kernel[((p + 15) // 16, b, h)](
                theirs.q_state, theirs.shared_exp, theirs.micro_exp, x, dt, bias, A, B, C, D, None, y_ref, tmp, h // g,
                *theirs.q_state.stride(), *theirs.shared_exp.stride(), *theirs.micro_exp.stride(), *x.stride(), *dt.stride(),
                *A.stride(), *B.stride(), *C.stride(), *D.stride(), 0, 0, 0, *y_ref.stride(), p, n, True,
                HAS_DT_BIAS=True, HAS_D=True, HAS_Z=False, FORMAT_BITS=4, STOCHASTIC=True, RNG_SEED=0, RNG_OFFSET=off,
                BLOCK_SIZE_M=16, BLOCK_SIZE_N=n)
            rmk._requantize_mx4_kernel[(b * h * p * (n // 16),)](tmp, theirs.q_state, theirs.shared_exp, theirs.micro_exp,
                                                                 b * h * p, n, True, 0, off)
            theirs.step += 1
        torch.cuda.synchronize()
        err = ((y_lq.float() - y_ref.float()).abs().max() / y_ref.float().abs().max()).item()
        qd = (ours.q_state != theirs.q_state)
        step_off = (ours.q_state.int() - theirs.q_state.int()).abs().max().item()
        _report(test="mx_fused_update", bits=bits, step=s, y_rel_err_vs_triton=err, codes_differ=qd.float().mean().item(),
                exps_differ=(ours.shared_exp != theirs.shared_exp).float().mean().item(), max_code_step=step_off)
        assert err <= 2.0 ** -7  # bf16 outputs
        assert qd.float().mean().item() < 5e-3 and step_off <= 1
        # continue both from the same state: differences must not compound into the next comparison
        for name in ("q_state", "shared_exp", "micro_exp"):
            getattr(theirs, name).copy_(getattr(ours, name))
    assert ours.step == theirs.step == steps

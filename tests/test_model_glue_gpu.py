"""The patch functions and the attention forward replacement running inside a model on the GPU: a
small Nemotron-H-shaped torch model (tests/nemotron_h_shim.py) is decoded unpatched (bf16 KV, bf16
SSM state) and patched (INT4 KV cache, MX8 / MX4 state), the way run_nemotron_8b_decode_degradation.py
drives the real model: prefill, register the state caches, then one token per step."""
import copy

import numpy as np
import pytest
import torch

import oracle
from tests import nemotron_h_shim as shim

pytestmark = pytest.mark.gpu

CTX, STEPS, BATCH = 48, 24, 3


def _model(seed=0):
    torch.manual_seed(seed)
    cfg = shim.tiny_config()
    model = shim.NemotronHShimForCausalLM(cfg)
    for p in model.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.05)
    return model.to("cuda", torch.bfloat16).eval(), cfg


def _decode(model, cfg, ids, mode_by_layer=None):
    """Prefill CTX tokens, then STEPS single-token steps; returns last-position logits per step and the cache."""
    from layer_quant_b200.mamba_state_8b_kernel import register_mamba_state_kernel_caches
    shim._mamba_decode_state_kernel_caches = {}
    cache = shim.HybridMambaAttentionDynamicCache(cfg, ids.shape[0], torch.bfloat16, device=ids.device)
    logits = []
    with torch.inference_mode():
        model(ids[:, :CTX], cache_params=cache, cache_position=torch.arange(CTX, device=ids.device))
        if mode_by_layer:
            register_mamba_state_kernel_caches(model, cache, mode_by_layer)
        for s in range(STEPS):
            pos = CTX + s
            out = model(ids[:, pos:pos + 1], cache_params=cache, cache_position=torch.tensor([pos], device=ids.device))
            logits.append(out.logits[:, -1].float())
    torch.cuda.synchronize()
    return torch.stack(logits, dim=1), cache


def _kl(p_logits, q_logits):
    p = torch.log_softmax(p_logits, -1)
    q = torch.log_softmax(q_logits, -1)
    return float((p.exp() * (p - q)).sum(-1).mean())


@pytest.fixture(scope="module")
def runs():
    from layer_quant_b200.int4_8b_attention import patch_nemotron_h_attention_int4_kv
    from layer_quant_b200.mamba_state_8b_kernel import patch_nemotron_h_mamba_decode_state_kernel
    original_ssu = shim.selective_state_update
    for name in ("_mx_state_kernel_patched", "_mx_state_kernel_original"):
        if hasattr(shim, name):
            delattr(shim, name)
    model, cfg = _model()
    ids = torch.randint(0, cfg.vocab_size, (BATCH, CTX + STEPS + 1), generator=torch.Generator().manual_seed(1)).cuda()
    mamba = [i for i, k in enumerate(cfg.hybrid_override_pattern) if k == "M"]
    out = {"cfg": cfg, "mamba": mamba}
    out["base"] = _decode(model, cfg, ids)
    int4_model = copy.deepcopy(model)
    patch_nemotron_h_attention_int4_kv(int4_model, group_size=32)
    out["int4"] = _decode(int4_model, cfg, ids)
    patch_nemotron_h_mamba_decode_state_kernel(model, 16, stochastic=False, seed=0)
    out["mx8"] = _decode(model, cfg, ids, {i: "mx8" for i in mamba})
    out["mx8_kernel_caches"] = dict(model._mamba_decode_state_kernel_caches)
    out["mx8_meta"] = dict(model._mamba_decode_state_kernel_meta)
    patch_nemotron_h_mamba_decode_state_kernel(int4_model, 16, stochastic=True, seed=1234)
    out["both"] = _decode(int4_model, cfg, ids, {i: "mx8" for i in mamba})
    out["mx4"] = _decode(model, cfg, ids, {i: "mx4" for i in mamba[:1]})
    yield out
    shim.selective_state_update = original_ssu


def test_int4_kv_decode_tracks_the_bf16_model(runs):
    base, _ = runs["base"]
    got, cache = runs["int4"]
    assert torch.isfinite(got).all()
    assert _kl(base, got) < 0.02
    assert (base.argmax(-1) == got.argmax(-1)).float().mean() > 0.85
    layer_caches = cache._int4_kv_layer_caches
    attn = [i for i, k in enumerate(runs["cfg"].hybrid_override_pattern) if k == "*"]
    assert sorted(layer_caches) == attn
    for c in layer_caches.values():
        assert c.length == CTX + STEPS and c.k_packed.shape[2] >= CTX + STEPS
    # the first attention layer sees bit-identical inputs in both runs (nothing upstream is quantised), so its
    # INT4 rows must be the oracle codec applied to the bf16 keys / values the unpatched model cached
    first = attn[0]
    k_bf16 = runs["base"][1].key_cache[first].float().cpu().numpy()
    v_bf16 = runs["base"][1].value_cache[first].float().cpu().numpy()
    n = CTX + STEPS
    for src, packed, scale in ((k_bf16, layer_caches[first].k_packed, layer_caches[first].k_scale),
                               (v_bf16, layer_caches[first].v_packed, layer_caches[first].v_scale)):
        q, s = oracle.int4_encode(src, 32)
        assert np.array_equal(packed[:, :, :n].cpu().numpy(), oracle.int4_pack_nibbles(q))
        assert np.array_equal(scale[:, :, :n].cpu().numpy(), s)


def test_mx8_state_decode_tracks_the_bf16_model(runs):
    base, base_cache = runs["base"]
    got, cache = runs["mx8"]
    assert torch.isfinite(got).all()
    assert _kl(base, got) < 0.02
    kernel_caches = runs["mx8_kernel_caches"]
    assert len(kernel_caches) == len(runs["mamba"])
    assert set(runs["mx8_meta"]) == set(runs["mamba"])
    for i in runs["mamba"]:
        kc = kernel_caches[id(cache.ssm_states[i])]
        assert kc.step == STEPS and kc.format_bits == 8 and kc.layer == i
        ref_state = base_cache.ssm_states[i].float()
        err = (kc.dequantize() - ref_state).abs().max() / ref_state.abs().max()
        assert err < 0.1, f"layer {i}: MX8 state drifted {err:.3f} from the bf16 state"


def test_int4_plus_stochastic_mx8_and_mx4(runs):
    base, _ = runs["base"]
    both, _ = runs["both"]
    mx4, _ = runs["mx4"]
    assert torch.isfinite(both).all() and torch.isfinite(mx4).all()
    assert _kl(base, both) < 0.05
    assert _kl(base, mx4) < 0.5  # one layer at 4 bits: coarse, but the same distribution family
    assert _kl(base, mx4) > _kl(base, runs["mx8"][0]) * 0.5  # and visibly coarser than MX8


def test_unregistered_states_fall_through_to_the_original_update(runs):
    """After the patch, a state tensor that was never registered still goes through the model's own
    selective_state_update (the reference's dispatch-by-id rule)."""
    assert getattr(shim, "_mx_state_kernel_patched", False)
    shim._mamba_decode_state_kernel_caches = {}
    state = torch.zeros((1, 8, 64, 128), device="cuda", dtype=torch.bfloat16)
    x = torch.ones((1, 8, 64), device="cuda", dtype=torch.bfloat16)
    dt = torch.ones((1, 8, 64), device="cuda", dtype=torch.bfloat16)
    A = -torch.ones((8, 64, 128), device="cuda")
    B = torch.ones((1, 2, 128), device="cuda", dtype=torch.bfloat16)
    y = shim.selective_state_update(state, x, dt, A, B, B)
    assert torch.allclose(y.float(), torch.full_like(y.float(), 128.0)) and float(state.float().mean()) == 1.0

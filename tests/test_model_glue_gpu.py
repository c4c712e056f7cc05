"""The patch functions and the attention forward replacement running inside a model on the GPU: a
small Nemotron-H-shaped torch model (tests/models/nemotron_h_shim) is decoded unpatched (bf16 KV, bf16
SSM state) and patched (INT4 KV cache, MX8 / MX4 state), the way run_nemotron_8b_decode_degradation.py
drives the real model: prefill, register the state caches, then one token per step."""
import copy

import numpy as np
import pytest
import torch

import oracle
from tests.models.nemotron_h_shim import modeling_nemotron_h_shim as shim

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


def test_whole_decode_step_replays_from_a_cuda_graph():
    """INT4 KV + MX8 state decode with the positions and step counts on the device: the whole model step
    (embedding to logits) is recorded once and replayed for every token; logits must track the eager,
    host-synchronised run of the same patched model, and the caches must end up at the same lengths."""
    from layer_quant_b200 import int4_8b_attention as ia
    from layer_quant_b200 import mamba_state_8b_kernel as mk
    from layer_quant_b200 import _lib
    original_ssu = shim.selective_state_update
    for name in ("_mx_state_kernel_patched", "_mx_state_kernel_original"):
        if hasattr(shim, name):
            delattr(shim, name)
    try:
        model, cfg = _model(seed=3)
        ids = torch.randint(0, cfg.vocab_size, (BATCH, CTX + STEPS + 1), generator=torch.Generator().manual_seed(4)).cuda()
        mamba = [i for i, k in enumerate(cfg.hybrid_override_pattern) if k == "M"]
        ia.patch_nemotron_h_attention_int4_kv(model, group_size=32)
        mk.patch_nemotron_h_mamba_decode_state_kernel(model, 16, stochastic=False, seed=0)
        eager, eager_cache = _decode(model, cfg, ids, {i: "mx8" for i in mamba})

        shim._mamba_decode_state_kernel_caches = {}
        cache = shim.HybridMambaAttentionDynamicCache(cfg, BATCH, torch.bfloat16, device=ids.device)
        token = torch.zeros((BATCH, 1), dtype=ids.dtype, device=ids.device)
        with torch.inference_mode():
            model(ids[:, :CTX], cache_params=cache, cache_position=torch.arange(CTX, device=ids.device))
            mk.register_mamba_state_kernel_caches(model, cache, {i: "mx8" for i in mamba})
            ia.prepare_graph_decode(cache, CTX + STEPS)
            mk.prepare_graph_decode(model)
            # one step outside the recording (allocates the scratch), undone on the device-side counters
            snap = [(c.length_counter.clone()) for c in ia._cache_dict(cache).values()]
            snap_state = [(k.q_state.clone(), k.shared_exp.clone(), k.micro_exp.clone(), k.step_counter.clone())
                          for k in model._mamba_decode_state_kernel_caches.values()]
            conv = [c.clone() for c in cache.conv_states]
            token.copy_(ids[:, CTX:CTX + 1])
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                model(token, cache_params=cache)
            torch.cuda.current_stream().wait_stream(side)
            for c, n in zip(ia._cache_dict(cache).values(), snap):
                c.length_counter.copy_(n)
            for k, (q, e, m, st) in zip(model._mamba_decode_state_kernel_caches.values(), snap_state):
                k.q_state.copy_(q), k.shared_exp.copy_(e), k.micro_exp.copy_(m), k.step_counter.copy_(st)
            for dst, src in zip(cache.conv_states, conv):
                dst.copy_(src)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_logits = model(token, cache_params=cache).logits
            got = []
            for s in range(STEPS):
                token.copy_(ids[:, CTX + s:CTX + s + 1])
                graph.replay()
                got.append(static_logits[:, -1].float().clone())
        torch.cuda.synchronize()
        got = torch.stack(got, dim=1)
        scale = float(eager.abs().max())
        assert float((got - eager).abs().max()) <= 2e-2 * scale, float((got - eager).abs().max()) / scale
        assert _kl(eager, got) < 1e-3
        ia.sync_graph_decode(cache)
        assert all(c.length == CTX + STEPS for c in ia._cache_dict(cache).values())
        assert set(mk.graph_decode_steps(model).values()) == {STEPS}
        assert _lib.device_status() == 0
        # the INT4 rows appended by the replays are the rows the eager run appended (same K/V up to MX/attention noise
        # upstream, so compare the prefill rows exactly and the shapes of the rest)
        for idx, c in ia._cache_dict(cache).items():
            ref = ia._cache_dict(eager_cache)[idx]
            assert torch.equal(c.k_packed[:, :, :CTX], ref.k_packed[:, :, :CTX])
            assert torch.equal(c.v_scale[:, :, :CTX], ref.v_scale[:, :, :CTX])
    finally:
        shim.selective_state_update = original_ssu
        shim._mamba_decode_state_kernel_caches = {}


def test_prefill_from_the_quantised_cache_in_the_forward():
    """With PREFILL_FROM_INT4_CACHE the attention forward serves a prompt from the packed cache; the prompt's
    last-position logits must track the default path (SDPA over the un-quantised K / V) closely: the only
    difference is INT4 rounding of K / V inside the prompt."""
    from layer_quant_b200 import int4_8b_attention as ia
    model, cfg = _model(seed=5)
    ia.patch_nemotron_h_attention_int4_kv(model, group_size=32)
    ids = torch.randint(0, cfg.vocab_size, (BATCH, CTX), generator=torch.Generator().manual_seed(6)).cuda()
    outs = []
    try:
        for flag in (False, True):
            ia.PREFILL_FROM_INT4_CACHE = flag
            cache = shim.HybridMambaAttentionDynamicCache(cfg, BATCH, torch.bfloat16, device=ids.device)
            with torch.inference_mode():
                outs.append(model(ids, cache_params=cache, cache_position=torch.arange(CTX, device=ids.device)).logits.float())
            assert all(c.length == CTX for c in ia._cache_dict(cache).values())
    finally:
        ia.PREFILL_FROM_INT4_CACHE = False
    assert not torch.equal(outs[0], outs[1])
    assert _kl(outs[0][:, -1:], outs[1][:, -1:]) < 5e-3
    scale = float(outs[0].abs().max())
    assert float((outs[0] - outs[1]).abs().max()) < 0.1 * scale

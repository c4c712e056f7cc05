"""Alias of :mod:`layer_quant_b200.int4_8b_attention` under the reference's module path."""
from layer_quant_b200.int4_8b_attention import *  # noqa: F401,F403
from layer_quant_b200.int4_8b_attention import (  # noqa: F401
    Int4KVLayerCache, _allocate_layer_cache, _append_decode_attention, _cache_dict, _decode_attention,
    _decode_attention_mask, _ensure_layer_cache, _forward_fused_int4_kv, _pack_kv_into_cache, _positions, _prefill_attention,
    int4_quant_dequant, patch_nemotron_h_attention_int4_kv,
)

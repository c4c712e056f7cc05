"""Alias of :mod:`layer_quant_b200.nemotron_8b_decode_eval` under the reference's module path."""
from layer_quant_b200.nemotron_8b_decode_eval import (  # noqa: F401
    DeviceList, adjacent_mamba_layers, layer_groups, make_hybrid_cache, patch_attention_cache_in_blocks,
)

"""Helpers of the decode evaluation loop: host-side mirror of the reference module
``hybrid_quant/nemotron_8b_decode_eval.py`` (phcool/Layer_Quant), the immediate caller of the two
hot paths.  Same names and behaviour:

====================================  =========================================
here                                  reference (nemotron_8b_decode_eval.py)
====================================  =========================================
``patch_attention_cache_in_blocks``   :8-50   block.forward that hands the cache to attention mixers
``DeviceList``                        :53-56
``make_hybrid_cache``                 :59-66
``layer_groups``                      :69-74
``adjacent_mamba_layers``             :77-86
====================================  =========================================
"""
from __future__ import annotations

from types import MethodType

import torch


def _mixer_call(block, hidden_states, cache_params, cache_position, attention_mask):
    """Run the block's mixer with the arguments its kind takes; attention gets the cache as past_key_value."""
    kind = block.block_type
    if kind == "mlp":
        return block.mixer(hidden_states)
    if kind == "mamba":
        return block.mixer(hidden_states, cache_params=cache_params, cache_position=cache_position, attention_mask=attention_mask)
    if kind == "attention":
        out = block.mixer(hidden_states, attention_mask=attention_mask, past_key_value=cache_params,
                          use_cache=cache_params is not None, cache_position=cache_position)
        return out[0]
    raise ValueError(f"Invalid block_type: {kind}")


def _block_forward_with_cache(self, hidden_states, cache_params=None, cache_position=None, attention_mask=None):
    device = hidden_states.device
    with torch.cuda.stream(torch.cuda.default_stream(device)):
        normed = self.norm(hidden_states.to(dtype=self.norm.weight.dtype))
        skip = hidden_states.to(torch.float32) if self.residual_in_fp32 else hidden_states
        return skip + _mixer_call(self, normed, cache_params, cache_position, attention_mask)


def patch_attention_cache_in_blocks(model) -> None:
    """Give every block of ``model.backbone.layers`` a forward that passes ``cache_params`` to attention
    mixers as ``past_key_value`` (the remote Nemotron-H block drops it) and runs on the device's default
    stream, as the reference does (:8-50)."""
    for block in model.backbone.layers:
        if not getattr(block, "_decode_eval_block_patched", False):
            block.forward = MethodType(_block_forward_with_cache, block)
            block._decode_eval_block_patched = True


class DeviceList(list):
    """A list that also answers ``.device`` (what the remote cache's tensors-or-lists are asked for)."""

    def __init__(self, values, device):
        super().__init__(values)
        self.device = device


def make_hybrid_cache(model, batch_size: int):
    """The remote module's ``HybridMambaAttentionDynamicCache`` for ``model`` in bf16, its state lists
    wrapped in :class:`DeviceList`."""
    module = __import__(model.__class__.__module__, fromlist=["HybridMambaAttentionDynamicCache"])
    cache = module.HybridMambaAttentionDynamicCache(model.config, batch_size, torch.bfloat16, device=model.device)
    cache.conv_kernel_size = model.config.conv_kernel
    cache.conv_states = DeviceList(cache.conv_states, model.device)
    cache.ssm_states = DeviceList(cache.ssm_states, model.device)
    return cache


def layer_groups(config) -> tuple[list[int], list[int], list[int]]:
    """Indices of the Mamba2 ('M'), attention ('*') and MLP ('-') blocks of ``hybrid_override_pattern``."""
    pattern = config.hybrid_override_pattern
    pick = lambda kind: [i for i, c in enumerate(pattern) if c == kind]
    return pick("M"), pick("*"), pick("-")


def adjacent_mamba_layers(mamba_layers: list[int], attention_layers: list[int]) -> set[int]:
    """The Mamba2 layers directly before and after each attention layer."""
    out: set[int] = set()
    for attn in attention_layers:
        before = [i for i in mamba_layers if i < attn]
        after = [i for i in mamba_layers if i > attn]
        if before:
            out.add(before[-1])
        if after:
            out.add(after[0])
    return out

"""Alias of :mod:`layer_quant_b200.mamba_state_8b_kernel` under the reference's module path."""
from layer_quant_b200.mamba_state_8b_kernel import *  # noqa: F401,F403
from layer_quant_b200.mamba_state_8b_kernel import (  # noqa: F401
    MX4_BLOCK_SIZE, MX4_MANTISSA_MAX, MX4_PAIR_SIZE, MX8_BLOCK_SIZE, MX8_MANTISSA_MAX, MX8_PAIR_SIZE,
    MambaStateKernelCache, _quantize_initial_state_mx, allocate_state_kernel_cache, mx4_state_selective_update,
    mx8_state_selective_update, mx_state_selective_update, patch_nemotron_h_mamba_decode_state_kernel,
    register_mamba_state_kernel_caches,
)

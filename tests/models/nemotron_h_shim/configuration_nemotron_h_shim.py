"""Configuration of the Nemotron-H-shaped stand-in model (tests and the benchmark's model case)."""
from transformers import PretrainedConfig


class NemotronHShimConfig(PretrainedConfig):
    """Field names follow what the reference's helpers read from the real model's config:
    ``hybrid_override_pattern`` ('M' Mamba2, '*' attention, '-' MLP) and ``conv_kernel``."""

    model_type = "nemotron_h_shim"

    def __init__(self, hybrid_override_pattern="M-M*-M-*M", hidden_size=1024, vocab_size=512, intermediate_size=2048,
                 num_attention_heads=8, num_key_value_heads=2, head_dim=128, mamba_num_heads=8, mamba_head_dim=64,
                 mamba_intermediate=512, ssm_state_size=128, n_groups=2, conv_kernel=4, initializer_range=0.05, **kwargs):
        self.hybrid_override_pattern = hybrid_override_pattern
        self.hidden_size, self.vocab_size, self.intermediate_size = hidden_size, vocab_size, intermediate_size
        self.num_attention_heads, self.num_key_value_heads, self.head_dim = num_attention_heads, num_key_value_heads, head_dim
        self.mamba_num_heads, self.mamba_head_dim, self.mamba_intermediate = mamba_num_heads, mamba_head_dim, mamba_intermediate
        self.ssm_state_size, self.n_groups, self.conv_kernel = ssm_state_size, n_groups, conv_kernel
        self.initializer_range = initializer_range
        self.num_hidden_layers = len(hybrid_override_pattern)
        kwargs.setdefault("tie_word_embeddings", False)
        super().__init__(**kwargs)


def nemotron_h_8b_config() -> NemotronHShimConfig:
    """The 8B shape: 52 blocks = 24 Mamba2 + 4 attention + 24 MLP, hidden 4096, vocab 131072, FFN 21504,
    32 query / 8 kv heads of 128, Mamba2 with 128 heads of 64, state 128, 8 groups, conv kernel 4."""
    return NemotronHShimConfig(
        hybrid_override_pattern="M-M-M-M*-M-M-M-M-M*-M-M-M-M-M*-M-M-M-M-M*-M-M-M-M-M-", hidden_size=4096, vocab_size=131072,
        intermediate_size=21504, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        mamba_num_heads=128, mamba_head_dim=64, mamba_intermediate=8192, ssm_state_size=128, n_groups=8, conv_kernel=4,
        initializer_range=0.02)


def tiny_config(pattern="M-M*-M-*M", hidden=1024) -> NemotronHShimConfig:
    """The test shape.  hidden = attention heads x head_dim (8 x 128), as in the real model: the reference's attention
    forward reshapes its output to [batch, q_len, hidden_size] (int4_8b_attention.py:689,712)."""
    return NemotronHShimConfig(hybrid_override_pattern=pattern, hidden_size=hidden, intermediate_size=2 * hidden)

"""CPU restatement of the two Layer_Quant decode hot paths (TEST INFRASTRUCTURE ONLY).

This package is the checker for the CUDA library, never a product code path: only the
tests, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import it.
The shipped package (``layer_quant_b200``) never imports it and has no CPU fallback.

Every function restates, in numpy, one piece of the reference
(``hybrid_quant/int4_8b_attention.py`` and ``hybrid_quant/mamba_state_8b_kernel.py`` of
phcool/Layer_Quant) and cites the reference lines it follows.  The reference has no tests
and no golden vectors of its own; the oracle is pinned instead against outputs of the
reference's own kernels executed on CPU under ``TRITON_INTERPRET=1``, committed as
``tests/golden/*.npz`` together with the script that generated them
(``tests/golden/make_golden.py``).  The Philox generator lives in a third-party
dependency of the reference (Triton, ``triton/language/random.py``; the reference pins
torch==2.8.0 which ships triton 3.4.x, the fixtures were generated with triton 3.6.0);
its published algorithm (Philox4x32-10, Salmon et al. 2011) is restated in
``oracle/philox.py`` and pinned by known-answer words in the same fixtures.
``oracle/dense_state.py`` (the unquantised baselines, third-party mamba-ssm / causal-conv1d
behaviour) is the one part whose parity is unpinned; its header says why.
"""
from .philox import philox4x32_10, tl_randint, tl_rand, words_to_uniform  # noqa: F401
from .mx_codec import (  # noqa: F401
    mx_encode, mx_decode, mx_pack_micro_bits, mx_unpack_micro_bits, mx4_pack_nibbles,
    mx4_unpack_nibbles, ceil_log2_f32, native_sr_encode,
)
from .mx_state import mx_state_update, reference_rng_offsets, layered4_words  # noqa: F401
from .int4_kv import (  # noqa: F401
    int4_encode, int4_decode, int4_pack_nibbles, int4_unpack_nibbles, int4_quant_dequant,
    int4_decode_attention, decode_attention_mask, int4_prefill_attention,
)
from .dense_state import dense_state_update, causal_conv1d_update  # noqa: F401

"""Drop-in import path: ``hybrid_quant.int4_8b_attention`` and ``hybrid_quant.mamba_state_8b_kernel``
resolve to the layer_quant_b200 implementations, so scripts written against phcool/Layer_Quant's
``hybrid_quant`` package import them unchanged."""

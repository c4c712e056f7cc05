"""layer_quant_b200: B200 (sm_100a) kernels for the two Nemotron-H-8B decode hot paths of
phcool/Layer_Quant, behind the reference's own Python call signatures.

* ``layer_quant_b200.int4_8b_attention``      mirrors ``hybrid_quant/int4_8b_attention.py``
* ``layer_quant_b200.mamba_state_8b_kernel``  mirrors ``hybrid_quant/mamba_state_8b_kernel.py``
* ``layer_quant_b200.sharding``               batch sharding over ranks (one process per GPU)

The kernels live in ``liblayer_quant_b200.so`` (C ABI, ``include/layer_quant_b200.h``), built by
``python -m layer_quant_b200.build``.  There is no Triton, CPU or eager fallback.
"""
__version__ = "0.1.0"

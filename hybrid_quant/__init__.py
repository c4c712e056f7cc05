"""Drop-in import path: ``hybrid_quant.int4_8b_attention`` and ``hybrid_quant.mamba_state_8b_kernel``
resolve to the layer_quant_b200 implementations, so scripts written against phcool/Layer_Quant's
``hybrid_quant`` package import them unchanged.

Only those two modules are replaced.  Every other module of the reference's package
(``hybrid_quant.data``, ``hybrid_quant.env``, ``hybrid_quant.nemotron_8b_decode_eval`` ...) is looked up
in the ``hybrid_quant`` directories that come LATER on ``sys.path``: put this repository first and a
checkout of the reference after it, and the reference's scripts run with its own helpers around the
two replaced hot paths.
"""
from pkgutil import extend_path

__path__ = extend_path(__path__, __name__)

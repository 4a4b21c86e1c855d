"""eptq_b200 -- B200 (sm_100a) inference path for EPTQ-quantized linear layers.

Public surface, named as in the reference package:
  eptq_b200.config.QuantizedLayerData          (reference: config.py:98-159)
  eptq_b200.quantizers.E8LatticeQuantizer/E8D4Quantizer  (codebook + dequant only)
  eptq_b200.kernels.e8_forward / e8d4_forward / dequantize_layer
  eptq_b200.kernels.linear.EPTQLinear          (reference: kernels/linear.py:20)
  eptq_b200.kernels.patch.load_quantized_model (reference: kernels/patch.py:24)

All compute goes through the C-ABI library built from ``csrc/``; there is no
CPU or PyTorch fallback.
"""
from .config import QuantizedLayerData  # noqa: F401

__all__ = ["QuantizedLayerData"]

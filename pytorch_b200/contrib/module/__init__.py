"""Quantized linear layers with the reference's names and constructor signatures
(``torch_npu/contrib/module/__init__.py:17-19``)."""
from .linear_a8w8_quant import LinearA8W8Quant
from .linear_quant import LinearQuant
from .linear_weight_quant import LinearWeightQuant

__all__ = ["LinearA8W8Quant", "LinearQuant", "LinearWeightQuant"]

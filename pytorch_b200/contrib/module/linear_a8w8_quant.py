"""``LinearA8W8Quant``: the deprecated alias of ``LinearQuant`` with its stricter dtype checks
(``torch_npu/contrib/module/linear_a8w8_quant.py:12-120``; messages at ``:91-111``)."""
import warnings

import torch
import torch.nn as nn
from torch import Tensor

from .linear_quant import init_quant_linear, quant_linear_forward

__all__ = ["LinearA8W8Quant"]


class LinearA8W8Quant(nn.Module):
    def __init__(self, in_features: int, out_features: int, *, bias: bool = True, offset: bool = False,
                 pertoken_scale: bool = False, device=None, dtype=None, output_dtype=None) -> None:
        super().__init__()
        warnings.warn("LinearA8W8Quant is deprecated and will be removed in a future version. "
                      "Use LinearQuant instead.", FutureWarning)
        init_quant_linear(self, in_features, out_features, bias, offset, pertoken_scale, device, output_dtype)

    def forward(self, linear_quant_input: Tensor) -> Tensor:
        def bad(what, allowed, got):
            return ValueError(f"{what} should be {allowed} datatype, but now it is {got}.")

        if self.scale.dtype not in [torch.int64, torch.float32, torch.bfloat16]:
            raise bad("scale", "torch.int64, torch.float32 or torch.bfloat16", self.scale.dtype)
        if self.offset is not None and self.offset.dtype is not torch.float32:
            raise bad("offset", "torch.float32", self.offset.dtype)
        if self.bias is not None and self.bias.dtype not in [torch.int32, torch.bfloat16, torch.float16,
                                                               torch.float32]:
            raise bad("bias", "torch.int32, torch.bfloat16, torch.float16 or torch.float32", self.bias.dtype)
        if self.pertoken_scale is not None and self.pertoken_scale.dtype is not torch.float32:
            raise bad("pertoken_scale", "torch.float32", self.pertoken_scale.dtype)
        if self.output_dtype is not None and self.output_dtype not in [torch.int8, torch.float16, torch.bfloat16]:
            raise ValueError("output_dtype should be torch.int8, torch.float16 or torch.bfloat16, "
                             f"but now it is {self.output_dtype}.")
        return quant_linear_forward(self, linear_quant_input)

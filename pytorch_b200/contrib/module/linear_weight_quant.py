"""``LinearWeightQuant``: weight-only quantised linear (W8A16 / int4-packed W4A16) over
``npu_weight_quant_batchmatmul``.  Mirrors ``torch_npu/contrib/module/linear_weight_quant.py:10-109``:
same constructor, weight stored ``[out,in]`` and passed as its transposed view, 2-D antiquant
parameters stored ``[out, groups]`` and transposed to ``[groups, out]`` for the call."""
import torch
import torch.nn as nn
from torch import Tensor
from torch.nn.parameter import Parameter

__all__ = ["LinearWeightQuant"]


class LinearWeightQuant(nn.Module):
    in_features: int
    out_features: int
    weight: Tensor
    antiquant_scale: Tensor
    antiquant_offset: Tensor
    quant_scale: Tensor
    quant_offset: Tensor

    def __init__(self, in_features, out_features, bias: bool = True, device=None, dtype=None,
                 antiquant_offset: bool = False, quant_scale: bool = False, quant_offset: bool = False,
                 antiquant_group_size: int = 0, inner_precise: int = 0, weight_dtype=None) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = Parameter(torch.empty((out_features, in_features), device=device), False)
        self.antiquant_scale = Parameter(torch.empty(out_features, device=device), False)
        for name, present in (("antiquant_offset", antiquant_offset), ("quant_scale", quant_scale),
                              ("quant_offset", quant_offset), ("bias", bias)):
            if present:
                setattr(self, name, Parameter(torch.empty(out_features, device=device), False))
            else:
                self.register_parameter(name, None)
        self.antiquant_group_size = antiquant_group_size
        self.inner_precise = inner_precise
        self.weight_dtype = weight_dtype

    def forward(self, x: Tensor) -> Tensor:
        scale = self.antiquant_scale
        offset = self.antiquant_offset
        if scale.dim() == 2:
            scale = scale.transpose(-1, -2)
        if offset is not None and offset.dim() == 2:
            offset = offset.transpose(-1, -2)
        return torch.ops.npu.npu_weight_quant_batchmatmul(
            x, self.weight.transpose(-1, -2), scale, offset, self.quant_scale, self.quant_offset, self.bias,
            self.antiquant_group_size, self.inner_precise, weight_dtype=self.weight_dtype)

"""``LinearQuant``: int8 x int8 linear layer over ``npu_quant_matmul``.

Mirrors ``torch_npu/contrib/module/linear_quant.py:11-112``: the same constructor signature
(frozen in ``test/torch_npu_schema.json:26-39``), the same non-trainable parameters
(``weight [out,in]``, ``scale [out]``, ``offset [out]`` fp32, ``pertoken_scale`` fp32,
``bias [out]`` int32), the same dtype gate and the same call: the weight is handed to the
operator as its transposed view, which is the K-major layout the tensor-core kernel reads
without a copy.
"""
import torch
import torch.nn as nn
from torch import Tensor
from torch.nn.parameter import Parameter

__all__ = ["LinearQuant"]


def quant_linear_forward(mod, x: Tensor) -> Tensor:
    ops = torch.ops.npu
    if not ((x.dtype == torch.int32 and mod.weight.dtype == torch.int32) or
            (x.dtype == torch.int8 and mod.weight.dtype == torch.int8)):
        raise ValueError("input and weight should be both torch.int32 or both torch.int8 datatype, "
                         f"but now input is {x.dtype}, weight is {mod.weight.dtype}.")
    scale = mod.scale
    fp32_scale_needs_packing = (mod.scale.dtype == torch.float32 and
                                mod.output_dtype not in [torch.bfloat16, torch.int32])
    if mod.pertoken_scale is None and fp32_scale_needs_packing:
        scale = ops.npu_trans_quant_param(mod.scale, mod.offset)
    w = mod.weight
    return ops.npu_quant_matmul(x, w.transpose(w.dim() - 2, w.dim() - 1), scale, offset=mod.offset,
                                pertoken_scale=mod.pertoken_scale, bias=mod.bias,
                                output_dtype=mod.output_dtype)


def init_quant_linear(mod, in_features, out_features, bias, offset, pertoken_scale, device, output_dtype):
    mod.in_features = in_features
    mod.out_features = out_features
    mod.weight = Parameter(torch.empty((out_features, in_features), device=device), False)
    mod.scale = Parameter(torch.empty(out_features, device=device), False)
    mod.output_dtype = output_dtype
    if offset:
        mod.offset = Parameter(torch.empty(out_features, dtype=torch.float32, device=device), False)
    else:
        mod.register_parameter("offset", None)
    if pertoken_scale:
        mod.pertoken_scale = Parameter(torch.empty(out_features, dtype=torch.float32, device=device), False)
    else:
        mod.register_parameter("pertoken_scale", None)
    if bias:
        mod.bias = Parameter(torch.empty(out_features, dtype=torch.int32, device=device), False)
    else:
        mod.register_parameter("bias", None)


class LinearQuant(nn.Module):
    r"""``y = dequant(x @ weight^T)`` with int8 (A8W8) operands.

    Parameters are placeholders to be overwritten with quantised values
    (``module.weight.data = w_int8`` ...), exactly as with the reference module.

    Example::
        >>> m = LinearQuant(5120, 13824, bias=False, output_dtype=torch.bfloat16).cuda()
        >>> m.weight.data = w_int8            # [13824, 5120]
        >>> m.scale.data = w_scale            # [13824] fp32
        >>> y = m(x_int8)                     # [..., 13824] bf16
    """
    in_features: int
    out_features: int
    weight: Tensor
    scale: Tensor
    offset: Tensor
    pertoken_scale: Tensor
    bias: Tensor

    def __init__(self, in_features: int, out_features: int, *, bias: bool = True, offset: bool = False,
                 pertoken_scale: bool = False, device=None, dtype=None, output_dtype=None) -> None:
        super().__init__()
        init_quant_linear(self, in_features, out_features, bias, offset, pertoken_scale, device, output_dtype)

    def forward(self, linear_quant_input: Tensor) -> Tensor:
        return quant_linear_forward(self, linear_quant_input)

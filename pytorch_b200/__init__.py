"""B200-native implementation of torch_npu's quantized-inference operator path.

Importing the package loads the in-tree PyTorch extension, which registers the operators
under the reference's own names (``torch.ops.npu.npu_dynamic_quant`` and friends) and, as
the reference does in ``torch_npu/_init/core/_exports.py:45-51``, re-exports every one of them
as an attribute of this package: ``pytorch_b200.npu_quant_matmul is torch.ops.npu.npu_quant_matmul``.

There is no CPU, Triton or eager fallback.  If the extension has not been built the import
raises; build it with ``python pytorch_b200/_build.py``.
"""
from __future__ import annotations

import os as _os

import torch as _torch

_LIBDIR = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "lib")
_TORCH_LIB = _os.path.join(_LIBDIR, "libb200q_torch.so")

OPS = (
    "npu_dynamic_quant",
    "npu_quant_matmul",
    "npu_weight_quant_batchmatmul",
    "npu_convert_weight_to_int4pack",
    "npu_trans_quant_param",
    "npu_dynamic_quant_asymmetric",
    "npu_anti_quant",
    "npu_swiglu_quant",
    "npu_mm_reduce_scatter_base",
    "npu_all_gather_base_mm",
    "npu_mm_all_reduce_base",
)


def _load() -> None:
    if not _os.path.exists(_TORCH_LIB):
        raise ImportError(
            f"{_TORCH_LIB} is missing: build the extension with `python pytorch_b200/_build.py`; "
            "the operators have no fallback implementation")
    _torch.ops.load_library(_TORCH_LIB)


_load()

npu_dynamic_quant = _torch.ops.npu.npu_dynamic_quant
npu_quant_matmul = _torch.ops.npu.npu_quant_matmul
npu_weight_quant_batchmatmul = _torch.ops.npu.npu_weight_quant_batchmatmul
npu_convert_weight_to_int4pack = _torch.ops.npu.npu_convert_weight_to_int4pack
npu_trans_quant_param = _torch.ops.npu.npu_trans_quant_param
npu_dynamic_quant_asymmetric = _torch.ops.npu.npu_dynamic_quant_asymmetric
npu_anti_quant = _torch.ops.npu.npu_anti_quant
npu_swiglu_quant = _torch.ops.npu.npu_swiglu_quant

from . import collective_ops  # noqa: E402,F401  (defines the three collective-fused operators in torch.ops.npu)

npu_mm_reduce_scatter_base = _torch.ops.npu.npu_mm_reduce_scatter_base
npu_all_gather_base_mm = _torch.ops.npu.npu_all_gather_base_mm
npu_mm_all_reduce_base = _torch.ops.npu.npu_mm_all_reduce_base

from . import contrib  # noqa: E402,F401

__all__ = list(OPS) + ["contrib", "OPS"]

"""A W8A8 SwiGLU MLP block as a chain of the quantized operators.

The reference tree has no function of this name; it ships the pieces (``npu_dynamic_quant``,
``npu_quant_matmul``, ``npu_swiglu`` at ``torch_npu/_inductor/decomposition.py:186-188`` and the fused
``npu_swiglu_quant`` named in ``docs/zh/release_notes.md:303``) and leaves the chaining to the model
code.  This is that chain with the activations quantised in flight: the only tensors written to HBM
between the two GEMMs are the bf16 gate/up projection and the int8 activation."""
from __future__ import annotations

import torch


def w8a8_swiglu_mlp(x: torch.Tensor, smooth_in: torch.Tensor | None, w_gate_up: torch.Tensor,
                    scale_gate_up: torch.Tensor, smooth_act: torch.Tensor | None, w_down: torch.Tensor,
                    scale_down: torch.Tensor, output_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``down( quant( silu(gate(x)) * up(x) ) )`` with int8 weights and per-token dynamic activations.

    ``w_gate_up`` is ``[2F, K]`` (gate rows first, then up rows; the layout ``LinearQuant`` keeps its
    weight in), ``w_down`` is ``[H, F]``; ``scale_*`` are the per-channel weight scales ``[2F]`` / ``[H]``;
    ``smooth_in`` ``[K]`` and ``smooth_act`` ``[F]`` are optional smooth-quant vectors."""
    ops = torch.ops.npu
    q, s = ops.npu_dynamic_quant(x, smooth_scales=smooth_in)
    gu = ops.npu_quant_matmul(q, w_gate_up.transpose(-2, -1), scale_gate_up, pertoken_scale=s.reshape(-1),
                              output_dtype=torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float16)
    qa, sa = ops.npu_swiglu_quant(gu, smooth_scales=smooth_act, activate_left=True, quant_mode=1)
    return ops.npu_quant_matmul(qa, w_down.transpose(-2, -1), scale_down, pertoken_scale=sa.reshape(-1),
                                output_dtype=output_dtype)

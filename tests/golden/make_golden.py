"""Regenerates the fixtures in this directory.  Run from the repository root:

    python tests/golden/make_golden.py --reference <path to the Ascend/pytorch tree>

``reference_goldens.npz`` is produced by the REFERENCE's own CPU golden helpers:
the helper functions are cut out of the reference's test files by name with
``ast`` (those files import ``torch_npu`` at the top and so cannot be imported on
a machine without an Ascend device) and executed unchanged on small seeded
inputs.  The tests then require the oracle to reproduce those outputs:

* ``unpack_int4``                       test/custom_ops/test_npu_anti_quant.py:12-24
* ``TestAntiQuant.custom_op_exec``      test/custom_ops/test_npu_anti_quant.py:29-42 (int4 and int8 inputs,
                                        fp16 and bf16 outputs, with and without offset)
* ``cpu_linear_weight_quant``           test/contrib/test_linear_weight_quant.py:20-28
* ``_get_global_tensor`` (int8 dequant) test/distributed/tensor/test_matrix_ops.py:21-40
* ``TestMmReduceScatterBaseOp._get_global_tensor`` (per-rank int8 products, dequantised and added in rank
                                        order)  test/distributed/tensor/test_matrix_ops.py:86-110

``oracle_kat.npz`` holds known-answer vectors computed by ``oracle/quant_oracle.py``
for config 1 and a few small cases, so that the GPU tests can be held against
committed bytes as well as against the live oracle.  bf16 tensors are stored as
their uint16 bit patterns.
"""
from __future__ import annotations

import argparse
import ast
import os
import sys
import textwrap

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import quant_oracle as oracle          # noqa: E402
from pytorch_b200 import workloads                 # noqa: E402


def _cut(path, name, cls=None):
    """Source text of function ``name`` (inside class ``cls`` if given)."""
    src = open(path).read()
    tree = ast.parse(src)
    body = tree.body
    if cls is not None:
        body = next(n for n in body if isinstance(n, ast.ClassDef) and n.name == cls).body
    fn = next(n for n in body if isinstance(n, ast.FunctionDef) and n.name == name)
    return textwrap.dedent(ast.get_source_segment(src, fn, padded=True))


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def reference_goldens(ref):
    from ml_dtypes import int4
    out = {}
    g = torch.Generator().manual_seed(77)

    ns = {"np": np, "torch": torch, "int4": int4}
    f_anti = os.path.join(ref, "test/custom_ops/test_npu_anti_quant.py")
    exec(_cut(f_anti, "unpack_int4"), ns)
    exec(_cut(f_anti, "custom_op_exec", "TestAntiQuant"), ns)
    packed = torch.randint(-2**31, 2**31 - 1, (6, 10), generator=g, dtype=torch.int64).to(torch.int32)
    out["unpack_in"] = packed.numpy()
    out["unpack_out"] = ns["unpack_int4"](packed).numpy()
    scale = torch.rand(80, generator=g) * 200 - 100
    offs = torch.rand(80, generator=g) * 200 - 100
    out["anti_scale"], out["anti_offset"] = scale.numpy(), offs.numpy()
    out["anti_out_f16"] = ns["custom_op_exec"](None, packed, scale, offs, torch.float16, None).numpy()
    # int8 input, both output types, with and without offset (shapes of test_npu_anti_quant.py:49-58)
    g8 = torch.Generator().manual_seed(78)      # its own stream: the draws below keep their values
    x8 = torch.randint(-127, 128, (10, 100), generator=g8, dtype=torch.int64).to(torch.int8)
    sc8 = torch.rand(100, generator=g8) * 200 - 100
    of8 = torch.rand(100, generator=g8) * 200 - 100
    out["anti8_x"], out["anti8_scale"], out["anti8_offset"] = x8.numpy(), sc8.numpy(), of8.numpy()
    out["anti8_out_f16"] = ns["custom_op_exec"](None, x8, sc8, of8, torch.float16, torch.int8).numpy()
    out["anti8_out_bf16"] = bits(ns["custom_op_exec"](None, x8, sc8, of8, torch.bfloat16, torch.int8))
    out["anti8_out_nooff_f16"] = ns["custom_op_exec"](None, x8, sc8, None, torch.float16, None).numpy()
    out["anti_out_bf16"] = bits(ns["custom_op_exec"](None, packed, scale, offs, torch.bfloat16, None))

    ns2 = {"np": np, "torch": torch}
    f_wq = os.path.join(ref, "test/contrib/test_linear_weight_quant.py")
    exec(_cut(f_wq, "cpu_linear_weight_quant", "TestLinearWeightQuant"), ns2)
    m, k, n = 8, 96, 40
    x = torch.randn((m, k), generator=g).to(torch.float16)
    w = torch.randn((n, k), generator=g).mul(20).to(torch.int8)
    a_s = torch.randn(n, generator=g).to(torch.float16)
    a_o = torch.randn(n, generator=g).to(torch.float16)
    out["wq_x"], out["wq_w_nk"] = x.numpy(), w.numpy()
    out["wq_scale"], out["wq_offset"] = a_s.numpy(), a_o.numpy()
    out["wq_out"] = ns2["cpu_linear_weight_quant"](None, w.to(torch.float16).t(), x, a_s, a_o)

    ns3 = {"torch": torch}
    f_mm = os.path.join(ref, "test/distributed/tensor/test_matrix_ops.py")
    exec(_cut(f_mm, "_get_global_tensor", "TestAllGatherBaseMmOp"), ns3)
    m, k, n = 6, 64, 24
    x1 = torch.randint(-127, 128, (m, k), generator=g).to(torch.float32)
    x2 = torch.randint(-127, 128, (k, n), generator=g).to(torch.float32)
    b = torch.randint(-50, 50, (n,), generator=g).to(torch.float32)
    s1 = torch.rand((m, 1), generator=g) * 1e-2
    s2 = torch.rand((1, n), generator=g) * 1e-2
    _, _, deq, _ = ns3["_get_global_tensor"](None, [x1], [x2], [b], [s1], [s2])
    out["mm_x1"], out["mm_x2"] = x1.to(torch.int8).numpy(), x2.to(torch.int8).numpy()
    out["mm_bias"] = b.to(torch.int32).numpy()
    out["mm_s1"], out["mm_s2"], out["mm_out"] = s1.numpy(), s2.numpy(), deq.numpy()

    # quantised reduce-scatter golden: three ranks, each with its own K slice and scales (own generator, so
    # that the draws above keep their values)
    ns4 = {"torch": torch}
    exec(_cut(f_mm, "_get_global_tensor", "TestMmReduceScatterBaseOp"), ns4)
    g4 = torch.Generator().manual_seed(79)
    ranks, m, k, n = 3, 6, 48, 32
    x1l = [torch.randint(-127, 128, (m, k), generator=g4).to(torch.int8) for _ in range(ranks)]
    x2l = [torch.randint(-127, 128, (k, n), generator=g4).to(torch.int8) for _ in range(ranks)]
    s1l = [torch.rand((m, 1), generator=g4) * 1e-2 for _ in range(ranks)]
    s2l = [torch.rand((1, n), generator=g4) * 1e-2 for _ in range(ranks)]
    _, _, rs = ns4["_get_global_tensor"](None, x1l, x2l, None, s1l, s2l)
    out["rs_x1"] = torch.stack(x1l).numpy()
    out["rs_x2"] = torch.stack(x2l).numpy()
    out["rs_s1"] = torch.stack(s1l).numpy()
    out["rs_s2"] = torch.stack(s2l).numpy()
    out["rs_out"] = rs.numpy()
    np.savez_compressed(os.path.join(HERE, "reference_goldens.npz"), **out)


def oracle_kat():
    out = {}
    c1 = workloads.config1()
    q, s = oracle.dynamic_quant(c1["x"])
    y = oracle.quant_matmul(q, c1["x2"], c1["scale"], pertoken_scale=s, output_dtype=torch.bfloat16)
    acc = oracle.quant_matmul(q, c1["x2"], c1["scale"], output_dtype=torch.int32)
    out.update(c1_x=bits(c1["x"]), c1_x2=c1["x2"].numpy(), c1_scale=c1["scale"].numpy(),
               c1_q=q.numpy(), c1_pertoken=s.numpy(), c1_acc=acc.numpy(), c1_out=bits(y))

    d = workloads.w8a8_linear(5, 136, 24, 11)
    q, s = oracle.dynamic_quant(d["x"], d["smooth_scales"])
    out.update(dq_x=bits(d["x"]), dq_smooth=d["smooth_scales"].numpy(), dq_q=q.numpy(), dq_scale=s.numpy())

    b = workloads.batched_w8a8(2, 3, 48, 16, 12)
    y = oracle.quant_matmul(b["x1"], b["x2"], b["scale"], offset=b["offset"],
                            pertoken_scale=b["pertoken_scale"], bias=b["bias"], output_dtype=torch.float16)
    y8 = oracle.quant_matmul(b["x1"], b["x2"], b["scale"], offset=b["offset"], bias=b["bias"])
    out.update({f"b_{k}": v.numpy() for k, v in b.items()})
    out.update(b_out_f16=y.numpy(), b_out_i8=y8.numpy())

    w = workloads.w4a16(3, 256, 32, 128, 13)
    packed = oracle.convert_weight_to_int4pack(w["w_int4"])
    y = oracle.weight_quant_batchmatmul(w["x"], packed, w["antiquant_scale"], w["antiquant_offset"],
                                        antiquant_group_size=128)
    out.update(w4_x=bits(w["x"]), w4_w=w["w_int4"].numpy(), w4_packed=packed.numpy(),
               w4_scale=bits(w["antiquant_scale"]), w4_offset=bits(w["antiquant_offset"]), w4_out=bits(y))
    np.savez_compressed(os.path.join(HERE, "oracle_kat.npz"), **out)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="reference tree; omit to rebuild only oracle_kat.npz")
    a = ap.parse_args()
    if a.reference:
        reference_goldens(a.reference)
    oracle_kat()
    print("fixtures written to", HERE)

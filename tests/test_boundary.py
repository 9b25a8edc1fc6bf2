"""Host-side checks that need no GPU: the C ABI exports every symbol the header declares, the
operators are registered under the reference's names with its keyword names, FakeTensor/meta
shape contracts (mirroring test/test_fake_tensor.py:1670-1686,1883-1943 of the reference), the
modules' constructor signatures and dtype gates, and the absence of any CPU fallback."""
import ctypes
import inspect
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def pkg():
    import pytorch_b200
    return pytorch_b200


def test_cabi_exports_every_declared_symbol():
    from pytorch_b200 import _cabi
    header = open(os.path.join(ROOT, "include", "b200q.h")).read()
    declared = set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in the header"
    lib = ctypes.CDLL(os.path.join(ROOT, "pytorch_b200", "lib", "libb200q.so"))
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in b200q.h but not exported"
    assert declared == set(_cabi.EXPORTS)
    assert _cabi.lib().b200q_version() >= 100
    assert _cabi.lib().b200q_status_string(2) == b"unsupported"


def test_struct_layout_matches_header():
    from pytorch_b200 import _cabi
    assert ctypes.sizeof(_cabi.QuantMatmulArgs) == 23 * 8
    assert ctypes.sizeof(_cabi.WeightQuantMatmulArgs) == 16 * 8


def test_ops_are_registered_under_reference_names(pkg):
    for name in pkg.OPS:
        assert getattr(pkg, name) is getattr(torch.ops.npu, name)
    s = str(torch.ops.npu.npu_quant_matmul.default._schema)
    for kw in ("offset", "pertoken_scale", "bias", "output_dtype"):
        assert kw in s
    s = str(torch.ops.npu.npu_weight_quant_batchmatmul.default._schema)
    for kw in ("antiquant_scale", "antiquant_offset", "quant_scale", "quant_offset", "bias",
               "antiquant_group_size", "inner_precise", "weight_dtype"):
        assert kw in s
    s = str(torch.ops.npu.npu_dynamic_quant.default._schema)
    for kw in ("smooth_scales", "group_index", "dst_type"):
        assert kw in s


def test_no_cpu_fallback(pkg):
    with pytest.raises(NotImplementedError):
        pkg.npu_dynamic_quant(torch.zeros(2, 8, dtype=torch.bfloat16))
    with pytest.raises(NotImplementedError):
        pkg.npu_quant_matmul(torch.zeros(2, 16, dtype=torch.int8), torch.zeros(16, 8, dtype=torch.int8), torch.ones(1))
    from pytorch_b200 import _cabi
    with pytest.raises(_cabi.B200QError):
        _cabi.dynamic_quant(torch.zeros(2, 8, dtype=torch.bfloat16))


def meta(*shape, dtype):
    return torch.empty(*shape, dtype=dtype, device="meta")


def test_dynamic_quant_meta_contract(pkg):
    x = meta(4, 2048, 1024, dtype=torch.float16)
    y, s = pkg.npu_dynamic_quant(x, smooth_scales=meta(1024, dtype=torch.float16))
    assert y.dtype == torch.int8 and y.shape == (4, 2048, 1024) and y.device == x.device
    assert s.dtype == torch.float32 and s.shape == (4, 2048)
    y, s = pkg.npu_dynamic_quant(x, smooth_scales=None, dst_type=torch.int8)
    assert y.shape == x.shape
    with pytest.raises(RuntimeError, match="group_index"):
        pkg.npu_dynamic_quant(x, group_index=meta(4, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="dst_type"):
        pkg.npu_dynamic_quant(x, dst_type=torch.int32)
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        pkg.npu_dynamic_quant(meta(2, 8, dtype=torch.float32))
    with pytest.raises(RuntimeError, match="smooth_scales"):
        pkg.npu_dynamic_quant(x, smooth_scales=meta(512, dtype=torch.float16))


def test_quant_matmul_meta_contract(pkg):
    x1 = meta(1, 1, 1024, dtype=torch.int8)
    x2 = meta(1, 1024, 100, dtype=torch.int8)
    scale, offset = meta(1, dtype=torch.float32), meta(1, dtype=torch.float32)
    r = pkg.npu_quant_matmul(x1, x2, scale, offset=offset, bias=meta(1, 1, 100, dtype=torch.int32))
    assert r.shape == (1, 1, 100) and r.dtype == torch.int8
    r = pkg.npu_quant_matmul(x1, x2, meta(1, dtype=torch.bfloat16), offset=None,
                             bias=meta(1, 1, 100, dtype=torch.bfloat16), output_dtype=torch.bfloat16)
    assert r.shape == (1, 1, 100) and r.dtype == torch.bfloat16
    r = pkg.npu_quant_matmul(x1, x2, scale, offset=None, pertoken_scale=meta(1, dtype=torch.float32),
                             bias=meta(1, 1, 100, dtype=torch.float32), output_dtype=torch.float16)
    assert r.shape == (1, 1, 100) and r.dtype == torch.float16
    r = pkg.npu_quant_matmul(x1, x2, scale, offset=None, pertoken_scale=None,
                             bias=meta(1, 1, 100, dtype=torch.int32), output_dtype=torch.int32)
    assert r.shape == (1, 1, 100) and r.dtype == torch.int32
    # int4-packed int32 operands: shape inference only
    r = pkg.npu_quant_matmul(meta(16, 8, dtype=torch.int32), meta(64, 5, dtype=torch.int32), scale, offset=None,
                             bias=meta(40, dtype=torch.int32), output_dtype=torch.float16)
    assert r.shape == (16, 40) and r.dtype == torch.float16
    # batch dimensions of x1 fold into m
    r = pkg.npu_quant_matmul(meta(8, 512, 5120, dtype=torch.int8), meta(5120, 13824, dtype=torch.int8),
                             meta(13824, dtype=torch.float32), pertoken_scale=meta(4096, dtype=torch.float32),
                             output_dtype=torch.float16)
    assert r.shape == (8, 512, 13824)
    with pytest.raises(RuntimeError, match="scale should be"):
        pkg.npu_quant_matmul(x1, x2, meta(1, dtype=torch.float16))
    with pytest.raises(RuntimeError, match="inner dimensions"):
        pkg.npu_quant_matmul(meta(4, 32, dtype=torch.int8), meta(64, 8, dtype=torch.int8), scale)
    with pytest.raises(RuntimeError, match="output_dtype"):
        pkg.npu_quant_matmul(x1, x2, scale, output_dtype=torch.float32)


def test_weight_quant_and_pack_meta_contract(pkg):
    x = meta(32, 8192, dtype=torch.bfloat16)
    w = meta(8192, 28672 // 8, dtype=torch.int32)
    sc = meta(64, 28672, dtype=torch.bfloat16)
    r = pkg.npu_weight_quant_batchmatmul(x, w, sc, sc, None, None, None, 128)
    assert r.shape == (32, 28672) and r.dtype == torch.bfloat16
    r = pkg.npu_weight_quant_batchmatmul(meta(16, 32, dtype=torch.float16), meta(32, 128, dtype=torch.int8),
                                         meta(128, dtype=torch.float16))
    assert r.shape == (16, 128) and r.dtype == torch.float16
    with pytest.raises(RuntimeError, match="quant_scale"):
        pkg.npu_weight_quant_batchmatmul(x, w, sc, sc, meta(28672, dtype=torch.float32), None, None, 128)
    with pytest.raises(RuntimeError, match="weight_dtype"):
        pkg.npu_weight_quant_batchmatmul(x, w, sc, sc, None, None, None, 128, 0, weight_dtype=torch.int8)
    p = pkg.npu_convert_weight_to_int4pack(meta(8192, 28672, dtype=torch.int32))
    assert p.shape == (8192, 3584) and p.dtype == torch.int32
    with pytest.raises(RuntimeError, match="multiple of 8"):
        pkg.npu_convert_weight_to_int4pack(meta(4, 12, dtype=torch.int32))


def test_sibling_ops_meta_contract(pkg):
    # npu_dynamic_quant_asymmetric: test/test_fake_tensor.py:1690-1709
    x = meta(4, 2048, 1024, dtype=torch.float16)
    y, s, o = pkg.npu_dynamic_quant_asymmetric(x, smooth_scales=meta(1024, dtype=torch.float16))
    assert y.shape == (4, 2048, 1024) and y.dtype == torch.int8
    assert s.shape == (4, 2048) and s.dtype == torch.float32 and o.shape == (4, 2048) and o.dtype == torch.float32
    # group_index: one smooth row per group (test/onnx/test_wrapper_onnx_ops.py:1335-1392)
    y, s = pkg.npu_dynamic_quant(x, smooth_scales=meta(10, 1024, dtype=torch.float16),
                                 group_index=meta(10, dtype=torch.int32))
    assert y.shape == (4, 2048, 1024) and s.shape == (4, 2048)
    with pytest.raises(RuntimeError, match="group_index"):
        pkg.npu_dynamic_quant(x, smooth_scales=meta(1024, dtype=torch.float16), group_index=meta(10, dtype=torch.int32))
    # npu_anti_quant: test/test_fake_tensor.py:1949-1959
    q = meta(20, 100, dtype=torch.int8)
    r = pkg.npu_anti_quant(q, meta(100, dtype=torch.float32), offset=meta(100, dtype=torch.float32),
                           dst_dtype=torch.float16)
    assert r.shape == q.shape and r.dtype == torch.float16
    r = pkg.npu_anti_quant(meta(10, 25, dtype=torch.int32), meta(200, dtype=torch.float32), dst_dtype=torch.bfloat16)
    assert r.shape == (10, 200) and r.dtype == torch.bfloat16
    with pytest.raises(RuntimeError, match="dst_dtype"):
        pkg.npu_anti_quant(q, meta(100, dtype=torch.float32), dst_dtype=torch.float32)
    # npu_swiglu_quant (dynamic mode): the last dimension halves
    y, s = pkg.npu_swiglu_quant(meta(4, 128, 57344, dtype=torch.bfloat16), smooth_scales=meta(28672, dtype=torch.float32),
                                activate_left=True, quant_mode=1)
    assert y.shape == (4, 128, 28672) and y.dtype == torch.int8 and s.shape == (4, 128) and s.dtype == torch.float32
    with pytest.raises(RuntimeError, match="quant_mode"):
        pkg.npu_swiglu_quant(meta(4, 64, dtype=torch.bfloat16))


def test_trans_quant_param_meta_contract(pkg):
    r = pkg.npu_trans_quant_param(meta(1, dtype=torch.float32), meta(4, dtype=torch.float32))
    assert r.shape == (4,) and r.dtype == torch.int64
    r = pkg.npu_trans_quant_param(meta(1, 4, dtype=torch.float32), meta(1, 4, dtype=torch.float32))
    assert r.shape == (1, 4) and r.dtype == torch.int64


def test_fake_tensor_mode(pkg):
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(4, 64, dtype=torch.bfloat16, device="cuda")
        y, s = pkg.npu_dynamic_quant(x)
        out = pkg.npu_quant_matmul(y, torch.empty(64, 32, dtype=torch.int8, device="cuda"),
                                   torch.empty(32, device="cuda"), pertoken_scale=s, output_dtype=torch.bfloat16)
        assert out.shape == (4, 32) and out.dtype == torch.bfloat16 and out.device.type == "cuda"


def test_module_signatures_and_dtype_gates(pkg):
    from pytorch_b200.contrib.module import LinearA8W8Quant, LinearQuant, LinearWeightQuant
    sig = inspect.signature(LinearQuant.__init__)
    assert list(sig.parameters)[1:] == ["in_features", "out_features", "bias", "offset", "pertoken_scale", "device",
                                        "dtype", "output_dtype"]
    assert sig.parameters["bias"].kind is inspect.Parameter.KEYWORD_ONLY
    sig = inspect.signature(LinearWeightQuant.__init__)
    assert list(sig.parameters)[1:] == ["in_features", "out_features", "bias", "device", "dtype", "antiquant_offset",
                                        "quant_scale", "quant_offset", "antiquant_group_size", "inner_precise",
                                        "weight_dtype"]
    m = LinearQuant(64, 32, bias=True, offset=True, pertoken_scale=True, device="meta", output_dtype=torch.bfloat16)
    assert m.weight.shape == (32, 64) and m.bias.dtype == torch.int32 and m.offset.dtype == torch.float32
    assert not any(p.requires_grad for p in m.parameters())
    with pytest.raises(ValueError, match="both torch.int32 or both torch.int8"):
        m(torch.empty(4, 64, dtype=torch.int8, device="meta"))          # weight is still float
    m.weight.data = torch.empty(32, 64, dtype=torch.int8, device="meta")
    m.pertoken_scale.data = torch.empty(4, dtype=torch.float32, device="meta")
    assert m(torch.empty(4, 64, dtype=torch.int8, device="meta")).shape == (4, 32)
    # without pertoken_scale and with a non-bf16 output the fp32 scale goes through npu_trans_quant_param
    m2 = LinearQuant(64, 32, bias=False, device="meta")
    m2.weight.data = torch.empty(32, 64, dtype=torch.int8, device="meta")
    out = m2(torch.empty(2, 3, 64, dtype=torch.int8, device="meta"))
    assert out.shape == (2, 3, 32) and out.dtype == torch.int8
    with pytest.warns(FutureWarning):
        a = LinearA8W8Quant(64, 32, bias=False, device="meta", output_dtype=torch.int32)
    a.weight.data = torch.empty(32, 64, dtype=torch.int8, device="meta")
    with pytest.raises(ValueError, match="output_dtype should be"):       # int32 output is refused by this module
        a(torch.empty(4, 64, dtype=torch.int8, device="meta"))
    with pytest.warns(FutureWarning):
        a = LinearA8W8Quant(64, 32, bias=False, device="meta")
    a.weight.data = torch.empty(32, 64, dtype=torch.int8, device="meta")
    a.scale.data = torch.empty(32, dtype=torch.float16, device="meta")
    with pytest.raises(ValueError, match="scale should be"):               # fp16 scale is refused
        a(torch.empty(4, 64, dtype=torch.int8, device="meta"))
    w = LinearWeightQuant(64, 32, bias=False, device="meta", antiquant_offset=True, antiquant_group_size=32)
    w.weight.data = torch.empty(32, 64, dtype=torch.int8, device="meta")
    w.antiquant_scale.data = torch.empty(32, 2, dtype=torch.float16, device="meta")
    w.antiquant_offset.data = torch.empty(32, 2, dtype=torch.float16, device="meta")
    assert w(torch.empty(5, 64, dtype=torch.float16, device="meta")).shape == (5, 32)


def test_collective_fused_operators_meta_contracts(pkg):
    """Shape/dtype contracts of the collective-fused operators (reference: test/test_fake_tensor.py:1555-1583 for
    npu_mm_all_reduce_base; schemas torch_npu/distributed/tensor/_matrix_ops.py:471-476,556-561)."""
    x1 = torch.empty(128, 256, dtype=torch.int8, device="meta")
    x2 = torch.empty(256, 128, dtype=torch.int8, device="meta")
    out = pkg.npu_mm_all_reduce_base(x1, x2, "fake group info", reduce_op="sum",
                                     dequant_scale=torch.empty(128, dtype=torch.int64, device="meta"))
    assert out.shape == (128, 128) and out.dtype == torch.float16
    out = pkg.npu_mm_all_reduce_base(x1, x2, "fake group info", reduce_op="sum",
                                     dequant_scale=torch.empty(128, dtype=torch.bfloat16, device="meta"))
    assert out.shape == (128, 128) and out.dtype == torch.bfloat16
    out = pkg.npu_mm_reduce_scatter_base(x1, x2, "g", 4, x1_scale=torch.empty(128, 1, device="meta"),
                                         x2_scale=torch.empty(1, 128, device="meta"), output_dtype=torch.bfloat16)
    assert out.shape == (32, 128) and out.dtype == torch.bfloat16
    out, gathered = pkg.npu_all_gather_base_mm(x1, x2, "g", 4)
    assert out.shape == (512, 128) and gathered.shape == (512, 256) and gathered.dtype == torch.int8
    s = str(torch.ops.npu.npu_mm_reduce_scatter_base.default._schema)
    for kw in ("hcom", "world_size", "reduce_op", "bias", "x1_scale", "x2_scale", "comm_turn", "output_dtype", "comm_mode"):
        assert kw in s
    s = str(torch.ops.npu.npu_all_gather_base_mm.default._schema)
    for kw in ("gather_index", "gather_output", "x1_scale", "x2_scale"):
        assert kw in s


def test_collective_fused_operators_have_no_cpu_path(pkg):
    with pytest.raises(NotImplementedError):
        pkg.npu_mm_reduce_scatter_base(torch.zeros(4, 16, dtype=torch.int8), torch.zeros(16, 8, dtype=torch.int8), "g", 2)

"""Argument validation of the C ABI: every entry point refuses bad arguments with a status code and a
message before it touches the device, so these checks run without a GPU (no kernel is launched: sizes
are zero or the call fails first)."""
import ctypes as C

import pytest

from pytorch_b200 import _cabi as cabi


@pytest.fixture(scope="module")
def lib():
    return cabi.lib()


def last(lib):
    return lib.b200q_last_error().decode()


def test_dynamic_quant_argument_checks(lib):
    assert lib.b200q_dynamic_quant(None, cabi.F32, None, cabi.NONE, None, None, 4, 8, None) == cabi.ERR_UNSUPPORTED
    assert "bf16 or f16" in last(lib)
    assert lib.b200q_dynamic_quant(None, cabi.BF16, None, cabi.NONE, None, None, -1, 8, None) == cabi.ERR_BAD_ARG
    assert lib.b200q_dynamic_quant(None, cabi.BF16, None, cabi.NONE, None, None, 0, 8, None) == cabi.OK   # no rows
    assert lib.b200q_dynamic_quant(None, cabi.BF16, None, cabi.NONE, None, None, 4, 8, None) == cabi.ERR_BAD_ARG
    assert "NULL" in last(lib)
    # extended entry: group_index needs smooth scales
    gi = (C.c_int32 * 2)(1, 2)
    rc = lib.b200q_dynamic_quant_ext(None, cabi.BF16, None, cabi.NONE, gi, 2, None, None, None, 4, 8, None)
    assert rc == cabi.ERR_BAD_ARG and "group_index" in last(lib)


def test_anti_quant_argument_checks(lib):
    assert lib.b200q_anti_quant(None, 5, None, None, cabi.F32, None, cabi.F16, 2, 16, None) == cabi.ERR_UNSUPPORTED
    assert "src_bits" in last(lib)
    assert lib.b200q_anti_quant(None, 4, None, None, cabi.F32, None, cabi.F16, 2, 12, None) == cabi.ERR_BAD_ARG
    assert "multiple of 8" in last(lib)
    assert lib.b200q_anti_quant(None, 8, None, None, cabi.F16, None, cabi.F16, 2, 16, None) == cabi.ERR_UNSUPPORTED
    assert lib.b200q_anti_quant(None, 8, None, None, cabi.F32, None, cabi.F32, 2, 16, None) == cabi.ERR_UNSUPPORTED
    assert "dst_dtype" in last(lib)
    assert lib.b200q_anti_quant(None, 8, None, None, cabi.F32, None, cabi.F16, 0, 16, None) == cabi.OK     # empty
    assert lib.b200q_anti_quant(None, 8, None, None, cabi.F32, None, cabi.F16, 2, 16, None) == cabi.ERR_BAD_ARG


def test_swiglu_quant_argument_checks(lib):
    assert lib.b200q_swiglu_quant(None, cabi.F32, None, cabi.NONE, 1, None, None, 2, 16, None) == cabi.ERR_UNSUPPORTED
    assert lib.b200q_swiglu_quant(None, cabi.BF16, None, cabi.NONE, 1, None, None, 0, 16, None) == cabi.OK
    one = (C.c_float * 4)()
    assert lib.b200q_swiglu_quant(None, cabi.BF16, None, cabi.NONE, 1, None, one, 2, 16, None) == cabi.ERR_BAD_ARG
    x = (C.c_uint8 * 256)()
    y = (C.c_int8 * 64)()
    rc = lib.b200q_swiglu_quant(x, cabi.BF16, None, cabi.NONE, 1, y, one, 2, 20, None)
    assert rc == cabi.ERR_UNSUPPORTED and "multiple of 8" in last(lib)


def test_matmul_argument_checks(lib):
    assert lib.b200q_quant_matmul(None, None) == cabi.ERR_BAD_ARG and "NULL" in last(lib)
    assert lib.b200q_weight_quant_matmul(None, None) == cabi.ERR_BAD_ARG
    a = cabi.WeightQuantMatmulArgs()
    a.m, a.k, a.n, a.x_dtype, a.weight_bits = 4, 64, 64, cabi.F32, 4
    assert lib.b200q_weight_quant_matmul(C.byref(a), None) == cabi.ERR_UNSUPPORTED and "bf16 or f16" in last(lib)
    a.x_dtype, a.weight_bits = cabi.BF16, 3
    assert lib.b200q_weight_quant_matmul(C.byref(a), None) == cabi.ERR_UNSUPPORTED and "weight_bits" in last(lib)
    a.weight_bits, a.n = 4, 60
    assert lib.b200q_weight_quant_matmul(C.byref(a), None) == cabi.ERR_BAD_ARG and "multiple of 8" in last(lib)
    assert lib.b200q_int4pack(None, None, 2, 12, None) == cabi.ERR_BAD_ARG and "multiple of 8" in last(lib)
    assert lib.b200q_int4pack(None, None, 0, 16, None) == cabi.OK
    assert lib.b200q_trans_quant_param(None, 0, None, 4, None) == cabi.ERR_BAD_ARG
    assert lib.b200q_trans_quant_param(None, 3, None, 4, None) == cabi.ERR_BAD_ARG and "elements" in last(lib)
    # a successful call clears the message
    assert lib.b200q_int4pack(None, None, 0, 16, None) == cabi.OK and last(lib) == ""

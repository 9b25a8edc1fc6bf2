"""CPU checks of the oracle for the operators next to the hot path: npu_anti_quant against the
reference's own golden function (fixtures from tests/golden/make_golden.py), the asymmetric dynamic
quantisation and group_index against their defining properties."""
import os

import numpy as np
import pytest
import torch

from oracle import quant_oracle as oracle


@pytest.fixture(scope="module")
def ref(golden_dir):
    return np.load(os.path.join(golden_dir, "reference_goldens.npz"))


def bf16_bits(t):
    return t.view(torch.int16).numpy().view(np.uint16)


def test_anti_quant_int8_matches_reference_golden(ref):
    x = torch.from_numpy(ref["anti8_x"])
    sc, of = torch.from_numpy(ref["anti8_scale"]), torch.from_numpy(ref["anti8_offset"])
    assert np.array_equal(oracle.anti_quant(x, sc, of, torch.float16).numpy(), ref["anti8_out_f16"])
    assert np.array_equal(bf16_bits(oracle.anti_quant(x, sc, of, torch.bfloat16)), ref["anti8_out_bf16"])
    assert np.array_equal(oracle.anti_quant(x, sc, None, torch.float16).numpy(), ref["anti8_out_nooff_f16"])


def test_anti_quant_int4_matches_reference_golden(ref):
    x = torch.from_numpy(ref["unpack_in"])
    sc, of = torch.from_numpy(ref["anti_scale"]), torch.from_numpy(ref["anti_offset"])
    assert np.array_equal(oracle.anti_quant(x, sc, of, torch.float16).numpy(), ref["anti_out_f16"])
    assert np.array_equal(bf16_bits(oracle.anti_quant(x, sc, of, torch.bfloat16)), ref["anti_out_bf16"])


def test_asymmetric_quant_properties():
    g = torch.Generator().manual_seed(5)
    x = (torch.randn((7, 256), generator=g) * 3 + 1.5).to(torch.float16)
    sm = (torch.rand(256, generator=g) + 0.5).to(torch.float16)
    y, s, o = oracle.dynamic_quant_asymmetric(x, sm)
    assert y.dtype == torch.int8 and y.shape == x.shape and s.shape == (7,) and o.shape == (7,)
    xs = x.float() * sm.float()
    # the row maximum maps to 127 and the minimum to -128; the whole int8 range is used
    assert torch.equal(y.max(-1).values, torch.full((7,), 127, dtype=torch.int8))
    assert torch.equal(y.min(-1).values, torch.full((7,), -128, dtype=torch.int8))
    # dequantisation error is at most half a step
    back = (y.float() - o[:, None]) * s[:, None]
    assert float((back - xs).abs().max()) <= float(s.max()) * 0.5 * 1.001
    # a constant row: scale 0, offset 0, y 0
    y0, s0, o0 = oracle.dynamic_quant_asymmetric(torch.full((2, 16), 3.0, dtype=torch.bfloat16))
    assert int(y0.abs().max()) == 0 and float(s0.abs().max()) == 0 and float(o0.abs().max()) == 0


def test_group_index_selects_the_smooth_row():
    g = torch.Generator().manual_seed(6)
    x = torch.randn((12, 64), generator=g).to(torch.bfloat16)
    sm = (torch.rand((3, 64), generator=g) + 0.5).to(torch.bfloat16)
    gi = torch.tensor([4, 4, 12], dtype=torch.int32)        # group 1 is empty
    y, s = oracle.dynamic_quant(x, sm, gi)
    ya, sa = oracle.dynamic_quant(x[:4], sm[0])
    yb, sb = oracle.dynamic_quant(x[4:], sm[2])
    assert torch.equal(y, torch.cat([ya, yb])) and torch.equal(s, torch.cat([sa, sb]))
    # rows past the last entry use the last row
    y2, _ = oracle.dynamic_quant(x, sm, torch.tensor([4, 6, 8], dtype=torch.int32))
    yc, _ = oracle.dynamic_quant(x[6:], sm[2])
    assert torch.equal(y2[6:], yc)
    y3, s3, o3 = oracle.dynamic_quant_asymmetric(x, sm, gi)
    y3b, s3b, o3b = oracle.dynamic_quant_asymmetric(x[4:], sm[2])
    assert torch.equal(y3[4:], y3b) and torch.equal(s3[4:], s3b) and torch.equal(o3[4:], o3b)


def test_swiglu_quant_oracle_properties():
    g = torch.Generator().manual_seed(8)
    x = torch.randn((5, 128), generator=g).to(torch.bfloat16)
    sm = (torch.rand(64, generator=g) + 0.5).to(torch.bfloat16)
    y, s = oracle.swiglu_quant(x, sm, activate_left=True)
    act = torch.nn.functional.silu(x[:, :64].float()) * x[:, 64:].float() * sm.float()
    assert y.shape == (5, 64) and s.shape == (5,)
    assert torch.allclose(s, act.abs().max(-1).values / 127, rtol=1e-5)
    assert int((y.float() - torch.round(act / s[:, None])).abs().max()) <= 1
    # the other half activated: same as swapping the halves
    y2, s2 = oracle.swiglu_quant(torch.cat([x[:, 64:], x[:, :64]], -1), sm, activate_left=False)
    assert torch.equal(y, y2) and torch.equal(s, s2)

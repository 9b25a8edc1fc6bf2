"""GPU parity of the operators next to the hot path (npu_anti_quant, npu_dynamic_quant_asymmetric,
group_index) against the CPU oracle and the reference's golden vectors: bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import quant_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pb():
    import pytorch_b200
    assert torch.cuda.is_available()
    return pytorch_b200


@pytest.fixture(scope="module")
def ref(golden_dir):
    return np.load(os.path.join(golden_dir, "reference_goldens.npz"))


@pytest.fixture(autouse=True)
def no_device_error():
    yield
    from pytorch_b200 import _cabi
    torch.cuda.synchronize()
    assert _cabi.device_error() == 0


def same_bits(a, b):
    return torch.equal(a.cpu().view(torch.int16), b.view(torch.int16))


def test_anti_quant_reference_golden(pb, ref):
    x8 = torch.from_numpy(ref["anti8_x"]).cuda()
    sc, of = torch.from_numpy(ref["anti8_scale"]).cuda(), torch.from_numpy(ref["anti8_offset"]).cuda()
    out = pb.npu_anti_quant(x8, sc, offset=of, dst_dtype=torch.float16, src_dtype=torch.int8)
    assert np.array_equal(out.cpu().numpy(), ref["anti8_out_f16"])
    out = pb.npu_anti_quant(x8, sc, offset=of, dst_dtype=torch.bfloat16)
    assert np.array_equal(out.cpu().view(torch.int16).numpy().view(np.uint16), ref["anti8_out_bf16"])
    out = pb.npu_anti_quant(x8, sc)                                   # defaults: no offset, fp16
    assert out.dtype == torch.float16 and np.array_equal(out.cpu().numpy(), ref["anti8_out_nooff_f16"])
    x4 = torch.from_numpy(ref["unpack_in"]).cuda()
    sc4, of4 = torch.from_numpy(ref["anti_scale"]).cuda(), torch.from_numpy(ref["anti_offset"]).cuda()
    out = pb.npu_anti_quant(x4, sc4, offset=of4, dst_dtype=torch.float16)
    assert out.shape == (6, 80) and np.array_equal(out.cpu().numpy(), ref["anti_out_f16"])


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("pdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("odtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(3, 5, 1024), (257, 4096), (9, 104)])
def test_anti_quant_matches_oracle(pb, bits, pdtype, odtype, shape):
    g = torch.Generator().manual_seed(hash((bits, shape)) % 1000)
    n = shape[-1]
    if bits == 8:
        x = torch.randint(-128, 128, shape, generator=g, dtype=torch.int64).to(torch.int8)
    else:
        x = torch.randint(-2 ** 31, 2 ** 31 - 1, (*shape[:-1], n // 8), generator=g, dtype=torch.int64).to(torch.int32)
    sc = (torch.rand(n, generator=g) * 4 - 2).to(pdtype)
    of = (torch.rand(n, generator=g) * 20 - 10).to(pdtype)
    for offset in (of, None):
        got = pb.npu_anti_quant(x.cuda(), sc.cuda(), offset=None if offset is None else offset.cuda(), dst_dtype=odtype)
        want = oracle.anti_quant(x, sc, offset, odtype)
        assert got.shape == want.shape and got.dtype == odtype
        assert same_bits(got, want)


def test_anti_quant_rejects_bad_arguments(pb):
    x = torch.zeros((2, 16), dtype=torch.int8, device="cuda")
    sc = torch.ones(16, device="cuda")
    with pytest.raises(RuntimeError, match="dst_dtype"):
        pb.npu_anti_quant(x, sc, dst_dtype=torch.float32)
    with pytest.raises(RuntimeError, match="scale must have"):
        pb.npu_anti_quant(x, torch.ones(8, device="cuda"))
    with pytest.raises(RuntimeError, match="same device"):
        pb.npu_anti_quant(x, sc, offset=torch.zeros(16))
    e = pb.npu_anti_quant(torch.zeros((0, 16), dtype=torch.int8, device="cuda"), sc)
    assert e.shape == (0, 16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,smooth", [((4, 33, 1024), "x"), ((64, 8192), "f32"), ((5, 200), None),
                                          ((3, 100), "x"), ((16, 11008), "x"), ((2, 40960), None)])
def test_dynamic_quant_asymmetric_matches_oracle(pb, dtype, shape, smooth):
    g = torch.Generator().manual_seed(shape[-1])
    x = (torch.randn(shape, generator=g) * 2 + 0.7).to(dtype)
    sm = None
    if smooth is not None:
        sm = (torch.rand(shape[-1], generator=g) * 1.5 + 0.5).to(dtype if smooth == "x" else torch.float32)
    y, s, o = pb.npu_dynamic_quant_asymmetric(x.cuda(), smooth_scales=None if sm is None else sm.cuda())
    yo, so, oo = oracle.dynamic_quant_asymmetric(x, sm)
    assert y.shape == x.shape and s.shape == x.shape[:-1] and o.shape == x.shape[:-1]
    assert torch.equal(s.cpu().view(torch.int32), so.view(torch.int32))
    assert torch.equal(o.cpu().view(torch.int32), oo.view(torch.int32))
    assert torch.equal(y.cpu(), yo)


def test_dynamic_quant_asymmetric_rows_far_from_zero(pb):
    """Rows whose values sit far from zero compared with their spread: the offset is huge, the sum with it rounds
    coarsely and the clamp to [-128, 127] matters.  Must still equal the oracle bit for bit."""
    g = torch.Generator().manual_seed(31)
    x = (1000.0 + torch.randn((6, 1024), generator=g) * 0.02).to(torch.float16)
    x[3] = (torch.randn(1024, generator=g) * 3).to(torch.float16)           # an ordinary row among them
    y, s, o = pb.npu_dynamic_quant_asymmetric(x.cuda())
    yo, so, oo = oracle.dynamic_quant_asymmetric(x)
    assert torch.equal(s.cpu().view(torch.int32), so.view(torch.int32)) and torch.equal(o.cpu().view(torch.int32), oo.view(torch.int32))
    assert torch.equal(y.cpu(), yo)


def test_dynamic_quant_asymmetric_constant_and_empty_rows(pb):
    x = torch.full((3, 64), -2.5, dtype=torch.bfloat16)
    x[1] = torch.linspace(-1, 1, 64).to(torch.bfloat16)
    y, s, o = pb.npu_dynamic_quant_asymmetric(x.cuda())
    yo, so, oo = oracle.dynamic_quant_asymmetric(x)
    assert torch.equal(y.cpu(), yo) and torch.equal(s.cpu(), so) and torch.equal(o.cpu(), oo)
    assert float(s[0]) == 0 and int(y[0].abs().max()) == 0
    y, s, o = pb.npu_dynamic_quant_asymmetric(torch.zeros((0, 64), dtype=torch.float16, device="cuda"))
    assert y.shape == (0, 64) and s.shape == (0,) and o.shape == (0,)


@pytest.mark.parametrize("k", [512, 4096, 100])
def test_group_index_matches_oracle(pb, k):
    # ten groups with sorted random boundaries, the last one the row count (the reference's ONNX test
    # builds its inputs this way: test/onnx/test_wrapper_onnx_ops.py:1344-1354)
    g = torch.Generator().manual_seed(k)
    x = (torch.rand((4, 64, k), generator=g) * 6 - 3).to(torch.float16)
    sm = (torch.rand((10, k), generator=g) * 6 - 3).to(torch.float16)
    rows = 4 * 64
    gi = torch.sort(torch.randint(0, rows, (10,), generator=g)).values.to(torch.int32)
    gi[-1] = rows
    y, s = pb.npu_dynamic_quant(x.cuda(), smooth_scales=sm.cuda(), group_index=gi.cuda())
    yo, so = oracle.dynamic_quant(x, sm, gi)
    assert torch.equal(y.cpu(), yo) and torch.equal(s.cpu().view(torch.int32), so.view(torch.int32))
    y, s, o = pb.npu_dynamic_quant_asymmetric(x.cuda(), smooth_scales=sm.cuda(), group_index=gi.cuda().long())
    yo, so, oo = oracle.dynamic_quant_asymmetric(x, sm, gi)
    assert torch.equal(y.cpu(), yo) and torch.equal(s.cpu(), so) and torch.equal(o.cpu(), oo)
    with pytest.raises(RuntimeError, match="group_index"):
        pb.npu_dynamic_quant(x.cuda(), group_index=gi.cuda())


def close_int8(got, want, scale_got, scale_want):
    """exp() differs in the last bits between the host and the device, so a value that lands on a rounding
    boundary may move by one step: scales to 1e-5 relative, values within 1, at most 1 % of them different."""
    assert torch.allclose(scale_got.cpu(), scale_want, rtol=1e-5, atol=1e-12)
    d = (got.cpu().to(torch.int16) - want.to(torch.int16)).abs()
    assert int(d.max()) <= 1 and float((d > 0).float().mean()) <= 0.01


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,smooth,left", [((3, 17, 512), "x", True), ((64, 16384), "f32", True),
                                               ((9, 57344), None, True), ((33, 2048 + 64), "x", False),
                                               ((4, 16), None, False), ((2, 65536), "f32", True)])
def test_swiglu_quant_matches_oracle(pb, dtype, shape, smooth, left):
    g = torch.Generator().manual_seed(shape[-1])
    x = (torch.randn(shape, generator=g) * 1.5).to(dtype)
    f = shape[-1] // 2
    sm = None
    if smooth is not None:
        sm = (torch.rand(f, generator=g) * 1.5 + 0.5).to(dtype if smooth == "x" else torch.float32)
    y, s = pb.npu_swiglu_quant(x.cuda(), smooth_scales=None if sm is None else sm.cuda(), activate_left=left,
                               quant_mode=1)
    yo, so = oracle.swiglu_quant(x, sm, activate_left=left)
    assert y.shape == (*shape[:-1], f) and y.dtype == torch.int8 and s.shape == shape[:-1]
    close_int8(y, yo, s, so)


def test_swiglu_quant_rejects_unsupported(pb):
    x = torch.zeros((2, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="quant_mode"):
        pb.npu_swiglu_quant(x)                                        # the default is the static mode
    with pytest.raises(RuntimeError, match="even"):
        pb.npu_swiglu_quant(torch.zeros((2, 63), dtype=torch.bfloat16, device="cuda"), quant_mode=1)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        pb.npu_swiglu_quant(torch.zeros((2, 20), dtype=torch.bfloat16, device="cuda"), quant_mode=1)
    y, s = pb.npu_swiglu_quant(torch.zeros((0, 64), dtype=torch.bfloat16, device="cuda"), quant_mode=1)
    assert y.shape == (0, 32) and s.shape == (0,)


def test_w8a8_swiglu_mlp_matches_oracle_chain(pb):
    from pytorch_b200.contrib.function import w8a8_swiglu_mlp
    g = torch.Generator().manual_seed(21)
    m, k, f, h = 48, 256, 384, 128
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    sm_in = (torch.rand(k, generator=g) + 0.5)
    sm_act = (torch.rand(f, generator=g) + 0.5)
    w_gu = torch.randint(-127, 128, (2 * f, k), generator=g).to(torch.int8)
    w_dn = torch.randint(-127, 128, (h, f), generator=g).to(torch.int8)
    s_gu = torch.rand(2 * f, generator=g) * 2e-3 + 1e-3
    s_dn = torch.rand(h, generator=g) * 2e-3 + 1e-3
    got = w8a8_swiglu_mlp(x.cuda(), sm_in.cuda(), w_gu.cuda(), s_gu.cuda(), sm_act.cuda(), w_dn.cuda(), s_dn.cuda())
    q, s = oracle.dynamic_quant(x, sm_in)
    gu = oracle.quant_matmul(q, w_gu.t(), s_gu, pertoken_scale=s, output_dtype=torch.bfloat16)
    qa, sa = oracle.swiglu_quant(gu, sm_act, activate_left=True)
    want = oracle.quant_matmul(qa, w_dn.t(), s_dn, pertoken_scale=sa, output_dtype=torch.bfloat16)
    assert got.shape == (m, h) and got.dtype == torch.bfloat16
    # int8 activations may differ by one step in a few places (see close_int8): bf16 output within 2^-6
    assert oracle.max_mixed_error(got.cpu(), want) <= 2.0 ** -6

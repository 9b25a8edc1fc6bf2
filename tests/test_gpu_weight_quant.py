"""Parity of npu_weight_quant_batchmatmul (W4A16 int4-packed and W8A16) with the CPU oracle,
through the C ABI.  Outputs are bf16/fp16: bound 2**-7 under the atol-OR-rtol rule."""
import os

import numpy as np
import pytest
import torch

from oracle import quant_oracle as oracle
from pytorch_b200 import workloads

pytestmark = pytest.mark.gpu
TOL = 2.0 ** -7


@pytest.fixture(scope="module")
def cabi():
    from pytorch_b200 import _cabi
    _cabi.lib()
    assert torch.cuda.is_available()
    return _cabi


@pytest.fixture(autouse=True)
def no_device_error(cabi):
    yield
    torch.cuda.synchronize()
    assert cabi.device_error() == 0


def dev(t):
    return None if t is None else t.cuda()


def check(cabi, x, w, scale, offset, gs, bias=None, w_dev=None):
    got = cabi.weight_quant_matmul(dev(x), dev(w) if w_dev is None else w_dev, dev(scale), dev(offset), bias=dev(bias),
                                   antiquant_group_size=gs).cpu()
    want = oracle.weight_quant_batchmatmul(x, w, scale, offset, bias=bias, antiquant_group_size=gs)
    assert got.dtype == x.dtype and got.shape == want.shape
    err = oracle.max_mixed_error(got, want)
    assert err <= TOL, err


def test_w4a16_golden_fixture(cabi, golden_dir):
    kat = np.load(os.path.join(golden_dir, "oracle_kat.npz"))
    bf = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    got = cabi.weight_quant_matmul(bf(kat["w4_x"]).cuda(), torch.from_numpy(kat["w4_packed"]).cuda(),
                                   bf(kat["w4_scale"]).cuda(), bf(kat["w4_offset"]).cuda(), antiquant_group_size=128)
    assert oracle.max_mixed_error(got.cpu(), bf(kat["w4_out"])) <= TOL


@pytest.mark.parametrize("m,k,n,gs", [(1, 512, 128, 128), (16, 1024, 256, 128), (32, 1024, 384, 128), (17, 512, 160, 64),
                                      (64, 2048, 128, 0), (100, 512, 256, 256), (256, 512, 256, 128),
                                      (300, 256, 128, 128), (5, 8192, 512, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_w4a16_int4_packed(cabi, m, k, n, gs, dtype):
    d = workloads.w4a16(m, k, n, gs, 300 + m + n, x_dtype=dtype)
    packed = cabi.int4pack(d["w_int4"].cuda())
    assert torch.equal(packed.cpu(), oracle.convert_weight_to_int4pack(d["w_int4"]))
    check(cabi, d["x"], packed.cpu(), d["antiquant_scale"], d["antiquant_offset"], gs, w_dev=packed)
    check(cabi, d["x"], packed.cpu(), d["antiquant_scale"], None, gs, w_dev=packed)


@pytest.mark.parametrize("m,k,n,gs", [(1, 512, 256, 0), (3, 1024, 288, 128), (8, 2048, 1024, 64), (9, 2048, 544, 128),
                                      (16, 4096, 2080, 256), (12, 8192, 1056, 128), (7, 96, 32, 0)])
@pytest.mark.parametrize("ksplit", ["", "1", "3", "8"])
def test_w4a16_few_tokens_streaming_kernel(cabi, monkeypatch, m, k, n, gs, ksplit):
    """Up to 16 tokens take the streaming warp-MMA kernel: ragged column strips (n not a multiple of 128),
    warps that start inside a scale group, every split of K over a cluster, bias, both dtypes' roundings."""
    if ksplit:
        monkeypatch.setenv("B200Q_WQ_KSPLIT", ksplit)
    d = workloads.w4a16(m, k, n, gs, 900 + m + n)
    packed = cabi.int4pack(d["w_int4"].cuda())
    g = torch.Generator().manual_seed(m)
    bias = workloads.rand_uniform((n,), g, -1, 1, torch.bfloat16)
    check(cabi, d["x"], packed.cpu(), d["antiquant_scale"], d["antiquant_offset"], gs, bias=bias, w_dev=packed)
    check(cabi, d["x"], packed.cpu(), d["antiquant_scale"], None, gs, w_dev=packed)
    # the tcgen05 kernel dequantises to the same 16-bit values; the fp32 sums are taken in another order, which
    # can move an output by one unit in the last place of its 16-bit format (at most 2**-7 relative)
    got = cabi.weight_quant_matmul(d["x"].cuda(), packed, d["antiquant_scale"].cuda(), d["antiquant_offset"].cuda(),
                                   antiquant_group_size=gs)
    monkeypatch.setenv("B200Q_WQ_STREAM", "0")
    other = cabi.weight_quant_matmul(d["x"].cuda(), packed, d["antiquant_scale"].cuda(), d["antiquant_offset"].cuda(),
                                     antiquant_group_size=gs)
    assert oracle.max_mixed_error(got.cpu(), other.cpu()) <= TOL


@pytest.mark.parametrize("m,k,n,gs", [(1, 512, 128, 0), (33, 1024, 272, 0), (128, 512, 256, 128), (260, 1024, 128, 64)])
@pytest.mark.parametrize("layout", ["nk_view", "kn"])
def test_w8a16_int8(cabi, m, k, n, gs, layout):
    g = torch.Generator().manual_seed(m + k)
    x = workloads.randn_bf16((m, k), g, torch.float16)
    w_nk = workloads.rand_int8((n, k), g, -128, 127)
    groups = k // gs if gs else 1
    scale = workloads.rand_uniform((groups, n), g, 5e-3, 2e-2, torch.float16)
    offset = workloads.rand_uniform((groups, n), g, -1, 1, torch.float16)
    bias = workloads.rand_uniform((n,), g, -1, 1, torch.float16)
    w = w_nk.t() if layout == "nk_view" else w_nk.t().contiguous()
    w_dev = w_nk.cuda().t() if layout == "nk_view" else w.cuda()
    check(cabi, x, w, scale, offset, gs, w_dev=w_dev)
    check(cabi, x, w, scale[0] if groups == 1 else scale, None, gs, bias=bias, w_dev=w_dev)


def test_reference_golden_shape_w8a16_per_channel_offset(cabi):
    """The one weight-only case the reference checks numerically (fp16, int8 weight stored [n,k], per-channel
    scale and offset, rtol 1e-2), at a reduced size."""
    m, k, n = 256, 2816, 416
    g = torch.Generator().manual_seed(1)
    x = torch.randn((m, k), generator=g).to(torch.float16)
    w_nk = torch.randn((n, k), generator=g).mul(30).to(torch.int8)
    scale = torch.randn(n, generator=g).to(torch.float16)
    offset = torch.randn(n, generator=g).to(torch.float16)
    got = cabi.weight_quant_matmul(x.cuda(), w_nk.cuda().t(), scale.cuda(), offset.cuda()).cpu()
    want = oracle.weight_quant_batchmatmul(x, w_nk.t(), scale, offset)
    assert oracle.max_mixed_error(got, want) <= TOL
    n_abs, n_rel = oracle.count_outside(got, want, 1e-2)
    assert min(n_abs, n_rel) <= got.numel() * 1e-2


def test_unaligned_shapes_take_the_generic_kernel(cabi):
    g = torch.Generator().manual_seed(2)
    x = workloads.randn_bf16((3, 100), g)
    w = workloads.rand_int8((100, 24), g)
    sc = workloads.rand_uniform((24,), g, 5e-3, 2e-2, torch.bfloat16)
    of = workloads.rand_uniform((24,), g, -1, 1, torch.bfloat16)
    check(cabi, x, w, sc, of, 0)
    d = workloads.w4a16(2, 64, 8, 32, 9)
    packed = oracle.convert_weight_to_int4pack(d["w_int4"])
    check(cabi, d["x"], packed, d["antiquant_scale"], d["antiquant_offset"], 32)


@pytest.mark.parametrize("mi", [0, 1, 2])
def test_config3_w4a16_full_size(cabi, mi):
    """x bf16 [M,8192], int4 weight packed to [8192,3584], group size 128.  The kernel runs at full size;
    the oracle checks a 2048-column slice (its fp64 matmul over all 28672 columns would take minutes)."""
    d = workloads.config3_case(mi)
    packed = cabi.int4pack(d["w_int4"].cuda())
    y = cabi.weight_quant_matmul(d["x"].cuda(), packed, d["antiquant_scale"].cuda(), d["antiquant_offset"].cuda(),
                                 antiquant_group_size=128).cpu()
    assert y.shape == (workloads.C3_M[mi], workloads.C3_N)
    for n0 in (0, 13312, 26624):
        sl = slice(n0, n0 + 2048)
        want = oracle.weight_quant_batchmatmul(
            d["x"], oracle.convert_weight_to_int4pack(d["w_int4"][:, sl]), d["antiquant_scale"][:, sl],
            d["antiquant_offset"][:, sl], antiquant_group_size=128)
        err = oracle.max_mixed_error(y[:, sl], want)
        assert err <= TOL, (n0, err)
    # linearity in x: doubling the activations doubles every output exactly (power of two)
    y2 = cabi.weight_quant_matmul((d["x"].float() * 2).to(torch.bfloat16).cuda(), packed, d["antiquant_scale"].cuda(),
                                  d["antiquant_offset"].cuda(), antiquant_group_size=128).cpu()
    assert torch.equal(y2.float(), y.float() * 2)

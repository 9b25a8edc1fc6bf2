"""The operators as a user of the reference calls them: torch.ops.npu.* / pytorch_b200.npu_* and the
quantised linear modules, compared with the CPU oracle and with each other (the reference's module tests
check module output against a direct operator call: test/contrib/test_linear_quant.py:23-63)."""
import pytest
import torch

from oracle import quant_oracle as oracle
from pytorch_b200 import workloads

pytestmark = pytest.mark.gpu
TOL = 2.0 ** -7


@pytest.fixture(scope="module")
def pb():
    import pytorch_b200
    assert torch.cuda.is_available()
    return pytorch_b200


@pytest.fixture(autouse=True)
def no_device_error():
    yield
    from pytorch_b200 import _cabi
    torch.cuda.synchronize()
    assert _cabi.device_error() == 0


def test_dynamic_quant_op_matches_oracle(pb):
    g = torch.Generator().manual_seed(1)
    x = workloads.randn_bf16((4, 96, 1024), g, torch.float16)
    sm = workloads.rand_uniform((1024,), g, 0.5, 2, torch.float16)
    y, s = pb.npu_dynamic_quant(x.cuda(), smooth_scales=sm.cuda())
    yo, so = oracle.dynamic_quant(x, sm)
    assert y.shape == (4, 96, 1024) and s.shape == (4, 96)
    assert torch.equal(y.cpu(), yo) and torch.equal(s.cpu().view(torch.int32), so.view(torch.int32))
    xt = x.cuda().transpose(0, 1)                    # non-contiguous input
    y2, s2 = pb.npu_dynamic_quant(xt)
    yo2, so2 = oracle.dynamic_quant(x.transpose(0, 1))
    assert torch.equal(y2.cpu(), yo2) and torch.equal(s2.cpu(), so2)


def test_quant_matmul_batched_x2_and_bias_shapes(pb):
    g = torch.Generator().manual_seed(2)
    x1 = workloads.rand_int8((3, 20, 64), g)
    x2 = workloads.rand_int8((3, 64, 48), g)
    scale = workloads.rand_uniform((48,), g, 1e-3, 1e-2)
    bias = torch.randint(-100, 100, (3, 1, 48), generator=g, dtype=torch.int32)
    got = pb.npu_quant_matmul(x1.cuda(), x2.cuda(), scale.cuda(), bias=bias.cuda(), output_dtype=torch.float16).cpu()
    want = oracle.quant_matmul(x1, x2, scale, bias=bias, output_dtype=torch.float16)
    assert got.shape == (3, 20, 48) and torch.equal(got, want)
    # the reference's meta-test shapes, with real data: [1,1,1024] x [1,1024,100]
    a = workloads.rand_int8((1, 1, 1024), g)
    b = workloads.rand_int8((1, 1024, 100), g)
    sc, of = torch.tensor([2e-4]), torch.tensor([1.5])
    bi = torch.randint(-50, 50, (1, 1, 100), generator=g, dtype=torch.int32)
    got = pb.npu_quant_matmul(a.cuda(), b.cuda(), sc.cuda(), offset=of.cuda(), bias=bi.cuda()).cpu()
    assert got.dtype == torch.int8 and torch.equal(got, oracle.quant_matmul(a, b, sc, offset=of, bias=bi))


def test_quant_matmul_single_batch_x2_serves_every_batch_of_x1(pb):
    """x1 [B>1, M, K] against x2 [1, K, N]: one weight for all batches, every row of the [B, M, N] output is
    written (pertoken_scale has B*M elements, bias [1,1,N])."""
    g = torch.Generator().manual_seed(12)
    x1 = workloads.rand_int8((3, 20, 64), g)
    x2 = workloads.rand_int8((1, 64, 48), g)
    scale = workloads.rand_uniform((48,), g, 1e-3, 1e-2)
    pt = workloads.rand_uniform((60,), g, 1e-3, 1e-2)
    bias = torch.randint(-100, 100, (1, 1, 48), generator=g, dtype=torch.int32)
    got = pb.npu_quant_matmul(x1.cuda(), x2.cuda(), scale.cuda(), pertoken_scale=pt.cuda(), bias=bias.cuda(),
                              output_dtype=torch.bfloat16).cpu()
    want = oracle.quant_matmul(x1.reshape(60, 64), x2[0], scale, pertoken_scale=pt, bias=bias.reshape(-1),
                               output_dtype=torch.bfloat16).reshape(3, 20, 48)
    assert got.shape == (3, 20, 48) and torch.equal(got.view(torch.int16), want.view(torch.int16))
    acc = pb.npu_quant_matmul(x1.cuda(), x2.cuda(), scale.cuda(), output_dtype=torch.int32).cpu()
    assert torch.equal(acc, oracle.quant_matmul(x1.reshape(60, 64), x2[0], scale, output_dtype=torch.int32).reshape(3, 20, 48))


def test_linear_quant_module_equals_op_and_oracle(pb):
    from pytorch_b200.contrib.module import LinearA8W8Quant, LinearQuant
    g = torch.Generator().manual_seed(3)
    k, n = 5120, 1280
    x = workloads.rand_int8((8, 64, k), g)
    w = workloads.rand_int8((n, k), g)
    scale = workloads.rand_uniform((n,), g, 1e-3, 1e-2)
    offset = workloads.rand_uniform((n,), g, -4, 4)
    bias = torch.randint(-1000, 1001, (n,), generator=g, dtype=torch.int32)
    pt = workloads.rand_uniform((8 * 64,), g, 1e-3, 1e-2)
    m = LinearQuant(k, n, bias=True, offset=True, pertoken_scale=True, output_dtype=torch.float16).cuda()
    m.weight.data, m.scale.data, m.offset.data = w.cuda(), scale.cuda(), offset.cuda()
    m.bias.data, m.pertoken_scale.data = bias.cuda(), pt.cuda()
    y = m(x.cuda())
    direct = pb.npu_quant_matmul(x.cuda(), w.cuda().t(), scale.cuda(), offset=offset.cuda(), pertoken_scale=pt.cuda(),
                                 bias=bias.cuda(), output_dtype=torch.float16)
    assert torch.equal(y, direct)
    want = oracle.quant_matmul(x, w.t(), scale, offset=offset, pertoken_scale=pt, bias=bias, output_dtype=torch.float16)
    assert oracle.max_mixed_error(y.cpu(), want) <= TOL
    # int8 output without pertoken_scale: the fp32 scale is packed by npu_trans_quant_param first
    small = workloads.rand_uniform((n,), g, 2e-5, 1e-4)
    m8 = LinearQuant(k, n, bias=False).cuda()
    m8.weight.data, m8.scale.data = w.cuda(), small.cuda()
    y8 = m8(x.cuda())
    assert y8.dtype == torch.int8 and torch.equal(y8.cpu(), oracle.quant_matmul(x, w.t(), small))
    # int32 output through LinearQuant; refused by the deprecated A8W8 module
    m32 = LinearQuant(k, n, bias=False, output_dtype=torch.int32).cuda()
    m32.weight.data, m32.scale.data = w.cuda(), scale.cuda()
    assert torch.equal(m32(x.cuda()).cpu(), oracle.quant_matmul(x, w.t(), scale, output_dtype=torch.int32))
    with pytest.warns(FutureWarning):
        a = LinearA8W8Quant(k, n, bias=False, output_dtype=torch.int32).cuda()
    a.weight.data = w.cuda()
    with pytest.raises(ValueError):
        a(x.cuda())
    with pytest.raises(RuntimeError, match="scale should be"):
        pb.npu_quant_matmul(x.cuda(), w.cuda().t(), scale.cuda().half())


def test_linear_weight_quant_module(pb):
    from pytorch_b200.contrib.module import LinearWeightQuant
    g = torch.Generator().manual_seed(4)
    m_, k, n = 64, 1024, 384
    x = torch.randn((m_, k), generator=g).to(torch.float16)
    w_nk = workloads.rand_int8((n, k), g, -128, 127)
    sc = workloads.rand_uniform((n,), g, 5e-3, 2e-2, torch.float16)
    of = workloads.rand_uniform((n,), g, -1, 1, torch.float16)
    mod = LinearWeightQuant(k, n, bias=False, antiquant_offset=True).cuda()
    mod.weight.data, mod.antiquant_scale.data, mod.antiquant_offset.data = w_nk.cuda(), sc.cuda(), of.cuda()
    y = mod(x.cuda())
    want = oracle.weight_quant_batchmatmul(x, w_nk.t(), sc, of)
    assert oracle.max_mixed_error(y.cpu(), want) <= TOL
    # per-group parameters are stored [n, groups] by the module and transposed for the call
    scg = workloads.rand_uniform((n, k // 128), g, 5e-3, 2e-2, torch.float16)
    ofg = workloads.rand_uniform((n, k // 128), g, -1, 1, torch.float16)
    mod = LinearWeightQuant(k, n, bias=False, antiquant_offset=True, antiquant_group_size=128).cuda()
    mod.weight.data, mod.antiquant_scale.data, mod.antiquant_offset.data = w_nk.cuda(), scg.cuda(), ofg.cuda()
    y = mod(x.cuda())
    want = oracle.weight_quant_batchmatmul(x, w_nk.t(), scg.t(), ofg.t(), antiquant_group_size=128)
    assert oracle.max_mixed_error(y.cpu(), want) <= TOL


def test_int4pack_and_w4a16_ops(pb):
    d = workloads.w4a16(32, 1024, 256, 128, 77)
    packed = pb.npu_convert_weight_to_int4pack(d["w_int4"].cuda())
    assert torch.equal(packed.cpu(), oracle.convert_weight_to_int4pack(d["w_int4"]))
    y = pb.npu_weight_quant_batchmatmul(d["x"].cuda(), packed, d["antiquant_scale"].cuda(), d["antiquant_offset"].cuda(),
                                        None, None, None, 128)
    want = oracle.weight_quant_batchmatmul(d["x"], packed.cpu(), d["antiquant_scale"], d["antiquant_offset"],
                                           antiquant_group_size=128)
    assert oracle.max_mixed_error(y.cpu(), want) <= TOL


def test_trans_quant_param_op(pb):
    s = torch.tensor([0.0123, 4.5, 1e-3, 2.0])
    p = pb.npu_trans_quant_param(s.cuda(), torch.zeros(4).cuda())
    assert torch.equal(p.cpu(), oracle.trans_quant_param(s))


def test_mixed_device_is_rejected(pb):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    x = torch.zeros(4, 64, dtype=torch.int8, device="cuda:0")
    w = torch.zeros(64, 32, dtype=torch.int8, device="cuda:0")
    with pytest.raises(RuntimeError, match="Expected all tensors to be on the same device"):
        pb.npu_quant_matmul(x, w, torch.ones(32, device="cuda:1"))

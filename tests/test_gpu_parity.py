"""Parity of the CUDA kernels with the CPU oracle, called through the C ABI (ctypes).

Integer outputs (int8 quantised values, int32 accumulators, packed int4 words) and the fp32
per-token scale must match bit for bit; bf16/fp16 outputs must be within 2**-7 under the
atol-OR-rtol rule (``oracle.max_mixed_error``).  Cases the oracle cannot finish in seconds
are checked through size-independent properties (a Freivalds product check on the int32
accumulators, sampled rows for the epilogue).
"""
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
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return _cabi


@pytest.fixture(autouse=True)
def no_device_error(cabi):
    yield
    torch.cuda.synchronize()
    assert cabi.device_error() == 0, "a kernel gave up a bounded wait"


def dev(t):
    return None if t is None else t.cuda()


# ------------------------------------------------------------------ dynamic quant
def check_dq(cabi, x, smooth):
    q, s = cabi.dynamic_quant(dev(x), dev(smooth))
    qo, so = oracle.dynamic_quant(x, smooth)
    assert q.dtype == torch.int8 and s.dtype == torch.float32
    assert q.shape == x.shape and s.shape == x.shape[:-1]
    assert torch.equal(s.cpu().view(torch.int32), so.view(torch.int32)), "per-token scale differs"
    assert torch.equal(q.cpu(), qo), f"int8 differs at {(q.cpu() != qo).sum().item()} places"


def test_dynamic_quant_config1_and_golden(cabi, golden_dir):
    kat = np.load(os.path.join(golden_dir, "oracle_kat.npz"))
    c1 = workloads.config1()
    q, s = cabi.dynamic_quant(c1["x"].cuda())
    assert np.array_equal(q.cpu().numpy(), kat["c1_q"])
    assert np.array_equal(s.cpu().numpy().view(np.uint32), kat["c1_pertoken"].view(np.uint32))


@pytest.mark.parametrize("m,k", [(1, 4096), (16, 4096), (128, 11008), (2048, 4096), (33, 8192), (5, 28672),
                                 (3, 8), (9, 520), (2, 65536)])
def test_dynamic_quant_smooth_fp32(cabi, m, k):
    d = workloads.w8a8_linear(m, k, 8, 100 + m)
    check_dq(cabi, d["x"], d["smooth_scales"])
    check_dq(cabi, d["x"], None)


def test_dynamic_quant_fp16_and_same_dtype_smooth(cabi):
    g = torch.Generator().manual_seed(5)
    x = workloads.randn_bf16((4, 96, 1024), g, torch.float16)
    sm = workloads.rand_uniform((1024,), g, 0.5, 2.0, torch.float16)
    check_dq(cabi, x, sm)
    xb = workloads.randn_bf16((7, 2048), g)
    check_dq(cabi, xb, workloads.rand_uniform((2048,), g, 0.5, 2.0, torch.bfloat16))


def test_dynamic_quant_ragged_and_degenerate(cabi):
    g = torch.Generator().manual_seed(6)
    check_dq(cabi, workloads.randn_bf16((7, 1001), g), workloads.rand_uniform((1001,), g, 0.5, 2.0))   # k % 8 != 0
    check_dq(cabi, workloads.randn_bf16((3, 131080), g), None)                                          # beyond the register path
    check_dq(cabi, torch.zeros(4, 256, dtype=torch.bfloat16), None)                                     # all-zero rows
    x = workloads.randn_bf16((6, 512), g)
    x[2] = 0
    check_dq(cabi, x, None)
    q, s = cabi.dynamic_quant(torch.empty(0, 64, dtype=torch.bfloat16, device="cuda"))
    assert q.shape == (0, 64) and s.shape == (0,)
    # exact ties: scale is 1, halves round to even
    x = torch.tensor([[0.5, -1.5, 2.5, -127.0, 3.5, 4.5, -0.5, 1.0]], dtype=torch.float16)
    q, s = cabi.dynamic_quant(x.cuda())
    assert q.cpu().tolist() == [[0, -2, 2, -127, 4, 4, 0, 1]] and s.item() == 1.0


def test_dynamic_quant_rejects(cabi):
    with pytest.raises(cabi.B200QError) as e:
        cabi.dynamic_quant(torch.zeros(2, 8, device="cuda"))
    assert e.value.status == cabi.ERR_UNSUPPORTED
    with pytest.raises(cabi.B200QError):
        cabi.dynamic_quant(torch.zeros(2, 8, dtype=torch.bfloat16))          # CPU tensor: no CPU path


# ----------------------------------------------------------------------- int4 pack
def test_int4pack_matches_oracle_and_reference_unpack(cabi, golden_dir):
    g = torch.Generator().manual_seed(7)
    w = torch.randint(-8, 8, (129, 264), generator=g, dtype=torch.int32)
    p = cabi.int4pack(w.cuda()).cpu()
    assert p.dtype == torch.int32 and p.shape == (129, 33)
    assert torch.equal(p, oracle.convert_weight_to_int4pack(w))
    assert torch.equal(oracle.unpack_int4(p).to(torch.int32), w)
    ref = np.load(os.path.join(golden_dir, "reference_goldens.npz"))
    vals = torch.from_numpy(ref["unpack_out"].astype(np.int32))
    assert np.array_equal(cabi.int4pack(vals.cuda()).cpu().numpy(), ref["unpack_in"])
    with pytest.raises(cabi.B200QError):
        cabi.int4pack(torch.zeros(4, 12, dtype=torch.int32, device="cuda"))
    assert cabi.int4pack(torch.zeros(0, 16, dtype=torch.int32, device="cuda")).shape == (0, 2)


# -------------------------------------------------------------------- quant matmul
def run_qmm(cabi, x1, x2, scale, **kw):
    out = cabi.quant_matmul(dev(x1), dev(x2), dev(scale), offset=dev(kw.get("offset")),
                            pertoken_scale=dev(kw.get("pertoken_scale")), bias=dev(kw.get("bias")),
                            output_dtype=kw.get("output_dtype"))
    return out.cpu()


def check_qmm(cabi, x1, x2, scale, **kw):
    got = run_qmm(cabi, x1, x2, scale, **kw)
    want = oracle.quant_matmul(x1, x2, scale, **kw)
    assert got.dtype == want.dtype and got.shape == want.shape
    if want.dtype in (torch.int8, torch.int32):
        assert torch.equal(got, want), f"{(got != want).sum().item()} integer outputs differ"
    else:
        err = oracle.max_mixed_error(got, want)
        assert err <= TOL, err
        # the epilogue repeats the oracle's fp32 steps, so it should in fact agree to the bit
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def cuda_view(x2_nk):
    """The transposed view of an [n,k] weight, as LinearQuant passes it."""
    return x2_nk.cuda().t()


def test_config1_pipeline_and_golden(cabi, golden_dir):
    kat = np.load(os.path.join(golden_dir, "oracle_kat.npz"))
    c1 = workloads.config1()
    q, s = cabi.dynamic_quant(c1["x"].cuda())
    acc = cabi.quant_matmul(q, c1["x2"].cuda(), c1["scale"].cuda(), output_dtype=torch.int32)
    assert np.array_equal(acc.cpu().numpy(), kat["c1_acc"])
    y = cabi.quant_matmul(q, c1["x2"].cuda(), c1["scale"].cuda(), pertoken_scale=s, output_dtype=torch.bfloat16)
    assert np.array_equal(y.cpu().view(torch.int16).numpy().view(np.uint16), kat["c1_out"])
    # same weight handed over as the transposed view of [n,k]
    y2 = cabi.quant_matmul(q, c1["x2"].t().contiguous().cuda().t(), c1["scale"].cuda(), pertoken_scale=s,
                           output_dtype=torch.bfloat16)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("m", [1, 7, 16, 17, 64, 128, 129, 300])
@pytest.mark.parametrize("k,n", [(128, 256), (512, 384), (1040, 200), (4096, 1024)])
@pytest.mark.parametrize("layout", ["nk", "kn"])
def test_quant_matmul_int32_exact(cabi, m, k, n, layout):
    g = torch.Generator().manual_seed(m * 7 + k + n)
    x1 = workloads.rand_int8((m, k), g, -128, 127)
    w = workloads.rand_int8((n, k), g, -128, 127)
    x2 = w.t() if layout == "nk" else w.t().contiguous()
    got = cabi.quant_matmul(x1.cuda(), x2.cuda() if layout == "kn" else cuda_view(w), torch.ones(1, device="cuda"),
                            output_dtype=torch.int32).cpu()
    want = oracle.quant_matmul(x1, x2, torch.ones(1), output_dtype=torch.int32)
    assert torch.equal(got, want), f"{(got != want).sum().item()} of {got.numel()} accumulators differ"


@pytest.mark.parametrize("m", [1, 16, 100, 128, 200, 513])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, None, torch.int32])
def test_quant_matmul_epilogue_variants(cabi, m, out_dtype):
    k, n = 640, 272
    g = torch.Generator().manual_seed(m + 31)
    x1 = workloads.rand_int8((m, k), g)
    w = workloads.rand_int8((n, k), g)
    scale = workloads.rand_uniform((n,), g, 1e-3, 1e-2)
    small = workloads.rand_uniform((n,), g, 2e-5, 1e-4)       # keeps int8 outputs inside [-128, 127] mostly
    offset = workloads.rand_uniform((n,), g, -4, 4)
    pt = workloads.rand_uniform((m,), g, 1e-3, 1e-2)
    ibias = torch.randint(-1000, 1001, (n,), generator=g, dtype=torch.int32)
    fbias = workloads.rand_uniform((n,), g, -2, 2)
    x2 = w.t()
    if out_dtype == torch.int32:
        check_qmm(cabi, x1, x2, scale, bias=ibias, output_dtype=out_dtype)
        return
    if out_dtype is None:                                     # int8 output (the operator's default)
        check_qmm(cabi, x1, x2, small, offset=offset, bias=ibias)
        check_qmm(cabi, x1, x2, small[:1].clone(), offset=offset[:1].clone())
        return
    check_qmm(cabi, x1, x2, scale, pertoken_scale=pt, output_dtype=out_dtype)
    check_qmm(cabi, x1, x2, scale, offset=offset, pertoken_scale=pt, bias=ibias, output_dtype=out_dtype)
    check_qmm(cabi, x1, x2, scale, bias=fbias.to(out_dtype), output_dtype=out_dtype)
    check_qmm(cabi, x1, x2, scale, bias=fbias, pertoken_scale=pt, output_dtype=out_dtype)
    check_qmm(cabi, x1, x2, scale[:1].clone(), output_dtype=out_dtype)                 # per-tensor scale
    check_qmm(cabi, x1, x2, scale.to(torch.bfloat16), output_dtype=torch.bfloat16)     # bf16 scale
    check_qmm(cabi, x1, x2, oracle.trans_quant_param(scale), output_dtype=out_dtype)   # int64 scale


def test_quant_matmul_unaligned_shapes_take_the_generic_kernel(cabi):
    g = torch.Generator().manual_seed(9)
    for m, k, n in [(1, 5, 127), (3, 2, 128), (9, 100, 33), (4, 24, 8)]:
        x1 = workloads.rand_int8((m, k), g)
        w = workloads.rand_int8((n, k), g)
        sc = workloads.rand_uniform((n,), g, 1e-3, 1e-2)
        check_qmm(cabi, x1, w.t(), sc, output_dtype=torch.float16)
        check_qmm(cabi, x1, w.t().contiguous(), sc, output_dtype=torch.int32)
    e = cabi.quant_matmul(torch.zeros(0, 64, dtype=torch.int8, device="cuda"),
                          torch.zeros(64, 32, dtype=torch.int8, device="cuda"), torch.ones(1, device="cuda"))
    assert e.shape == (0, 32)


def test_quant_matmul_rejects(cabi):
    x1 = torch.zeros(4, 64, dtype=torch.int8, device="cuda")
    x2 = torch.zeros(64, 32, dtype=torch.int8, device="cuda")
    with pytest.raises(cabi.B200QError):                      # fp16 scale is not accepted by the operator
        cabi.quant_matmul(x1, x2, torch.ones(32, dtype=torch.float16, device="cuda"))
    with pytest.raises(cabi.B200QError):
        cabi.quant_matmul(x1, x2, torch.ones(7, device="cuda"))
    with pytest.raises(cabi.B200QError):
        cabi.quant_matmul(x1, x2, torch.ones(1, device="cuda"), output_dtype=torch.float64)


@pytest.mark.parametrize("mi", [0, 1, 2, 3])
@pytest.mark.parametrize("si", [0, 1, 2, 3])
def test_config2_llama7b_linears(cabi, mi, si):
    """Full-size config 2: dynamic quant with smooth scales then W8A8 GEMM, bf16 out.  The int8
    activations and fp32 scales are compared in full; the GEMM through a Freivalds check on the
    int32 accumulators and up to 64 full rows of the bf16 output against the oracle."""
    d = workloads.config2_case(mi, si)
    m, k = d["x"].shape
    n = d["scale"].numel()
    q, s = cabi.dynamic_quant(d["x"].cuda(), d["smooth_scales"].cuda())
    qo, so = oracle.dynamic_quant(d["x"], d["smooth_scales"])
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu().view(torch.int32), so.view(torch.int32))
    wv = cuda_view(d["weight_nk"])
    acc = cabi.quant_matmul(q, wv, torch.ones(1, device="cuda"), output_dtype=torch.int32)
    g = torch.Generator().manual_seed(1)
    v = torch.randint(-3, 4, (n,), generator=g, dtype=torch.int64)
    lhs = acc.cpu().to(torch.int64) @ v
    rhs = qo.to(torch.int64) @ (d["weight_nk"].to(torch.int64).t() @ v)
    assert torch.equal(lhs, rhs), "Freivalds check of the int32 accumulators failed"
    y = cabi.quant_matmul(q, wv, d["scale"].cuda(), pertoken_scale=s, output_dtype=torch.bfloat16).cpu()
    rows = torch.randperm(m, generator=g)[:64]
    want = oracle.quant_matmul(qo[rows], d["x2"], d["scale"], pertoken_scale=so[rows], output_dtype=torch.bfloat16)
    assert oracle.max_mixed_error(y[rows], want) <= TOL
    assert torch.equal(y[rows].view(torch.int16), want.view(torch.int16))


def test_config4_batched_offset_bias_fp16(cabi):
    d = workloads.config4()
    b, m, k = d["x1"].shape
    n = d["scale"].numel()
    x2 = d["x2"].cuda()
    y = cabi.quant_matmul(d["x1"].cuda(), x2, d["scale"].cuda(), offset=d["offset"].cuda(),
                          pertoken_scale=d["pertoken_scale"].cuda(), bias=d["bias"].cuda(),
                          output_dtype=torch.float16).cpu()
    assert y.shape == (b, m, n) and y.dtype == torch.float16
    g = torch.Generator().manual_seed(2)
    rows = torch.randperm(b * m, generator=g)[:48]
    want = oracle.quant_matmul(d["x1"].reshape(-1, k)[rows], d["x2"], d["scale"], offset=d["offset"],
                               pertoken_scale=d["pertoken_scale"][rows], bias=d["bias"], output_dtype=torch.float16)
    assert oracle.max_mixed_error(y.reshape(-1, n)[rows], want) <= TOL
    acc = cabi.quant_matmul(d["x1"].cuda(), x2, torch.ones(1, device="cuda"), bias=d["bias"].cuda(),
                            output_dtype=torch.int32).cpu().reshape(-1, n)
    v = torch.randint(-3, 4, (n,), generator=g, dtype=torch.int64)
    rhs = d["x1"].reshape(-1, k).to(torch.int64) @ (d["x2"].to(torch.int64) @ v) + (d["bias"].to(torch.int64) @ v)
    assert torch.equal(acc.to(torch.int64) @ v, rhs)


def test_dynamic_quant_tiny_rows_keep_ieee_division(cabi):
    """Rows whose maximum is so small that 1/scale overflows (bf16 inputs reach 1e-38): the reciprocal path
    must hand over to true division and still agree with the oracle bit for bit."""
    g = torch.Generator().manual_seed(8)
    for amp in (1e-38, 3e-37, 1e-33, 1e-28):
        x = (torch.randn((5, 2048), generator=g) * amp).to(torch.bfloat16)
        x[1] = 0
        check_dq(cabi, x, None)
        check_dq(cabi, x[:, :520].contiguous(), None)          # register kernel (k < 1024)


@pytest.mark.parametrize("m,k,n", [(1, 4096, 4096), (16, 8192, 2048), (7, 1024, 9472), (16, 11008, 4096),
                                   (3, 11008, 9600), (128, 1024, 22016), (64, 11008, 4096), (100, 2048, 12288)])
def test_quant_matmul_decode_cluster_split_k(cabi, m, k, n):
    """The paths for few tokens.  By default: one or two tokens a warp per channel (first shape), three to sixteen
    tokens the warp-MMA streaming kernel (second to fifth shape), both one launch without scratch;
    more tokens the swapped tcgen05 kernel with K split over independent CTAs.  Then, forced by the library's
    tuning switches, every shape through the cluster split-K kernel (partial tiles added through distributed
    shared memory; cluster sizes 1..8, token tiles 16..128, several rounds per cluster) and through the
    independent-CTA split.  int32 accumulators in full and the fused epilogue must match the oracle exactly."""
    g = torch.Generator().manual_seed(m + k + n)
    x1 = workloads.rand_int8((m, k), g, -128, 127)
    w = workloads.rand_int8((n, k), g, -128, 127)
    if m <= 16:
        assert cabi.lib().b200q_quant_matmul_workspace_bytes(m, k, n, 1, k) == 0  # no scratch, no second kernel
    got = cabi.quant_matmul(x1.cuda(), cuda_view(w), torch.ones(1, device="cuda"), output_dtype=torch.int32).cpu()
    want = oracle.quant_matmul(x1, w.t(), torch.ones(1), output_dtype=torch.int32)
    assert torch.equal(got, want), f"{(got != want).sum().item()} of {got.numel()} accumulators differ"
    scale = workloads.rand_uniform((n,), g, 1e-3, 1e-2)
    pt = workloads.rand_uniform((m,), g, 1e-3, 1e-2)
    bias = torch.randint(-1000, 1001, (n,), generator=g, dtype=torch.int32)
    check_qmm(cabi, x1, w.t(), scale, pertoken_scale=pt, bias=bias, output_dtype=torch.bfloat16)
    for _ in range(3):                                          # persistent clusters reuse their barriers and buffers
        again = cabi.quant_matmul(x1.cuda(), cuda_view(w), torch.ones(1, device="cuda"), output_dtype=torch.int32).cpu()
        assert torch.equal(again, want)
    # The cluster kernel on every shape of the list (larger token tiles, several rounds per cluster), forced by
    # the library's tuning switches; the default rule only picks it where it was measured faster.
    os.environ["B200Q_W8A8_DECODE"], os.environ["B200Q_W8A8_GEMV"], os.environ["B200Q_W8A8_SMALL_M"] = "1", "0", "0"
    try:
        forced = cabi.quant_matmul(x1.cuda(), cuda_view(w), torch.ones(1, device="cuda"), output_dtype=torch.int32).cpu()
        assert torch.equal(forced, want)
        check_qmm(cabi, x1, w.t(), scale, pertoken_scale=pt, bias=bias, output_dtype=torch.float16)
    finally:
        del os.environ["B200Q_W8A8_DECODE"], os.environ["B200Q_W8A8_GEMV"], os.environ["B200Q_W8A8_SMALL_M"]
    # ... and the K-split over independent CTAs (int32 scratch, atomics, second kernel), the path of 17..128 tokens
    os.environ["B200Q_W8A8_DECODE"], os.environ["B200Q_W8A8_GEMV"], os.environ["B200Q_W8A8_SMALL_M"] = "0", "0", "0"
    try:
        legacy = cabi.quant_matmul(x1.cuda(), cuda_view(w), torch.ones(1, device="cuda"), output_dtype=torch.int32).cpu()
        assert torch.equal(legacy, want)
    finally:
        del os.environ["B200Q_W8A8_DECODE"], os.environ["B200Q_W8A8_GEMV"], os.environ["B200Q_W8A8_SMALL_M"]


def freivalds_and_rows(cabi, q, qo, so, s, weight_nk, scale, seed, rows_checked=64):
    """Full-size GEMM check: (X W) v == X (W v) on the int32 accumulators in int64, and `rows_checked` full
    rows of the bf16 output against the oracle."""
    m, n = q.shape[0], weight_nk.shape[0]
    wv = cuda_view(weight_nk)
    acc = cabi.quant_matmul(q, wv, torch.ones(1, device="cuda"), output_dtype=torch.int32)
    g = torch.Generator().manual_seed(seed)
    v = torch.randint(-3, 4, (n,), generator=g, dtype=torch.int64)
    lhs = (acc.to(torch.float64) @ v.cuda().to(torch.float64)).cpu().to(torch.int64)       # |sum| < 2^53: exact
    del acc
    # W v and X (W v) in float64, a slice of W at a time: every partial sum is an integer below 2^53, so exact
    k = weight_nk.shape[1]
    wv_host = torch.zeros(k, dtype=torch.float64)
    vf = v.to(torch.float64)
    for lo in range(0, n, 8192):
        wv_host += weight_nk[lo:lo + 8192].to(torch.float64).t() @ vf[lo:lo + 8192]
    rhs = (qo.to(torch.float64) @ wv_host).to(torch.int64)
    assert torch.equal(lhs, rhs), "Freivalds check of the int32 accumulators failed"
    y = cabi.quant_matmul(q, wv, scale.cuda(), pertoken_scale=s, output_dtype=torch.bfloat16)
    rows = torch.randperm(m, generator=g)[:rows_checked]
    got = y[rows.cuda()].cpu()
    del y
    want = oracle.quant_matmul(qo[rows], weight_nk.t(), scale, pertoken_scale=so[rows], output_dtype=torch.bfloat16)
    assert oracle.max_mixed_error(got, want) <= TOL
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_config5_llama70b_mlp_full_size(cabi):
    """Config 5 at full size on one GPU (the shapes the benchmark is quoted on): dynamic quant of x [4096,8192]
    and x_down [4096,28672] compared with the oracle in full, bit for bit; gate/up GEMM 4096x8192x57344 and down
    GEMM 4096x28672x8192 through the Freivalds product check on all int32 accumulators plus 64 full bf16 rows."""
    d = workloads.config5_shard(0, 1)
    q, s = cabi.dynamic_quant(d["x"].cuda(), d["smooth_scales"].cuda())
    qo, so = oracle.dynamic_quant(d["x"], d["smooth_scales"])
    assert torch.equal(s.cpu().view(torch.int32), so.view(torch.int32)) and torch.equal(q.cpu(), qo)
    freivalds_and_rows(cabi, q, qo, so, s, d["gate_up_weight_nk"], d["gate_up_scale"], 51)
    del q, s
    q2, s2 = cabi.dynamic_quant(d["x_down"].cuda(), d["smooth_scales_down"].cuda())
    q2o, s2o = oracle.dynamic_quant(d["x_down"], d["smooth_scales_down"])
    assert torch.equal(s2.cpu().view(torch.int32), s2o.view(torch.int32)) and torch.equal(q2.cpu(), q2o)
    freivalds_and_rows(cabi, q2, q2o, s2o, s2, d["down_weight_nk"], d["down_scale"], 52)


def test_int4pack_flags_values_outside_int4(cabi):
    w = torch.zeros(4, 16, dtype=torch.int32, device="cuda")
    w[2, 5] = 9                                                 # no int4 representation
    cabi.int4pack(w)
    torch.cuda.synchronize()
    assert cabi.device_error(reset=True) == 0x201
    w[2, 5] = -8
    cabi.int4pack(w)
    torch.cuda.synchronize()
    assert cabi.device_error() == 0

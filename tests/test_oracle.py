"""The oracle against the reference's own CPU goldens (fixtures produced by
tests/golden/make_golden.py from the reference's helper functions), against its
committed known-answer vectors, and against independent integer arithmetic."""
import os

import numpy as np
import pytest
import torch

from oracle import quant_oracle as oracle
from pytorch_b200 import workloads


@pytest.fixture(scope="module")
def ref(golden_dir):
    return np.load(os.path.join(golden_dir, "reference_goldens.npz"))


@pytest.fixture(scope="module")
def kat(golden_dir):
    return np.load(os.path.join(golden_dir, "oracle_kat.npz"))


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def test_unpack_int4_matches_reference_helper(ref):
    got = oracle.unpack_int4(torch.from_numpy(ref["unpack_in"]))
    assert np.array_equal(got.numpy(), ref["unpack_out"])


def test_int4pack_is_inverse_of_reference_unpack(ref):
    vals = torch.from_numpy(ref["unpack_out"].astype(np.int32))
    packed = oracle.convert_weight_to_int4pack(vals)
    assert packed.dtype == torch.int32 and packed.shape == (6, 10)
    assert np.array_equal(packed.numpy(), ref["unpack_in"])


def test_int4pack_rejects_bad_input():
    with pytest.raises(ValueError):
        oracle.convert_weight_to_int4pack(torch.zeros(2, 12, dtype=torch.int32))
    with pytest.raises(ValueError):
        oracle.convert_weight_to_int4pack(torch.full((2, 8), 8, dtype=torch.int32))


def test_antiquant_matches_reference_golden(ref):
    # (x + offset) * scale on int4-packed input, per-channel fp32 scale/offset, fp16 out
    w = oracle.dequant_weight(torch.from_numpy(ref["unpack_in"]), torch.from_numpy(ref["anti_scale"]),
                              torch.from_numpy(ref["anti_offset"]))
    assert np.array_equal(torch.from_numpy(w).to(torch.float16).numpy(), ref["anti_out_f16"])


def test_weight_quant_matmul_matches_reference_golden(ref):
    # The reference golden is handed fp16 tensors, so it rounds (w+offset) and the product
    # to fp16 before its fp32 matmul.  The oracle's default does the same and must agree to
    # fp16 rounding of the result (fp32 vs fp64 summation); with an all-fp32 dequantisation the
    # difference is the golden's own fp16 rounding of the weights.
    args = (torch.from_numpy(ref["wq_x"]), torch.from_numpy(ref["wq_w_nk"]).t(),
            torch.from_numpy(ref["wq_scale"]), torch.from_numpy(ref["wq_offset"]))
    want = torch.from_numpy(ref["wq_out"])
    got16 = oracle.weight_quant_batchmatmul(*args)
    assert got16.dtype == torch.float16
    assert oracle.max_mixed_error(got16, want) <= 2 ** -10
    got = oracle.weight_quant_batchmatmul(*args, dequant_dtype=None)
    assert oracle.max_mixed_error(got, want) <= 2 ** -5


def test_quant_matmul_dequant_matches_reference_golden(ref):
    # x1_scale * x2_scale * (x1 @ x2 + bias): the oracle multiplies in the other order,
    # so the comparison is to fp32 rounding (2 ulp), not to the bit
    got = oracle.quant_matmul(
        torch.from_numpy(ref["mm_x1"]), torch.from_numpy(ref["mm_x2"]), torch.from_numpy(ref["mm_s2"]).reshape(-1),
        pertoken_scale=torch.from_numpy(ref["mm_s1"]).reshape(-1), bias=torch.from_numpy(ref["mm_bias"]),
        output_dtype=torch.float16)
    want = torch.from_numpy(ref["mm_out"])
    assert oracle.max_mixed_error(got, want.to(torch.float16)) <= 2 ** -10
    acc = oracle.quant_matmul(torch.from_numpy(ref["mm_x1"]), torch.from_numpy(ref["mm_x2"]),
                              torch.ones(1), bias=torch.from_numpy(ref["mm_bias"]), output_dtype=torch.int32)
    exact = ref["mm_x1"].astype(np.int64) @ ref["mm_x2"].astype(np.int64) + ref["mm_bias"]
    assert np.array_equal(acc.numpy(), exact.astype(np.int32))


def test_config1_known_answers(kat):
    c1 = workloads.config1()
    assert np.array_equal(c1["x"].view(torch.int16).numpy().view(np.uint16), kat["c1_x"])
    q, s = oracle.dynamic_quant(c1["x"])
    assert np.array_equal(q.numpy(), kat["c1_q"])
    assert np.array_equal(s.numpy().view(np.uint32), kat["c1_pertoken"].view(np.uint32))
    acc = oracle.quant_matmul(q, c1["x2"], c1["scale"], output_dtype=torch.int32)
    assert np.array_equal(acc.numpy(), kat["c1_acc"])
    y = oracle.quant_matmul(q, c1["x2"], c1["scale"], pertoken_scale=s, output_dtype=torch.bfloat16)
    assert torch.equal(y, bf16(kat["c1_out"]))


def test_dynamic_quant_scalar_restatement():
    """Pure-Python loop restatement on a small case: amax/127, rint, clamp."""
    d = workloads.w8a8_linear(3, 40, 8, 5)
    x = d["x"].float().numpy()
    sm = d["smooth_scales"].numpy()
    q, s = oracle.dynamic_quant(d["x"], d["smooth_scales"])
    for r in range(3):
        xs = [np.float32(x[r, c]) * np.float32(sm[c]) for c in range(40)]
        amax = max(abs(v) for v in xs)
        sc = np.float32(amax) / np.float32(127.0)
        assert np.float32(s[r].item()) == sc
        for c in range(40):
            want = int(np.clip(np.rint(np.float32(xs[c]) / sc), -128, 127))
            assert q[r, c].item() == want


def test_dynamic_quant_edge_cases():
    z = torch.zeros(2, 16, dtype=torch.bfloat16)
    q, s = oracle.dynamic_quant(z)
    assert q.abs().max() == 0 and s.abs().max() == 0
    x = torch.tensor([[0.5, -1.5, 2.5, -127.0]], dtype=torch.float16)
    q, s = oracle.dynamic_quant(x)          # scale = 1 -> ties go to even
    assert q.tolist() == [[0, -2, 2, -127]] and s.item() == 1.0
    q, s = oracle.dynamic_quant(torch.randn(4, 2048, 8, dtype=torch.float16))
    assert q.shape == (4, 2048, 8) and s.shape == (4, 2048) and s.dtype == torch.float32
    assert int(q.to(torch.int32).abs().amax(-1).min()) == 127   # the amax element maps to +-127


def test_quant_matmul_int32_exact_vs_integer_matmul():
    g = torch.Generator().manual_seed(3)
    a = workloads.rand_int8((33, 200), g, -128, 127)
    b = workloads.rand_int8((200, 17), g, -128, 127)
    acc = oracle.quant_matmul(a, b, torch.ones(1), output_dtype=torch.int32)
    assert np.array_equal(acc.numpy(), (a.numpy().astype(np.int64) @ b.numpy().astype(np.int64)).astype(np.int32))


def test_quant_matmul_batched_known_answers(kat):
    b = {k[2:]: torch.from_numpy(kat[k]) for k in kat.files if k.startswith("b_") and "out" not in k}
    y = oracle.quant_matmul(b["x1"], b["x2"], b["scale"], offset=b["offset"],
                            pertoken_scale=b["pertoken_scale"], bias=b["bias"], output_dtype=torch.float16)
    assert y.shape == (2, 3, 16) and np.array_equal(y.numpy(), kat["b_out_f16"])
    y8 = oracle.quant_matmul(b["x1"], b["x2"], b["scale"], offset=b["offset"], bias=b["bias"])
    assert y8.dtype == torch.int8 and np.array_equal(y8.numpy(), kat["b_out_i8"])


def test_w4a16_known_answers_and_linearity(kat):
    x = bf16(kat["w4_x"])
    packed = torch.from_numpy(kat["w4_packed"])
    assert np.array_equal(oracle.convert_weight_to_int4pack(torch.from_numpy(kat["w4_w"])).numpy(), kat["w4_packed"])
    sc, of = bf16(kat["w4_scale"]), bf16(kat["w4_offset"])
    y = oracle.weight_quant_batchmatmul(x, packed, sc, of, antiquant_group_size=128)
    assert torch.equal(y, bf16(kat["w4_out"]))
    y2 = oracle.weight_quant_batchmatmul((x.float() * 2).to(torch.bfloat16), packed, sc, of, antiquant_group_size=128)
    assert torch.equal(y2.float(), y.float() * 2)       # scaling x by 2 is exact in bf16


def test_trans_quant_param_contract():
    p = oracle.trans_quant_param(torch.randn(1), torch.randn(4))
    assert p.shape == (4,) and p.dtype == torch.int64
    p = oracle.trans_quant_param(torch.randn(1, 4), torch.randn(1, 4))
    assert p.shape == (1, 4) and p.dtype == torch.int64
    s = torch.tensor([0.0123, 4.5])
    assert np.array_equal(oracle.trans_quant_param_decode(oracle.trans_quant_param(s))[0], s.numpy())


def test_reduce_scatter_oracle_matches_reference_golden(golden_dir):
    """The reference's own TestMmReduceScatterBaseOp._get_global_tensor (test/distributed/tensor/test_matrix_ops.py:86-110)
    on three ranks of seeded int8 operands: the oracle's rank-ordered fp32 sum must agree to fp32 rounding (the
    golden multiplies the two scales first, the oracle scales the accumulator one factor at a time)."""
    ref = np.load(os.path.join(golden_dir, "reference_goldens.npz"))
    x1 = [torch.from_numpy(a) for a in ref["rs_x1"]]
    x2 = [torch.from_numpy(a) for a in ref["rs_x2"]]
    s1 = [torch.from_numpy(a) for a in ref["rs_s1"]]
    s2 = [torch.from_numpy(a) for a in ref["rs_s2"]]
    got = torch.cat(oracle.mm_reduce_scatter(x1, x2, s1, s2, output_dtype=torch.float32))
    want = torch.from_numpy(ref["rs_out"])
    assert got.shape == want.shape
    assert torch.allclose(got, want, rtol=4e-7, atol=1e-6)
    # after the cast the two orders give the same bf16 except where the fp32 value sits on a rounding boundary
    b = torch.cat(oracle.mm_reduce_scatter(x1, x2, s1, s2, output_dtype=torch.bfloat16))
    assert oracle.max_mixed_error(b, want.to(torch.bfloat16)) <= 2.0 ** -7
    # all-reduce form: same sum, replicated
    ar = oracle.mm_all_reduce(x1, x2, torch.from_numpy(ref["rs_s2"][0]).reshape(-1), output_dtype=torch.float32)
    assert ar.shape == (6, 32)

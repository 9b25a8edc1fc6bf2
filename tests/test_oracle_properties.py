"""Property tests of the CPU oracle on random shapes (hypothesis): the size-independent identities the
GPU parity tests rely on at full size must hold for the checker itself."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from oracle import quant_oracle as oracle

SETTINGS = dict(max_examples=25, deadline=None, derandomize=True)   # same examples on every run


def rand(shape, seed, dtype=torch.bfloat16, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@settings(**SETTINGS)
@given(rows=st.integers(1, 9), k=st.integers(1, 70), seed=st.integers(0, 10 ** 6),
       dtype=st.sampled_from([torch.bfloat16, torch.float16]))
def test_dynamic_quant_range_and_reconstruction(rows, k, seed, dtype):
    x = rand((rows, k), seed, dtype, 3.0)
    y, s = oracle.dynamic_quant(x)
    assert y.dtype == torch.int8 and s.dtype == torch.float32 and s.shape == (rows,)
    # the largest magnitude of every row maps to +-127, nothing leaves [-127, 127]
    nz = s > 0
    assert torch.equal(y.abs().max(-1).values[nz], torch.full((int(nz.sum()),), 127, dtype=torch.int8))
    assert int(y.abs().max()) <= 127
    # reconstruction error at most half a step (plus fp32 rounding of the quotient)
    err = (y.float() * s[:, None] - x.float()).abs().max(-1).values
    assert bool((err <= s * 0.5 * (1 + 1e-5)).all())


@settings(**SETTINGS)
@given(rows=st.integers(1, 6), k=st.integers(2, 64), seed=st.integers(0, 10 ** 6), p=st.integers(-3, 3))
def test_dynamic_quant_is_invariant_under_powers_of_two(rows, k, seed, p):
    x = rand((rows, k), seed, torch.float16, 1.0)
    y1, s1 = oracle.dynamic_quant(x)
    y2, s2 = oracle.dynamic_quant((x.float() * 2.0 ** p).to(torch.float16))
    assert torch.equal(y1, y2) and torch.equal(s1 * 2.0 ** p, s2)


@settings(**SETTINGS)
@given(rows=st.integers(1, 5), words=st.integers(1, 9), seed=st.integers(0, 10 ** 6))
def test_int4_pack_unpack_roundtrip(rows, words, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randint(-8, 8, (rows, words * 8), generator=g, dtype=torch.int32)
    packed = oracle.convert_weight_to_int4pack(w)
    assert packed.shape == (rows, words) and packed.dtype == torch.int32
    assert torch.equal(oracle.unpack_int4(packed).to(torch.int32), w)


@settings(**SETTINGS)
@given(m=st.integers(1, 6), k=st.integers(1, 48), n=st.integers(1, 12), seed=st.integers(0, 10 ** 6))
def test_int8_gemm_matches_integer_arithmetic_and_is_linear(m, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-128, 128, (m, k), generator=g, dtype=torch.int32).to(torch.int8)
    b = torch.randint(-128, 128, (k, n), generator=g, dtype=torch.int32).to(torch.int8)
    b2 = torch.randint(-64, 64, (k, n), generator=g, dtype=torch.int32).to(torch.int8)
    acc = oracle.int8_gemm_int32(a, b)
    assert np.array_equal(acc, a.numpy().astype(np.int64) @ b.numpy().astype(np.int64))
    both = oracle.int8_gemm_int32(a, b) + oracle.int8_gemm_int32(a, b2)
    wide = a.numpy().astype(np.int64) @ (b.numpy().astype(np.int64) + b2.numpy().astype(np.int64))
    assert np.array_equal(both, wide)


@settings(**SETTINGS)
@given(rows=st.integers(1, 6), n8=st.integers(1, 6), seed=st.integers(0, 10 ** 6),
       dst=st.sampled_from([torch.float16, torch.bfloat16]))
def test_anti_quant_int4_equals_int8_of_the_unpacked_values(rows, n8, seed, dst):
    g = torch.Generator().manual_seed(seed)
    packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, n8), generator=g, dtype=torch.int64).to(torch.int32)
    sc = torch.rand(n8 * 8, generator=g) * 4 - 2
    of = torch.rand(n8 * 8, generator=g) * 10 - 5
    a = oracle.anti_quant(packed, sc, of, dst)
    b = oracle.anti_quant(oracle.unpack_int4(packed), sc, of, dst)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


@settings(**SETTINGS)
@given(rows=st.integers(1, 6), k=st.integers(2, 64), seed=st.integers(0, 10 ** 6))
def test_asymmetric_quant_uses_the_whole_range(rows, k, seed):
    x = rand((rows, k), seed, torch.bfloat16, 2.0) + 0.75
    y, s, o = oracle.dynamic_quant_asymmetric(x)
    live = s > 0
    assert bool((y.max(-1).values[live] == 127).all()) and bool((y.min(-1).values[live] == -128).all())
    back = (y.float() - o[:, None]) * s[:, None]
    assert bool(((back - x.float()).abs().max(-1).values <= s * 0.5 * 1.001 + 1e-6).all())

"""Seeded synthetic inputs for the five benchmark configurations of the
quantized-inference path (shapes, dtypes and value distributions only; no data
set is involved).  Tensors are generated on the CPU with a fixed
``torch.Generator`` seed (``1000 * config + case``; config 1 uses seed 0) so that
the GPU path, the CPU oracle and the committed golden fixtures all see the same
bits.

Names: C1 plumbing, C2 Llama-7B-shaped W8A8 linears, C3 W4A16 weight-only,
C4 batched W8A8 with offset and bias, C5 Llama-70B-shaped N-sharded W8A8 MLP.
"""
from __future__ import annotations

import torch

C2_M = (1, 16, 128, 2048)
C2_KN = ((4096, 12288), (4096, 4096), (4096, 22016), (11008, 4096))
C3_M = (1, 32, 256)
C3_K, C3_N, C3_GS = 8192, 28672, 128
C4_SHAPE = (8, 512, 5120, 13824)           # batch, m, k, n
C5_M, C5_HIDDEN, C5_FFN = 4096, 8192, 28672


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def randn_bf16(shape, g, dtype=torch.bfloat16):
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype)


def rand_int8(shape, g, lo=-127, hi=127):
    return torch.randint(lo, hi + 1, shape, generator=g, dtype=torch.int32).to(torch.int8)


def rand_uniform(shape, g, lo, hi, dtype=torch.float32):
    return (torch.rand(shape, generator=g, dtype=torch.float32) * (hi - lo) + lo).to(dtype)


def config1():
    """x bf16 [16,512] ~N(0,1), seed 0; x2 int8 [512,256]; scale fp32 [256]."""
    g = _gen(0)
    return dict(
        x=randn_bf16((16, 512), g),
        x2=rand_int8((512, 256), g),
        scale=rand_uniform((256,), g, 1e-3, 1e-2),
    )


def w8a8_linear(m, k, n, seed, *, smooth=True, weight_layout="nk", x_dtype=torch.bfloat16):
    """One W8A8 linear: x [m,k], smooth_scales fp32 [k] in [0.5,2], weight int8 and
    per-channel fp32 scale [n] in [1e-3,1e-2].  ``weight_layout`` "nk" stores the
    weight as ``[n,k]`` (what ``LinearQuant`` holds; the op then sees the
    transposed view), "kn" stores a contiguous ``[k,n]``."""
    g = _gen(seed)
    d = dict(x=randn_bf16((m, k), g, x_dtype))
    d["smooth_scales"] = rand_uniform((k,), g, 0.5, 2.0) if smooth else None
    w = rand_int8((n, k), g)
    d["weight_nk"] = w
    d["x2"] = w.t() if weight_layout == "nk" else w.t().contiguous()
    d["scale"] = rand_uniform((n,), g, 1e-3, 1e-2)
    return d


def config2_case(mi: int, si: int, **kw):
    m = C2_M[mi]
    k, n = C2_KN[si]
    return w8a8_linear(m, k, n, 2000 + 4 * mi + si, **kw)


def w4a16(m, k, n, gs, seed, x_dtype=torch.bfloat16):
    """x [m,k]; int4 weight values in [-8,7] held one per int32 element ``[k,n]``
    (to be packed by ``npu_convert_weight_to_int4pack``); antiquant scale
    [k/gs,n] in [5e-3,2e-2] and offset [k/gs,n] in [-1,1], both in ``x_dtype``."""
    g = _gen(seed)
    groups = k // gs if gs > 0 else 1
    return dict(
        x=randn_bf16((m, k), g, x_dtype),
        w_int4=torch.randint(-8, 8, (k, n), generator=g, dtype=torch.int32),
        antiquant_scale=rand_uniform((groups, n), g, 5e-3, 2e-2, x_dtype),
        antiquant_offset=rand_uniform((groups, n), g, -1.0, 1.0, x_dtype),
        antiquant_group_size=gs,
    )


def config3_case(mi: int):
    return w4a16(C3_M[mi], C3_K, C3_N, C3_GS, 3000 + mi)


def batched_w8a8(b, m, k, n, seed):
    """x1 int8 [b,m,k]; x2 int8 [k,n]; scale, offset fp32 [n]; int32 bias [n];
    pertoken_scale fp32 [b*m]."""
    g = _gen(seed)
    return dict(
        x1=rand_int8((b, m, k), g),
        x2=rand_int8((k, n), g),
        scale=rand_uniform((n,), g, 1e-3, 1e-2),
        offset=rand_uniform((n,), g, -4.0, 4.0),
        bias=torch.randint(-1000, 1001, (n,), generator=g, dtype=torch.int32),
        pertoken_scale=rand_uniform((b * m,), g, 1e-3, 1e-2),
    )


def config4():
    b, m, k, n = C4_SHAPE
    return batched_w8a8(b, m, k, n, 4000)


def config5_shard(rank: int, world: int, *, m=C5_M, hidden=C5_HIDDEN, ffn=C5_FFN, seed=5000):
    """Rank ``rank``'s slice of the column-sharded MLP.  Activations and
    smooth scales are replicated (same seed on every rank); the gate/up weight
    ``[2*ffn, hidden]`` and the down weight ``[hidden, ffn]`` (both stored
    ``[n,k]``) are cut along n with their per-channel scales.  Each shard is
    generated from its own seed, so no rank ever materialises the full weight."""
    g = _gen(seed)
    d = dict(
        x=randn_bf16((m, hidden), g),
        smooth_scales=rand_uniform((hidden,), g, 0.5, 2.0),
        x_down=randn_bf16((m, ffn), g),
        smooth_scales_down=rand_uniform((ffn,), g, 0.5, 2.0),
    )
    n_gu, n_dn = 2 * ffn // world, hidden // world
    gs = _gen(seed + 1 + rank + 16 * world)
    d["gate_up_weight_nk"] = rand_int8((n_gu, hidden), gs)
    d["gate_up_scale"] = rand_uniform((n_gu,), gs, 1e-3, 1e-2)
    d["down_weight_nk"] = rand_int8((n_dn, ffn), gs)
    d["down_scale"] = rand_uniform((n_dn,), gs, 1e-3, 1e-2)
    return d


def quant_matmul_flops(m, k, n):
    """2*M*K*N, the reference's own matmul FLOP convention
    (``torch_npu/profiler/_flops_formulas.py:319-325``)."""
    return 2.0 * m * k * n


def dynamic_quant_bytes(m, k, in_bytes=2, smooth=True):
    """Algorithmic HBM bytes of one dynamic-quant call: read x, write int8 y and
    the fp32 scale per row, read the fp32 smooth vector once."""
    return m * k * in_bytes + m * k + 4 * m + (4 * k if smooth else 0)


def quant_matmul_bytes(m, k, n, out_bytes=2, pertoken=True, bias=False, offset=False):
    return (m * k + k * n + 4 * n + (4 * m if pertoken else 0) + (4 * n if bias else 0)
            + (4 * n if offset else 0) + m * n * out_bytes)


def w4a16_bytes(m, k, n, gs):
    groups = k // gs if gs else 1
    return 2 * m * k + k * n // 2 + 2 * groups * n * 2 + 2 * m * n


def config5_row_parallel_down(rank: int, world: int, *, hidden=C5_HIDDEN, ffn=C5_FFN, seed=5000):
    """The down projection of the same MLP cut along K instead of N (the reference's tensor-parallel
    form, ``npu_mm_reduce_scatter_base``): rank ``rank`` holds ``[hidden, ffn/world]`` of the ``[n,k]``
    weight, the matching slice of the activation's columns, and its own per-channel scale."""
    gs = _gen(seed + 101 + rank + 16 * world)
    kr = ffn // world
    return dict(down_weight_nk=rand_int8((hidden, kr), gs), down_scale=rand_uniform((hidden,), gs, 1e-3, 1e-2))

"""CPU oracle for torch_npu's quantized-inference operator path.

TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are compared
with; nothing in the shipped package imports it.  Only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may call it.

The arithmetic of the four operators lives in the un-vendored ``op-plugin``
submodule of the reference (``.gitmodules:1-4``, no commit pinned) and, below
that, in closed aclnn kernels.  What follows therefore restates the algorithm
from the CPU golden compositions the reference keeps in its own tests:

* symmetric int8 quantisation ``scale = max/127``, ``round`` (half to even),
  ``clip(-128, 127)``: ``test/custom_ops/test_npu_ifmr.py:38-45``,
  ``test/contrib/test_linear_weight_quant.py:13-16``; rounding mode "rint":
  ``torch_npu/contrib/module/quant_conv2d.py:101``.
* int8 GEMM dequantisation ``x1_scale * x2_scale * (x1 @ x2)`` with the bias
  added to the accumulator before scaling:
  ``test/distributed/tensor/test_matrix_ops.py:28-37,93-110``.
* weight-only dequantisation ``(w + offset) * scale`` followed by an fp32
  matmul and a cast: ``test/contrib/test_linear_weight_quant.py:20-28``,
  ``test/custom_ops/test_npu_anti_quant.py:29-42``.
* int4 nibble order inside an int32 (low nibble first, sign-extended):
  ``test/custom_ops/test_npu_anti_quant.py:12-24``.

PARITY STATUS: the reference holds no known-answer vectors for
``npu_dynamic_quant`` (symmetric or asymmetric), ``npu_quant_matmul``,
``npu_convert_weight_to_int4pack`` or group-wise W4A16 -> for those ops parity is
UNPINNED.  ``npu_anti_quant`` is pinned by the reference's own golden function.  Pinned pieces: the
int4 unpack convention, the ``(w+offset)*scale`` weight-only golden and the
``x1_scale*x2_scale*(x1@x2)`` dequant golden, all three checked against the
reference's own helper functions through ``tests/golden/reference_goldens.npz``.

Every float step below is done in IEEE binary32 with numpy (one rounding per
operation, no fused multiply-add), in the order the CUDA kernels use, so that
integer outputs and fp32 scales can be compared bit for bit.
"""
from __future__ import annotations

import numpy as np
import torch

F32 = np.float32


def _to_f32(t) -> np.ndarray:
    """bf16/fp16/fp32 torch tensor (or ndarray) -> float32 ndarray, exact."""
    if isinstance(t, torch.Tensor):
        return t.detach().cpu().to(torch.float32).numpy()
    return np.asarray(t, dtype=F32)


def _cast_out(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    """float32 ndarray -> torch tensor of ``dtype`` (round to nearest even)."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=F32)).to(dtype)


# --------------------------------------------------------------------------- A1
def _smoothed(x, smooth_scales, group_index):
    """fp32 ``x * smooth``; with ``group_index`` (sorted cumulative end rows, one smooth row per
    group; rows past the last entry use the last row: ``test/onnx/test_wrapper_onnx_ops.py:1345-1354``)."""
    xs = _to_f32(x)
    if smooth_scales is None:
        return xs
    sm = _to_f32(smooth_scales)
    if group_index is None:
        return xs * sm                               # fp32 multiply, one rounding
    gi = np.asarray(group_index.detach().cpu().numpy() if isinstance(group_index, torch.Tensor) else group_index)
    flat = xs.reshape(-1, xs.shape[-1])
    g = np.minimum(np.searchsorted(gi, np.arange(flat.shape[0]), side="right"), len(gi) - 1)
    return (flat * sm[g]).reshape(xs.shape)


def dynamic_quant(x, smooth_scales=None, group_index=None):
    """``npu_dynamic_quant(input, smooth_scales=None, group_index=None)`` -> (int8 y, fp32 scale).

    Per row of the last dimension: ``xs = x * smooth`` (fp32), ``amax = max|xs|``,
    ``scale = amax / 127`` (true division), ``y = clip(rint(xs / scale), -128, 127)``.
    An all-zero row gives ``scale = 0`` and ``y = 0``.  Output contract
    (int8 of the input's shape, fp32 of ``shape[:-1]``):
    ``test/test_fake_tensor.py:1671-1686``; formula: see the module docstring.
    """
    xs = _smoothed(x, smooth_scales, group_index)
    amax = np.max(np.abs(xs), axis=-1) if xs.shape[-1] else np.zeros(xs.shape[:-1], F32)
    scale = (amax / F32(127.0)).astype(F32)
    safe = np.where(scale == 0, F32(1.0), scale)[..., None]
    with np.errstate(invalid="ignore", over="ignore"):
        q = np.rint(xs / safe)
    q = np.where(scale[..., None] == 0, F32(0.0), q)
    y = np.clip(q, -128, 127).astype(np.int8)
    return torch.from_numpy(y), torch.from_numpy(scale.astype(F32))


def dynamic_quant_asymmetric(x, smooth_scales=None, group_index=None):
    """``npu_dynamic_quant_asymmetric`` -> (int8 y, fp32 scale, fp32 offset); contract
    ``test/test_fake_tensor.py:1690-1709``.  PARITY UNPINNED: the reference tree holds the output
    contract only; the formula is the published one of the aclnn dynamic-quant operator it calls:
    per row ``scale = (max(xs) - min(xs)) / 255``, ``offset = 127 - max(xs) / scale``,
    ``y = clip(rint(xs / scale + offset), -128, 127)``, each step one fp32 rounding.  A constant
    row gives ``scale = 0``, ``offset = 0``, ``y = 0`` (this build's choice)."""
    xs = _smoothed(x, smooth_scales, group_index)
    mx = np.max(xs, axis=-1).astype(F32)
    mn = np.min(xs, axis=-1).astype(F32)
    scale = ((mx - mn).astype(F32) / F32(255.0)).astype(F32)
    zero = scale == 0
    safe = np.where(zero, F32(1.0), scale)
    offset = np.where(zero, F32(0.0), (F32(127.0) - (mx / safe).astype(F32)).astype(F32)).astype(F32)
    with np.errstate(invalid="ignore", over="ignore"):
        q = np.rint(((xs / safe[..., None]).astype(F32) + offset[..., None]).astype(F32))
    q = np.where(zero[..., None], F32(0.0), q)
    y = np.clip(q, -128, 127).astype(np.int8)
    return torch.from_numpy(y), torch.from_numpy(scale), torch.from_numpy(offset)


def swiglu_quant(x, smooth_scales=None, activate_left=True):
    """``npu_swiglu_quant`` in dynamic mode -> (int8 y, fp32 scale): ``act = silu(a) * b`` in fp32 with
    ``a, b`` the halves of the last dimension (``a`` the left one when ``activate_left``; the reference's
    ``npu_swiglu`` activates the left half: ``torch_npu/_inductor/decomposition.py:186-188``), then
    ``act * smooth`` and the per-token quantisation of :func:`dynamic_quant`.  PARITY UNPINNED: the fused
    operator is only named in the reference tree (``docs/zh/release_notes.md:303``).  ``exp`` is the
    platform's fp32 one, so a GPU result is compared with a tolerance, not bit for bit."""
    xf = _to_f32(x)
    f = xf.shape[-1] // 2
    a, b = (xf[..., :f], xf[..., f:]) if activate_left else (xf[..., f:], xf[..., :f])
    with np.errstate(over="ignore"):
        s = (F32(1.0) / (F32(1.0) + np.exp(-a).astype(F32))).astype(F32)
    act = ((a * s).astype(F32) * b).astype(F32)
    if smooth_scales is not None:
        act = (act * _to_f32(smooth_scales)).astype(F32)
    return dynamic_quant(torch.from_numpy(np.ascontiguousarray(act)))


def anti_quant(x, scale, offset=None, dst_dtype=torch.float16, src_dtype=None):
    """``npu_anti_quant(x, scale, offset=None, dst_dtype, src_dtype)``: int8, or int32 words of eight
    int4 values, to fp16/bf16: ``cast((float(x) + offset) * scale)`` with an fp32 sum and an fp32
    product (``test/custom_ops/test_npu_anti_quant.py:29-42``)."""
    if x.dtype == torch.int32:
        x = unpack_int4(x)
    xf = x.detach().cpu().numpy().astype(F32)
    sc = np.broadcast_to(_to_f32(scale), xf.shape)
    if offset is not None:
        xf = (xf + np.broadcast_to(_to_f32(offset), xf.shape)).astype(F32)
    return _cast_out((xf * sc).astype(F32), dst_dtype)


# --------------------------------------------------------------------------- A2
def int8_gemm_int32(x1: torch.Tensor, x2: torch.Tensor) -> np.ndarray:
    """Exact ``x1 @ x2`` for int8 operands, int32 result.

    Runs as a float64 GEMM: every product and partial sum is an integer below
    2**53 (|acc| <= 128*128*K), so the result is exact in any summation order.
    """
    a = x1.detach().cpu().to(torch.float64)
    b = x2.detach().cpu().to(torch.float64)
    return torch.matmul(a, b).numpy().astype(np.int64).astype(np.int32)


def quant_matmul(x1, x2, scale, *, offset=None, pertoken_scale=None, bias=None,
                 output_dtype=None):
    """``npu_quant_matmul``: int8 x int8 -> int32, fused dequantisation.

    ``acc = x1 @ x2 (+ int32 bias[n])``; int32 output returns ``acc``.  Otherwise
    ``v = float(acc) * scale[n]``, then ``* pertoken_scale[m]`` if given, then
    a floating bias is added, then ``+ offset[n]`` if given; each step one fp32
    rounding; ``v`` is cast to bf16/fp16 (nearest even) or, for int8 (the default),
    ``clip(rint(v), -128, 127)``.  Dequant order follows
    ``test/distributed/tensor/test_matrix_ops.py:28-37`` (bias before scaling);
    output dtypes ``test/test_fake_tensor.py:1884-1925``.
    """
    out_dtype = torch.int8 if output_dtype is None else output_dtype
    acc = int8_gemm_int32(x1, x2)                                   # [..., M, N]
    n = acc.shape[-1]
    fbias = None
    if bias is not None:
        if bias.dtype == torch.int32:
            acc = (acc.astype(np.int64) + bias.detach().cpu().numpy().astype(np.int64)
                   .reshape(bias.shape if bias.dim() > 1 else (n,))).astype(np.int32)
        else:
            fbias = _to_f32(bias).reshape(bias.shape if bias.dim() > 1 else (n,))
    if out_dtype == torch.int32:
        return torch.from_numpy(acc)
    if scale.dtype == torch.int64:
        sc = trans_quant_param_decode(scale)[0]
    else:
        sc = _to_f32(scale)
    v = acc.astype(F32) * sc.reshape(-1)                            # int32->fp32 RNE, then mul
    if pertoken_scale is not None:
        pt = _to_f32(pertoken_scale).reshape(-1)
        v = (v.reshape(-1, n) * pt[:, None]).reshape(acc.shape)
    if fbias is not None:
        v = v + fbias
    if offset is not None:
        v = v + _to_f32(offset).reshape(-1)
    v = v.astype(F32)
    if out_dtype == torch.int8:
        return torch.from_numpy(np.clip(np.rint(v), -128, 127).astype(np.int8))
    return _cast_out(v, out_dtype)


# --------------------------------------------------------------- collective-fused forms
def mm_reduce_scatter(x1_list, x2_list, x1_scale_list=None, x2_scale_list=None, bias_list=None,
                      output_dtype=torch.bfloat16):
    """``npu_mm_reduce_scatter_base`` (int8 form) for every rank at once: rank i holds ``x1_list[i]``
    ``[m, k_i]`` and ``x2_list[i]`` ``[k_i, n]``; returns the list of per-rank outputs ``[m/g, n]``.

    Follows ``TestMmReduceScatterBaseOp._get_global_tensor``
    (``test/distributed/tensor/test_matrix_ops.py:86-110``): each rank's product (+ its int32 bias) is
    dequantised with its own ``x1_scale [m,1]`` and ``x2_scale [1,n]``, the fp32 partials are added in rank
    order starting from zero, and the sum is cast once.  The dequantisation of one partial is
    ``quant_matmul`` above, i.e. ``(float(acc) * x2_scale[n]) * x1_scale[m]``; the golden multiplies the two
    scales first, which differs by fp32 rounding only (checked against the golden in the tests)."""
    g = len(x1_list)
    total = None
    for i in range(g):
        n = x2_list[i].shape[1]
        sc = x2_scale_list[i].reshape(-1) if x2_scale_list is not None else torch.ones(1)
        pt = x1_scale_list[i].reshape(-1) if x1_scale_list is not None else None
        part = quant_matmul(x1_list[i], x2_list[i], sc, pertoken_scale=pt,
                            bias=None if bias_list is None else bias_list[i], output_dtype=torch.float32).numpy()
        total = part.astype(F32) if total is None else (total + part).astype(F32)
    m = total.shape[0]
    if m % g:
        raise ValueError(f"m={m} is not divisible by the number of ranks {g}")
    out = _cast_out(total, output_dtype)
    return [out[r * (m // g):(r + 1) * (m // g)] for r in range(g)]


def mm_all_reduce(x1_list, x2_list, dequant_scale, pertoken_scale=None, output_dtype=None):
    """``npu_mm_all_reduce_base`` (int8 form): the rank-ordered fp32 sum of the dequantised partial
    products, the same ``[m, n]`` on every rank.  Output type: bf16 for a bf16 ``dequant_scale``, else fp16
    (``test/test_fake_tensor.py:1555-1583``)."""
    if output_dtype is None:
        output_dtype = torch.bfloat16 if dequant_scale.dtype == torch.bfloat16 else torch.float16
    total = None
    for x1, x2 in zip(x1_list, x2_list):
        part = quant_matmul(x1, x2, dequant_scale, pertoken_scale=pertoken_scale, output_dtype=torch.float32).numpy()
        total = part.astype(F32) if total is None else (total + part).astype(F32)
    return _cast_out(total, output_dtype)


def all_gather_mm(x1_list, x2_list, x1_scale_list=None, x2_scale_list=None, bias_list=None,
                  output_dtype=torch.bfloat16):
    """``npu_all_gather_base_mm`` (int8 form) for every rank at once: ``x1_list[i]`` ``[m_i, k]`` is
    gathered along rows, rank i multiplies the gathered matrix by its ``x2_list[i]`` ``[k, n_i]``.  Returns
    ``([out_i [m, n_i]], gathered x1)`` as ``TestAllGatherBaseMmOp._get_global_tensor`` defines them
    (``test/distributed/tensor/test_matrix_ops.py:21-40``): bias joins the accumulator, then
    ``x1_scale * x2_scale * acc``."""
    x1 = torch.cat(list(x1_list), dim=0)
    pt = torch.cat([s.reshape(-1) for s in x1_scale_list]) if x1_scale_list is not None else None
    outs = []
    for i, x2 in enumerate(x2_list):
        sc = x2_scale_list[i].reshape(-1) if x2_scale_list is not None else torch.ones(1)
        outs.append(quant_matmul(x1, x2, sc, pertoken_scale=pt, bias=None if bias_list is None else bias_list[i],
                                 output_dtype=output_dtype))
    return outs, x1


def trans_quant_param(scale, offset=None):
    """``npu_trans_quant_param(scale, offset=None)`` -> int64 dequant parameter.

    Shape/dtype contract: ``test/test_fake_tensor.py:1929-1943`` (result has the
    broadcast shape of scale and offset, dtype int64).  The bit layout is not
    present in the reference tree; the layout used here keeps the fp32 bit
    pattern of ``scale`` in bits [0,32) and leaves the upper word zero.  The
    offset stays a separate fp32 argument of ``npu_quant_matmul`` (that is how
    ``torch_npu/contrib/module/linear_quant.py:110-112`` passes it), so it only
    contributes its shape.
    """
    s = _to_f32(scale)
    shape = s.shape
    if offset is not None:
        shape = np.broadcast_shapes(s.shape, tuple(offset.shape))
    bits = np.broadcast_to(s, shape).astype(F32).view(np.uint32).astype(np.int64)
    return torch.from_numpy(np.ascontiguousarray(bits))


def trans_quant_param_decode(param):
    bits = param.detach().cpu().numpy().astype(np.int64)
    lo = (bits & 0xFFFFFFFF).astype(np.uint32)
    return np.ascontiguousarray(lo).view(F32).reshape(-1), None


# --------------------------------------------------------------------------- A4
def convert_weight_to_int4pack(w: torch.Tensor) -> torch.Tensor:
    """Pack int4 values (one per int32 element, range [-8, 7]) eight per int32
    along the last dimension; element ``j`` of each group of eight occupies bits
    ``[4j, 4j+4)``.  Inverse of ``unpack_int4`` below."""
    a = w.detach().cpu().numpy().astype(np.int64)
    if a.shape[-1] % 8:
        raise ValueError("last dimension must be a multiple of 8")
    if a.min(initial=0) < -8 or a.max(initial=0) > 7:
        raise ValueError("int4 values must lie in [-8, 7]")
    g = (a & 0xF).reshape(*a.shape[:-1], a.shape[-1] // 8, 8)
    packed = np.zeros(g.shape[:-1], dtype=np.int64)
    for j in range(8):
        packed |= g[..., j] << (4 * j)
    return torch.from_numpy(packed.astype(np.uint32).view(np.int32).reshape(g.shape[:-1]))


def unpack_int4(p: torch.Tensor) -> torch.Tensor:
    """int32 [..., N/8] -> int8 [..., N]: bytes in memory order, low nibble first,
    nibbles sign-extended (``test/custom_ops/test_npu_anti_quant.py:12-24``)."""
    a = np.ascontiguousarray(p.detach().cpu().numpy().astype(np.int32))
    b = a.view(np.uint8).reshape(*a.shape, 4)
    lo = (b & 0xF).astype(np.int8)
    hi = (b >> 4).astype(np.int8)
    nib = np.stack([lo, hi], axis=-1).reshape(*a.shape[:-1], a.shape[-1] * 8)
    return torch.from_numpy(np.where(nib > 7, nib - 16, nib).astype(np.int8))


# --------------------------------------------------------------------------- A3
def dequant_weight(weight, antiquant_scale, antiquant_offset=None, antiquant_group_size=0,
                   dequant_dtype=None):
    """``(w + offset) * scale`` of an int8 ``[K,N]`` or int4-packed int32 ``[K,N/8]`` weight, returned
    as fp32.  Scale/offset are per channel (``[N]`` / ``[1,N]``) or per group of
    ``antiquant_group_size`` rows of K (``[K/gs, N]``).

    ``dequant_dtype`` is the type the two steps are carried out in.  The reference's golden for the
    weight-only matmul works on the tensors it is given, i.e. in fp16/bf16: the sum ``w + offset`` is
    rounded to that type, then the product with ``scale`` is rounded again, and only then is the
    result widened for the fp32 matmul (``test/contrib/test_linear_weight_quant.py:21-26``).  Passing
    the activation dtype reproduces that; ``None`` keeps both steps in fp32 (the order used by
    ``test/custom_ops/test_npu_anti_quant.py:36-41``)."""
    w = unpack_int4(weight) if weight.dtype == torch.int32 else weight.detach().cpu()
    k, n = w.shape[-2], w.shape[-1]

    def expand(p, dt):
        a = p.detach().cpu().to(dt)
        if a.dim() == 2 and a.shape[0] > 1:
            gs = antiquant_group_size if antiquant_group_size > 0 else k // a.shape[0]
            a = a.repeat_interleave(gs, dim=0)[:k]
        return a.reshape(-1, n)

    dt = torch.float32 if dequant_dtype is None else dequant_dtype
    wl = w.to(dt)
    if antiquant_offset is not None:
        wl = wl + expand(antiquant_offset, dt)
    wl = wl * expand(antiquant_scale, dt)
    return wl.to(torch.float32).numpy()


def weight_quant_batchmatmul(x, weight, antiquant_scale, antiquant_offset=None,
                             quant_scale=None, quant_offset=None, bias=None,
                             antiquant_group_size=0, inner_precise=0, dequant_dtype="x"):
    """``npu_weight_quant_batchmatmul``: ``x @ ((w + offset) * scale) (+ bias)``, result in ``x.dtype``.

    Follows the reference's golden, ``test/contrib/test_linear_weight_quant.py:20-28``: the weight is
    dequantised in the activation dtype (``dequant_dtype="x"``, see ``dequant_weight``), widened to
    fp32, multiplied and cast.  The product is accumulated in float64 and rounded once to fp32 so
    that the value does not depend on the host's summation order.  ``dequant_dtype=None`` gives the
    all-fp32 dequantisation instead."""
    if quant_scale is not None or quant_offset is not None or inner_precise != 0:
        raise NotImplementedError("requantised output / inner_precise are outside the path")
    if isinstance(dequant_dtype, str):
        dequant_dtype = x.dtype
    wd = dequant_weight(weight, antiquant_scale, antiquant_offset, antiquant_group_size, dequant_dtype)
    xf = x.detach().cpu().to(torch.float64)
    out = torch.matmul(xf, torch.from_numpy(wd).to(torch.float64)).to(torch.float32).numpy()
    if bias is not None:
        out = out + _to_f32(bias).reshape(-1)
    return _cast_out(out, x.dtype)


# ------------------------------------------------------------------ comparison
def max_mixed_error(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """Largest per-element ``min(|d|, |d| / max(|a|, |e|))``: the atol-OR-rtol rule of
    ``torch_npu/testing/testcase.py:161-175`` expressed as one number, to be held
    against a single bound (2**-7 for bf16/fp16 outputs)."""
    a = actual.detach().cpu().to(torch.float64)
    e = expected.detach().cpu().to(torch.float64)
    d = (a - e).abs()
    den = torch.maximum(a.abs(), e.abs()).clamp_min(1e-30)
    return float(torch.minimum(d, d / den).max()) if d.numel() else 0.0


def count_outside(actual, expected, prec: float, floor: float = 6e-8):
    """Element counts failing the absolute and the relative criterion of the
    reference's ``assertRtolEqual`` (``torch_npu/testing/testcase.py:161-175``): that
    helper fails only when BOTH counts exceed ``size * prec``."""
    a = actual.detach().cpu().to(torch.float64).numpy()
    e = expected.detach().cpu().to(torch.float64).numpy()
    d = np.abs(a - e)
    den = np.maximum(np.abs(a), np.abs(e)) + floor
    return int((d > prec).sum()), int((d / den > prec).sum())

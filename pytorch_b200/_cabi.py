"""ctypes binding of ``include/b200q.h``.

This is the same boundary a binding in any other host language would use: plain device
pointers, sizes and enums.  The helpers below take torch CUDA tensors only to obtain those
pointers (``data_ptr()``) and the current stream; they allocate outputs and workspace with
torch and pass them down.  There is no CPU path: loading fails loudly when the library has
not been built, and every compute call needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libb200q.so")

OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_LAUNCH, ERR_WORKSPACE, ERR_DEVICE = range(6)
BF16, F16, F32, I8, I32, I64, NONE = 0, 1, 2, 3, 4, 5, -1
DTYPE = {torch.bfloat16: BF16, torch.float16: F16, torch.float32: F32, torch.int8: I8,
         torch.int32: I32, torch.int64: I64}

EXPORTS = (
    "b200q_version", "b200q_last_error", "b200q_status_string", "b200q_device_error",
    "b200q_dynamic_quant", "b200q_quant_matmul_workspace_bytes", "b200q_quant_matmul",
    "b200q_static_scratch_bytes", "b200q_quant_matmul_static_scratch",
    "b200q_weight_quant_matmul_workspace_bytes", "b200q_weight_quant_matmul", "b200q_int4pack",
    "b200q_trans_quant_param", "b200q_scatter_columns", "b200q_dynamic_quant_ext", "b200q_anti_quant",
    "b200q_swiglu_quant", "b200q_enable_host_error_word", "b200q_peek_device_error", "b200q_selftest_expire_wait",
    "b200q_peer_barrier", "b200q_reduce_slots", "b200q_copy_columns",
)


class QuantMatmulArgs(C.Structure):
    _fields_ = [
        ("x1", C.c_void_p), ("x2", C.c_void_p),
        ("m", C.c_int64), ("k", C.c_int64), ("n", C.c_int64),
        ("x2_stride_k", C.c_int64), ("x2_stride_n", C.c_int64),
        ("scale", C.c_void_p), ("scale_dtype", C.c_int), ("scale_len", C.c_int64),
        ("offset", C.c_void_p), ("offset_len", C.c_int64),
        ("pertoken_scale", C.c_void_p),
        ("bias", C.c_void_p), ("bias_dtype", C.c_int),
        ("out", C.c_void_p), ("out_dtype", C.c_int),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("out_row_stride", C.c_int64),
        ("peer_out", C.POINTER(C.c_void_p)), ("n_peer_out", C.c_int), ("route_rows", C.c_int64),
    ]


class WeightQuantMatmulArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("x_dtype", C.c_int),
        ("weight", C.c_void_p), ("weight_bits", C.c_int),
        ("m", C.c_int64), ("k", C.c_int64), ("n", C.c_int64),
        ("w_stride_k", C.c_int64), ("w_stride_n", C.c_int64),
        ("antiquant_scale", C.c_void_p), ("antiquant_offset", C.c_void_p),
        ("group_size", C.c_int64),
        ("bias", C.c_void_p),
        ("out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class B200QError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"b200q status {status}: {message}")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """Loads ``lib/libb200q.so`` (raises if it has not been built)."""
    global _lib
    if _lib is None:
        path = os.environ.get("B200Q_LIB", _LIB_PATH)      # override: a differently built libb200q.so
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: run `python pytorch_b200/_build.py` "
                              "(there is no fallback implementation)")
        l = C.CDLL(path)
        l.b200q_version.restype = C.c_int
        l.b200q_last_error.restype = C.c_char_p
        l.b200q_status_string.restype = C.c_char_p
        l.b200q_status_string.argtypes = [C.c_int]
        l.b200q_device_error.argtypes = [C.POINTER(C.c_uint), C.c_int]
        l.b200q_dynamic_quant.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                          C.c_int64, C.c_int64, C.c_void_p]
        l.b200q_quant_matmul_workspace_bytes.restype = C.c_size_t
        l.b200q_quant_matmul_workspace_bytes.argtypes = [C.c_int64] * 5
        l.b200q_quant_matmul.argtypes = [C.POINTER(QuantMatmulArgs), C.c_void_p]
        l.b200q_static_scratch_bytes.restype = C.c_size_t
        l.b200q_quant_matmul_static_scratch.argtypes = [C.POINTER(QuantMatmulArgs), C.c_void_p]
        l.b200q_weight_quant_matmul_workspace_bytes.restype = C.c_size_t
        l.b200q_weight_quant_matmul_workspace_bytes.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.c_int]
        l.b200q_weight_quant_matmul.argtypes = [C.POINTER(WeightQuantMatmulArgs), C.c_void_p]
        l.b200q_int4pack.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        l.b200q_trans_quant_param.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p]
        l.b200q_dynamic_quant_ext.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int64,
                                              C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        l.b200q_swiglu_quant.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                         C.c_int64, C.c_int64, C.c_void_p]
        l.b200q_anti_quant.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                       C.c_int64, C.c_int64, C.c_void_p]
        l.b200q_peek_device_error.restype = C.c_uint
        l.b200q_selftest_expire_wait.argtypes = [C.c_uint64, C.c_void_p]
        l.b200q_peer_barrier.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_uint32, C.c_uint64, C.c_void_p]
        l.b200q_reduce_slots.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_int,
                                         C.POINTER(C.c_void_p), C.c_int, C.c_void_p]
        l.b200q_scatter_columns.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int64, C.c_int64, C.c_int64,
                                            C.c_int64, C.c_void_p]
        l.b200q_copy_columns.argtypes = l.b200q_scatter_columns.argtypes
        _lib = l
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise B200QError(status, lib().b200q_last_error().decode() or
                         lib().b200q_status_string(status).decode())


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise B200QError(ERR_BAD_ARG, "tensors must live on a CUDA device (there is no CPU path)")


def device_error(reset: bool = True) -> int:
    code = C.c_uint(0)
    lib().b200q_device_error(C.byref(code), int(reset))
    return code.value


def dynamic_quant(x: torch.Tensor, smooth_scales: torch.Tensor | None = None):
    _need_cuda(x, smooth_scales)
    x = x.contiguous()
    k = x.shape[-1]
    rows = x.numel() // k if k else (x.numel() if x.dim() == 0 else int(torch.Size(x.shape[:-1]).numel()))
    y = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scale = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    sm = None if smooth_scales is None else smooth_scales.contiguous()
    check(lib().b200q_dynamic_quant(_ptr(x), DTYPE[x.dtype], _ptr(sm), NONE if sm is None else DTYPE[sm.dtype],
                                    _ptr(y), _ptr(scale), rows, k, _stream()))
    return y, scale


def dynamic_quant_ext(x: torch.Tensor, smooth_scales: torch.Tensor | None = None,
                      group_index: torch.Tensor | None = None, asymmetric: bool = False):
    """``b200q_dynamic_quant_ext``: per-group smooth scales and/or the asymmetric variant.
    Returns (y, scale) or, with ``asymmetric``, (y, scale, offset)."""
    _need_cuda(x, smooth_scales, group_index)
    x = x.contiguous()
    k = x.shape[-1]
    rows = x.numel() // k if k else int(torch.Size(x.shape[:-1]).numel())
    y = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scale = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    offset = torch.empty_like(scale) if asymmetric else None
    sm = None if smooth_scales is None else smooth_scales.contiguous()
    gi = None if group_index is None else group_index.to(torch.int32).contiguous()
    check(lib().b200q_dynamic_quant_ext(_ptr(x), DTYPE[x.dtype], _ptr(sm), NONE if sm is None else DTYPE[sm.dtype],
                                        _ptr(gi), 0 if gi is None else gi.numel(), _ptr(y), _ptr(scale), _ptr(offset),
                                        rows, k, _stream()))
    return (y, scale, offset) if asymmetric else (y, scale)


def swiglu_quant(x: torch.Tensor, smooth_scales: torch.Tensor | None = None, activate_left: bool = True):
    """``b200q_swiglu_quant``: silu(a) * b of the two halves of the last dimension, then per-token int8."""
    _need_cuda(x, smooth_scales)
    x = x.contiguous()
    f = x.shape[-1] // 2
    rows = x.numel() // (2 * f) if f else int(torch.Size(x.shape[:-1]).numel())
    y = torch.empty((*x.shape[:-1], f), dtype=torch.int8, device=x.device)
    scale = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    sm = None if smooth_scales is None else smooth_scales.contiguous()
    check(lib().b200q_swiglu_quant(_ptr(x), DTYPE[x.dtype], _ptr(sm), NONE if sm is None else DTYPE[sm.dtype],
                                   int(activate_left), _ptr(y), _ptr(scale), rows, f, _stream()))
    return y, scale


def anti_quant(x: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor | None = None,
               dst_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """``b200q_anti_quant``: int8, or int32 words of eight int4 values, to fp16/bf16."""
    _need_cuda(x, scale, offset)
    x = x.contiguous()
    bits = 4 if x.dtype == torch.int32 else 8
    n = x.shape[-1] * (8 if bits == 4 else 1)
    out = torch.empty((*x.shape[:-1], n), dtype=dst_dtype, device=x.device)
    rows = out.numel() // n if n else 0
    sc = scale.contiguous()
    of = None if offset is None else offset.contiguous()
    check(lib().b200q_anti_quant(_ptr(x), bits, _ptr(sc), _ptr(of), DTYPE[sc.dtype], _ptr(out), DTYPE[dst_dtype],
                                 rows, n, _stream()))
    return out


def quant_matmul(x1, x2, scale, *, offset=None, pertoken_scale=None, bias=None, output_dtype=None,
                 workspace: torch.Tensor | None = None, out: torch.Tensor | None = None,
                 static_scratch: bool = False, peer_out=None, route_rows: int = 0, out_row_stride: int = 0):
    """2-D ``x2`` only (any strides); leading dimensions of ``x1`` are folded into m.

    ``peer_out`` (device addresses) with ``route_rows == 0``: the epilogue also stores the block at each
    of those addresses (the same block inside the peers' matrices).  With ``route_rows > 0`` row r goes to
    row ``r % route_rows`` of ``peer_out[r // route_rows]`` and ``out`` is not written (returns None).

    ``static_scratch=True`` goes through ``b200q_quant_matmul_static_scratch``: no workspace is
    allocated or passed; the library's built-in scratch array is used instead (``out`` should then be
    supplied by a caller that truly cannot allocate)."""
    _need_cuda(x1, x2, scale, offset, pertoken_scale, bias)
    out_dtype = torch.int8 if output_dtype is None else output_dtype
    x1c = x1.contiguous()
    k, n = x2.shape
    m = x1c.numel() // k if k else int(torch.Size(x1c.shape[:-1]).numel())
    if out is None and not route_rows:
        out = torch.empty((*x1c.shape[:-1], n), dtype=out_dtype, device=x1.device)
    need = lib().b200q_quant_matmul_workspace_bytes(m, k, n, x2.stride(0), x2.stride(1))
    if workspace is None and need and not static_scratch:
        workspace = torch.empty(need, dtype=torch.uint8, device=x1.device)
    a = QuantMatmulArgs()
    a.x1, a.x2 = x1c.data_ptr(), x2.data_ptr()
    a.m, a.k, a.n = m, k, n
    a.x2_stride_k, a.x2_stride_n = x2.stride(0), x2.stride(1)
    sc = scale.contiguous()
    a.scale, a.scale_dtype, a.scale_len = sc.data_ptr(), DTYPE.get(sc.dtype, 99), sc.numel()
    keep = [sc]
    if offset is not None:
        of = offset.contiguous(); keep.append(of)
        a.offset, a.offset_len = of.data_ptr(), of.numel()
    if pertoken_scale is not None:
        pt = pertoken_scale.contiguous(); keep.append(pt)
        a.pertoken_scale = pt.data_ptr()
    a.bias_dtype = NONE
    if bias is not None:
        b = bias.contiguous(); keep.append(b)
        a.bias, a.bias_dtype = b.data_ptr(), DTYPE.get(b.dtype, 99)
    a.out, a.out_dtype = (None if out is None else out.data_ptr()), DTYPE.get(out_dtype, 99)
    if out is not None and out.dim() >= 2 and out.stride(-1) == 1 and out.stride(-2) != n and m > 1:
        a.out_row_stride = out.stride(-2)      # a column slice of a wider matrix
    if out_row_stride:
        a.out_row_stride = out_row_stride
    if peer_out is not None:
        arr = (C.c_void_p * max(len(peer_out), 1))(*[C.c_void_p(int(p)) for p in peer_out])
        keep.append(arr)
        a.peer_out, a.n_peer_out, a.route_rows = arr, len(peer_out), route_rows
    if static_scratch:
        check(lib().b200q_quant_matmul_static_scratch(C.byref(a), _stream()))
        return out
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    check(lib().b200q_quant_matmul(C.byref(a), _stream()))
    return out


def weight_quant_matmul(x, weight, antiquant_scale, antiquant_offset=None, *, bias=None,
                        antiquant_group_size=0, workspace=None):
    _need_cuda(x, weight, antiquant_scale, antiquant_offset, bias)
    xc = x.contiguous()
    k = xc.shape[-1]
    m = xc.numel() // k
    a = WeightQuantMatmulArgs()
    if weight.dtype == torch.int32:
        w = weight.contiguous()
        n = w.shape[-1] * 8
        a.weight_bits, a.w_stride_k, a.w_stride_n = 4, 0, 0
    else:
        w = weight
        n = w.shape[-1]
        a.weight_bits, a.w_stride_k, a.w_stride_n = 8, w.stride(0), w.stride(1)
    out = torch.empty((*xc.shape[:-1], n), dtype=x.dtype, device=x.device)
    sc = antiquant_scale.contiguous()
    of = None if antiquant_offset is None else antiquant_offset.contiguous()
    b = None if bias is None else bias.contiguous()
    need = lib().b200q_weight_quant_matmul_workspace_bytes(m, k, n, a.weight_bits)
    if workspace is None and need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    a.x, a.x_dtype, a.weight = xc.data_ptr(), DTYPE.get(x.dtype, 99), w.data_ptr()
    a.m, a.k, a.n = m, k, n
    a.antiquant_scale = sc.data_ptr()
    a.antiquant_offset = None if of is None else of.data_ptr()
    a.group_size = antiquant_group_size
    a.bias = None if b is None else b.data_ptr()
    a.out = out.data_ptr()
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    check(lib().b200q_weight_quant_matmul(C.byref(a), _stream()))
    return out


def int4pack(w: torch.Tensor) -> torch.Tensor:
    _need_cuda(w)
    wc = w.contiguous()
    cols = wc.shape[-1]
    rows = wc.numel() // cols if cols else 0
    if cols % 8:
        raise B200QError(ERR_BAD_ARG, f"int4pack: last dimension ({cols}) must be a multiple of 8")
    out = torch.empty((*wc.shape[:-1], cols // 8), dtype=torch.int32, device=w.device)
    check(lib().b200q_int4pack(_ptr(wc), _ptr(out), rows, cols, _stream()))
    return out


def trans_quant_param(scale: torch.Tensor, out_shape) -> torch.Tensor:
    _need_cuda(scale)
    sc = scale.contiguous().to(torch.float32)
    out = torch.empty(tuple(out_shape), dtype=torch.int64, device=scale.device)
    check(lib().b200q_trans_quant_param(_ptr(sc), sc.numel(), _ptr(out), out.numel(), _stream()))
    return out


def scatter_columns(full: torch.Tensor, peer_ptrs, col_lo: int, col_hi: int) -> None:
    """Pushes columns [col_lo, col_hi) of the local row-major matrix ``full`` to the same place in the
    matrices at the device addresses ``peer_ptrs`` (peers' copies of ``full``, mapped for peer access)."""
    _need_cuda(full)
    if full.dim() != 2 or not full.is_contiguous():
        raise B200QError(ERR_BAD_ARG, "scatter_columns: a contiguous 2-D matrix is required")
    es = full.element_size()
    arr = (C.c_void_p * max(len(peer_ptrs), 1))(*[C.c_void_p(int(p)) for p in peer_ptrs])
    check(lib().b200q_scatter_columns(_ptr(full), arr, len(peer_ptrs), full.shape[0], full.shape[1] * es,
                                      col_lo * es, (col_hi - col_lo) * es, _stream()))


def copy_columns(full: torch.Tensor, peer_ptrs, col_lo: int, col_hi: int) -> None:
    """``b200q_copy_columns``: the push of :func:`scatter_columns` as one copy-engine transfer per peer,
    queued on the current stream."""
    _need_cuda(full)
    if full.dim() != 2 or not full.is_contiguous():
        raise B200QError(ERR_BAD_ARG, "copy_columns: a contiguous 2-D matrix is required")
    es = full.element_size()
    arr = (C.c_void_p * max(len(peer_ptrs), 1))(*[C.c_void_p(int(p)) for p in peer_ptrs])
    check(lib().b200q_copy_columns(_ptr(full), arr, len(peer_ptrs), full.shape[0], full.shape[1] * es,
                                   col_lo * es, (col_hi - col_lo) * es, _stream()))


def reduce_slots(slots: torch.Tensor, out: torch.Tensor, peer_out=()) -> torch.Tensor:
    """``b200q_reduce_slots``: ``out = cast(slots[0] + slots[1] + ...)`` (fp32 adds in slot order); the result
    is also stored at the device addresses ``peer_out`` (the same rows in the peers' matrices)."""
    _need_cuda(slots, out)
    if slots.dtype != torch.float32 or not slots.is_contiguous() or not out.is_contiguous():
        raise B200QError(ERR_BAD_ARG, "reduce_slots: contiguous fp32 slots and a contiguous output are required")
    n_slots, rows, n = slots.shape
    arr = (C.c_void_p * max(len(peer_out), 1))(*[C.c_void_p(int(p)) for p in peer_out])
    check(lib().b200q_reduce_slots(_ptr(slots), n_slots, rows, n, _ptr(out), DTYPE.get(out.dtype, 99), arr,
                                   len(peer_out), _stream()))
    return out


def peer_barrier(flag_ptrs, rank: int, epoch: int, timeout_ns: int = 0) -> None:
    """``b200q_peer_barrier`` over the flag arrays at the device addresses ``flag_ptrs`` (one per rank)."""
    arr = (C.c_void_p * len(flag_ptrs))(*[C.c_void_p(int(p)) for p in flag_ptrs])
    check(lib().b200q_peer_barrier(arr, len(flag_ptrs), rank, epoch & 0xFFFFFFFF, timeout_ns, _stream()))


def selftest_expire_wait(limit_ns: int) -> None:
    check(lib().b200q_selftest_expire_wait(limit_ns, _stream()))

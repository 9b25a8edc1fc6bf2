"""Collective-fused quantised matmuls under the reference's operator names.

``npu_mm_reduce_scatter_base``, ``npu_all_gather_base_mm`` and ``npu_mm_all_reduce_base`` are the
reference's tensor-parallel building blocks (schemas: ``torch_npu/distributed/tensor/_matrix_ops.py:471-476,
556-561``; ``torch_npu/onnx/wrapper_onnx_ops.py:723-737``; goldens ``test/distributed/tensor/test_matrix_ops.py:21-40,
86-110,204-247``; meta contracts ``test/test_fake_tensor.py:1555-1583``).  Only their int8 (quantised) forms lie
on this path and are implemented; floating-point operands are rejected.

How they run here, one process per GPU of an NVLink node:

* reduce-scatter: the W8A8 GEMM's epilogue stores each fp32 partial row block straight into the staging
  slot of the rank that owns those rows (``route_rows`` of the C ABI: plain 128-bit stores to peer-mapped
  memory, overlapped with the main loop), one bounded barrier, then ``b200q_reduce_slots`` adds the
  ``world`` partials in rank order in fp32 - the order of the reference's golden - and casts once.
* all-reduce: the same, and the reducing kernel also stores its rows into every peer's result matrix.
* all-gather + matmul: the rows of ``x1`` (and of ``x1_scale``) are pushed to the peers, barrier, GEMM.

``hcom`` is the name of a ``torch.distributed`` process group (``hcom_name(group)``), the counterpart of
the HCCL communicator name the reference passes.  Buffers in peer-mapped memory are created per group on
first use and reused (two of each, alternating, so that a call never overwrites what a slower peer is
still reading from the call before).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _cabi
from .sharded import PeerGroup

_LIB = torch.library.Library("npu", "FRAGMENT")
_LIB.define("npu_mm_reduce_scatter_base(Tensor self, Tensor x2, str hcom, int world_size, *, str reduce_op='sum', "
            "Tensor? bias=None, Tensor? x1_scale=None, Tensor? x2_scale=None, int comm_turn=0, "
            "ScalarType? output_dtype=None, str? comm_mode=None) -> Tensor")
_LIB.define("npu_all_gather_base_mm(Tensor self, Tensor x2, str hcom, int world_size, *, Tensor? bias=None, "
            "Tensor? x1_scale=None, Tensor? x2_scale=None, int gather_index=0, bool gather_output=True, "
            "int comm_turn=0, ScalarType? output_dtype=None, str? comm_mode=None) -> (Tensor, Tensor)")
_LIB.define("npu_mm_all_reduce_base(Tensor x1, Tensor x2, str hcom, *, str reduce_op='sum', Tensor? bias=None, "
            "Tensor? antiquant_scale=None, Tensor? antiquant_offset=None, Tensor? x3=None, Tensor? dequant_scale=None, "
            "Tensor? pertoken_scale=None, Tensor? comm_quant_scale_1=None, Tensor? comm_quant_scale_2=None, "
            "int antiquant_group_size=0, int comm_turn=0) -> Tensor")


def hcom_name(group=None) -> str:
    """The string to pass as ``hcom``: the process group's registered name."""
    g = dist.group.WORLD if group is None else group
    return g.group_name


class _Context:
    """Per process group: the peer group (barrier, symmetric allocation) and named alternating buffers."""

    def __init__(self, group, device):
        self.peers = PeerGroup(device, group)
        self.buffers = {}

    def buffer(self, name: str, nbytes: int):
        """The next of the two peer-mapped byte buffers called ``name`` (grown, collectively, when too
        small): ``(uint8 tensor, [address of every rank's copy])``."""
        ent = self.buffers.get(name)
        if ent is None or ent["size"] < nbytes:
            size = max(1 << 20, 1 << (nbytes - 1).bit_length())
            if ent is not None:
                self.peers.barrier()                  # nobody still writes into the buffers being replaced
                torch.cuda.synchronize()
            ent = {"size": size, "cur": 0, "bufs": [self.peers.symmetric((size,), torch.uint8)[:2] for _ in range(2)]}
            self.buffers[name] = ent
        ent["cur"] ^= 1
        return ent["bufs"][ent["cur"]]


_contexts: dict[str, _Context] = {}


def _context(hcom: str, device) -> _Context:
    ctx = _contexts.get(hcom)
    if ctx is None:
        if not dist.is_initialized():
            raise RuntimeError("collective-fused operators need an initialised torch.distributed process group")
        try:
            group = dist.distributed_c10d._resolve_process_group(hcom)
        except Exception as exc:                      # noqa: BLE001
            raise RuntimeError(f"hcom '{hcom}' is not the name of a process group (use hcom_name(group))") from exc
        ctx = _contexts[hcom] = _Context(group, device)
    return ctx


def release_contexts() -> None:
    """Drops every cached peer-mapped buffer (call before destroying the process group)."""
    _contexts.clear()


def _require_int8(op, x1, x2):
    if x1.dtype != torch.int8 or x2.dtype != torch.int8:
        raise NotImplementedError(f"{op}: only the int8 (quantised) form is implemented, got {x1.dtype} and {x2.dtype}")
    if x1.dim() != 2 or x2.dim() != 2 or x1.shape[1] != x2.shape[0]:
        raise ValueError(f"{op}: x1 [m,k] and x2 [k,n] expected, got {tuple(x1.shape)} and {tuple(x2.shape)}")


def _flat_scale(t, length, name, op):
    if t is None:
        return None
    if t.dtype != torch.float32 or t.numel() != length:
        raise ValueError(f"{op}: {name} must be float32 with {length} elements, got {t.dtype} {tuple(t.shape)}")
    return t.reshape(-1).contiguous()


def _routed_partials(ctx, name, x1, x2, x2_scale, x1_scale, bias):
    """Runs the GEMM whose epilogue sends row block d of the fp32 partial product to rank d's staging slot
    for this rank; returns this rank's staging area as ``[world, m/world, n]`` after the barrier."""
    g, r = ctx.peers.world, ctx.peers.rank
    m, n = x1.shape[0], x2.shape[1]
    rows = m // g
    nbytes = g * rows * n * 4
    stage, ptrs = ctx.buffer(name, nbytes)
    dest = [int(ptrs[d]) + r * rows * n * 4 for d in range(g)]
    scale = x2_scale if x2_scale is not None else torch.ones(1, dtype=torch.float32, device=x1.device)
    _cabi.quant_matmul(x1, x2, scale, pertoken_scale=x1_scale, bias=bias, output_dtype=torch.float32,
                       peer_out=dest, route_rows=rows, out_row_stride=n)
    ctx.peers.barrier()
    return stage[:nbytes].view(torch.float32).view(g, rows, n)


def _mm_reduce_scatter(x1, x2, hcom, world_size, reduce_op="sum", bias=None, x1_scale=None, x2_scale=None,
                       comm_turn=0, output_dtype=None, comm_mode=None):
    op = "npu_mm_reduce_scatter_base"
    _require_int8(op, x1, x2)
    if reduce_op != "sum":
        raise NotImplementedError(f"{op} only support reduce_op='sum' now, but got {reduce_op}.")
    ctx = _context(hcom, x1.device)
    g = ctx.peers.world
    m, n = x1.shape[0], x2.shape[1]
    if world_size != g:
        raise ValueError(f"{op}: world_size {world_size} differs from the group's {g}")
    if m % g:
        raise ValueError(f"{op}: m={m} must be divisible by the world size {g}")
    if bias is not None and bias.dtype != torch.int32:
        raise NotImplementedError(f"{op}: with int8 operands the bias must be int32")
    slots = _routed_partials(ctx, "reduce_scatter", x1.contiguous(), x2, _flat_scale(x2_scale, n, "x2_scale", op),
                             _flat_scale(x1_scale, m, "x1_scale", op), bias)
    out = torch.empty((m // g, n), dtype=output_dtype or torch.bfloat16, device=x1.device)
    return _cabi.reduce_slots(slots, out)


def _mm_all_reduce(x1, x2, hcom, reduce_op="sum", bias=None, antiquant_scale=None, antiquant_offset=None, x3=None,
                   dequant_scale=None, pertoken_scale=None, comm_quant_scale_1=None, comm_quant_scale_2=None,
                   antiquant_group_size=0, comm_turn=0):
    op = "npu_mm_all_reduce_base"
    _require_int8(op, x1, x2)
    if reduce_op != "sum":
        raise NotImplementedError(f"{op} only support reduce_op='sum' now, but got {reduce_op}.")
    for name, t in (("antiquant_scale", antiquant_scale), ("antiquant_offset", antiquant_offset), ("x3", x3),
                    ("comm_quant_scale_1", comm_quant_scale_1), ("comm_quant_scale_2", comm_quant_scale_2), ("bias", bias)):
        if t is not None:
            raise NotImplementedError(f"{op}: {name} is not supported")
    if dequant_scale is None:
        raise ValueError(f"{op}: int8 operands need dequant_scale")
    ctx = _context(hcom, x1.device)
    g, r = ctx.peers.world, ctx.peers.rank
    m, n = x1.shape[0], x2.shape[1]
    if m % g:
        raise ValueError(f"{op}: m={m} must be divisible by the world size {g}")
    out_dtype = torch.bfloat16 if dequant_scale.dtype == torch.bfloat16 else torch.float16
    pt = _flat_scale(pertoken_scale, m, "pertoken_scale", op)
    if dequant_scale.numel() not in (1, n):
        raise ValueError(f"{op}: dequant_scale must have 1 or n={n} elements")
    x1c = x1.contiguous()
    gs, rk = g, r
    rows = m // gs
    nbytes = gs * rows * n * 4
    stage, ptrs = ctx.buffer("all_reduce", nbytes)
    dest = [int(ptrs[d]) + rk * rows * n * 4 for d in range(gs)]
    _cabi.quant_matmul(x1c, x2, dequant_scale.reshape(-1).contiguous(), pertoken_scale=pt, output_dtype=torch.float32,
                       peer_out=dest, route_rows=rows, out_row_stride=n)
    ctx.peers.barrier()
    slots = stage[:nbytes].view(torch.float32).view(gs, rows, n)
    es = torch.empty((), dtype=out_dtype).element_size()
    full, fptrs = ctx.buffer("all_reduce_out", m * n * es)
    mine = full[:m * n * es].view(out_dtype).view(m, n)[rk * rows:(rk + 1) * rows]
    _cabi.reduce_slots(slots, mine, ctx.peers.peers_after(fptrs, rk * rows * n * es))
    ctx.peers.barrier()
    return full[:m * n * es].view(out_dtype).view(m, n).clone()


def _all_gather_mm(x1, x2, hcom, world_size, bias=None, x1_scale=None, x2_scale=None, gather_index=0,
                   gather_output=True, comm_turn=0, output_dtype=None, comm_mode=None):
    op = "npu_all_gather_base_mm"
    _require_int8(op, x1, x2)
    if gather_index != 0:
        raise NotImplementedError(f"{op} only support gather_index=0 now, but got {gather_index}.")
    ctx = _context(hcom, x1.device)
    g, r = ctx.peers.world, ctx.peers.rank
    if world_size != g:
        raise ValueError(f"{op}: world_size {world_size} differs from the group's {g}")
    mr, k = x1.shape
    n = x2.shape[1]
    if (mr * k) % 16 or (x1_scale is not None and mr % 4):
        raise NotImplementedError(f"{op}: the local block of x1 must be a multiple of 16 bytes (and m of 4 with x1_scale)")
    if bias is not None and bias.dtype != torch.int32:
        raise NotImplementedError(f"{op}: with int8 operands the bias must be int32")
    s1 = _flat_scale(x1_scale, mr, "x1_scale", op)
    nb_x, nb_s = g * mr * k, g * mr * 4
    buf, ptrs = ctx.buffer("all_gather", nb_x + nb_s)           # [g*mr*k int8 | g*mr fp32]
    gathered = buf[:nb_x].view(torch.int8).view(g * mr, k)
    gathered[r * mr:(r + 1) * mr].copy_(x1)
    peers = ctx.peers.peers_after(ptrs)
    lib, C = _cabi.lib(), _cabi.C
    arr = (C.c_void_p * max(len(peers), 1))(*[C.c_void_p(p) for p in peers])
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _cabi.check(lib.b200q_scatter_columns(buf.data_ptr(), arr, len(peers), 1, buf.numel(), r * mr * k, mr * k, st))
    gs = None
    if s1 is not None:
        gs = buf[nb_x:nb_x + nb_s].view(torch.float32)
        gs[r * mr:(r + 1) * mr].copy_(s1)
        _cabi.check(lib.b200q_scatter_columns(buf.data_ptr(), arr, len(peers), 1, buf.numel(), nb_x + r * mr * 4,
                                              mr * 4, st))
    ctx.peers.barrier()
    scale = _flat_scale(x2_scale, n, "x2_scale", op)
    if scale is None:
        scale = torch.ones(1, dtype=torch.float32, device=x1.device)
    out = _cabi.quant_matmul(gathered, x2, scale, pertoken_scale=gs, bias=bias, output_dtype=output_dtype or torch.bfloat16)
    gather_out = gathered.clone() if gather_output else torch.empty((0,), dtype=x1.dtype, device=x1.device)
    return out, gather_out


def _meta_reduce_scatter(x1, x2, hcom, world_size, reduce_op="sum", bias=None, x1_scale=None, x2_scale=None,
                         comm_turn=0, output_dtype=None, comm_mode=None):
    dt = output_dtype or (torch.bfloat16 if x1.dtype == torch.int8 else x1.dtype)
    return x1.new_empty((x1.shape[0] // world_size, x2.shape[1]), dtype=dt)


def _meta_all_gather_mm(x1, x2, hcom, world_size, bias=None, x1_scale=None, x2_scale=None, gather_index=0,
                        gather_output=True, comm_turn=0, output_dtype=None, comm_mode=None):
    dt = output_dtype or (torch.bfloat16 if x1.dtype == torch.int8 else x1.dtype)
    m = x1.shape[0] * world_size
    return (x1.new_empty((m, x2.shape[1]), dtype=dt),
            x1.new_empty((m, x1.shape[1]) if gather_output else (0,)))


def _meta_all_reduce(x1, x2, hcom, reduce_op="sum", bias=None, antiquant_scale=None, antiquant_offset=None, x3=None,
                     dequant_scale=None, pertoken_scale=None, comm_quant_scale_1=None, comm_quant_scale_2=None,
                     antiquant_group_size=0, comm_turn=0):
    # contract of test/test_fake_tensor.py:1555-1583: [m, n]; int64 dequant_scale -> float16, bfloat16 -> bfloat16
    if x1.dtype == torch.int8:
        dt = torch.bfloat16 if (dequant_scale is not None and dequant_scale.dtype == torch.bfloat16) else torch.float16
    else:
        dt = x1.dtype
    return x1.new_empty((*x1.shape[:-1], x2.shape[-1]), dtype=dt)


_LIB.impl("npu_mm_reduce_scatter_base", _mm_reduce_scatter, "CUDA")
_LIB.impl("npu_all_gather_base_mm", _all_gather_mm, "CUDA")
_LIB.impl("npu_mm_all_reduce_base", _mm_all_reduce, "CUDA")
_LIB.impl("npu_mm_reduce_scatter_base", _meta_reduce_scatter, "Meta")
_LIB.impl("npu_all_gather_base_mm", _meta_all_gather_mm, "Meta")
_LIB.impl("npu_mm_all_reduce_base", _meta_all_reduce, "Meta")

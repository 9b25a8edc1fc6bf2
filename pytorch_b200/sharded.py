"""Column-sharded (N-sharded) W8A8 linear across the GPUs of one node.

The reference's own sharding rule for a matmul is ``(Replicate, Shard(last)) -> Shard(last)``
(``torch_npu/distributed/tensor/_matrix_ops.py:143-146``) with the per-channel scales following
their operand (``:495-500``): rank r of g holds rows ``[r*N/g, (r+1)*N/g)`` of the ``[N,K]``
weight and the matching slice of ``scale`` / ``offset`` / ``bias``; activations, smooth scales
and the per-token scale are replicated.  The only exchange step is an all-gather of the
``[M, N/g]`` outputs along N, which the reference issues as ``hcclAllGather``
(``torch_npu/csrc/distributed/ProcessGroupHCCL.cpp:5896-5956``) and which runs here as
``ncclAllGather`` over NVLink through ``torch.distributed``.  With a world size of one no
collective is issued.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(n: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open column range of ``rank``; ``n`` must divide evenly."""
    if n % world:
        raise ValueError(f"n={n} is not divisible by the world size {world}")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_weight(weight_nk: torch.Tensor, *per_channel: torch.Tensor | None, rank: int, world: int):
    """Cuts an ``[N,K]`` weight and its per-channel vectors (``[N]``) for ``rank``."""
    lo, hi = shard_bounds(weight_nk.shape[0], rank, world)
    return (weight_nk[lo:hi].contiguous(),
            *[None if p is None else (p if p.numel() == 1 else p[lo:hi].contiguous()) for p in per_channel])


class ColumnShardedOutput:
    """Reusable buffers for gathering ``[M, N/g]`` shards into ``[M, N]``.

    ``all_gather_into_tensor`` delivers ``[g, M, N/g]`` (rank-major); one strided copy
    re-interleaves the column blocks into the row-major ``[M, N]`` the caller expects."""

    def __init__(self, m: int, n: int, dtype: torch.dtype, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.m, self.n = m, n
        if self.world > 1:
            # concatenation along dim 0 ([g*M, N/g]) is the output form every backend accepts
            self.staging = torch.empty((self.world * m, n // self.world), dtype=dtype, device=device)
            self.full = torch.empty((m, n), dtype=dtype, device=device)

    def gather(self, shard: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return shard
        dist.all_gather_into_tensor(self.staging, shard.contiguous(), group=self.group)
        per = self.n // self.world
        self.full.view(self.m, self.world, per).copy_(self.staging.view(self.world, self.m, per).permute(1, 0, 2))
        return self.full


class PeerColumnGather:
    """The same exchange without NCCL and without the re-interleave copy: every rank keeps its
    ``[M, N]`` result in symmetric (peer-mapped) memory, the GEMM writes the rank's column block
    straight into the local matrix (``out_row_stride = N``), ``b200q_scatter_columns`` pushes that
    block into every peer's matrix over NVLink with plain 128-bit stores, and a device-side barrier
    on the symmetric-memory signal pads tells every rank that all blocks have landed.

    Usage per step: ``y = self.local_block()`` (a ``[M, N/g]`` view to hand to the GEMM as ``out``),
    then ``full = self.gather()``.  ``full`` is overwritten by the next step's pushes: finish reading
    it (or copy it) before any rank starts that step.  No rank may leave while a step is in flight."""

    def __init__(self, m: int, n: int, dtype: torch.dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = dist.group.WORLD if group is None else group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.m, self.n = m, n
        self.lo, self.hi = shard_bounds(n, self.rank, self.world)
        self.full = symm_mem.empty((m, n), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.full, self.group)
        ptrs = list(self.handle.buffer_ptrs)
        # staggered order: rank r starts with r+1, so the switch sees an all-to-all, not a hot spot
        self.peer_ptrs = [ptrs[(self.rank + 1 + i) % self.world] for i in range(self.world - 1)]

    def local_block(self) -> torch.Tensor:
        return self.full[:, self.lo:self.hi]

    def gather(self) -> torch.Tensor:
        from . import _cabi
        _cabi.scatter_columns(self.full, self.peer_ptrs, self.lo, self.hi)
        self.handle.barrier(channel=0)
        return self.full


class ShardedW8A8LinearPlan:
    """One column-sharded W8A8 linear with every buffer and C-ABI argument block prepared once:
    dynamic quant of ``x`` (replicated), GEMM of this rank's columns written straight into the
    peer-mapped ``[M, N]`` matrix, push to the peers, barrier.  ``run()`` then issues four C-ABI
    calls and one barrier with no allocation and almost no Python work, which matters when eight
    ranks share one host and a step lasts about a millisecond."""

    def __init__(self, x: torch.Tensor, smooth_scales: torch.Tensor, weight_nk_shard: torch.Tensor,
                 scale_shard: torch.Tensor, gather: PeerColumnGather):
        import ctypes as C
        from . import _cabi
        self._C, self._cabi, self._lib = C, _cabi, _cabi.lib()
        self.gather = gather
        m, k = x.shape
        n = weight_nk_shard.shape[0]
        assert m == gather.m and n == gather.hi - gather.lo and weight_nk_shard.shape[1] == k
        dev = x.device
        self.x, self.smooth = x, smooth_scales.contiguous()
        self.q = torch.empty((m, k), dtype=torch.int8, device=dev)
        self.s = torch.empty((m,), dtype=torch.float32, device=dev)
        self.w, self.scale = weight_nk_shard, scale_shard.contiguous()
        need = self._lib.b200q_quant_matmul_workspace_bytes(m, k, n, 1, k)
        self.ws = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
        out = gather.local_block()
        a = _cabi.QuantMatmulArgs()
        a.x1, a.x2, a.m, a.k, a.n = self.q.data_ptr(), self.w.data_ptr(), m, k, n
        a.x2_stride_k, a.x2_stride_n = 1, k
        a.scale, a.scale_dtype, a.scale_len = self.scale.data_ptr(), _cabi.DTYPE[self.scale.dtype], self.scale.numel()
        a.pertoken_scale, a.bias_dtype = self.s.data_ptr(), _cabi.NONE
        a.out, a.out_dtype, a.out_row_stride = out.data_ptr(), _cabi.DTYPE[out.dtype], out.stride(0)
        if need:
            a.workspace, a.workspace_bytes = self.ws.data_ptr(), need
        self.args = a
        self.m, self.k = m, k
        es = gather.full.element_size()
        self.peers = (C.c_void_p * max(len(gather.peer_ptrs), 1))(*[C.c_void_p(int(p)) for p in gather.peer_ptrs])
        self.n_peers = len(gather.peer_ptrs)
        self.row_bytes, self.col_off, self.block = gather.n * es, gather.lo * es, (gather.hi - gather.lo) * es

    def run(self, x: torch.Tensor | None = None, exchange: bool = True) -> torch.Tensor:
        C, cabi, lib = self._C, self._cabi, self._lib
        xs = self.x if x is None else x
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        cabi.check(lib.b200q_dynamic_quant(xs.data_ptr(), cabi.DTYPE[xs.dtype], self.smooth.data_ptr(),
                                           cabi.DTYPE[self.smooth.dtype], self.q.data_ptr(), self.s.data_ptr(),
                                           self.m, self.k, st))
        cabi.check(lib.b200q_quant_matmul(C.byref(self.args), st))
        if exchange:
            cabi.check(lib.b200q_scatter_columns(self.gather.full.data_ptr(), self.peers, self.n_peers, self.m,
                                                 self.row_bytes, self.col_off, self.block, st))
            self.gather.handle.barrier(channel=0)
        return self.gather.full


def sharded_w8a8_linear(x: torch.Tensor, smooth_scales, weight_nk_shard: torch.Tensor, scale_shard: torch.Tensor,
                        gather: ColumnShardedOutput, *, output_dtype=torch.bfloat16, quantized=None):
    """dynamic quant (replicated) -> W8A8 GEMM on this rank's columns -> all-gather along N.

    ``quantized`` may carry the ``(int8, scale)`` pair of an earlier call on the same ``x``."""
    ops = torch.ops.npu
    q, s = quantized if quantized is not None else ops.npu_dynamic_quant(x, smooth_scales=smooth_scales)
    y = ops.npu_quant_matmul(q, weight_nk_shard.t(), scale_shard, pertoken_scale=s, output_dtype=output_dtype)
    return gather.gather(y)

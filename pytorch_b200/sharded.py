"""Column-sharded (N-sharded) W8A8 linear across the GPUs of one node.

The reference's own sharding rule for a matmul is ``(Replicate, Shard(last)) -> Shard(last)``
(``torch_npu/distributed/tensor/_matrix_ops.py:143-146``) with the per-channel scales following
their operand (``:495-500``): rank r of g holds rows ``[r*N/g, (r+1)*N/g)`` of the ``[N,K]``
weight and the matching slice of ``scale`` / ``offset`` / ``bias``; activations, smooth scales
and the per-token scale are replicated.  The only exchange step is an all-gather of the
``[M, N/g]`` outputs along N, which the reference issues as ``hcclAllGather``
(``torch_npu/csrc/distributed/ProcessGroupHCCL.cpp:5896-5956``).  Here the GEMM kernel itself
stores every finished tile into the peers' matrices over NVLink (``peer_out`` of the C ABI), so
the exchange overlaps the main loop, and one bounded cross-rank barrier ends the step.  An NCCL
all-gather variant is kept for set-ups without peer-mapped memory.  With a world size of one no
exchange is issued.
"""
from __future__ import annotations

import ctypes as C

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
    """Reusable buffers for gathering ``[M, N/g]`` shards into ``[M, N]`` with NCCL.

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


def _ptr_array(ptrs):
    return (C.c_void_p * max(len(ptrs), 1))(*[C.c_void_p(int(p)) for p in ptrs])


class PeerGroup:
    """The ranks of one node that address each other's memory, plus the cross-rank barrier
    (``b200q_peer_barrier``) over a small array of flag words in peer-mapped memory.

    The barrier kernel has a time budget (10 s unless ``timeout_ns`` says otherwise): when a peer never
    arrives the kernel records a code in the device error word and returns, so a rank whose peer has
    died gets a ``B200QError`` from :meth:`check` instead of a spinning kernel."""

    def __init__(self, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self._symm = symm_mem
        self.group = dist.group.WORLD if group is None else group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device
        self.flags = symm_mem.empty((64,), dtype=torch.int32, device=device)
        self.flags.zero_()
        torch.cuda.synchronize(device)
        self._flags_handle = symm_mem.rendezvous(self.flags, self.group)
        dist.barrier(self.group)                      # every rank's flags are zero before anyone signals
        self._flag_ptrs = _ptr_array(self._flags_handle.buffer_ptrs)
        self.epoch = 0

    def symmetric(self, shape, dtype):
        """A tensor in peer-mapped memory and the device addresses of every rank's copy."""
        t = self._symm.empty(tuple(shape), dtype=dtype, device=self.device)
        handle = self._symm.rendezvous(t, self.group)
        return t, list(handle.buffer_ptrs), handle

    def peers_after(self, ptrs, byte_offset: int = 0):
        """The other ranks' pointers in a rank-staggered order (rank r starts with r+1), so that at any
        moment the ranks write to different peers and the switch sees an all-to-all, not a hot spot."""
        return [int(ptrs[(self.rank + 1 + i) % self.world]) + byte_offset for i in range(self.world - 1)]

    def barrier(self, timeout_ns: int = 0) -> None:
        from . import _cabi
        self.epoch += 1
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        _cabi.check(_cabi.lib().b200q_peer_barrier(self._flag_ptrs, self.world, self.rank, self.epoch & 0xFFFFFFFF,
                                                   timeout_ns, st))

    def check(self) -> None:
        """Raises if a kernel on this device gave up a bounded wait (synchronises the device)."""
        from . import _cabi
        code = _cabi.device_error(reset=True)
        if code:
            raise _cabi.B200QError(_cabi.ERR_DEVICE, f"a kernel gave up a bounded wait (device error 0x{code:x})")


class PeerColumnGather:
    """``[M, N]`` result matrices in peer-mapped memory, ``buffers`` of them used in rotation.

    Per step the caller takes ``local_block()`` (the ``[M, N/g]`` view of the current matrix the GEMM
    writes) and ``peer_blocks()`` (the addresses of the same block in every peer's current matrix, which
    the GEMM's epilogue writes too), runs the GEMM, and ends the step with ``finish()``: one barrier,
    after which ``full`` holds every rank's columns.  With two buffers the matrix a step has produced
    stays untouched while the next step runs: peers only write into it again two steps later, and by
    then the barrier in between has ordered that after everything this rank had queued on its stream
    before it, a device-to-host copy of ``full`` included."""

    def __init__(self, m: int, n: int, dtype: torch.dtype, device, peers: PeerGroup | None = None, group=None,
                 buffers: int = 2):
        self.peers = peers if peers is not None else PeerGroup(device, group)
        self.world, self.rank = self.peers.world, self.peers.rank
        self.m, self.n = m, n
        self.lo, self.hi = shard_bounds(n, self.rank, self.world)
        self.es = torch.empty((), dtype=dtype).element_size()
        self.bufs = []
        for _ in range(buffers):
            t, ptrs, handle = self.peers.symmetric((m, n), dtype)
            self.bufs.append((t, ptrs, handle))
        self.cur = 0

    @property
    def full(self) -> torch.Tensor:
        return self.bufs[self.cur][0]

    @property
    def peer_ptrs(self):
        return self.peers.peers_after(self.bufs[self.cur][1])

    def advance(self) -> None:
        self.cur = (self.cur + 1) % len(self.bufs)

    def local_block(self) -> torch.Tensor:
        return self.full[:, self.lo:self.hi]

    def peer_blocks(self):
        return self.peers.peers_after(self.bufs[self.cur][1], self.lo * self.es)

    def push(self) -> None:
        """Stand-alone push of the current block (for a producer that could not write to the peers itself)."""
        from . import _cabi
        _cabi.scatter_columns(self.full, self.peer_ptrs, self.lo, self.hi)

    def push_copy_engine(self, part: int = 0, parts: int = 1) -> None:
        """The same push as one copy-engine transfer per peer on the current stream (no SM involved);
        ``part`` of ``parts`` takes every ``parts``-th peer of the rank-staggered order."""
        from . import _cabi
        _cabi.copy_columns(self.full, self.peer_ptrs[part::parts], self.lo, self.hi)

    def finish(self) -> torch.Tensor:
        self.peers.barrier()
        return self.full

    def gather(self) -> torch.Tensor:
        """Push kernel + barrier: the exchange as a separate step after a GEMM that wrote only locally."""
        self.push()
        return self.finish()


class PipelinedExchange:
    """The exchange of a step on the copy engines, one step behind the kernels.

    The GEMMs of a step write only their own column blocks (``fused_push=False`` plans).  After each GEMM the
    caller calls :meth:`produced`: an event is recorded on the compute stream and, on a side stream, the
    column block is copied into every peer's matrix behind that event.  :meth:`end_step` queues the
    cross-rank barrier behind the copies, on the side stream too, and rotates the result buffers.  The
    compute stream never waits for NVLink: with two result buffers per gather the kernels of step i+1 run
    while the blocks of step i cross the links, and step i+2 (which writes the buffers of step i again)
    first waits for step i's copies.  :meth:`drain` makes the compute stream wait for everything queued.

    Whoever reads a gathered matrix of step i must (a) wait for ``done_event(i)`` and (b) have finished, or be
    queued on the side stream through :meth:`before_next_barrier`, before this rank joins the barrier of step
    i+1: peers write that matrix again in their step i+2, which they start once that barrier has passed."""

    def __init__(self, peers: PeerGroup, gathers, device, copy_streams: int = 1):
        self.peers, self.gathers = peers, list(gathers)
        # The copies to different peers can be spread over several streams (the barrier follows on the first).
        # One stream is the default: with two, the ranks' rank-staggered transfers no longer stay in step, two
        # senders meet at one receiver, and the four-GPU step measured 0.73 ms against 0.67 ms.
        self.sides = [torch.cuda.Stream(device=device) for _ in range(max(1, min(copy_streams, peers.world - 1)))]
        self.side = self.sides[0]
        nbuf = len(self.gathers[0].bufs)
        assert nbuf >= 2 and all(len(g.bufs) == nbuf for g in self.gathers)
        self._done = [torch.cuda.Event() for _ in range(nbuf)]
        self._produced = [[torch.cuda.Event() for _ in self.gathers] for _ in range(nbuf)]
        self._copied = [[torch.cuda.Event() for _ in self.sides[1:]] for _ in range(nbuf)]
        self._steps = 0
        self._prev_done = None
        self._readers = [[] for _ in range(nbuf)]
        self._last_b = 0

    def begin_step(self) -> None:
        """Before the first kernel that writes this step's result buffers: their last use (the copies out of
        them two steps ago, and every registered reader of that step's gathered matrices) must be over."""
        b = self.gathers[0].cur
        cur = torch.cuda.current_stream()
        if self._steps >= len(self._done):
            cur.wait_event(self._done[b])
        for ev in self._readers[b]:
            cur.wait_event(ev)
        self._readers[b] = []

    def produced(self, index: int) -> None:
        """The GEMM of gather ``index`` has been queued on the current stream."""
        g = self.gathers[index]
        ev = self._produced[g.cur][index]
        ev.record(torch.cuda.current_stream())
        for j, st in enumerate(self.sides):
            with torch.cuda.stream(st):
                st.wait_event(ev)
                if j > 0 and self._prev_done is not None:
                    st.wait_event(self._prev_done)        # like the first stream: not before the previous step's barrier
                g.push_copy_engine(j, len(self.sides))

    def before_next_barrier(self, event: torch.cuda.Event) -> None:
        """A reader of the gathered matrices of the step that ended last has recorded ``event`` when it was done:
        this rank joins the next barrier only after it (peers write those matrices again once that barrier has
        passed), and this rank's own kernels write them again only after it (see :meth:`begin_step`)."""
        self.side.wait_event(event)
        self._readers[self._last_b].append(event)

    def end_step(self) -> torch.cuda.Event:
        b = self.gathers[0].cur
        for j, st in enumerate(self.sides[1:]):
            self._copied[b][j].record(st)
            self.side.wait_event(self._copied[b][j])
        with torch.cuda.stream(self.side):
            self.peers.barrier()
            self._done[b].record(self.side)
        for g in self.gathers:
            g.advance()
        self._steps += 1
        self._prev_done = self._done[b]
        self._last_b = b
        return self._done[b]

    def drain(self) -> None:
        for st in self.sides:
            torch.cuda.current_stream().wait_stream(st)


class LocalOutput:
    """The single-GPU stand-in for :class:`PeerColumnGather`: plain ``[M, N]`` result matrices, no peers, so
    that :class:`ShardedW8A8LinearPlan` can drive an unsharded linear through the same prepared C-ABI calls."""

    def __init__(self, m: int, n: int, dtype: torch.dtype, device, buffers: int = 2):
        self.world, self.rank, self.m, self.n, self.lo, self.hi = 1, 0, m, n, 0, n
        self.bufs = [(torch.empty((m, n), dtype=dtype, device=device), [], None) for _ in range(buffers)]
        self.cur = 0

    @property
    def full(self) -> torch.Tensor:
        return self.bufs[self.cur][0]

    def advance(self) -> None:
        self.cur = (self.cur + 1) % len(self.bufs)

    def local_block(self) -> torch.Tensor:
        return self.full

    def peer_blocks(self):
        return []

    def push(self) -> None:
        pass

    def finish(self) -> torch.Tensor:
        return self.full


class ShardedW8A8LinearPlan:
    """One column-sharded W8A8 linear with every buffer and C-ABI argument block prepared once:
    dynamic quant of ``x`` (replicated), then one GEMM launch that writes this rank's columns into the
    local ``[M, N]`` matrix and into every peer's.  ``run()`` issues two C-ABI calls with no allocation
    and almost no Python work, which matters when eight ranks share one host and a step lasts well under
    a millisecond.  The caller ends the step with ``gather.finish()`` (one barrier for all linears of the
    step that share a :class:`PeerGroup`)."""

    def __init__(self, x: torch.Tensor, smooth_scales: torch.Tensor, weight_nk_shard: torch.Tensor,
                 scale_shard: torch.Tensor, gather: PeerColumnGather, fused_push: bool = True):
        from . import _cabi
        self._cabi, self._lib = _cabi, _cabi.lib()
        self.gather = gather
        self.fused_push = fused_push
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
        self.m, self.k = m, k
        self.args, self._keep = [], []
        for b in range(len(gather.bufs)):            # one argument block per result buffer
            gather.cur = b
            out = gather.local_block()
            a = _cabi.QuantMatmulArgs()
            a.x1, a.x2, a.m, a.k, a.n = self.q.data_ptr(), self.w.data_ptr(), m, k, n
            a.x2_stride_k, a.x2_stride_n = 1, k
            a.scale, a.scale_dtype, a.scale_len = self.scale.data_ptr(), _cabi.DTYPE[self.scale.dtype], self.scale.numel()
            a.pertoken_scale, a.bias_dtype = self.s.data_ptr(), _cabi.NONE
            a.out, a.out_dtype, a.out_row_stride = out.data_ptr(), _cabi.DTYPE[out.dtype], out.stride(0)
            if need:
                a.workspace, a.workspace_bytes = self.ws.data_ptr(), need
            if fused_push and gather.world > 1:
                arr = _ptr_array(gather.peer_blocks())
                self._keep.append(arr)
                a.peer_out, a.n_peer_out = arr, gather.world - 1
            self.args.append(a)
        gather.cur = 0

    def quant(self, x: torch.Tensor | None = None) -> None:
        cabi = self._cabi
        xs = self.x if x is None else x
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        cabi.check(self._lib.b200q_dynamic_quant(xs.data_ptr(), cabi.DTYPE[xs.dtype], self.smooth.data_ptr(),
                                                 cabi.DTYPE[self.smooth.dtype], self.q.data_ptr(), self.s.data_ptr(),
                                                 self.m, self.k, st))

    def matmul(self, push: bool = True) -> None:
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        self._cabi.check(self._lib.b200q_quant_matmul(C.byref(self.args[self.gather.cur]), st))
        if push and not self.fused_push and self.gather.world > 1:
            self.gather.push()

    def run(self, x: torch.Tensor | None = None) -> torch.Tensor:
        self.quant(x)
        self.matmul()
        return self.gather.full


def sharded_w8a8_linear(x: torch.Tensor, smooth_scales, weight_nk_shard: torch.Tensor, scale_shard: torch.Tensor,
                        gather: ColumnShardedOutput, *, output_dtype=torch.bfloat16, quantized=None):
    """dynamic quant (replicated) -> W8A8 GEMM on this rank's columns -> all-gather along N (NCCL variant).

    ``quantized`` may carry the ``(int8, scale)`` pair of an earlier call on the same ``x``."""
    ops = torch.ops.npu
    q, s = quantized if quantized is not None else ops.npu_dynamic_quant(x, smooth_scales=smooth_scales)
    y = ops.npu_quant_matmul(q, weight_nk_shard.t(), scale_shard, pertoken_scale=s, output_dtype=output_dtype)
    return gather.gather(y)

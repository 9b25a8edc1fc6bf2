"""GPU side of the column-sharded linear: writing a shard into its place of a wider matrix
(out_row_stride) and the peer push kernel, emulated on one GPU with several local buffers standing in
for the peers' matrices; on a box with two or more GPUs also the real two-rank exchange over
symmetric memory, checked against the unsharded oracle."""
import os
import socket
import sys

import pytest
import torch

from oracle import quant_oracle as oracle
from pytorch_b200 import workloads

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def cabi():
    from pytorch_b200 import _cabi
    _cabi.lib()
    assert torch.cuda.is_available()
    return _cabi


@pytest.mark.parametrize("m", [16, 640])
def test_shards_written_in_place_and_pushed(cabi, m):
    world, k, n = 4, 512, 1024
    d = workloads.w8a8_linear(m, k, n, 321)
    q, s = oracle.dynamic_quant(d["x"], d["smooth_scales"])
    want = oracle.quant_matmul(q, d["x2"], d["scale"], pertoken_scale=s, output_dtype=torch.bfloat16)
    qd, sd = q.cuda(), s.cuda()
    fulls = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    per = n // world
    for r in range(world):                               # "rank" r computes its columns into its own matrix
        w = d["weight_nk"][r * per:(r + 1) * per].cuda()
        view = fulls[r][:, r * per:(r + 1) * per]
        out = cabi.quant_matmul(qd, w.t(), d["scale"][r * per:(r + 1) * per].cuda(), pertoken_scale=sd,
                                output_dtype=torch.bfloat16, out=view)
        assert out.data_ptr() == view.data_ptr()
        assert torch.isnan(fulls[r][:, :r * per].float()).all() and torch.isnan(fulls[r][:, (r + 1) * per:].float()).all()
    for r in range(world):                               # ... and pushes them to the other three
        peers = [fulls[(r + 1 + i) % world].data_ptr() for i in range(world - 1)]
        cabi.scatter_columns(fulls[r], peers, r * per, (r + 1) * per)
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(fulls[r].cpu().view(torch.int16), want.view(torch.int16))
    with pytest.raises(cabi.B200QError):
        cabi.scatter_columns(fulls[0], [fulls[1].data_ptr()], 4, 4 + 3)      # 6-byte block: not a 16-byte multiple


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), TORCH_SYMM_MEM_DISABLE_MULTICAST="1",
                      NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    import pytorch_b200 as pb
    from pytorch_b200 import _cabi, collective_ops, sharded
    try:
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        m, k, n = 256, 1024, 2048
        d = workloads.w8a8_linear(m, k, n, 77)
        q, s = oracle.dynamic_quant(d["x"], d["smooth_scales"])
        want = oracle.quant_matmul(q, d["x2"], d["scale"], pertoken_scale=s, output_dtype=torch.bfloat16)
        peers = sharded.PeerGroup(dev)
        gat = sharded.PeerColumnGather(m, n, torch.bfloat16, dev, peers)
        w, sc = sharded.shard_weight(d["weight_nk"], d["scale"], rank=rank, world=world)
        ok = True
        # (a) separate push kernel after a GEMM that wrote locally; (b) the GEMM's own epilogue writes to the peer
        for step in range(4):                             # result matrices and flags are reused from step to step
            if step % 2 == 0:
                _cabi.quant_matmul(q.to(dev), w.to(dev).t(), sc.to(dev), pertoken_scale=s.to(dev),
                                   output_dtype=torch.bfloat16, out=gat.local_block())
                full = gat.gather()
            else:
                _cabi.quant_matmul(q.to(dev), w.to(dev).t(), sc.to(dev), pertoken_scale=s.to(dev),
                                   output_dtype=torch.bfloat16, out=gat.local_block(), peer_out=gat.peer_blocks())
                full = gat.finish()
            torch.cuda.synchronize()
            ok = ok and torch.equal(full.cpu().view(torch.int16), want.view(torch.int16))
            gat.advance()
        # the prepared-argument plan the benchmark uses
        plan = sharded.ShardedW8A8LinearPlan(d["x"].to(dev), d["smooth_scales"].to(dev), w.to(dev), sc.to(dev), gat)
        for _ in range(3):
            plan.run()
            full = gat.finish()
            torch.cuda.synchronize()
            ok = ok and torch.equal(full.cpu().view(torch.int16), want.view(torch.int16))
            gat.advance()
        # the exchange on the copy engines, one step behind the kernels (two steps in flight, buffers reused)
        nop = sharded.ShardedW8A8LinearPlan(d["x"].to(dev), d["smooth_scales"].to(dev), w.to(dev), sc.to(dev), gat,
                                            fused_push=False)
        pipe = sharded.PipelinedExchange(peers, (gat,), dev)
        fulls, dones = [], []
        for _ in range(5):
            pipe.begin_step()
            nop.quant()
            nop.matmul(push=False)
            pipe.produced(0)
            fulls.append(gat.full)
            dones.append(pipe.end_step())
        pipe.drain()
        torch.cuda.synchronize()
        dist.barrier()
        for full in fulls[-2:]:                           # the two result matrices hold the last two steps
            ok = ok and torch.equal(full.cpu().view(torch.int16), want.view(torch.int16))
        # ... with a reader of every step's gathered matrix (a device-to-host copy on a third stream) and inputs that
        # change from step to step: a matrix overwritten too early by a peer's later step would show up as a mismatch
        xs = [workloads.w8a8_linear(m, k, n, 500 + i)["x"] for i in range(3)]
        wants = []
        for xi in xs:
            qi, si = oracle.dynamic_quant(xi, d["smooth_scales"])
            wants.append(oracle.quant_matmul(qi, d["x2"], d["scale"], pertoken_scale=si, output_dtype=torch.bfloat16))
        xs_dev = [xi.to(dev) for xi in xs]
        reader = torch.cuda.Stream(device=dev)
        host = [torch.empty((m, n), dtype=torch.bfloat16).pin_memory() for _ in range(7)]
        for step in range(7):
            pipe.begin_step()
            nop.quant(xs_dev[step % 3])
            nop.matmul(push=False)
            pipe.produced(0)
            full = gat.full
            done = pipe.end_step()
            with torch.cuda.stream(reader):
                reader.wait_event(done)
                host[step].copy_(full, non_blocking=True)
                read = torch.cuda.Event()
                read.record(reader)
            pipe.before_next_barrier(read)
        pipe.drain()
        torch.cuda.synchronize()
        dist.barrier()
        for step in range(7):
            ok = ok and torch.equal(host[step].view(torch.int16), wants[step % 3].view(torch.int16))
        # collective-fused operators against the oracle of all ranks' inputs (same seed on every rank)
        g = torch.Generator().manual_seed(5)
        mm, kk, nn = 128, 256, 256
        x1l = [workloads.rand_int8((mm, kk), g) for _ in range(world)]
        wl = [workloads.rand_int8((nn, kk), g) for _ in range(world)]
        s1l = [workloads.rand_uniform((mm, 1), g, 1e-3, 1e-2) for _ in range(world)]
        s2l = [workloads.rand_uniform((1, nn), g, 1e-3, 1e-2) for _ in range(world)]
        hcom = collective_ops.hcom_name()
        rs_want = oracle.mm_reduce_scatter(x1l, [t.t() for t in wl], s1l, s2l)
        ar_want = oracle.mm_all_reduce(x1l, [t.t() for t in wl], s2l[0].reshape(-1).to(torch.bfloat16), s1l[0].reshape(-1))
        ag_want, ag_x1 = oracle.all_gather_mm(x1l, [t.t() for t in wl], s1l, s2l)
        for _ in range(3):                                # staging buffers alternate between calls
            rs = pb.npu_mm_reduce_scatter_base(x1l[rank].to(dev), wl[rank].to(dev).t(), hcom, world,
                                               x1_scale=s1l[rank].to(dev), x2_scale=s2l[rank].to(dev),
                                               output_dtype=torch.bfloat16, comm_mode="aiv")
            ar = pb.npu_mm_all_reduce_base(x1l[rank].to(dev), wl[rank].to(dev).t(), hcom, reduce_op="sum",
                                           dequant_scale=s2l[0].reshape(-1).to(torch.bfloat16).to(dev),
                                           pertoken_scale=s1l[0].reshape(-1).to(dev))
            ag, gx = pb.npu_all_gather_base_mm(x1l[rank].to(dev), wl[rank].to(dev).t(), hcom, world,
                                               x1_scale=s1l[rank].to(dev), x2_scale=s2l[rank].to(dev))
            torch.cuda.synchronize()
            ok = ok and torch.equal(rs.cpu().view(torch.int16), rs_want[rank].view(torch.int16))
            ok = ok and torch.equal(ar.cpu().view(torch.int16), ar_want.view(torch.int16))
            ok = ok and torch.equal(ag.cpu().view(torch.int16), ag_want[rank].view(torch.int16))
            ok = ok and torch.equal(gx.cpu(), ag_x1)
        peers.check()
        dist.barrier()
        results.put((rank, "ok" if ok else "mismatch"))
        collective_ops.release_contexts()
        dist.destroy_process_group()
    except Exception as e:                                # pragma: no cover
        results.put((rank, f"fail:{type(e).__name__}:{e}"))


def test_two_rank_peer_gather_and_collective_ops_match_unsharded_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import queue
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(2):
            try:
                r, msg = results.get(timeout=240)
            except queue.Empty:
                break
            out[r] = msg
            if msg != "ok":                                # the other rank's barrier will run out; do not wait for it
                break
    finally:
        for p in procs:
            p.join(timeout=30)
        for p in procs:                                    # never leave a child (and its kernels) behind
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
    assert out == {0: "ok", 1: "ok"}, out

"""Host logic of the N-sharded linear on CPU ranks (gloo, world size 2): shard bounds, slicing of
the per-channel vectors, the all-gather and re-interleave into [M, N], and the failure mode of a
rank that never joins the collective (bounded by the process-group timeout, no GPU involved).
The arithmetic on each shard comes from the CPU oracle here; the CUDA kernels are covered by the
GPU tests."""
import datetime
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    from oracle import quant_oracle as oracle
    from pytorch_b200 import sharded, workloads
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
        if mode == "gather":
            m, k, n = 12, 64, 48
            d = workloads.w8a8_linear(m, k, n, 99)                      # same seed -> same tensors on every rank
            q, s = oracle.dynamic_quant(d["x"], d["smooth_scales"])
            w_shard, sc_shard = sharded.shard_weight(d["weight_nk"], d["scale"], rank=rank, world=world)
            lo, hi = sharded.shard_bounds(n, rank, world)
            assert w_shard.shape == (n // world, k) and torch.equal(sc_shard, d["scale"][lo:hi])
            y = oracle.quant_matmul(q, w_shard.t(), sc_shard, pertoken_scale=s, output_dtype=torch.bfloat16)
            gat = sharded.ColumnShardedOutput(m, n, torch.bfloat16, "cpu")
            full = gat.gather(y)
            want = oracle.quant_matmul(q, d["x2"], d["scale"], pertoken_scale=s, output_dtype=torch.bfloat16)
            assert full.shape == (m, n) and torch.equal(full, want)
            full2 = gat.gather(y * 2)                                    # buffers are reusable
            assert torch.equal(full2.float(), want.float() * 2)
            results.put((rank, "ok"))
        elif mode == "absent":
            if rank == 1:
                results.put((rank, "left"))                                    # leaves between steps, nothing in flight
                return
            gat = sharded.ColumnShardedOutput(4, 8, torch.float32, "cpu")
            try:
                gat.gather(torch.zeros(4, 4))
                results.put((rank, "no error"))
            except Exception as e:                                       # the collective ends with an error
                results.put((rank, "error:" + type(e).__name__))
    except Exception as e:                                               # pragma: no cover
        results.put((rank, f"fail:{type(e).__name__}:{e}"))
    finally:
        if dist.is_initialized() and mode == "gather":
            dist.destroy_process_group()


def _run(mode, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    return out


def test_shard_bounds():
    sys.path.insert(0, ROOT)
    from pytorch_b200 import sharded
    assert sharded.shard_bounds(57344, 3, 8) == (21504, 28672)
    assert sharded.shard_bounds(8192, 0, 1) == (0, 8192)
    with pytest.raises(ValueError):
        sharded.shard_bounds(10, 0, 4)
    w = torch.arange(24).reshape(6, 4)
    ws, sc, none, one = sharded.shard_weight(w, torch.arange(6.0), None, torch.ones(1), rank=1, world=3)
    assert torch.equal(ws, w[2:4]) and torch.equal(sc, torch.tensor([2.0, 3.0])) and none is None and one.numel() == 1


def test_two_rank_gather_matches_unsharded_oracle():
    assert _run("gather") == {0: "ok", 1: "ok"}


def test_rank_that_never_joins_ends_the_collective_with_an_error():
    out = _run("absent")
    assert out[1] == "left" and out[0].startswith("error:"), out

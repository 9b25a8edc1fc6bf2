#!/usr/bin/env python
"""Benchmark of the W8A8 quantized-inference path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload at every N: the Llama-70B-shaped W8A8 MLP of the benchmark configurations
(x bf16 [4096,8192] -> dynamic quant with smooth scales -> gate/up GEMM against an int8
[8192,57344] weight; x_down bf16 [4096,28672] -> dynamic quant -> down GEMM against an int8
[28672,8192] weight; bf16 outputs), the weights column-sharded over the N ranks with their
per-channel scales and the outputs all-gathered over NVLink when N > 1.  One step is one pass
of that path over one batch of 4096 tokens; total work is fixed, so scaling is "strong".
At N = 1 the line also carries the Llama-7B-shaped linears at M = 2048 and the dynamic-quant
bandwidth as extra keys.

Prints ONE JSON line on rank 0.  `value` is whole-job TOPS (2*M*K*N summed over the two GEMMs
and divided by the max-over-ranks device time per step) with inputs resident in HBM; `e2e`
repeats the measurement through torch.ops.npu.* from pinned host buffers with the host->device
copy of the activations and the device->host copy of both outputs inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, HIDDEN, FFN = 4096, 8192, 28672
METRIC = "w8a8_quant_matmul_tops"
UNIT = "TOPS"


def step_flops():
    return 2.0 * M * HIDDEN * (2 * FFN) + 2.0 * M * FFN * HIDDEN


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) every few ms."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, device_index: int):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.handle = None

    def run(self):
        if self.handle is None:
            return
        while not self._stop_evt.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.handle, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(0.004)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_inputs(rank: int, world: int, device):
    """Synthetic tensors of the configuration's shapes and value ranges, created on the device
    (activations and smooth scales from a seed shared by all ranks, weight shards per rank)."""
    g = torch.Generator(device=device)
    g.manual_seed(5000)
    d = {}
    d["x"] = torch.randn((M, HIDDEN), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    d["smooth"] = torch.rand((HIDDEN,), generator=g, device=device) * 1.5 + 0.5
    d["x_down"] = torch.randn((M, FFN), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    d["smooth_down"] = torch.rand((FFN,), generator=g, device=device) * 1.5 + 0.5
    g.manual_seed(5001 + rank + 16 * world)
    n_gu, n_dn = 2 * FFN // world, HIDDEN // world
    d["w_gu"] = torch.randint(-127, 128, (n_gu, HIDDEN), generator=g, device=device, dtype=torch.int8)
    d["s_gu"] = torch.rand((n_gu,), generator=g, device=device) * 9e-3 + 1e-3
    d["w_dn"] = torch.randint(-127, 128, (n_dn, FFN), generator=g, device=device, dtype=torch.int8)
    d["s_dn"] = torch.rand((n_dn,), generator=g, device=device) * 9e-3 + 1e-3
    return d


def time_events(pairs):
    return sum(a.elapsed_time(b) for a, b in pairs)


def run_b200(args):
    import torch.distributed as dist
    import pytorch_b200  # noqa: F401  (registers torch.ops.npu.*; raises if the extension is missing)
    from pytorch_b200 import sharded, workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ops = torch.ops.npu
    d = make_inputs(rank, world, device)
    w_gu_t, w_dn_t = d["w_gu"].t(), d["w_dn"].t()
    exchange = "none"
    gat_gu = gat_dn = None
    if world > 1:
        # Preferred exchange: GEMM writes its column block into a peer-mapped [M, N] matrix and
        # b200q_scatter_columns pushes it to the peers over NVLink.  NCCL all-gather + re-interleave copy
        # is used only where symmetric memory cannot be set up (BENCH_EXCHANGE=nccl forces it).
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        try:
            if os.environ.get("BENCH_EXCHANGE", "p2p") != "p2p":
                raise RuntimeError("NCCL exchange requested")
            gat_gu = sharded.PeerColumnGather(M, 2 * FFN, torch.bfloat16, device)
            gat_dn = sharded.PeerColumnGather(M, HIDDEN, torch.bfloat16, device)
            exchange = "p2p_scatter"
        except Exception as exc:                                   # noqa: BLE001
            if rank == 0:
                print(f"[bench] peer-memory exchange unavailable ({exc}); using NCCL all-gather", file=sys.stderr)
            gat_gu = sharded.ColumnShardedOutput(M, 2 * FFN, torch.bfloat16, device)
            gat_dn = sharded.ColumnShardedOutput(M, HIDDEN, torch.bfloat16, device)
            exchange = "nccl_all_gather"
        flag = torch.tensor([1 if exchange == "p2p_scatter" else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)                # all ranks must agree
        if int(flag.item()) == 0 and exchange == "p2p_scatter":
            gat_gu = sharded.ColumnShardedOutput(M, 2 * FFN, torch.bfloat16, device)
            gat_dn = sharded.ColumnShardedOutput(M, HIDDEN, torch.bfloat16, device)
            exchange = "nccl_all_gather"
    from pytorch_b200 import _cabi
    plans = None
    if exchange == "p2p_scatter":
        plans = (sharded.ShardedW8A8LinearPlan(d["x"], d["smooth"], d["w_gu"], d["s_gu"], gat_gu),
                 sharded.ShardedW8A8LinearPlan(d["x_down"], d["smooth_down"], d["w_dn"], d["s_dn"], gat_dn))
    gemm_events, dq_events = [], []

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # high priority: the exchange kernel is small and must get its CTAs resident before the next GEMM fills the SMs
    comm = torch.cuda.Stream(device=device, priority=-1) if world > 1 else None

    def gemm(q, w_t, scale, s, gat):
        if exchange == "p2p_scatter":      # C-ABI call with the output placed inside the peer-mapped matrix
            return _cabi.quant_matmul(q, w_t, scale, pertoken_scale=s, output_dtype=torch.bfloat16, out=gat.local_block())
        return ops.npu_quant_matmul(q, w_t, scale, pertoken_scale=s, output_dtype=torch.bfloat16)

    comm_events = []

    def gather_async(gat, y, record=False):
        """Exchange on the side stream so that it overlaps the next GEMM (independent data)."""
        if world == 1:
            return y
        main = torch.cuda.current_stream()
        # The peer push runs in stream order after its GEMM: measured on 8 GPUs, overlapping it with the next
        # dynamic quant + GEMM slowed the push five-fold, while back to back it runs at the link rate.
        # The NCCL variant keeps its side stream (its kernels cannot share an SM with the GEMM's CTAs anyway).
        side = main if exchange == "p2p_scatter" else comm
        side.wait_stream(main)
        with torch.cuda.stream(side):
            if record:
                a, b = ev(), ev()
                a.record()
            if exchange == "p2p_scatter":
                out = gat.gather()
            else:
                y.record_stream(comm)
                out = gat.gather(y)
            if record:
                b.record()
                comm_events.append((a, b))
            return out

    def step(x, x_down, record=False):
        if plans is not None and not record:
            # lean launch path: prepared argument blocks, C-ABI calls only (dynamic quant, GEMM into the
            # peer-mapped matrix, push, barrier) for each projection
            return plans[0].run(x), plans[1].run(x_down)
        e = [ev() for _ in range(6)] if record else None
        if record: e[0].record()
        q, s = ops.npu_dynamic_quant(x, smooth_scales=d["smooth"])
        if record: e[1].record()
        y1 = gemm(q, w_gu_t, d["s_gu"], s, gat_gu if world > 1 else None)
        if record: e[2].record()
        o1 = gather_async(gat_gu, y1, record)
        if record: e[3].record()
        q2, s2 = ops.npu_dynamic_quant(x_down, smooth_scales=d["smooth_down"])
        if record: e[4].record()
        y2 = gemm(q2, w_dn_t, d["s_dn"], s2, gat_dn if world > 1 else None)
        if record: e[5].record()
        o2 = gather_async(gat_dn, y2, record)
        if world > 1:
            torch.cuda.current_stream().wait_stream(comm)      # the step ends when both gathers have landed
        if record:
            dq_events.extend([(e[0], e[1]), (e[3], e[4])])
            gemm_events.extend([(e[1], e[2]), (e[4], e[5])])
        return o1, o2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident measurement
    for _ in range(args.warmup):
        step(d["x"], d["x_down"])
    barrier()
    # Only the rank that prints the line samples its GPU: eight processes polling NVML at this rate
    # would contend with each other's kernel launches.  The sampler is set up before the last barrier,
    # so that the rank that pays for the NVML start-up does not enter the timed region late.
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler is not None:
        sampler.start()
    barrier()
    t0, t1 = ev(), ev()
    t0.record()
    host_t0 = time.perf_counter()
    for _ in range(args.steps):
        step(d["x"], d["x_down"], record=plans is None)
    t1.record()
    host_ms_step = (time.perf_counter() - host_t0) * 1e3 / args.steps     # time the host needs to launch one step
    barrier()
    ms_total = max_over_ranks(t0.elapsed_time(t1))
    clocks = sampler.stop() if sampler is not None else None
    if plans is not None:
        # per-kernel events from three extra steps through the event-recording path (same kernels, same buffers)
        for _ in range(3):
            step(d["x"], d["x_down"], record=True)
        barrier()
    ms_step = ms_total / args.steps
    value = step_flops() / (ms_step * 1e-3) / 1e12

    gemm_ms = time_events(gemm_events) / len(gemm_events)
    dq_ms = time_events(dq_events) / len(dq_events)
    gemm_flops_per_launch = step_flops() / world / 2          # two GEMM launches per step on each rank
    dq_bytes_per_launch = (workloads.dynamic_quant_bytes(M, HIDDEN) + workloads.dynamic_quant_bytes(M, FFN)) / 2
    peaks = measured_peaks()
    int8_peak = 2.0 * peaks["bf16_sustained"]

    # ---- end to end from pinned host memory
    hx, hxd = d["x"].cpu().pin_memory(), d["x_down"].cpu().pin_memory()
    dx, dxd = torch.empty_like(d["x"]), torch.empty_like(d["x_down"])
    ho1 = torch.empty((M, 2 * FFN), dtype=torch.bfloat16).pin_memory()
    ho2 = torch.empty((M, HIDDEN), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        dx.copy_(hx, non_blocking=True)
        dxd.copy_(hxd, non_blocking=True)
        o1, o2 = step(dx, dxd)
        ho1.copy_(o1, non_blocking=True)
        ho2.copy_(o2, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    barrier()
    t0, t1 = ev(), ev()
    t0.record()
    for _ in range(e2e_steps):
        e2e_step()
    t1.record()
    barrier()
    e2e_ms = max_over_ranks(t0.elapsed_time(t1)) / e2e_steps
    e2e = {"value": round(step_flops() / (e2e_ms * 1e-3) / 1e12, 2), "unit": UNIT, "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": hx.numel() * 2 + hxd.numel() * 2, "d2h_bytes_per_step": ho1.numel() * 2 + ho2.numel() * 2}

    out = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "C5 Llama-70B-shaped W8A8 MLP, x bf16 [4096,8192] and [4096,28672], int8 weights "
                               "[8192,57344] and [28672,8192] column-sharded over the ranks, bf16 outputs all-gathered",
                   "tokens": M, "hidden": HIDDEN, "ffn": FFN, "parallelism": f"n-shard{world}",
                   "weight_layout": "[n,k] K-major (transposed view, as LinearQuant passes it)",
                   "l2": "weights streamed per step (705 MB / N per rank) exceed the 126 MB L2; no explicit flush"},
        "clocks": clocks,
        "host_launch_ms_per_step": round(host_ms_step, 4),
        "e2e": e2e,
        "gpu_launches": (4 if world == 1 else 6 if exchange == "p2p_scatter" else 4) * args.steps,
        "roofline": {"bound": "tensor", "kernel": "w8a8_umma_pair_kernel", "achieved": round(gemm_flops_per_launch / (gemm_ms * 1e-3) / 1e12, 1),
                     "peak": round(int8_peak, 1), "unit": "TOP/s", "frac": round(gemm_flops_per_launch / (gemm_ms * 1e-3) / 1e12 / int8_peak, 4),
                     "traffic": None,
                     "peak_source": f"2 x bf16_tflops_sustained ({peaks['source']}); int8 runs at twice the bf16 rate on B200",
                     "avg_launch_ms": round(gemm_ms, 4)},
        "roofline_dynamic_quant": {"bound": "hbm", "kernel": "dynamic_quant_rows", "achieved": round(dq_bytes_per_launch / (dq_ms * 1e-3) / 1e9, 1),
                                   "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                   "frac": round(dq_bytes_per_launch / (dq_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                                   "avg_launch_ms": round(dq_ms, 4), "peak_source": peaks["source"]},
    }
    if world > 1:
        compute_ms = 2 * gemm_ms + 2 * dq_ms
        out["compute_phase"] = {"ms_per_step": round(compute_ms, 4),
                                "value": round(step_flops() / (compute_ms * 1e-3) / 1e12, 2), "unit": UNIT,
                                "note": "rank-0 GEMM + dynamic-quant kernels only"}
        out["exposed_gather_ms_per_step"] = round(ms_step - compute_ms, 4)
        recv = (world - 1) / world * (M * 2 * FFN + M * HIDDEN) * 2
        out["gather_link_floor_ms"] = round(recv / 770e9 * 1e3, 4)
        if exchange == "p2p_scatter":
            # the same push measured on its own (no GEMM before it): kernel only, then kernel + barrier
            def timed(fn, n=5):
                fn(); barrier()
                a, b = ev(), ev()
                a.record()
                for _ in range(n):
                    fn()
                b.record(); torch.cuda.synchronize()
                return max_over_ranks(a.elapsed_time(b) / n)
            push_only = timed(lambda: _cabi.scatter_columns(gat_gu.full, gat_gu.peer_ptrs, gat_gu.lo, gat_gu.hi))
            push_barrier = timed(lambda: gat_gu.gather())
            out["exchange_isolated_ms"] = {"gate_up_push": round(push_only, 4), "gate_up_push_and_barrier": round(push_barrier, 4)}
        out["exchange"] = exchange
        out["exchange_ms"] = {"gate_up": round(time_events(comm_events[0::2]) / max(1, len(comm_events[0::2])), 4),
                                             "down": round(time_events(comm_events[1::2]) / max(1, len(comm_events[1::2])), 4)}
        out["gather_note"] = ("p2p_scatter: the GEMM writes its column block into a peer-mapped [M,N] matrix and "
                              "b200q_scatter_columns pushes it to every peer with 128-bit stores over NVLink, then a "
                              "device-side barrier; nccl_all_gather: all_gather_into_tensor plus one re-interleave copy. "
                              "link floor = bytes each GPU must receive / 770 GB/s")
    if rank == 0 and world == 1:
        out["c2_linears_m2048"] = bench_c2(ops, device, int8_peak)
        out["cpu_baseline"] = cpu_baseline(d, sample_rows=2048)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def bench_c2(ops, device, int8_peak):
    """The four Llama-7B-shaped linears at M = 2048 (dynamic quant + GEMM), timed one by one with a
    rotating set of weights larger than L2."""
    from pytorch_b200 import workloads
    res = []
    for (k, n) in workloads.C2_KN:
        copies = max(2, int(300e6 // (k * n)) + 1)
        ws = [torch.randint(-127, 128, (n, k), device=device, dtype=torch.int8) for _ in range(copies)]
        xs = [torch.randn((2048, k), device=device, dtype=torch.bfloat16) for _ in range(4)]
        sm = torch.rand((k,), device=device) + 0.5
        sc = torch.rand((n,), device=device) * 9e-3 + 1e-3
        q, s = ops.npu_dynamic_quant(xs[0], smooth_scales=sm)
        gemm, dq = [], []
        for it in range(3 + 20):
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record()
            q, s = ops.npu_dynamic_quant(xs[it % 4], smooth_scales=sm)
            e[1].record()
            ops.npu_quant_matmul(q, ws[it % copies].t(), sc, pertoken_scale=s, output_dtype=torch.bfloat16)
            e[2].record()
            if it >= 3:
                dq.append((e[0], e[1])); gemm.append((e[1], e[2]))
        torch.cuda.synchronize()
        g_ms = time_events(gemm) / len(gemm)
        d_ms = time_events(dq) / len(dq)
        tops = 2.0 * 2048 * k * n / (g_ms * 1e-3) / 1e12
        res.append({"k": k, "n": n, "gemm_us": round(g_ms * 1e3, 1), "tops": round(tops, 1),
                    "frac_of_int8_peak": round(tops / int8_peak, 3), "dynamic_quant_us": round(d_ms * 1e3, 1),
                    "dynamic_quant_gbs": round(workloads.dynamic_quant_bytes(2048, k) / (d_ms * 1e-3) / 1e9, 1)})
        del ws
    return res


def cpu_sample(x, smooth, w_nk, scale, oracle):
    q, s = oracle.dynamic_quant(x, smooth)
    return oracle.quant_matmul(q, w_nk.t(), scale, pertoken_scale=s, output_dtype=torch.bfloat16)


def cpu_baseline(d, sample_rows: int):
    """The CPU oracle on a bounded sample of the same step: `sample_rows` of the 4096 tokens through
    half of each weight's columns, all host threads torch uses."""
    from oracle import quant_oracle as oracle
    n_gu, n_dn = d["w_gu"].shape[0] // 2, d["w_dn"].shape[0] // 2
    x, xd = d["x"][:sample_rows].cpu(), d["x_down"][:sample_rows].cpu()
    w1, s1 = d["w_gu"][:n_gu].cpu(), d["s_gu"][:n_gu].cpu()
    w2, s2 = d["w_dn"][:n_dn].cpu(), d["s_dn"][:n_dn].cpu()
    sm, smd = d["smooth"].cpu(), d["smooth_down"].cpu()
    t = time.perf_counter()
    cpu_sample(x, sm, w1, s1, oracle)
    cpu_sample(xd, smd, w2, s2, oracle)
    dt = time.perf_counter() - t
    flops = 2.0 * sample_rows * (HIDDEN * n_gu + FFN * n_dn)
    return {"value": round(flops / dt / 1e12, 4), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "seconds": round(dt, 2),
            "sample": f"{sample_rows} of {M} tokens x first half of each weight's columns "
                      f"(gate/up {n_gu}, down {n_dn}); dynamic quant + exact int GEMM + dequant"}


def run_reference(args):
    """The reference's own implementation of this path is closed (aclnn kernels behind an un-vendored
    submodule), so the reference arm times the CPU oracle, which restates the reference's CPU golden
    compositions, on the host cores: each step is a bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1 for its children; the CPU arm uses every host core.
    torch.set_num_threads(os.cpu_count() or 1)
    from oracle import quant_oracle as oracle
    rows = 128
    g = torch.Generator().manual_seed(5000)
    n_gu, n_dn = FFN // 2, HIDDEN // 4
    x = torch.randn((rows, HIDDEN), generator=g).to(torch.bfloat16)
    xd = torch.randn((rows, FFN), generator=g).to(torch.bfloat16)
    sm, smd = torch.rand(HIDDEN, generator=g) * 1.5 + 0.5, torch.rand(FFN, generator=g) * 1.5 + 0.5
    w1 = torch.randint(-127, 128, (n_gu, HIDDEN), generator=g, dtype=torch.int32).to(torch.int8)
    w2 = torch.randint(-127, 128, (n_dn, FFN), generator=g, dtype=torch.int32).to(torch.int8)
    s1, s2 = torch.rand(n_gu, generator=g) * 9e-3 + 1e-3, torch.rand(n_dn, generator=g) * 9e-3 + 1e-3
    flops = 2.0 * rows * (HIDDEN * n_gu + FFN * n_dn)

    def step():
        cpu_sample(x, sm, w1, s1, oracle)
        cpu_sample(xd, smd, w2, s2, oracle)

    for _ in range(min(args.warmup, 3)):
        step()
    t = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t) / args.steps
    value = round(flops / dt / 1e12, 4)
    sample = (f"{rows} of {M} tokens x {n_gu} of {2 * FFN} gate/up columns and {n_dn} of {HIDDEN} down columns per step; "
              "dynamic quant + exact int GEMM + dequant on the host")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "C5 Llama-70B-shaped W8A8 MLP (bounded sample per step)", "tokens": M, "hidden": HIDDEN,
                   "ffn": FFN},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the W8A8 quantized-inference path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python bench.py --op {dq,dqa,sgq,aq,qmm,w4,suite} [--m M --k K --n N ...]     single-operator timing

Workload at every N: the Llama-70B-shaped W8A8 MLP of the benchmark configurations
(x bf16 [4096,8192] -> dynamic quant with smooth scales -> gate/up GEMM against an int8
[8192,57344] weight; x_down bf16 [4096,28672] -> dynamic quant -> down GEMM against an int8
[28672,8192] weight; bf16 outputs), the weights column-sharded over the N ranks with their
per-channel scales and the outputs gathered over NVLink when N > 1 (the GEMM's epilogue stores
its tiles into every peer's matrix).  One step is one pass of that path over one batch of 4096
tokens; total work is fixed, so scaling is "strong".  Inputs are seeded on the CPU
(pytorch_b200.workloads.config5_shard) and, outside the timed region, the outputs are compared
with the CPU oracle ("parity_checked").  At N = 1 the line also carries the other benchmark
configurations (Llama-7B-shaped linears, W4A16, batched W8A8) as extra keys, each timed alone by
CUDA-graph replay.

Prints ONE JSON line on rank 0.  `value` is whole-job TOPS (2*M*K*N summed over the two GEMMs
and divided by the max-over-ranks device time per step) with inputs resident in HBM; `e2e`
repeats the measurement from pinned host buffers with the host->device copy of the activations
and the device->host copy of the outputs inside the timed region.
"""
from __future__ import annotations

import argparse
import ctypes as C
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
NOMINAL_INT8_TOPS = 4500.0          # B200 dense int8, datasheet
L2_BYTES = 126e6

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the two kernels the rooflines are
# quoted on, from one ncu capture each on a smaller case of the same kernel, as a ratio to that case's
# algorithmic bytes; the bench scales the ratio to its own launches (traffic grows in proportion with the rows
# and columns processed).  Sources: profiles/w8a8_umma_pair_kernel_m4096_k8192_n7168.md,
# profiles/dynamic_quant_rows_m4096_k8192.md.
# GEMM: (101.18 + 39.22) MB measured / 151.04 MB algorithmic; dynamic quant: (67.16 + 4.72) MB / 100.71 MB (the
# int8 output of a launch is still in L2 when the kernel ends, so part of the write-back is not in its window).
NCU_TRAFFIC_RATIO = {"w8a8_umma_pair_kernel": 0.93, "dynamic_quant_rows": 0.71}


def step_flops():
    return 2.0 * M * HIDDEN * (2 * FFN) + 2.0 * M * FFN * HIDDEN


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def int8_peak(peaks, timed_seconds: float):
    """The tensor roofline's denominator.  No int8 figure is measured on this pool; the int8 pipe of B200 runs
    at twice the bf16 rate (4.5 against 2.25 PFLOP/s nominal), so the ceiling is twice the measured cuBLAS bf16
    rate: the burst figure for a timed region under a second (clocks have not settled under the power cap
    yet), the sustained one for longer regions."""
    if timed_seconds < 1.0:
        return 2.0 * peaks["bf16"], f"2 x bf16_tflops burst ({peaks['source']}); timed region {timed_seconds:.2f} s"
    return 2.0 * peaks["bf16_sustained"], f"2 x bf16_tflops_sustained ({peaks['source']}); timed region {timed_seconds:.1f} s"


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


def ev():
    return torch.cuda.Event(enable_timing=True)


def time_events(pairs):
    return sum(a.elapsed_time(b) for a, b in pairs)


# ------------------------------------------------------------------------------------------------
# Single-operator timing through the C ABI.  Argument structs are built once and the calls are replayed
# from a CUDA graph, so the figure is device time per call (all kernels of the call, no host launch
# overhead).  Operands rotate over more than the 126 MB L2 so that weight and activation reads come from
# HBM.  plain=True launches without a graph (what a profiler should be pointed at).
def graph_time(calls, iters, plain=False):
    n_buf = len(calls)
    stream = torch.cuda.Stream()
    sp = C.c_void_p(stream.cuda_stream)
    with torch.cuda.stream(stream):
        for i in range(3):
            calls[i % n_buf](sp)
        stream.synchronize()
        a, b = ev(), ev()
        if plain:
            a.record(stream)
            for i in range(iters):
                calls[i % n_buf](sp)
            b.record(stream)
        else:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(iters):
                    calls[i % n_buf](sp)
            g.replay()
            stream.synchronize()
            a.record(stream)
            g.replay()
            b.record(stream)
        stream.synchronize()
    return a.elapsed_time(b) / iters


def _copies(bytes_each, cap=64):
    return min(cap, max(2, int(3 * L2_BYTES // max(bytes_each, 1)) + 1))


def op_dq(cabi, m, k, iters=30, plain=False):
    from pytorch_b200 import workloads
    lib = cabi.lib()
    xs = [torch.randn(m, k, device="cuda", dtype=torch.bfloat16) for _ in range(_copies(m * k * 3))]
    sm = torch.rand(k, device="cuda") + 0.5
    y = torch.empty(m, k, device="cuda", dtype=torch.int8)
    s = torch.empty(m, device="cuda")
    calls = [(lambda sp, x=x: cabi.check(lib.b200q_dynamic_quant(x.data_ptr(), cabi.BF16, sm.data_ptr(), cabi.F32,
                                                                y.data_ptr(), s.data_ptr(), m, k, sp))) for x in xs]
    ms = graph_time(calls, iters, plain)
    by = workloads.dynamic_quant_bytes(m, k)
    return {"op": "dynamic_quant", "m": m, "k": k, "us": round(ms * 1e3, 2), "gbs": round(by / ms / 1e6, 1),
            "algorithmic_bytes": by}


def op_dq_asym(cabi, m, k, iters=30, plain=False):
    from pytorch_b200 import workloads
    lib = cabi.lib()
    xs = [torch.randn(m, k, device="cuda", dtype=torch.bfloat16) for _ in range(_copies(m * k * 3))]
    sm = torch.rand(k, device="cuda") + 0.5
    y = torch.empty(m, k, device="cuda", dtype=torch.int8)
    s, o = torch.empty(m, device="cuda"), torch.empty(m, device="cuda")
    calls = [(lambda sp, x=x: cabi.check(lib.b200q_dynamic_quant_ext(
        x.data_ptr(), cabi.BF16, sm.data_ptr(), cabi.F32, None, 0, y.data_ptr(), s.data_ptr(), o.data_ptr(), m, k, sp)))
        for x in xs]
    ms = graph_time(calls, iters, plain)
    by = workloads.dynamic_quant_bytes(m, k) + 4 * m
    return {"op": "dynamic_quant_asymmetric", "m": m, "k": k, "us": round(ms * 1e3, 2),
            "gbs": round(by / ms / 1e6, 1), "algorithmic_bytes": by}


def op_swiglu_quant(cabi, m, f, iters=30, plain=False):
    lib = cabi.lib()
    xs = [torch.randn(m, 2 * f, device="cuda", dtype=torch.bfloat16) for _ in range(_copies(m * f * 5))]
    sm = torch.rand(f, device="cuda") + 0.5
    y = torch.empty(m, f, device="cuda", dtype=torch.int8)
    s = torch.empty(m, device="cuda")
    calls = [(lambda sp, x=x: cabi.check(lib.b200q_swiglu_quant(x.data_ptr(), cabi.BF16, sm.data_ptr(), cabi.F32, 1,
                                                                y.data_ptr(), s.data_ptr(), m, f, sp))) for x in xs]
    ms = graph_time(calls, iters, plain)
    by = 4 * m * f + m * f + 4 * m + 4 * f
    return {"op": "swiglu_quant", "m": m, "f": f, "us": round(ms * 1e3, 2), "gbs": round(by / ms / 1e6, 1),
            "algorithmic_bytes": by}


def op_anti_quant(cabi, m, n, bits, iters=30, plain=False):
    lib = cabi.lib()
    in_bytes = m * n * bits // 8
    if bits == 8:
        xs = [torch.randint(-128, 128, (m, n), device="cuda", dtype=torch.int8) for _ in range(_copies(m * n * 3))]
    else:
        xs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (m, n // 8), device="cuda", dtype=torch.int32)
              for _ in range(_copies(m * n * 3))]
    sc, of = torch.rand(n, device="cuda") + 0.5, torch.rand(n, device="cuda")
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    calls = [(lambda sp, x=x: cabi.check(lib.b200q_anti_quant(x.data_ptr(), bits, sc.data_ptr(), of.data_ptr(), cabi.F32,
                                                              out.data_ptr(), cabi.BF16, m, n, sp))) for x in xs]
    ms = graph_time(calls, iters, plain)
    by = in_bytes + 2 * m * n + 8 * n
    return {"op": f"anti_quant_int{bits}", "m": m, "n": n, "us": round(ms * 1e3, 2), "gbs": round(by / ms / 1e6, 1),
            "algorithmic_bytes": by}


def op_qmm(cabi, m, k, n, iters=30, plain=False, out_dtype=torch.bfloat16, offset=False, int_bias=False):
    from pytorch_b200 import workloads
    lib = cabi.lib()
    wts = [torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8) for _ in range(_copies(k * n))]
    x1 = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8)
    sc = torch.rand(n, device="cuda") * 9e-3 + 1e-3
    pt = torch.rand(m, device="cuda") * 9e-3 + 1e-3
    of = torch.rand(n, device="cuda") * 8 - 4
    ib = torch.randint(-1000, 1001, (n,), device="cuda", dtype=torch.int32)
    out = torch.empty(m, n, dtype=out_dtype, device="cuda")
    ws = torch.empty(max(1, lib.b200q_quant_matmul_workspace_bytes(m, k, n, 1, k)), dtype=torch.uint8, device="cuda")
    args = []
    for w in wts:
        a = cabi.QuantMatmulArgs()
        a.x1, a.x2, a.m, a.k, a.n = x1.data_ptr(), w.data_ptr(), m, k, n
        a.x2_stride_k, a.x2_stride_n = 1, k
        a.scale, a.scale_dtype, a.scale_len = sc.data_ptr(), cabi.F32, n
        a.pertoken_scale, a.bias_dtype = pt.data_ptr(), cabi.NONE
        if offset:
            a.offset, a.offset_len = of.data_ptr(), n
        if int_bias:
            a.bias, a.bias_dtype = ib.data_ptr(), cabi.I32
        a.out, a.out_dtype = out.data_ptr(), cabi.DTYPE[out_dtype]
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        args.append(a)
    calls = [(lambda sp, a=a: cabi.check(lib.b200q_quant_matmul(C.byref(a), sp))) for a in args]
    ms = graph_time(calls, iters, plain)
    by = workloads.quant_matmul_bytes(m, k, n, bias=int_bias, offset=offset)
    return {"op": "quant_matmul", "m": m, "k": k, "n": n, "us": round(ms * 1e3, 2),
            "tops": round(2.0 * m * k * n / ms / 1e9, 1), "gbs": round(by / ms / 1e6, 1), "algorithmic_bytes": by}


def op_w4(cabi, m, k, n, gs, iters=30, plain=False):
    from pytorch_b200 import workloads
    lib = cabi.lib()
    packs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (k, n // 8), device="cuda", dtype=torch.int32)
             for _ in range(_copies(k * n // 2, 16))]
    groups = k // gs if gs else 1
    sc = (torch.rand(groups, n, device="cuda") * 1.5e-2 + 5e-3).to(torch.bfloat16)
    of = (torch.rand(groups, n, device="cuda") * 2 - 1).to(torch.bfloat16)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    ws = torch.empty(max(1, lib.b200q_weight_quant_matmul_workspace_bytes(m, k, n, 4)), dtype=torch.uint8, device="cuda")
    args = []
    for pk in packs:
        a = cabi.WeightQuantMatmulArgs()
        a.x, a.x_dtype, a.weight, a.weight_bits = x.data_ptr(), cabi.BF16, pk.data_ptr(), 4
        a.m, a.k, a.n = m, k, n
        a.antiquant_scale, a.antiquant_offset, a.group_size = sc.data_ptr(), of.data_ptr(), gs
        a.out = out.data_ptr()
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        args.append(a)
    calls = [(lambda sp, a=a: cabi.check(lib.b200q_weight_quant_matmul(C.byref(a), sp))) for a in args]
    ms = graph_time(calls, iters, plain)
    by = workloads.w4a16_bytes(m, k, n, gs)
    return {"op": "weight_quant_matmul_int4", "m": m, "k": k, "n": n, "gs": gs, "us": round(ms * 1e3, 2),
            "tflops": round(2.0 * m * k * n / ms / 1e9, 1), "gbs": round(by / ms / 1e6, 1), "algorithmic_bytes": by}


def run_op(a):
    """`--op`: one operator (or the whole suite) timed alone; one JSON line per measurement."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --op needs a CUDA device")
    from pytorch_b200 import _cabi as cabi
    from pytorch_b200 import workloads
    it, pl = a.iters, a.plain
    if a.op == "dq":
        print(json.dumps(op_dq(cabi, a.m, a.k, it, pl)))
    elif a.op == "dqa":
        print(json.dumps(op_dq_asym(cabi, a.m, a.k, it, pl)))
    elif a.op == "sgq":
        print(json.dumps(op_swiglu_quant(cabi, a.m, a.n, it, pl)))
    elif a.op == "aq":
        print(json.dumps(op_anti_quant(cabi, a.m, a.n, a.bits, it, pl)))
    elif a.op == "qmm":
        print(json.dumps(op_qmm(cabi, a.m, a.k, a.n, it, pl)))
    elif a.op == "w4":
        print(json.dumps(op_w4(cabi, a.m, a.k, a.n, a.gs, it, pl)))
    else:
        for (m, k) in [(2048, 4096), (2048, 11008), (4096, 8192), (4096, 28672), (16384, 8192)]:
            print(json.dumps(op_dq(cabi, m, k, it, pl)), flush=True)
        for m in workloads.C2_M + (4096,):
            for (k, n) in workloads.C2_KN:
                print(json.dumps(op_qmm(cabi, m, k, n, it, pl)), flush=True)
        for (m, k, n) in [(4096, 8192, 7168), (4096, 28672, 1024), (4096, 8192, 14336), (4096, 28672, 2048)]:
            print(json.dumps(op_qmm(cabi, m, k, n, it, pl)), flush=True)
        for m in workloads.C3_M:
            print(json.dumps(op_w4(cabi, m, workloads.C3_K, workloads.C3_N, workloads.C3_GS, it, pl)), flush=True)
        print(json.dumps(op_dq_asym(cabi, 4096, 8192, it, pl)), flush=True)
        print(json.dumps(op_swiglu_quant(cabi, 4096, 28672, it, pl)), flush=True)
        for bits in (8, 4):
            print(json.dumps(op_anti_quant(cabi, 8192, 8192, bits, it, pl)), flush=True)
    torch.cuda.synchronize()
    print(json.dumps({"device_error": cabi.device_error()}))


# ------------------------------------------------------------------------------------------------
# The benchmark proper.
def exact_matvec_check(acc_dev, q_cpu, weight_nk_cpu, seed):
    """Freivalds check of int32 accumulators `acc_dev` [m, n] = q @ weight^T: (acc v) == q (W v) for a random
    small-integer v, both sides exact (every partial sum is an integer below 2^53 in float64)."""
    n, k = weight_nk_cpu.shape
    g = torch.Generator().manual_seed(seed)
    v = torch.randint(-3, 4, (n,), generator=g, dtype=torch.int64).to(torch.float64)
    lhs = (acc_dev.to(torch.float64) @ v.to(acc_dev.device)).cpu()
    wv = torch.zeros(k, dtype=torch.float64)
    for lo in range(0, n, 8192):
        wv += weight_nk_cpu[lo:lo + 8192].to(torch.float64).t() @ v[lo:lo + 8192]
    return bool(torch.equal(lhs, q_cpu.to(torch.float64) @ wv))


def check_parity(rank, world, device, d, outs, cabi, dist):
    """Outside the timed region.  Every rank: its dynamic-quant outputs against the oracle in full (bit for bit)
    and a Freivalds check of the int32 accumulators of its own weight shards.  Rank 0: 64 full rows of both
    gathered bf16 outputs against the oracle, with every rank's weights regenerated from their seeds.  All
    ranks: the gathered matrices must be identical everywhere.  Returns True when everything agreed."""
    from oracle import quant_oracle as oracle
    from pytorch_b200 import workloads
    o_gu, o_dn = outs
    ok = True
    x, sm, xd, smd = d["x"], d["smooth_scales"], d["x_down"], d["smooth_scales_down"]
    q, s = cabi.dynamic_quant(x.to(device), sm.to(device))
    qo, so = oracle.dynamic_quant(x, sm)
    ok &= bool(torch.equal(q.cpu(), qo) and torch.equal(s.cpu().view(torch.int32), so.view(torch.int32)))
    q2, s2 = cabi.dynamic_quant(xd.to(device), smd.to(device))
    q2o, s2o = oracle.dynamic_quant(xd, smd)
    ok &= bool(torch.equal(q2.cpu(), q2o) and torch.equal(s2.cpu().view(torch.int32), s2o.view(torch.int32)))
    one = torch.ones(1, device=device)
    for qq, qq_cpu, w in ((q, qo, d["gate_up_weight_nk"]), (q2, q2o, d["down_weight_nk"])):
        acc = cabi.quant_matmul(qq, w.to(device).t(), one, output_dtype=torch.int32)
        ok &= exact_matvec_check(acc, qq_cpu, w, 7 + rank)
        del acc
    if rank == 0:
        g = torch.Generator().manual_seed(3)
        rows = torch.randperm(M, generator=g)[:64]
        shards = [d if r == 0 else workloads.config5_shard(r, world) for r in range(world)]
        for full, qq, ss, wk, sk in ((o_gu, qo, so, "gate_up_weight_nk", "gate_up_scale"),
                                     (o_dn, q2o, s2o, "down_weight_nk", "down_scale")):
            got = full[rows.to(device)].cpu()
            per = got.shape[1] // world
            for r in range(world):
                want = oracle.quant_matmul(qq[rows], shards[r][wk].t(), shards[r][sk], pertoken_scale=ss[rows],
                                           output_dtype=torch.bfloat16)
                ok &= bool(torch.equal(got[:, r * per:(r + 1) * per].view(torch.int16), want.view(torch.int16)))
        del shards
    if world > 1:
        for full in outs:                                  # identical gathered matrices on every rank
            h = full.view(torch.int16).to(torch.int64).sum().reshape(1)
            lo, hi = h.clone(), h.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            ok &= bool(lo.item() == hi.item())
        flag = torch.tensor([1 if ok else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(flag.item())
    return ok


def run_b200(args):
    import torch.distributed as dist
    import pytorch_b200  # noqa: F401  (registers torch.ops.npu.*; raises if the extension is missing)
    from pytorch_b200 import _cabi, sharded, workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dist.init_process_group("nccl", device_id=device)
        torch.set_num_threads(max(1, (os.cpu_count() or 8) // world))     # input generation and the parity check
    ops = torch.ops.npu
    d = workloads.config5_shard(rank, world)                               # CPU-seeded, the oracle sees the same bits
    x, x_down = d["x"].to(device), d["x_down"].to(device)
    smooth, smooth_down = d["smooth_scales"].to(device), d["smooth_scales_down"].to(device)
    w_gu, s_gu = d["gate_up_weight_nk"].to(device), d["gate_up_scale"].to(device)
    w_dn, s_dn = d["down_weight_nk"].to(device), d["down_scale"].to(device)

    exchange = "none"
    peers = gat_gu = gat_dn = plans = nopush = None
    if world > 1:
        # The GEMM's epilogue stores its column block into every peer's [M, N] matrix (peer-mapped memory);
        # an NCCL all-gather + re-interleave copy is used only where that memory cannot be set up
        # (BENCH_EXCHANGE=nccl forces it).
        try:
            if os.environ.get("BENCH_EXCHANGE", "p2p") not in ("p2p", "fused"):
                raise RuntimeError("NCCL exchange requested")
            peers = sharded.PeerGroup(device)
            gat_gu = sharded.PeerColumnGather(M, 2 * FFN, torch.bfloat16, device, peers)
            gat_dn = sharded.PeerColumnGather(M, HIDDEN, torch.bfloat16, device, peers)
            exchange = "copy_engine_pipelined" if os.environ.get("BENCH_EXCHANGE", "p2p") == "p2p" else "gemm_epilogue_peer_stores"
        except Exception as exc:                                   # noqa: BLE001
            if rank == 0:
                print(f"[bench] peer-memory exchange unavailable ({exc}); using NCCL all-gather", file=sys.stderr)
            exchange = "nccl_all_gather"
        flag = torch.tensor([1 if exchange != "nccl_all_gather" else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)                # all ranks must agree
        if int(flag.item()) == 0:
            exchange = "nccl_all_gather"
            peers = None
            gat_gu = sharded.ColumnShardedOutput(M, 2 * FFN, torch.bfloat16, device)
            gat_dn = sharded.ColumnShardedOutput(M, HIDDEN, torch.bfloat16, device)
    else:
        gat_gu = sharded.LocalOutput(M, 2 * FFN, torch.bfloat16, device)
        gat_dn = sharded.LocalOutput(M, HIDDEN, torch.bfloat16, device)
    if exchange != "nccl_all_gather":
        plans = (sharded.ShardedW8A8LinearPlan(x, smooth, w_gu, s_gu, gat_gu),
                 sharded.ShardedW8A8LinearPlan(x_down, smooth_down, w_dn, s_dn, gat_dn))
        if world > 1:
            nopush = (sharded.ShardedW8A8LinearPlan(x, smooth, w_gu, s_gu, gat_gu, fused_push=False),
                      sharded.ShardedW8A8LinearPlan(x_down, smooth_down, w_dn, s_dn, gat_dn, fused_push=False))
    gemm_events, dq_events = [], []
    pipe = sharded.PipelinedExchange(peers, (gat_gu, gat_dn), device) if exchange == "copy_engine_pipelined" else None

    def step_pipelined(xi, xdi, record=False):
        """The same four kernels writing only their own column blocks; each block goes to the peers on the copy
        engines behind its GEMM, on a side stream, followed there by the cross-rank barrier, while this
        stream goes on with the next step (two result buffers; step i+2 waits for step i's copies)."""
        e = [ev() for _ in range(5)] if record else None
        pipe.begin_step()
        if record: e[0].record()
        nopush[0].quant(xi)
        if record: e[1].record()
        nopush[1].quant(xdi)
        if record: e[2].record()
        nopush[0].matmul(push=False)
        if record: e[3].record()
        pipe.produced(0)
        nopush[1].matmul(push=False)
        if record: e[4].record()
        pipe.produced(1)
        o1, o2 = gat_gu.full, gat_dn.full
        pipe.end_step()
        if record:
            dq_events.extend([(e[0], e[1]), (e[1], e[2])])
            gemm_events.extend([(e[2], e[3]), (e[3], e[4])])
        return o1, o2

    def step(xi, xdi, record=False):
        """One pass of the path: both dynamic quantisations, then both GEMMs (the two projections of this
        configuration take independent inputs, so the order inside the step is free; quantising first keeps the
        bandwidth-bound kernels away from the write-back of the 470 MB gate/up output).  Four C-ABI calls on
        prepared argument blocks; at N > 1 each GEMM launch also writes the peers' matrices and one
        cross-rank barrier ends the step.  (NCCL variant: the public operators plus all_gather.)"""
        e = [ev() for _ in range(5)] if record else None
        if record: e[0].record()
        if plans is not None:
            plans[0].quant(xi)
            if record: e[1].record()
            plans[1].quant(xdi)
            if record: e[2].record()
            plans[0].matmul()
            if record: e[3].record()
            plans[1].matmul()
            if record: e[4].record()
            if peers is not None:
                peers.barrier()
            o1, o2 = gat_gu.full, gat_dn.full
            gat_gu.advance(); gat_dn.advance()
        else:
            o1, o2 = step_public(xi, xdi, e)
        if record:
            dq_events.extend([(e[0], e[1]), (e[1], e[2])])
            gemm_events.extend([(e[2], e[3]), (e[3], e[4])])
        return o1, o2

    def step_public(xi, xdi, e=None):
        """The same pass through the public operators torch.ops.npu.* (what a user of the reference calls)."""
        q, s = ops.npu_dynamic_quant(xi, smooth_scales=smooth)
        if e: e[1].record()
        q2, s2 = ops.npu_dynamic_quant(xdi, smooth_scales=smooth_down)
        if e: e[2].record()
        y1 = ops.npu_quant_matmul(q, w_gu.t(), s_gu, pertoken_scale=s, output_dtype=torch.bfloat16)
        if e: e[3].record()
        y2 = ops.npu_quant_matmul(q2, w_dn.t(), s_dn, pertoken_scale=s2, output_dtype=torch.bfloat16)
        if e: e[4].record()
        if world > 1:
            return gat_gu.gather(y1), gat_dn.gather(y2)
        return y1, y2

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

    headline_step = step_pipelined if pipe is not None else step

    def timed_steps(n, record=False):
        barrier()
        t0, t1 = ev(), ev()
        t0.record()
        h0 = time.perf_counter()
        for _ in range(n):
            headline_step(x, x_down, record)
        if pipe is not None:
            pipe.drain()                                   # the last steps' copies and barriers are inside the interval
        t1.record()
        host_ms = (time.perf_counter() - h0) * 1e3 / n
        barrier()
        return max_over_ranks(t0.elapsed_time(t1)), host_ms

    # ---- device-resident measurement
    for _ in range(args.warmup):
        headline_step(x, x_down)
    barrier()
    # Only the rank that prints the line samples its GPU: eight processes polling NVML at this rate
    # would contend with each other's kernel launches.  The sampler is set up before the last barrier,
    # so that the rank that pays for the NVML start-up does not enter the timed region late.
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler is not None:
        sampler.start()
    ms_total, host_ms_step = timed_steps(args.steps)
    clocks = sampler.stop() if sampler is not None else None
    ms_step = ms_total / args.steps
    value = step_flops() / (ms_step * 1e-3) / 1e12
    # per-kernel events from extra steps through the same path (same kernels, same buffers)
    timed_steps(4, record=True)
    outs = headline_step(x, x_down)
    barrier()
    gemm_ms = time_events(gemm_events) / len(gemm_events)
    dq_ms = time_events(dq_events) / len(dq_events)
    dev_err = _cabi.device_error()
    parity_ok = check_parity(rank, world, device, d, outs, _cabi, dist) if not args.no_parity else None
    if parity_ok is not None and dev_err != 0:
        parity_ok = False                                  # a kernel gave up a bounded wait: its output cannot be trusted
    if peers is not None:
        peers.check()

    # ---- the same step for at least three seconds: clocks settle under the power cap
    sustained = None
    if args.sustained_seconds > 0:
        n_sus = max(args.steps, int(args.sustained_seconds * 1e3 / ms_step) + 1)
        s2 = ClockSampler(local) if rank == 0 else None
        if s2 is not None:
            s2.start()
        ms_sus, _ = timed_steps(n_sus)
        c2 = s2.stop() if s2 is not None else None
        sustained = {"steps": n_sus, "seconds": round(ms_sus * 1e-3, 2), "ms_per_step": round(ms_sus / n_sus, 4),
                     "value": round(step_flops() / (ms_sus / n_sus * 1e-3) / 1e12, 2), "unit": UNIT, "clocks": c2}

    gemm_flops_per_launch = step_flops() / world / 2          # two GEMM launches per step on each rank
    dq_bytes_per_launch = (workloads.dynamic_quant_bytes(M, HIDDEN) + workloads.dynamic_quant_bytes(M, FFN)) / 2
    peaks = measured_peaks()
    peak_i8, peak_src = int8_peak(peaks, ms_total * 1e-3)
    return dict(world=world, rank=rank, device=device, d=d, dist=dist, peers=peers, plans=plans, nopush=nopush,
                gat=(gat_gu, gat_dn), step=step, step_public=step_public, barrier=barrier, max_over_ranks=max_over_ranks, x=x, x_down=x_down,
                exchange=exchange, clocks=clocks, ms_step=ms_step, ms_total=ms_total, value=value, host_ms_step=host_ms_step,
                gemm_ms=gemm_ms, dq_ms=dq_ms, dev_err=dev_err, parity_ok=parity_ok, sustained=sustained,
                gemm_flops_per_launch=gemm_flops_per_launch, dq_bytes_per_launch=dq_bytes_per_launch, peaks=peaks,
                peak_i8=peak_i8, peak_src=peak_src, timed_steps=timed_steps,
                tensors=dict(smooth=smooth, smooth_down=smooth_down, w_gu=w_gu, s_gu=s_gu, w_dn=w_dn, s_dn=s_dn))


def measure_e2e(c, args):
    """The same step end to end, as a serving loop would run it: every step copies its activations from pinned
    host memory to the device and its outputs back (each rank the column block it computed when N > 1, so that
    every output byte crosses PCIe once; the whole matrices at N = 1).  The three stages run on three streams
    with two sets of buffers, so that the upload of step i+1, the kernels of step i and the download of step
    i-1 overlap (PCIe is full duplex); every byte of every step is still copied inside the timed region.  At
    N = 1 the kernels are launched through the public operators torch.ops.npu.*."""
    world, rank, device = c["world"], c["rank"], c["device"]
    x, x_down = c["x"], c["x_down"]
    hx, hxd = x.cpu().pin_memory(), x_down.cpu().pin_memory()
    dx = [torch.empty_like(x) for _ in range(2)]
    dxd = [torch.empty_like(x_down) for _ in range(2)]
    n1, n2 = 2 * FFN // world, HIDDEN // world
    ho1 = [torch.empty((M, n1), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    ho2 = [torch.empty((M, n2), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    ev_in = [torch.cuda.Event() for _ in range(2)]        # upload of buffer set b has landed
    ev_used = [torch.cuda.Event() for _ in range(2)]      # the kernels have consumed buffer set b
    ev_out = [torch.cuda.Event() for _ in range(2)]       # download of the outputs of set b has finished
    for e_ in ev_used + ev_out:
        e_.record(main)
    state = {"i": 0}

    def e2e_step():
        b = state["i"] % 2
        state["i"] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_used[b])
            dx[b].copy_(hx, non_blocking=True)
            dxd[b].copy_(hxd, non_blocking=True)
            ev_in[b].record(s_in)
        main.wait_event(ev_in[b])
        main.wait_event(ev_out[b])                         # the result matrices of two steps ago have been read out
        if world > 1:
            # Peers write into this rank's result matrix of step i during their step i+2, which they may start once
            # this rank has joined the barrier of step i+1: that barrier must not be queued before step i's download.
            main.wait_event(ev_out[1 - b])
        o1, o2 = (c["step_public"] if world == 1 else c["step"])(dx[b], dxd[b])
        ev_used[b].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_used[b])
            ho1[b].copy_(o1[:, rank * n1:(rank + 1) * n1], non_blocking=True)
            ho2[b].copy_(o2[:, rank * n2:(rank + 1) * n2], non_blocking=True)
            ev_out[b].record(s_out)
        o1.record_stream(s_out)
        o2.record_stream(s_out)

    def drain():
        main.wait_stream(s_in)
        main.wait_stream(s_out)

    e2e_steps = max(4, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    drain()
    c["barrier"]()
    t0, t1 = ev(), ev()
    t0.record()
    for _ in range(e2e_steps):
        e2e_step()
    drain()
    t1.record()
    c["barrier"]()
    e2e_ms = c["max_over_ranks"](t0.elapsed_time(t1)) / e2e_steps
    return {"value": round(step_flops() / (e2e_ms * 1e-3) / 1e12, 2), "unit": UNIT, "ms_per_step": round(e2e_ms, 4),
            "h2d_bytes_per_step": world * (hx.numel() + hxd.numel()) * 2,
            "d2h_bytes_per_step": world * (ho1[0].numel() + ho2[0].numel()) * 2,
            "note": "every rank copies both activation tensors in (replicated inputs) and its own column blocks out; "
                    "upload, kernels and download of consecutive steps overlap on three streams (two buffer sets)"}


def measure_multi_gpu_extras(c, args):
    """N > 1 only: the compute phase alone (dynamic quant + GEMM with local stores only), and the reference's
    tensor-parallel form of the same MLP (column-parallel gate/up without a gather, row-parallel down projection
    with a reduce-scatter: npu_mm_reduce_scatter_base)."""
    import ctypes
    from oracle import quant_oracle as oracle
    from pytorch_b200 import _cabi, workloads
    world, rank, device, peers = c["world"], c["rank"], c["device"], c["peers"]
    nopush, barrier, mor = c["nopush"], c["barrier"], c["max_over_ranks"]
    out = {}
    # -- compute phase: same kernels, epilogue writes locally only
    def compute_only():
        nopush[0].quant(); nopush[0].matmul(push=False)
        nopush[1].quant(); nopush[1].matmul(push=False)
    for _ in range(3):
        compute_only()
    barrier()
    a, b = ev(), ev()
    a.record()
    for _ in range(args.steps):
        compute_only()
    b.record()
    barrier()
    cms = mor(a.elapsed_time(b)) / args.steps
    out["compute_phase"] = {"ms_per_step": round(cms, 4), "value": round(step_flops() / (cms * 1e-3) / 1e12, 2), "unit": UNIT,
                            "note": "dynamic quant + GEMM kernels with local stores only (no exchange), max over ranks"}
    out["exposed_exchange_ms_per_step"] = round(c["ms_step"] - cms, 4)
    recv = (world - 1) / world * (M * 2 * FFN + M * HIDDEN) * 2
    out["gather_link_floor_ms"] = round(recv / 770e9 * 1e3, 4)
    if c["exchange"] == "copy_engine_pipelined":
        # -- the same step with the exchange fused into the GEMM's epilogue (one kernel computes and stores to the peers)
        for _ in range(3):
            c["step"](c["x"], c["x_down"])
        barrier()
        a, b = ev(), ev()
        a.record()
        for _ in range(args.steps):
            c["step"](c["x"], c["x_down"])
        b.record()
        barrier()
        fms = mor(a.elapsed_time(b)) / args.steps
        out["fused_epilogue_form"] = {"ms_per_step": round(fms, 4), "value": round(step_flops() / (fms * 1e-3) / 1e12, 2),
                                      "unit": UNIT, "note": "exchange = gemm_epilogue_peer_stores: each GEMM launch also stores "
                                      "its tiles into every peer's matrix (TMA tensor stores), one barrier per step"}

    # -- tensor-parallel form
    lib = _cabi.lib()
    kr, rows = FFN // world, M // world
    tp = workloads.config5_row_parallel_down(rank, world)
    w_dn_k, s_dn_k = tp["down_weight_nk"].to(device), tp["down_scale"].to(device)
    xd_slice = c["x_down"][:, rank * kr:(rank + 1) * kr].contiguous()
    sm_slice = c["tensors"]["smooth_down"][rank * kr:(rank + 1) * kr].contiguous()
    q2 = torch.empty((M, kr), dtype=torch.int8, device=device)
    s2 = torch.empty((M,), dtype=torch.float32, device=device)
    stag = [peers.symmetric((world, rows, HIDDEN), torch.float32)[:2] for _ in range(2)]
    res = torch.empty((rows, HIDDEN), dtype=torch.bfloat16, device=device)
    blocks, keep = [], []
    for t, ptrs in stag:
        a_ = _cabi.QuantMatmulArgs()
        a_.x1, a_.x2, a_.m, a_.k, a_.n = q2.data_ptr(), w_dn_k.data_ptr(), M, kr, HIDDEN
        a_.x2_stride_k, a_.x2_stride_n = 1, kr
        a_.scale, a_.scale_dtype, a_.scale_len = s_dn_k.data_ptr(), _cabi.F32, HIDDEN
        a_.pertoken_scale, a_.bias_dtype = s2.data_ptr(), _cabi.NONE
        a_.out, a_.out_dtype, a_.out_row_stride = None, _cabi.F32, HIDDEN
        arr = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(ptrs[dst]) + rank * rows * HIDDEN * 4) for dst in range(world)])
        keep.append(arr)
        a_.peer_out, a_.n_peer_out, a_.route_rows = arr, world, rows
        blocks.append((a_, t))
    cur = [0]

    def tp_step():
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        nopush[0].quant(); nopush[0].matmul(push=False)                 # column-parallel gate/up: stays sharded
        _cabi.check(lib.b200q_dynamic_quant(xd_slice.data_ptr(), _cabi.BF16, sm_slice.data_ptr(), _cabi.F32, q2.data_ptr(),
                                            s2.data_ptr(), M, kr, st))
        a_, t = blocks[cur[0]]
        _cabi.check(lib.b200q_quant_matmul(ctypes.byref(a_), st))       # partial rows routed to their owners
        peers.barrier()
        _cabi.reduce_slots(t, res)
        cur[0] ^= 1

    for _ in range(3):
        tp_step()
    barrier()
    a, b = ev(), ev()
    a.record()
    for _ in range(args.steps):
        tp_step()
    b.record()
    barrier()
    tms = mor(a.elapsed_time(b)) / args.steps
    # parity of the reduce-scatter: rank 0 checks 16 of its rows against the oracle over every rank's K slice
    ok = True
    if rank == 0:
        g = torch.Generator().manual_seed(4)
        pick = torch.randperm(rows, generator=g)[:16]
        x1l, x2l, s1l, s2l = [], [], [], []
        xd_cpu, smd_cpu = c["d"]["x_down"], c["d"]["smooth_scales_down"]
        for r in range(world):
            tr = workloads.config5_row_parallel_down(r, world)
            qq, ss = oracle.dynamic_quant(xd_cpu[pick][:, r * kr:(r + 1) * kr], smd_cpu[r * kr:(r + 1) * kr])
            x1l.append(qq); s1l.append(ss.reshape(-1, 1))
            x2l.append(tr["down_weight_nk"].t()); s2l.append(tr["down_scale"].reshape(1, -1))
        want = torch.cat(oracle.mm_reduce_scatter(x1l, x2l, s1l, s2l, output_dtype=torch.bfloat16))
        ok = bool(torch.equal(res[pick.to(device)].cpu().view(torch.int16), want.view(torch.int16)))
    flag = torch.tensor([1 if ok else 0], device=device)
    c["dist"].all_reduce(flag, op=c["dist"].ReduceOp.MIN)
    recv_tp = (world - 1) / world * rows * world * HIDDEN * 4
    out["tensor_parallel_form"] = {
        "ms_per_step": round(tms, 4), "value": round(step_flops() / (tms * 1e-3) / 1e12, 2), "unit": UNIT,
        "parity_checked": bool(flag.item()), "link_floor_ms": round(recv_tp / 770e9 * 1e3, 4),
        "note": "same FLOPs: column-parallel gate/up kept sharded (no gather), row-parallel down projection "
                "[4096, 28672/N] x [28672/N, 8192] with per-rank dynamic quant, fp32 partial rows routed to their owner "
                "by the GEMM epilogue, one barrier, rank-ordered fp32 sum (npu_mm_reduce_scatter_base); output [4096/N, 8192] per rank"}
    return out


def other_configs(cabi, peaks):
    """N = 1 only: the benchmark configurations that are not the step itself, each operator timed alone (CUDA
    graph replay, operands rotated over more than L2): config 2 (Llama-7B-shaped linears, every M), config 3
    (W4A16, every M) and config 4 (batched W8A8 with offset, int32 bias, fp16 out).  Every entry says which
    roofline bounds it and the fraction reached."""
    from pytorch_b200 import workloads
    hbm, i8, bf = peaks["hbm_gbs"], 2.0 * peaks["bf16"], peaks["bf16"]
    res = {"note": "each call timed alone (all its kernels, device time); peaks: measured HBM copy, 2 x bf16 burst for int8, "
                   "bf16 burst for W4A16; a case is HBM-bound when its algorithmic bytes / HBM peak exceed its ops / tensor peak"}
    c2 = []
    for (k, n) in workloads.C2_KN:
        for m in workloads.C2_M:
            r = op_qmm(cabi, m, k, n, iters=20)
            t_mem, t_mma = r["algorithmic_bytes"] / (hbm * 1e9), 2.0 * m * k * n / (i8 * 1e12)
            bound = "hbm" if t_mem > t_mma else "tensor"
            frac = (r["gbs"] / hbm) if bound == "hbm" else (r["tops"] / i8)
            dq = op_dq(cabi, m, k, iters=20)
            c2.append({"m": m, "k": k, "n": n, "gemm_us": r["us"], "tops": r["tops"], "gbs": r["gbs"], "bound": bound,
                       "frac": round(frac, 3), "frac_of_nominal_int8": round(r["tops"] / NOMINAL_INT8_TOPS, 3),
                       "dynamic_quant_us": dq["us"], "dynamic_quant_gbs": dq["gbs"],
                       "dynamic_quant_frac_of_hbm": round(dq["gbs"] / hbm, 3)})
    res["c2_llama7b_linears"] = c2
    c3 = []
    for m in workloads.C3_M:
        r = op_w4(cabi, m, workloads.C3_K, workloads.C3_N, workloads.C3_GS, iters=20)
        t_mem, t_mma = r["algorithmic_bytes"] / (hbm * 1e9), 2.0 * m * workloads.C3_K * workloads.C3_N / (bf * 1e12)
        bound = "hbm" if t_mem > t_mma else "tensor"
        frac = (r["gbs"] / hbm) if bound == "hbm" else (r["tflops"] / bf)
        c3.append({"m": m, "k": workloads.C3_K, "n": workloads.C3_N, "us": r["us"], "tflops": r["tflops"], "gbs": r["gbs"],
                   "bound": bound, "frac": round(frac, 3)})
    res["c3_w4a16"] = c3
    b, mm, k, n = workloads.C4_SHAPE
    r = op_qmm(cabi, b * mm, k, n, iters=10, out_dtype=torch.float16, offset=True, int_bias=True)
    res["c4_batched_w8a8_offset_bias_fp16"] = {"m": b * mm, "k": k, "n": n, "us": r["us"], "tops": r["tops"], "bound": "tensor",
                                               "frac": round(r["tops"] / i8, 3),
                                               "frac_of_nominal_int8": round(r["tops"] / NOMINAL_INT8_TOPS, 3)}
    # host cost of one decode-shape call through the public operator (launch path, no device wait)
    ops = torch.ops.npu
    x1 = torch.randint(-127, 128, (1, 4096), device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (4096, 4096), device="cuda", dtype=torch.int8)
    sc = torch.rand(4096, device="cuda")
    for _ in range(10):
        ops.npu_quant_matmul(x1, w.t(), sc, output_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    t = time.perf_counter()
    for _ in range(200):
        ops.npu_quant_matmul(x1, w.t(), sc, output_dtype=torch.bfloat16)
    res["host_us_per_call_torch_ops_m1"] = round((time.perf_counter() - t) / 200 * 1e6, 1)
    torch.cuda.synchronize()
    return res


def cpu_sample(x, smooth, w_nk, scale, oracle):
    q, s = oracle.dynamic_quant(x, smooth)
    return oracle.quant_matmul(q, w_nk.t(), scale, pertoken_scale=s, output_dtype=torch.bfloat16)


CPU_SAMPLE_ROWS = int(os.environ.get("BENCH_CPU_SAMPLE_ROWS", "2048"))     # tokens of the CPU legs' sample


def cpu_sample_inputs():
    """The bounded sample both CPU legs time: CPU_SAMPLE_ROWS of the 4096 tokens through the first half of each
    weight's columns (seeded like the benchmark's own inputs)."""
    from pytorch_b200 import workloads
    d = workloads.config5_shard(0, 2)                    # rank 0 of 2 = first half of the columns of both weights
    return dict(x=d["x"][:CPU_SAMPLE_ROWS], xd=d["x_down"][:CPU_SAMPLE_ROWS], sm=d["smooth_scales"],
                smd=d["smooth_scales_down"], w1=d["gate_up_weight_nk"], s1=d["gate_up_scale"],
                w2=d["down_weight_nk"], s2=d["down_scale"])


def cpu_sample_flops(s):
    return 2.0 * s["x"].shape[0] * (HIDDEN * s["w1"].shape[0] + FFN * s["w2"].shape[0])


def cpu_sample_text(s):
    return (f"{s['x'].shape[0]} of {M} tokens x first half of each weight's columns (gate/up {s['w1'].shape[0]}, "
            f"down {s['w2'].shape[0]}); dynamic quant + exact int GEMM + dequant on the host")


def cpu_baseline():
    """The CPU oracle on a bounded sample of the same step, all host threads torch uses."""
    from oracle import quant_oracle as oracle
    torch.set_num_threads(os.cpu_count() or 1)
    s = cpu_sample_inputs()
    t = time.perf_counter()
    cpu_sample(s["x"], s["sm"], s["w1"], s["s1"], oracle)
    cpu_sample(s["xd"], s["smd"], s["w2"], s["s2"], oracle)
    dt = time.perf_counter() - t
    return {"value": round(cpu_sample_flops(s) / dt / 1e12, 4), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "seconds": round(dt, 2), "sample": cpu_sample_text(s)}


def run_and_print(args):
    c = run_b200(args)
    from pytorch_b200 import _cabi
    world, rank = c["world"], c["rank"]
    e2e = measure_e2e(c, args)
    multi = measure_multi_gpu_extras(c, args) if c["nopush"] is not None else {}
    peaks, peak_i8 = c["peaks"], c["peak_i8"]
    gemm_tops = c["gemm_flops_per_launch"] / (c["gemm_ms"] * 1e-3) / 1e12
    dq_gbs = c["dq_bytes_per_launch"] / (c["dq_ms"] * 1e-3) / 1e9
    gemm_alg_bytes = ((M * HIDDEN + HIDDEN * 2 * FFN / world + M * 2 * FFN / world * 2) +
                      (M * FFN + FFN * HIDDEN / world + M * HIDDEN / world * 2)) / 2
    tr_g, tr_d = NCU_TRAFFIC_RATIO["w8a8_umma_pair_kernel"], NCU_TRAFFIC_RATIO["dynamic_quant_rows"]
    frac = gemm_tops / peak_i8
    out = {
        "metric": METRIC, "value": round(c["value"], 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(c["ms_step"], 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "C5 Llama-70B-shaped W8A8 MLP, x bf16 [4096,8192] and [4096,28672], int8 weights "
                               "[8192,57344] and [28672,8192] column-sharded over the ranks, bf16 outputs gathered on every rank",
                   "tokens": M, "hidden": HIDDEN, "ffn": FFN, "parallelism": f"n-shard{world}",
                   "inputs": "seeded on the CPU (workloads.config5_shard), copied to the device before the timed region",
                   "weight_layout": "[n,k] K-major (transposed view, as LinearQuant passes it)",
                   "l2": "weights streamed per step (705 MB / N per rank) exceed the 126 MB L2; no explicit flush"},
        "clocks": c["clocks"],
        "parity_checked": c["parity_ok"],
        "device_error": c["dev_err"],
        "host_launch_ms_per_step": round(c["host_ms_step"], 4),
        "e2e": e2e,
        "gpu_launches": (4 if world == 1 else 5 if c["peers"] is not None else 4) * args.steps,
        "roofline": {"bound": "tensor", "kernel": "w8a8_umma_pair_kernel", "achieved": round(gemm_tops, 1),
                     "peak": round(peak_i8, 1), "unit": "TOP/s", "frac": round(frac, 4),
                     "frac_of_nominal_int8": round(gemm_tops / NOMINAL_INT8_TOPS, 4),
                     "frac_exceeds_1": bool(frac > 1.0),
                     "traffic": None if tr_g is None else round(tr_g * gemm_alg_bytes),
                     "algorithmic_bytes": round(gemm_alg_bytes),
                     "peak_source": c["peak_src"] + "; int8 runs at twice the bf16 rate on B200 (nominal 4500 TOP/s dense)",
                     "avg_launch_ms": round(c["gemm_ms"], 4),
                     "note": "at N > 1 the launch also stores its tiles into the peers' matrices, so its duration "
                             "includes the exchange" if world > 1 else "average of the gate/up and the down launch"},
        "roofline_dynamic_quant": {"bound": "hbm", "kernel": "dynamic_quant_rows", "achieved": round(dq_gbs, 1),
                                   "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(dq_gbs / peaks["hbm_gbs"], 4),
                                   "traffic": None if tr_d is None else round(tr_d * c["dq_bytes_per_launch"]),
                                   "algorithmic_bytes": round(c["dq_bytes_per_launch"]),
                                   "avg_launch_ms": round(c["dq_ms"], 4), "peak_source": peaks["source"]},
        "sustained": c["sustained"],
    }
    if world > 1:
        out.update(multi)
        out["exchange"] = c["exchange"]
        out["exchange_note"] = ("copy_engine_pipelined: every GEMM writes its own column block; behind it, on a side stream, "
                                "one strided copy-engine transfer per peer and the bounded cross-rank barrier, while the "
                                "kernels of the next step run (two result buffers; all copies and barriers of the timed "
                                "steps end inside the timed interval); gemm_epilogue_peer_stores: the GEMM's epilogue "
                                "stores each finished tile into the local [M,N] matrix and into every peer's (TMA tensor "
                                "stores), one bounded barrier per step; nccl_all_gather: all_gather_into_tensor plus one "
                                "re-interleave copy.  link floor = bytes each GPU must receive / 770 GB/s")
    if rank == 0 and world == 1 and not args.no_extras:
        out["other_configs"] = other_configs(_cabi, peaks)
        out["cpu_baseline"] = cpu_baseline()
    torch.cuda.synchronize()
    out["device_error_at_end"] = _cabi.device_error()
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        from pytorch_b200 import collective_ops
        collective_ops.release_contexts()
        c["dist"].barrier()
        c["dist"].destroy_process_group()


def run_reference(args):
    """The reference's own implementation of this path is closed (aclnn kernels behind an un-vendored
    submodule), so the reference arm times the CPU oracle, which restates the reference's CPU golden
    compositions, on the host cores: each step is the same bounded sample of the workload that the
    `cpu_baseline` leg of the other arm times."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1 for its children; the CPU arm uses every host core.
    torch.set_num_threads(os.cpu_count() or 1)
    from oracle import quant_oracle as oracle
    s = cpu_sample_inputs()
    flops = cpu_sample_flops(s)

    def step():
        cpu_sample(s["x"], s["sm"], s["w1"], s["s1"], oracle)
        cpu_sample(s["xd"], s["smd"], s["w2"], s["s2"], oracle)

    for _ in range(min(args.warmup, 1)):
        step()
    t = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t) / args.steps
    value = round(flops / dt / 1e12, 4)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "C5 Llama-70B-shaped W8A8 MLP (bounded sample per step)", "tokens": M, "hidden": HIDDEN,
                   "ffn": FFN},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": cpu_sample_text(s)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--sustained-seconds", type=float, default=3.0, help="length of the extra sustained run (0 = skip)")
    ap.add_argument("--no-extras", action="store_true", help="N = 1: skip the other configurations and the CPU baseline")
    ap.add_argument("--no-parity", action="store_true", help="skip the comparison with the CPU oracle")
    ap.add_argument("--op", default=None, choices=["dq", "dqa", "sgq", "aq", "qmm", "w4", "suite"],
                    help="time one operator alone instead of the benchmark step")
    ap.add_argument("--bits", type=int, default=8)
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--gs", type=int, default=128)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--plain", action="store_true", help="--op: launch without a CUDA graph (for a profiler)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.op:
        run_op(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_and_print(args)


if __name__ == "__main__":
    main()

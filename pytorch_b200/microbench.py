"""Single-operator timing through the C ABI:  python -m pytorch_b200.microbench <op> [sizes]

    dq   --m M --k K                  npu_dynamic_quant, bf16 in, fp32 smooth scales
    qmm  --m M --k K --n N            npu_quant_matmul, [n,k] weight view, per-token scale, bf16 out
    w4   --m M --k K --n N [--gs 128] npu_weight_quant_batchmatmul, int4-packed weight, bf16

Argument structs are built once and the calls are replayed from a CUDA graph, so the figure is
device time per call (all kernels of the call, no host launch overhead).  Operands rotate over
more than the 126 MB L2 so that weight and activation reads come from HBM.  `--plain` launches
without a graph (what a profiler should be pointed at); `--iters` sets the calls per measurement.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import torch

from . import _cabi as cabi
from . import workloads

L2_BYTES = 126e6


def _graph_time(calls, iters, plain):
    n_buf = len(calls)
    stream = torch.cuda.Stream()
    sp = C.c_void_p(stream.cuda_stream)
    with torch.cuda.stream(stream):
        for i in range(3):
            calls[i % n_buf](sp)
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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


def _copies(bytes_each):
    return max(2, int(3 * L2_BYTES // max(bytes_each, 1)) + 1)


def bench_dq(m, k, iters, plain):
    lib = cabi.lib()
    xs = [torch.randn(m, k, device="cuda", dtype=torch.bfloat16) for _ in range(min(_copies(m * k * 3), 64))]
    sm = torch.rand(k, device="cuda") + 0.5
    y = torch.empty(m, k, device="cuda", dtype=torch.int8)
    s = torch.empty(m, device="cuda")
    calls = [(lambda sp, x=x: cabi.check(lib.b200q_dynamic_quant(x.data_ptr(), cabi.BF16, sm.data_ptr(), cabi.F32,
                                                                y.data_ptr(), s.data_ptr(), m, k, sp))) for x in xs]
    ms = _graph_time(calls, iters, plain)
    by = workloads.dynamic_quant_bytes(m, k)
    return {"op": "dynamic_quant", "m": m, "k": k, "us": round(ms * 1e3, 2), "gbs": round(by / ms / 1e6, 1),
            "algorithmic_bytes": by}


def bench_dq_asym(m, k, iters, plain):
    lib = cabi.lib()
    xs = [torch.randn(m, k, device="cuda", dtype=torch.bfloat16) for _ in range(min(_copies(m * k * 3), 64))]
    sm = torch.rand(k, device="cuda") + 0.5
    y = torch.empty(m, k, device="cuda", dtype=torch.int8)
    s, o = torch.empty(m, device="cuda"), torch.empty(m, device="cuda")
    calls = [(lambda sp, x=x: cabi.check(lib.b200q_dynamic_quant_ext(
        x.data_ptr(), cabi.BF16, sm.data_ptr(), cabi.F32, None, 0, y.data_ptr(), s.data_ptr(), o.data_ptr(), m, k, sp)))
        for x in xs]
    ms = _graph_time(calls, iters, plain)
    by = workloads.dynamic_quant_bytes(m, k) + 4 * m
    return {"op": "dynamic_quant_asymmetric", "m": m, "k": k, "us": round(ms * 1e3, 2),
            "gbs": round(by / ms / 1e6, 1), "algorithmic_bytes": by}


def bench_swiglu_quant(m, f, iters, plain):
    lib = cabi.lib()
    xs = [torch.randn(m, 2 * f, device="cuda", dtype=torch.bfloat16) for _ in range(min(_copies(m * f * 5), 64))]
    sm = torch.rand(f, device="cuda") + 0.5
    y = torch.empty(m, f, device="cuda", dtype=torch.int8)
    s = torch.empty(m, device="cuda")
    calls = [(lambda sp, x=x: cabi.check(lib.b200q_swiglu_quant(x.data_ptr(), cabi.BF16, sm.data_ptr(), cabi.F32, 1,
                                                                y.data_ptr(), s.data_ptr(), m, f, sp))) for x in xs]
    ms = _graph_time(calls, iters, plain)
    by = 4 * m * f + m * f + 4 * m + 4 * f
    return {"op": "swiglu_quant", "m": m, "f": f, "us": round(ms * 1e3, 2), "gbs": round(by / ms / 1e6, 1),
            "algorithmic_bytes": by}


def bench_anti_quant(m, n, bits, iters, plain):
    lib = cabi.lib()
    in_bytes = m * n * bits // 8
    if bits == 8:
        xs = [torch.randint(-128, 128, (m, n), device="cuda", dtype=torch.int8)
              for _ in range(min(_copies(m * n * 3), 64))]
    else:
        xs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (m, n // 8), device="cuda", dtype=torch.int32)
              for _ in range(min(_copies(m * n * 3), 64))]
    sc, of = torch.rand(n, device="cuda") + 0.5, torch.rand(n, device="cuda")
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    calls = [(lambda sp, x=x: cabi.check(lib.b200q_anti_quant(x.data_ptr(), bits, sc.data_ptr(), of.data_ptr(), cabi.F32,
                                                              out.data_ptr(), cabi.BF16, m, n, sp))) for x in xs]
    ms = _graph_time(calls, iters, plain)
    by = in_bytes + 2 * m * n + 8 * n
    return {"op": f"anti_quant_int{bits}", "m": m, "n": n, "us": round(ms * 1e3, 2), "gbs": round(by / ms / 1e6, 1),
            "algorithmic_bytes": by}


def bench_qmm(m, k, n, iters, plain):
    lib = cabi.lib()
    wts = [torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8) for _ in range(min(_copies(k * n), 64))]
    x1 = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8)
    sc = torch.rand(n, device="cuda") * 9e-3 + 1e-3
    pt = torch.rand(m, device="cuda") * 9e-3 + 1e-3
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(max(1, lib.b200q_quant_matmul_workspace_bytes(m, k, n, 1, k)), dtype=torch.uint8, device="cuda")
    args = []
    for w in wts:
        a = cabi.QuantMatmulArgs()
        a.x1, a.x2, a.m, a.k, a.n = x1.data_ptr(), w.data_ptr(), m, k, n
        a.x2_stride_k, a.x2_stride_n = 1, k
        a.scale, a.scale_dtype, a.scale_len = sc.data_ptr(), cabi.F32, n
        a.pertoken_scale, a.bias_dtype = pt.data_ptr(), cabi.NONE
        a.out, a.out_dtype = out.data_ptr(), cabi.BF16
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        args.append(a)
    calls = [(lambda sp, a=a: cabi.check(lib.b200q_quant_matmul(C.byref(a), sp))) for a in args]
    ms = _graph_time(calls, iters, plain)
    by = workloads.quant_matmul_bytes(m, k, n)
    return {"op": "quant_matmul", "m": m, "k": k, "n": n, "us": round(ms * 1e3, 2),
            "tops": round(2.0 * m * k * n / ms / 1e9, 1), "gbs": round(by / ms / 1e6, 1), "algorithmic_bytes": by}


def bench_w4(m, k, n, gs, iters, plain):
    lib = cabi.lib()
    packs = [torch.randint(-2 ** 31, 2 ** 31 - 1, (k, n // 8), device="cuda", dtype=torch.int32)
             for _ in range(min(_copies(k * n // 2), 16))]
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
    ms = _graph_time(calls, iters, plain)
    by = workloads.w4a16_bytes(m, k, n, gs)
    return {"op": "weight_quant_matmul_int4", "m": m, "k": k, "n": n, "gs": gs, "us": round(ms * 1e3, 2),
            "tflops": round(2.0 * m * k * n / ms / 1e9, 1), "gbs": round(by / ms / 1e6, 1), "algorithmic_bytes": by}


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=["dq", "dqa", "sgq", "aq", "qmm", "w4", "suite"])
    ap.add_argument("--bits", type=int, default=8)
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--gs", type=int, default=128)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--plain", action="store_true")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    if a.op == "dq":
        print(json.dumps(bench_dq(a.m, a.k, a.iters, a.plain)))
    elif a.op == "dqa":
        print(json.dumps(bench_dq_asym(a.m, a.k, a.iters, a.plain)))
    elif a.op == "sgq":
        print(json.dumps(bench_swiglu_quant(a.m, a.n, a.iters, a.plain)))
    elif a.op == "aq":
        print(json.dumps(bench_anti_quant(a.m, a.n, a.bits, a.iters, a.plain)))
    elif a.op == "qmm":
        print(json.dumps(bench_qmm(a.m, a.k, a.n, a.iters, a.plain)))
    elif a.op == "w4":
        print(json.dumps(bench_w4(a.m, a.k, a.n, a.gs, a.iters, a.plain)))
    else:
        for (m, k) in [(2048, 4096), (2048, 11008), (4096, 8192), (4096, 28672), (16384, 8192)]:
            print(json.dumps(bench_dq(m, k, a.iters, a.plain)), flush=True)
        for m in workloads.C2_M + (4096,):
            for (k, n) in workloads.C2_KN:
                print(json.dumps(bench_qmm(m, k, n, a.iters, a.plain)), flush=True)
        for m in workloads.C3_M:
            print(json.dumps(bench_w4(m, workloads.C3_K, workloads.C3_N, workloads.C3_GS, a.iters, a.plain)), flush=True)
        print(json.dumps(bench_dq_asym(4096, 8192, a.iters, a.plain)), flush=True)
        print(json.dumps(bench_swiglu_quant(4096, 28672, a.iters, a.plain)), flush=True)
        for bits in (8, 4):
            print(json.dumps(bench_anti_quant(8192, 8192, bits, a.iters, a.plain)), flush=True)
        print(json.dumps({"device_error": cabi.device_error()}))


if __name__ == "__main__":
    main()

"""The multi-GPU forms of the GEMM epilogue and their helper kernels, exercised on ONE GPU: local buffers stand
in for the peers' memory (the kernels only see device addresses), and the "ranks" run one after the other.
Covered: the replicating epilogue (all-gather form) of the CTA-pair and the single-CTA kernel, the row-routed
fp32 epilogue plus b200q_reduce_slots (reduce-scatter form) against the oracle of npu_mm_reduce_scatter_base,
the bounded cross-rank barrier, and the path a device-side wait takes when it runs out: error word, host
mirror, operator-level exception.  Nothing here faults or traps the GPU."""
import pytest
import torch

from oracle import quant_oracle as oracle
from pytorch_b200 import workloads

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cabi():
    from pytorch_b200 import _cabi
    _cabi.lib()
    assert torch.cuda.is_available()
    return _cabi


@pytest.mark.parametrize("m,k,n,world", [(640, 512, 2048, 4), (100, 256, 1024, 2), (1024, 1024, 4096, 8),
                                         (300, 384, 512, 4)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_epilogue_replicates_the_column_block_to_every_peer(cabi, m, k, n, world, out_dtype):
    d = workloads.w8a8_linear(m, k, n, 900 + m)
    q, s = oracle.dynamic_quant(d["x"], d["smooth_scales"])
    want = oracle.quant_matmul(q, d["x2"], d["scale"], pertoken_scale=s, output_dtype=out_dtype)
    qd, sd = q.cuda(), s.cuda()
    fulls = [torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda") for _ in range(world)]
    per = n // world
    es = fulls[0].element_size()
    for r in range(world):                                # "rank" r: one launch writes its block everywhere
        w = d["weight_nk"][r * per:(r + 1) * per].cuda()
        peers = [fulls[(r + 1 + i) % world].data_ptr() + r * per * es for i in range(world - 1)]
        cabi.quant_matmul(qd, w.t(), d["scale"][r * per:(r + 1) * per].cuda(), pertoken_scale=sd, output_dtype=out_dtype,
                          out=fulls[r][:, r * per:(r + 1) * per], peer_out=peers)
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(fulls[r].cpu().view(torch.int16), want.view(torch.int16)), f"matrix of rank {r} differs"
    assert cabi.device_error() == 0


def test_copy_engine_push_writes_the_column_block_and_nothing_else(cabi):
    g = torch.Generator().manual_seed(11)
    full = torch.randn((300, 1000), generator=g).to(torch.bfloat16).cuda()
    peers = [torch.full((300, 1000), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    lo, hi = 250, 500
    cabi.copy_columns(full, [p.data_ptr() for p in peers], lo, hi)
    torch.cuda.synchronize()
    for p in peers:
        assert torch.equal(p[:, lo:hi], full[:, lo:hi])
        assert bool((p[:, :lo] == 7.0).all()) and bool((p[:, hi:] == 7.0).all())
    by_kernel = [torch.full((300, 1000), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    cabi.scatter_columns(full, [p.data_ptr() for p in by_kernel], 248, 504)   # the kernel push wants 16-byte multiples
    torch.cuda.synchronize()
    assert torch.equal(by_kernel[0][:, lo:hi], peers[0][:, lo:hi])


def test_replicating_epilogue_rejects_what_it_cannot_write(cabi):
    x1 = torch.zeros(64, 64, dtype=torch.int8, device="cuda")
    w = torch.zeros(96, 64, dtype=torch.int8, device="cuda")
    peer = torch.zeros(64, 96, dtype=torch.int8, device="cuda")
    with pytest.raises(cabi.B200QError) as e:             # int8 output: rows are not whole 128-byte lines
        cabi.quant_matmul(x1, w.t(), torch.ones(1, device="cuda"), peer_out=[peer.data_ptr()])
    assert e.value.status == cabi.ERR_UNSUPPORTED
    with pytest.raises(cabi.B200QError):                  # more destinations than one node has GPUs
        cabi.quant_matmul(x1, w[:64].t(), torch.ones(1, device="cuda"), output_dtype=torch.bfloat16,
                          peer_out=[peer.data_ptr()] * 9)


@pytest.mark.parametrize("m,k,n,world", [(512, 256, 256, 4), (64, 128, 128, 2), (1024, 512, 1024, 8)])
def test_routed_epilogue_and_slot_reduce_give_the_reduce_scatter(cabi, m, k, n, world):
    """Every rank's K slice: x1_r [m, k], x2_r [k, n] with its own per-token and per-channel scales.  The
    routed fp32 epilogue sends row block d of rank r's partial product to slot r of rank d's staging area;
    b200q_reduce_slots adds the slots in rank order.  Must equal the oracle bit for bit."""
    g = torch.Generator().manual_seed(m + world)
    x1 = [workloads.rand_int8((m, k), g) for _ in range(world)]
    w = [workloads.rand_int8((n, k), g) for _ in range(world)]
    s1 = [workloads.rand_uniform((m, 1), g, 1e-3, 1e-2) for _ in range(world)]
    s2 = [workloads.rand_uniform((1, n), g, 1e-3, 1e-2) for _ in range(world)]
    want = oracle.mm_reduce_scatter(x1, [t.t() for t in w], s1, s2, output_dtype=torch.bfloat16)
    rows = m // world
    staging = [torch.full((world, rows, n), float("nan"), device="cuda") for _ in range(world)]
    for r in range(world):
        dest = [staging[dst].data_ptr() + r * rows * n * 4 for dst in range(world)]
        out = cabi.quant_matmul(x1[r].cuda(), w[r].cuda().t(), s2[r].reshape(-1).cuda(),
                                pertoken_scale=s1[r].reshape(-1).cuda(), output_dtype=torch.float32, peer_out=dest,
                                route_rows=rows, out_row_stride=n)
        assert out is None
    for dst in range(world):
        out = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
        mirror = torch.empty_like(out)
        cabi.reduce_slots(staging[dst], out, [mirror.data_ptr()])
        torch.cuda.synchronize()
        assert torch.equal(out.cpu().view(torch.int16), want[dst].view(torch.int16)), f"rows of rank {dst} differ"
        assert torch.equal(mirror, out)
    assert cabi.device_error() == 0


def test_fp32_output_is_the_value_before_the_cast(cabi):
    g = torch.Generator().manual_seed(3)
    for m in (8, 200):
        x1, w = workloads.rand_int8((m, 256), g), workloads.rand_int8((192, 256), g)
        sc, pt = workloads.rand_uniform((192,), g, 1e-3, 1e-2), workloads.rand_uniform((m,), g, 1e-3, 1e-2)
        got = cabi.quant_matmul(x1.cuda(), w.cuda().t(), sc.cuda(), pertoken_scale=pt.cuda(), output_dtype=torch.float32)
        want = oracle.quant_matmul(x1, w.t(), sc, pertoken_scale=pt, output_dtype=torch.float32)
        assert torch.equal(got.cpu().view(torch.int32), want.view(torch.int32))


def test_peer_barrier_passes_when_the_peer_has_arrived_and_gives_up_when_it_has_not(cabi):
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(2)]
    ptrs = [f.data_ptr() for f in flags]
    flags[0][1] = 1                                       # "rank 1" has already announced barrier 1 to rank 0
    cabi.peer_barrier(ptrs, rank=0, epoch=1)
    torch.cuda.synchronize()
    assert flags[1][0].item() == 1 and cabi.device_error() == 0
    # barrier 2: nobody announces it.  The wait has one millisecond, then the kernel records 0x104 and returns.
    cabi.peer_barrier(ptrs, rank=0, epoch=2, timeout_ns=1_000_000)
    torch.cuda.synchronize()
    assert flags[1][0].item() == 2
    assert cabi.device_error(reset=True) == 0x104
    assert cabi.device_error() == 0
    # the context is intact: ordinary work still runs
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_expired_wait_sets_the_error_word_and_the_next_operator_call_raises(cabi):
    import pytorch_b200 as pb
    x = torch.randn(4, 64, device="cuda").to(torch.bfloat16)
    pb.npu_dynamic_quant(x)                               # first operator call on the device sets up the host mirror
    lib = cabi.lib()
    assert lib.b200q_peek_device_error() == 0
    cabi.selftest_expire_wait(200_000)                    # one warp waits 0.2 ms on a barrier nothing arrives on
    torch.cuda.synchronize()
    assert lib.b200q_peek_device_error() == 0x1FF         # read from pinned host memory, no device access
    with pytest.raises(RuntimeError, match="gave up a bounded wait"):
        pb.npu_dynamic_quant(x)
    assert lib.b200q_peek_device_error() == 0 and cabi.device_error() == 0      # raising cleared it
    q, s = pb.npu_dynamic_quant(x)                        # and the operators work again
    qo, so = oracle.dynamic_quant(x.cpu())
    assert torch.equal(q.cpu(), qo)
    with pytest.raises(cabi.B200QError):
        cabi.selftest_expire_wait(0)

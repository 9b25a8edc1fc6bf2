"""b200q_quant_matmul_static_scratch: the matmul entry point for hosts that cannot allocate device
memory when the call is made (all free HBM already pledged to a cache pool, a fixed memory plan owned
by another runtime, or a path where an allocation could synchronise the device).  It must give the
same bits as b200q_quant_matmul, which takes caller-allocated workspace, while using only the scratch
array built into the library, and it must do so on back-to-back calls that share that array.

Collected last on purpose (file name), so that a run stopping at the first failure has already been
through every other test.  It also passes when run alone in a fresh process."""
import pytest
import torch

from pytorch_b200 import workloads

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cabi():
    from pytorch_b200 import _cabi
    _cabi.lib()
    assert torch.cuda.is_available()
    return _cabi


def case(m, k, n, seed, layout):
    g = torch.Generator().manual_seed(seed)
    x1 = workloads.rand_int8((m, k), g).cuda()
    w = workloads.rand_int8((n, k), g).cuda()
    x2 = w.t() if layout == "nk" else w.t().contiguous()
    scale = workloads.rand_uniform((n,), g, 1e-3, 1e-2).cuda()
    pt = workloads.rand_uniform((m,), g, 1e-3, 1e-2).cuda()
    bias = torch.randint(-1000, 1001, (n,), generator=g, dtype=torch.int32).cuda()
    return x1, x2, scale, pt, bias


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row(cabi):
    lib = cabi.lib()
    assert lib.b200q_static_scratch_bytes() == 16 << 20
    # 17..128 tokens against few channel tiles split K across CTAs (int32 accumulators in scratch); a contiguous
    # [k,n] weight needs the re-layout scratch, whatever the token count.  All calls use the same built-in array.
    shapes = [(24, 4096, 1024, "nk"), (64, 1024, 2048, "kn"), (128, 4096, 512, "nk"), (3, 512, 384, "kn")]
    for rep in range(2):
        for i, (m, k, n, layout) in enumerate(shapes):
            x1, x2, scale, pt, bias = case(m, k, n, 100 * rep + i, layout)
            assert lib.b200q_quant_matmul_workspace_bytes(m, k, n, x2.stride(0), x2.stride(1)) > 0
            for out_dtype in (torch.bfloat16, torch.int32):
                kw = dict(bias=bias, output_dtype=out_dtype)
                if out_dtype != torch.int32:
                    kw["pertoken_scale"] = pt
                want = cabi.quant_matmul(x1, x2, scale, **kw)
                out = torch.empty_like(want)                    # allocated up front by the caller
                got = cabi.quant_matmul(x1, x2, scale, out=out, static_scratch=True, **kw)
                again = cabi.quant_matmul(x1, x2, scale, out=torch.empty_like(want), static_scratch=True, **kw)
                torch.cuda.synchronize()
                assert torch.equal(got, want), (rep, m, k, n, layout, out_dtype)
                assert torch.equal(again, want), "second call in a row differs"
    assert cabi.device_error() == 0


def test_static_scratch_needs_no_workspace_for_large_m_and_rejects_oversize(cabi):
    x1, x2, scale, pt, bias = case(256, 512, 256, 7, "nk")      # m > 128: no scratch at all
    want = cabi.quant_matmul(x1, x2, scale, pertoken_scale=pt, output_dtype=torch.float16)
    got = cabi.quant_matmul(x1, x2, scale, pertoken_scale=pt, output_dtype=torch.float16, static_scratch=True)
    assert torch.equal(got, want)
    # a contiguous [k,n] weight of 8192 x 4096 needs 32 MiB for its re-layout: over the 16 MiB limit
    x1 = torch.zeros(8, 8192, dtype=torch.int8, device="cuda")
    x2 = torch.zeros(8192, 4096, dtype=torch.int8, device="cuda")
    with pytest.raises(cabi.B200QError) as e:
        cabi.quant_matmul(x1, x2, torch.ones(1, device="cuda"), output_dtype=torch.int32, static_scratch=True)
    assert e.value.status == cabi.ERR_WORKSPACE and "16777216" in str(e.value)

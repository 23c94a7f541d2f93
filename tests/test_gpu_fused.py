"""The fused Strassen kernel against the separate passes.

One persistent launch multiplies all 7^depth operand blocks while extra warps of every CTA form the
later groups' operand blocks and recombine the quadrants of C. Its adder warps run the same device
code, position by position, as the stand-alone outer-group passes of the pipelined schedule, and the
products come from the same tensor-core main loop, so the two schedules must agree bit for bit; both
must sit within the usual bound of the oracle's model of the library's rounding points.
"""
import pytest
import torch

from oracle import strassen_oracle as so
from tests.conftest import seeded_pair

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_library):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from strassen_triton_b200 import ops as _ops

    return _ops


def rel(x, ref):
    return ((x.double() - ref.double()).norm() / ref.double().norm()).item()


@pytest.mark.parametrize("fuse", [1, 3])
@pytest.mark.parametrize("algo", ["classic", "winograd"])
@pytest.mark.parametrize("depth", [1, 2])
@pytest.mark.parametrize("beta", [0, 1])
def test_fused_matches_separate_passes(ops, fuse, algo, depth, beta):
    M, N, K = 768, 512, 1024
    A, B = seeded_pair(21, (M, K), (K, N), dist="uniform")
    A, B = A.bfloat16().cuda(), B.bfloat16().cuda()
    C0 = torch.randn(M, N, device="cuda").bfloat16()
    Cs, Cf = C0.clone(), C0.clone()
    ops.matmul_out(A, B, Cs, algo=algo, depth=depth, beta=beta, fuse=2, pipeline=1)
    ops.matmul_out(A, B, Cf, algo=algo, depth=depth, beta=beta, fuse=fuse)
    assert torch.equal(Cf, Cs)
    want = so.library_model(A.cpu(), B.cpu(), depth, algo, out_dtype=torch.float32)
    if beta:
        want = want + C0.cpu().float()
    assert rel(Cf.cpu(), want.bfloat16()) < 1.5e-3
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_fused_operand_majors_and_dtypes(ops, dtype, a_t, b_t):
    M, N, K = 512, 1024, 768
    A, B = seeded_pair(5, (M, K), (K, N), scale=K ** -0.5)
    A, B = A.to(dtype).cuda(), B.to(dtype).cuda()
    Av = A.t().contiguous().t() if a_t else A
    Bv = B.t().contiguous().t() if b_t else B
    want = ops.matmul(Av, Bv, algo="classic", depth=2, fuse=2, pipeline=1)
    got = ops.matmul(Av, Bv, algo="classic", depth=2, fuse=1)
    assert torch.equal(got, want)
    model = so.library_model(A.cpu(), B.cpu(), 2, "classic")
    assert rel(got.cpu(), model) < 1e-3
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("shape,depth", [((4096, 4096, 4096), 2), ((2048, 8192, 1024), 2), ((8192, 2048, 2048), 1)])
def test_fused_many_waves(ops, shape, depth):
    """Several hundred tiles per launch: every cluster crosses group boundaries, the adders run ahead
    of the products and the recombination trails them. Compared with the separate passes bit for bit
    and with fp64 through a probe vector (C x = A (B x))."""
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(3)
    A = (torch.rand((M, K), generator=g, device="cuda") * 2 - 1).bfloat16()
    B = (torch.rand((K, N), generator=g, device="cuda") * 2 - 1).bfloat16()
    want = ops.matmul(A, B, algo="classic", depth=depth, fuse=2, pipeline=2)
    for fuse in (1, 3):
        got = ops.matmul(A, B, algo="classic", depth=depth, fuse=fuse)
        again = ops.matmul(A, B, algo="classic", depth=depth, fuse=fuse)
        assert torch.equal(got, again)                     # no atomics on data: bit-identical repeats
        # the sequential schedule sums the recombination in one pass over all levels, the fused one
        # group by group: the fp32 sums can differ in the last bit before the one rounding to bf16
        assert rel(got, want) < 2e-4
    x = torch.randn(N, 1, device="cuda", dtype=torch.float64)
    ref = A.double() @ (B.double() @ x)
    assert rel(got.double() @ x, ref) < 2e-2      # the algorithm's own bf16 error at this depth
    assert ops.device_status() == (0, 0)


def test_fused_reuses_b_blocks_across_row_panels(ops):
    M, N, K = 1024, 2048, 2048
    A, B = seeded_pair(33, (M, K), (K, N), dist="uniform")
    A, B = A.bfloat16().cuda(), B.bfloat16().cuda()
    want = torch.cat([ops.matmul(A[256 * i:256 * (i + 1)], B, algo="classic", depth=2, fuse=2, pipeline=1)
                      for i in range(4)])
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    p, _, _ = ops.make_problem(A[:256], B, C[:256], "classic", 2, fuse=1)
    ws = torch.empty(ops.workspace_bytes(p), dtype=torch.uint8, device="cuda")
    for i in range(4):
        ops.matmul_out(A[256 * i:256 * (i + 1)], B, C[256 * i:256 * (i + 1)], algo="classic", depth=2, fuse=1,
                       b_blocks_ready=i > 0, workspace=ws)
    assert torch.equal(C, want)
    assert ops.device_status() == (0, 0)


def test_fused_request_that_cannot_be_met_is_refused(ops):
    A = torch.zeros(2, 256, 256, device="cuda", dtype=torch.bfloat16)
    C = torch.zeros(2, 256, 256, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.matmul_out(A, A, C, algo="classic", depth=1, fuse=1)        # batched
    with pytest.raises(ValueError):
        ops.matmul_out(A[0], A[0], C[0], algo="classic", depth=1, fuse=1, prod_dtype=torch.float32)

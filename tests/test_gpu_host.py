"""Products with operands and result in host memory (strassen_triton_b200.host): B first, A in row
panels, C back panel by panel on streams of their own. The arithmetic of a panel is that of
ops.matmul on the same rows, so the streamed product must equal the panel-wise product bit for bit
whatever the interleaving of copies and kernels, call after call on the same buffers."""
import pytest
import torch

from tests.conftest import seeded_pair

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods(built_library):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from strassen_triton_b200 import host, ops

    return host, ops


@pytest.mark.parametrize("M,N,K,panels,algo,depth", [
    (1024, 512, 768, 4, "classic", 2),      # four equal panels: B's blocks formed once, reused three times
    (1280, 768, 512, 3, "winograd", 1),     # ragged last panel
    (512, 1024, 1024, 1, "classic", 2),     # one panel
    (2048, 512, 512, 8, "dense", 0),
])
def test_streamed_product_equals_panelwise_product(mods, M, N, K, panels, algo, depth):
    host, ops = mods
    plan = host.HostStreamedMatmul(M, N, K, torch.bfloat16, algo=algo, depth=depth, panels=panels)
    assert plan.h2d_bytes == (M * K + K * N) * 2 and plan.d2h_bytes == M * N * 2
    for seed in (3, 4, 5):                  # repeated calls reuse every buffer and event
        A, B = seeded_pair(seed, (M, K), (K, N), dist="uniform")
        hA, hB = A.bfloat16().pin_memory(), B.bfloat16().pin_memory()
        hC = torch.full((M, N), float("nan"), dtype=torch.bfloat16).pin_memory()
        got = plan(hA, hB, hC)
        torch.cuda.current_stream().synchronize()
        assert got is hC
        dA, dB = hA.cuda(), hB.cuda()
        want = torch.cat([ops.matmul(dA[p0:p1], dB, algo=algo, depth=depth, pipeline=2, fuse=2)
                          for p0, p1 in plan.bounds]).cpu()
        assert torch.equal(hC, want)
        ref = A.bfloat16().double() @ B.bfloat16().double()
        assert ((hC.double() - ref).norm() / ref.norm()).item() < 2e-2
    assert ops.device_status() == (0, 0)


def test_matmul_from_host_allocates_pinned_result_and_rejects_device_tensors(mods):
    host, ops = mods
    A, B = seeded_pair(9, (512, 512), (512, 512))
    hA, hB = A.bfloat16(), B.bfloat16()      # pageable memory works too
    out = host.matmul_from_host(hA, hB, algo="classic", depth=1, panels=2)
    assert not out.is_cuda and out.is_pinned() and out.shape == (512, 512)
    want = torch.cat([ops.matmul(hA.cuda()[r:r + 256], hB.cuda(), algo="classic", depth=1, pipeline=2, fuse=2)
                      for r in (0, 256)]).cpu()
    assert torch.equal(out, want)
    with pytest.raises(ValueError):
        host.matmul_from_host(hA.cuda(), hB)
    with pytest.raises(ValueError):
        host.matmul_from_host(hA, hB[:, :100].t())

"""The row-sharded product on real GPUs. With one visible GPU the plan runs as a single-rank group:
the recombination kernel then stores into one destination (its own symmetric-memory C), which still
exercises the whole orchestration (panels, side stream, barriers, b200s_combine_peers)."""
import socket

import pytest
import torch
import torch.distributed as dist

from tests.conftest import seeded_pair

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture(scope="module")
def single_rank_group(built_library):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    torch.cuda.set_device(0)
    created = not dist.is_initialized()
    if created:
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{_free_port()}", rank=0, world_size=1,
                                device_id=torch.device("cuda", 0))
    yield dist.group.WORLD
    if created:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["store", "push", "copy"])
@pytest.mark.parametrize("panels", [1, 2])
def test_peer_sharded_plan_single_rank(single_rank_group, exchange, panels):
    from strassen_triton_b200 import ops
    from strassen_triton_b200.sharded import PeerShardedMatmul

    M, N, K = 1024, 512, 768
    A, B = seeded_pair(77, (M, K), (K, N), dist="uniform")
    A, B = A.bfloat16().cuda(), B.bfloat16().cuda()
    try:
        plan = PeerShardedMatmul(M, N, K, torch.bfloat16, group=single_rank_group, algo="classic", depth=2,
                                 panels=panels, exchange=exchange)
    except RuntimeError as e:  # symmetric memory not available in this environment
        pytest.skip(f"symmetric memory rendezvous unavailable: {e}")
    for _ in range(2):
        C = plan(A, B)
    torch.cuda.synchronize()
    pr = plan.prow
    want = torch.cat([ops.matmul(A[i * pr:(i + 1) * pr], B, algo="classic", depth=2) for i in range(M // pr)])
    assert torch.equal(C, want)
    ref = A.double() @ B.double()
    assert ((C.double() - ref).norm() / ref.norm()).item() < 2e-2
    assert ops.device_status() == (0, 0)


def test_nccl_sharded_matmul_single_rank(single_rank_group):
    from strassen_triton_b200 import ops
    from strassen_triton_b200.sharded import sharded_matmul

    M, N, K = 512, 512, 512
    A, B = seeded_pair(78, (M, K), (K, N), dist="uniform")
    A, B = A.bfloat16().cuda(), B.bfloat16().cuda()
    C = sharded_matmul(A, B, M, group=single_rank_group, panels=2, algo="classic", depth=1)
    ref = A.double() @ B.double()
    assert ((C.double() - ref).norm() / ref.norm()).item() < 1e-2

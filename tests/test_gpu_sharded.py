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


@pytest.mark.parametrize("exchange", ["store", "push", "copy", "overlap"])
@pytest.mark.parametrize("algo,depth,panels", [("classic", 2, 1), ("classic", 2, 2), ("dense", 0, 2), ("winograd", 1, 1)])
def test_peer_sharded_plan_single_rank(single_rank_group, exchange, algo, depth, panels):
    from strassen_triton_b200 import ops
    from strassen_triton_b200.sharded import PeerShardedMatmul

    M, N, K = 1024, 512, 768
    A, B = seeded_pair(77, (M, K), (K, N), dist="uniform")
    A, B = A.bfloat16().cuda(), B.bfloat16().cuda()
    try:
        plan = PeerShardedMatmul(M, N, K, torch.bfloat16, group=single_rank_group, algo=algo, depth=depth,
                                 panels=panels, exchange=exchange, barrier_ms=200)
    except RuntimeError as e:  # symmetric memory not available in this environment
        pytest.skip(f"symmetric memory rendezvous unavailable: {e}")
    if exchange == "overlap" and panels == 1:
        panels = 4              # the overlapped exchange needs several panels and takes four
    assert (plan.algo, plan.depth, plan.panels, plan.exchange) == (algo, depth, panels, exchange)
    for _ in range(2):
        C = plan(A, B)
    plan.check()
    pr = plan.prow
    want = torch.cat([plan.panel_product(A[i * pr:(i + 1) * pr], B) for i in range(M // pr)])
    assert torch.equal(C, want)
    ref = A.double() @ B.double()
    assert ((C.double() - ref).norm() / ref.norm()).item() < 2e-2
    assert ops.device_status() == (0, 0)


def test_peer_barrier_gives_up_on_a_rank_that_never_arrives(single_rank_group):
    """Two pads, this process plays rank 0, nobody plays rank 1: the barrier waits its limit, reports
    the timeout with its own waiter code and returns; the next launch on the device works."""
    import ctypes

    from strassen_triton_b200 import _lib, ops

    lib = _lib.load()
    pads = torch.zeros(2, 64, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(pads[0].data_ptr(), pads[1].data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.b200s_peer_barrier(ptrs, 0, 2, 1, 5_000_000, stream) == 0          # 5 ms
    assert ops.device_status() == (_lib.ERR_DEVICE_TIMEOUT, 8)
    assert pads[1, 0].item() == 1 and pads[0, 0].item() == 1                     # it did signal both pads
    assert ops.device_status() == (0, 0)
    # with the missing rank's slots filled in by hand the same barrier passes
    pads[0, 1] = 2
    assert lib.b200s_peer_barrier(ptrs, 0, 2, 2, 5_000_000, stream) == 0
    assert ops.device_status() == (0, 0)
    assert lib.b200s_peer_barrier(ptrs, 2, 2, 3, 5_000_000, stream) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_peer_barrier(None, 0, 2, 3, 5_000_000, stream) == _lib.ERR_NULL_POINTER


def test_nccl_gather_with_fp32_products_across_panels(single_rank_group):
    """Several panels with keyword arguments that change the scratch size: the shared buffer is sized
    for the real problem and B's blocks are reused only when they are really there."""
    from strassen_triton_b200 import ops
    from strassen_triton_b200.sharded import sharded_matmul

    M, N, K = 1024, 512, 512
    A, B = seeded_pair(79, (M, K), (K, N), dist="uniform")
    A, B = A.bfloat16().cuda(), B.bfloat16().cuda()
    C = sharded_matmul(A, B, M, group=single_rank_group, panels=4, algo="classic", depth=2, prod_dtype=torch.float32)
    want = torch.cat([ops.matmul(A[256 * i:256 * (i + 1)], B, algo="classic", depth=2, prod_dtype=torch.float32)
                      for i in range(4)])
    assert torch.equal(C, want)


def test_nccl_sharded_matmul_single_rank(single_rank_group):
    from strassen_triton_b200 import ops
    from strassen_triton_b200.sharded import sharded_matmul

    M, N, K = 512, 512, 512
    A, B = seeded_pair(78, (M, K), (K, N), dist="uniform")
    A, B = A.bfloat16().cuda(), B.bfloat16().cuda()
    C = sharded_matmul(A, B, M, group=single_rank_group, panels=2, algo="classic", depth=1)
    ref = A.double() @ B.double()
    assert ((C.double() - ref).norm() / ref.norm()).item() < 1e-2


def test_fsdp_gpt2_steps_single_rank(single_rank_group):
    """Two GPT-2 blocks under FSDP (bf16 mixed precision, use_orig_params) with every Linear a
    LinearStrassen: a few optimizer steps on random tokens run through the library's kernels in
    forward and backward, the loss starts at ln(vocab) and stays finite."""
    import math

    from strassen_triton_b200 import _lib, ops
    from strassen_triton_b200.fsdp_gpt2 import VOCAB_PADDED, build, train_steps

    torch.manual_seed(0)
    model = build(layers=2, seq=128, depth=None, device="cuda", world=1)
    n0 = _lib.load().b200s_launch_count()
    losses = train_steps(model, 4, batch=4, seq=128, rank=0)
    assert all(math.isfinite(x) for x in losses)
    assert abs(losses[0] - math.log(VOCAB_PADDED)) < 0.5
    assert losses[-1] < losses[0] + 0.5
    # 9 Linears (4 per block + lm_head), forward + two backward products each, 4 steps
    assert _lib.load().b200s_launch_count() - n0 >= 9 * 3 * 4
    assert ops.device_status() == (0, 0)

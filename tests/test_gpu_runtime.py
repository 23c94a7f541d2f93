"""Run-time services of the library on a GPU: the bounded wait giving up, the status words of the
no-allocation entry point, and the stage timing. None of these tests faults, traps or hangs the GPU:
the wait that runs out is a one-thread kernel with a limit of a few milliseconds and nothing in
flight."""
import ctypes

import pytest
import torch

from tests.conftest import seeded_pair

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib(built_library):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from strassen_triton_b200 import _lib

    return _lib.load()


def test_bounded_wait_runs_out_and_reports(lib):
    """A wait nobody satisfies returns after its limit, the status words carry the timeout and the
    role code of the waiter, reading them clears them, and the context stays usable."""
    from strassen_triton_b200 import _lib, ops

    assert ops.device_status() == (0, 0)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.b200s_wait_probe(0, stream) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_wait_probe(2_000_000_000, stream) == _lib.ERR_BAD_SHAPE       # the self-test is capped at 1 s
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.b200s_wait_probe(3_000_000, stream) == 0                            # 3 ms
    t1.record()
    torch.cuda.synchronize()
    assert 2.5 <= t0.elapsed_time(t1) < 500.0
    assert ops.device_status() == (_lib.ERR_DEVICE_TIMEOUT, 7)
    assert ops.device_status() == (0, 0)
    # the device still computes
    A, B = seeded_pair(1, (256, 256), (256, 256))
    C = ops.matmul(A.bfloat16().cuda(), B.bfloat16().cuda(), algo="dense", out_dtype=torch.float32)
    ref = A.bfloat16().double() @ B.bfloat16().double()
    assert ((C.cpu().double() - ref).norm() / ref.norm()).item() < 2e-6
    assert ops.device_status() == (0, 0)


def test_static_entry_has_a_status_reader_and_refuses_three_pass_tf32(lib):
    from strassen_triton_b200 import _lib, ops

    s, d = ctypes.c_int32(5), ctypes.c_int32(5)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.b200s_static_status(stream, ctypes.byref(s), ctypes.byref(d)) == 0
    assert (s.value, d.value) == (0, 0)
    assert lib.b200s_static_status(stream, None, None) == _lib.ERR_NULL_POINTER
    A = torch.zeros(256, 256, device="cuda")
    C = torch.zeros(256, 256, device="cuda")
    p, _, _ = ops.make_problem(A, A.t(), C, "classic", 1, precision="3xtf32")
    rc = lib.b200s_matmul_static(ctypes.byref(p), A.data_ptr(), A.data_ptr(), C.data_ptr(), stream)
    assert rc == _lib.ERR_BAD_DTYPE                     # refused, not run at lower precision


@pytest.mark.parametrize("fuse", [2, 3])
def test_stage_timing_covers_the_call(lib, fuse):
    """The four stage durations of the measured calls add up to (almost) the duration of the calls."""
    from strassen_triton_b200 import ops

    n = 8192                                            # large enough for launch gaps not to matter
    g = torch.Generator(device="cuda").manual_seed(0)
    A = (torch.rand((n, n), generator=g, device="cuda") * 2 - 1).bfloat16()
    B = (torch.rand((n, n), generator=g, device="cuda") * 2 - 1).bfloat16()
    C = torch.empty((n, n), device="cuda", dtype=torch.bfloat16)
    p, _, _ = ops.make_problem(A, B, C, "classic", 2, fuse=fuse, pipeline=2)
    ws = torch.empty(ops.workspace_bytes(p), dtype=torch.uint8, device="cuda")
    run = lambda: ops.matmul_out(A, B, C, algo="classic", depth=2, fuse=fuse, pipeline=2, workspace=ws)  # noqa: E731
    for _ in range(3):
        run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ops.stage_timing(8) as stages:
        e0.record()
        for _ in range(5):
            run()
        e1.record()
    total = e0.elapsed_time(e1) / 5
    assert stages["calls"] == 5
    parts = [stages[k] for k in ("operand_blocks_A", "operand_blocks_B", "products", "recombination")]
    assert all(x >= 0 for x in parts) and parts[2] > 0
    assert 0.8 * total <= sum(parts) <= 1.05 * total
    ops.matmul_out(A, B, C, algo="dense")
    with ops.stage_timing(2) as dense:                  # a dense product is all "products"
        ops.matmul_out(A, B, C, algo="dense")
    assert dense["calls"] == 1 and dense["products"] > 0
    assert dense["operand_blocks_A"] + dense["operand_blocks_B"] + dense["recombination"] < 0.05 * dense["products"]
    with ops.stage_timing(2) as none:                   # the multi-stream schedule records nothing
        ops.matmul_out(A, B, C, algo="classic", depth=2, fuse=2, pipeline=1)
    assert none["calls"] == 0


@pytest.mark.parametrize("algo,depth", [("dense", 0), ("classic", 2)])
def test_result_does_not_depend_on_how_many_sms_the_products_get(built_library, algo, depth):
    """b200s_set_product_sms leaves SMs to other kernels. More tiles than CTAs, so the tiles are
    dealt out differently on fewer SMs; the order of the additions along K is tied to the tile, not
    to the CTA that happens to run it, so every bit stays the same."""
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from strassen_triton_b200 import _lib, ops

    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(11)
    M, N, K = (4096, 4096, 2048) if depth == 0 else (8192, 8192, 4096)
    A = (torch.randn(M, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    B = (torch.randn(K, N, device="cuda", generator=g) / K ** 0.5).bfloat16()
    full = ops.matmul(A, B, algo=algo, depth=depth, pipeline=2, fuse=2)
    assert lib.b200s_set_product_sms(96) == 0
    try:
        fewer = ops.matmul(A, B, algo=algo, depth=depth, pipeline=2, fuse=2)
        assert lib.b200s_set_product_sms(30) == 96
        fewest = ops.matmul(A, B, algo=algo, depth=depth, pipeline=2, fuse=2)
    finally:
        lib.b200s_set_product_sms(0)
    assert torch.equal(fewer, full) and torch.equal(fewest, full)
    assert ops.device_status() == (0, 0)

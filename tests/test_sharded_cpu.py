"""The row-sharded product's orchestration on CPU ranks (gloo, world size 2), with the CPU
torch.mm standing in for the per-rank CUDA product."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from strassen_triton_b200.sharded import panel_bounds, row_block


def test_row_blocks_cover_the_matrix():
    for M, W in ((32768, 8), (1000, 3), (7, 8)):
        spans = [row_block(M, W, r) for r in range(W)]
        assert spans[0][0] == 0 and spans[-1][1] == M
        assert all(spans[i][1] == spans[i + 1][0] for i in range(W - 1))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1


def test_panel_bounds():
    assert panel_bounds(4096, 4, 64) == [(0, 1024), (1024, 2048), (2048, 3072), (3072, 4096)]
    assert panel_bounds(100, 4, 64) == [(0, 100)]
    assert panel_bounds(200, 4, 64) == [(0, 128), (128, 200)]
    assert panel_bounds(10, 1) == [(0, 10)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, panels, fail_rank, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from strassen_triton_b200.sharded import sharded_matmul

        g = torch.Generator().manual_seed(0)
        A = torch.randn(M, 96, generator=g)
        B = torch.randn(96, 64, generator=g)
        r0, r1 = row_block(M, world, rank)

        def per_rank(a, b):
            if rank == fail_rank:
                raise RuntimeError("injected failure before the exchange")
            return torch.mm(a, b)

        try:
            C = sharded_matmul(A[r0:r1], B, M, panels=panels, matmul_fn=per_rank)
            err = (C - A @ B).abs().max().item()
            q.put((rank, "ok", err))
        except Exception as e:  # noqa: BLE001
            q.put((rank, "error", type(e).__name__))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(world, M, panels, fail_rank=-1):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, panels, fail_rank, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    return sorted(results)


@pytest.mark.parametrize("M,panels", [(256, 1), (256, 2), (250, 1)])
def test_two_rank_gather_matches_single_process(M, panels):
    results = _run(2, M, panels)
    assert [r[1] for r in results] == ["ok", "ok"], results
    assert all(r[2] < 1e-4 for r in results)


def test_rank_failure_surfaces_as_an_error_not_a_hang():
    """A rank that raises before the exchange: it reports its own error, the other rank's
    collective ends with an error once the process-group timeout runs out."""
    results = _run(2, 256, 1, fail_rank=1)
    status = {r[0]: r[1] for r in results}
    assert status[1] == "error"
    assert status[0] in ("error", "ok")  # gloo may also complete rank 0's send side first


def test_balanced_row_counts():
    from strassen_triton_b200.sharded import balanced_row_counts as b

    assert b(32768, [7.0] * 8, [4096] * 8) == [4096] * 8                       # equal speed: equal blocks
    got = b(32768, [13.4, 11.1, 12.0, 11.5], [8192] * 4)
    assert sum(got) == 32768 and all(r % 256 == 0 for r in got)
    assert got[0] == min(got) and got[1] == max(got)                          # the slowest GPU gets the fewest rows
    # after the split the predicted times are closer together than before
    before = max(13.4, 11.1, 12.0, 11.5) / min(13.4, 11.1, 12.0, 11.5)
    after = [t / 8192 * r for t, r in zip([13.4, 11.1, 12.0, 11.5], got)]
    assert max(after) / min(after) < before
    assert b(1024, [1.0, 100.0], [512, 512]) == [768, 256]                    # nobody is left without rows
    import pytest
    with pytest.raises(ValueError):
        b(1000, [1.0, 1.0], [500, 500])

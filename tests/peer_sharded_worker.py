"""One rank of the multi-GPU check of the row-sharded product (started by test_gpu_multi.py through
torch.distributed.run, one process per GPU).

Every rank builds the same full A and B from a seed, keeps its row block of A, runs the plan, and
compares the WHOLE C it ends up with - its own rows and the rows every peer stored into it - bit for
bit with the panel products computed locally from the full A. It then checks the NCCL all-gather
variant the same way and prints one line, "ok <rank>" or the failure.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from strassen_triton_b200 import ops
    from strassen_triton_b200.sharded import PeerShardedMatmul, row_block, sharded_matmul

    M, N, K = 1024 * world, 1024, 768
    g = torch.Generator("cpu").manual_seed(5)
    A = (2 * torch.rand((M, K), generator=g) - 1).bfloat16().cuda()
    B = (2 * torch.rand((K, N), generator=g) - 1).bfloat16().cuda()
    r0, r1 = row_block(M, world, rank)
    failures = []
    for algo, depth, panels in (("classic", 2, 2), ("dense", 0, 1), ("classic", 1, 1), ("auto", -1, 2)):
        for exchange in ("store", "multicast", "senders", "overlap", "push", "copy"):    # multicast falls back to store without NVLS
            plan = PeerShardedMatmul(M, N, K, torch.bfloat16, algo=algo, depth=depth, panels=panels, exchange=exchange,
                                     barrier_ms=5000)
            for _ in range(2):              # the second call overwrites a C the peers have already read
                C = plan(A[r0:r1], B)
            plan.check()
            pr = plan.prow
            want = torch.cat([plan.panel_product(A[i * pr:(i + 1) * pr], B) for i in range(M // pr)])
            if not torch.equal(C, want):
                bad = (C != want).any(dim=1).nonzero().flatten()
                failures.append(f"{algo}/{depth}/{panels}/{exchange}: {bad.numel()} rows differ, first {bad[:4].tolist()}")
            del plan
    # unequal row blocks (a slower GPU gets fewer rows): rank r takes 768, 1280, 768, 1280, ... rows
    counts = [768 if r % 2 == 0 else 1280 for r in range(world)]
    for algo, depth in (("dense", 0), ("classic", 1)):
        plan = PeerShardedMatmul(M, N, K, torch.bfloat16, algo=algo, depth=depth, row_counts=counts, barrier_ms=5000)
        s0 = plan.row_start
        for _ in range(2):
            C = plan(A[s0:s0 + plan.rows], B)
        plan.check()
        want = torch.cat([plan.panel_product(A[plan.row_starts[r]:plan.row_starts[r] + counts[r]], B) for r in range(world)])
        if plan.panels != 1 or not torch.equal(C, want):
            failures.append(f"unequal row blocks, {algo}/{depth}: differs")
        del plan
    C = sharded_matmul(A[r0:r1], B, M, panels=2, algo="classic", depth=2)
    rows = (r1 - r0) // 2
    want = torch.cat([ops.matmul(A[i * rows:(i + 1) * rows], B, algo="classic", depth=2) for i in range(M // rows)])
    if not torch.equal(C, want):
        failures.append("nccl all-gather variant differs")
    ref = A.double() @ B.double()
    err = ((C.double() - ref).norm() / ref.norm()).item()
    if err > 2e-2:
        failures.append(f"error against fp64 {err}")
    torch.cuda.synchronize()
    dist.barrier()
    print(f"ok {rank}" if not failures else f"FAILED {rank}: " + "; ".join(failures), flush=True)
    dist.destroy_process_group()
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()

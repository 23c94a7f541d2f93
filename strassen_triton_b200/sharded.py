"""Row-sharded matrix product over the GPUs of one node.

A is split into contiguous row blocks, one per rank; B is replicated; every rank runs the whole
Strassen pipeline of libb200s.so on its (M/P) x K block and the bf16 row blocks of C are exchanged
with one all-gather (NCCL over NVLink on GPUs). Row panels let the gather of panel i overlap the
product of panel i+1. The reference has no multi-GPU product; this is the partition its
north-star configuration names (M = N = K = 32768 over 1/2/4/8 GPUs).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def row_block(M: int, world: int, rank: int) -> Tuple[int, int]:
    """[start, stop) rows of rank's block: M // world rows each, the remainder spread over the
    first ranks."""
    base, rem = divmod(M, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def panel_bounds(rows: int, panels: int, quantum: int = 1) -> List[Tuple[int, int]]:
    """Split ``rows`` into at most ``panels`` contiguous pieces whose sizes are multiples of
    ``quantum`` (the last piece takes the remainder)."""
    panels = max(1, min(panels, max(1, rows // max(quantum, 1))))
    step = -(-rows // panels)
    step = -(-step // quantum) * quantum
    out, r = [], 0
    while r < rows:
        out.append((r, min(rows, r + step)))
        r += step
    return out


def sharded_matmul(A_block: torch.Tensor, B: torch.Tensor, M: int, *, group=None, panels: int = 1,
                   matmul_fn: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None,
                   out: Optional[torch.Tensor] = None, **matmul_kwargs) -> torch.Tensor:
    """C = A @ B with A given as this rank's row block (``row_block(M, world, rank)``) and B whole.
    Returns the full M x N product on every rank.

    ``matmul_fn`` is the per-rank product; it defaults to ``strassen_triton_b200.ops.matmul`` and
    exists so the orchestration can be driven on CPU ranks (gloo) in tests."""
    if matmul_fn is None:
        from . import ops

        # One scratch buffer for all panels: B's operand blocks are formed by the first panel and
        # reused by the later ones of the same extent (b_blocks_ready).
        state = {"rows": None, "ws": matmul_kwargs.pop("workspace", None)}

        def matmul_fn(a, b):
            c = torch.empty((a.shape[0], b.shape[-1]), dtype=a.dtype, device=a.device)
            p, _, _ = ops.make_problem(a, b, c, matmul_kwargs.get("algo", "auto"), matmul_kwargs.get("depth", -1))
            need = ops.workspace_bytes(p)
            if need and (state["ws"] is None or state["ws"].numel() < need):
                state["ws"], state["rows"] = torch.empty(need, dtype=torch.uint8, device=a.device), None
            ready = state["rows"] == a.shape[0] and need > 0
            ops.matmul_out(a, b, c, b_blocks_ready=ready, workspace=state["ws"], **matmul_kwargs)
            state["rows"] = a.shape[0]
            return c
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    r0, r1 = row_block(M, world, rank)
    if A_block.shape[0] != r1 - r0:
        raise ValueError(f"rank {rank} holds {A_block.shape[0]} rows of A, expected {r1 - r0}")
    N = B.shape[-1]
    if out is None:
        out = torch.empty((M, N), dtype=A_block.dtype, device=A_block.device)
    elif out.shape != (M, N):
        raise ValueError("out has the wrong shape")
    if world == 1:
        for p0, p1 in panel_bounds(r1 - r0, panels, 64):
            out[p0:p1] = matmul_fn(A_block[p0:p1], B)
        return out

    even = M % world == 0
    use_cuda = A_block.is_cuda
    comm_stream = torch.cuda.Stream(A_block.device) if use_cuda else None
    works = []
    rows = r1 - r0
    bounds = panel_bounds(rows, panels if even else 1, 64)
    for p0, p1 in bounds:
        c_panel = matmul_fn(A_block[p0:p1], B)
        if even:
            # every rank's panel has the same extent: gather straight into the rows of C
            views = [out[r * rows + p0: r * rows + p1] for r in range(world)]
        else:
            views = [out[slice(*row_block(M, world, r))] for r in range(world)]
        if use_cuda:
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream(A_block.device))
            with torch.cuda.stream(comm_stream):
                comm_stream.wait_event(done)
                if even:
                    dist.all_gather(views, c_panel, group=group)
                else:
                    _all_gather_uneven(views, c_panel, group)
                c_panel.record_stream(comm_stream)
        else:
            if even:
                works.append(dist.all_gather(views, c_panel, group=group, async_op=True))
            else:
                _all_gather_uneven(views, c_panel, group)
    for w in works:
        w.wait()
    if use_cuda:
        torch.cuda.current_stream(A_block.device).wait_stream(comm_stream)
    return out


def _all_gather_uneven(views, mine, group):
    """Row blocks differ by one row when M is not a multiple of the world size: broadcast each
    block from its owner."""
    rank = dist.get_rank(group)
    for r, v in enumerate(views):
        if r == rank:
            v.copy_(mine)
        dist.broadcast(v, src=dist.get_global_rank(group, r) if group is not None else r, group=group)

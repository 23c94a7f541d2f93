"""Row-sharded matrix product over the GPUs of one node.

A is split into contiguous row blocks, one per rank; B is replicated; every rank runs the whole
Strassen pipeline of libb200s.so on its (M/P) x K block and the bf16 row blocks of C are exchanged
with one all-gather (NCCL over NVLink on GPUs). Row panels let the gather of panel i overlap the
product of panel i+1. The reference has no multi-GPU product; this is the partition its
multi-GPU configuration names (M = N = K = 32768 over 1/2/4/8 GPUs).
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


class PeerShardedMatmul:
    """Row-sharded C = A @ B whose exchange is fused into the recombination kernel.

    Every rank holds a full-size C in symmetric memory (``torch.distributed._symmetric_memory``:
    each rank's buffer is mapped into every other rank's address space). A rank forms its row block
    of the product panel by panel; the recombination kernel of a panel (``b200s_combine_peers``)
    stores each finished vector into all ranks' C at once with plain global stores over NVLink, on a
    side stream, while the tensor cores already work on the next panel. No all-gather pass and no
    staging copy remain. With ``exchange="copy"`` the kernel writes only the local C and the copy
    engines push the finished rows to the peers instead, which holds no SM during the transfer. Two device-side barriers per call order the ranks: nobody overwrites a
    peer's C before that peer has entered the call, nobody returns before all stores have landed.

    Build it once per shape (allocation and rendezvous are collective and slow), then call it with
    this rank's row block of A and the whole B. The result tensor is reused by every call.
    """

    def __init__(self, M: int, N: int, K: int, dtype=torch.bfloat16, group=None, algo: str = "classic",
                 depth: int = 2, panels: int = 2, device=None, exchange: str = "store"):
        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib, ops

        self._lib, self._ops = _lib, ops
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one node)")
        if M % self.world:
            raise ValueError("M must be a multiple of the number of ranks")
        if depth not in (1, 2):
            raise ValueError("depth must be 1 or 2 (a dense product has no recombination to fuse into)")
        self.M, self.N, self.K, self.dtype, self.algo, self.depth = M, N, K, dtype, algo, depth
        if exchange not in ("store", "copy", "push"):
            raise ValueError("exchange must be 'store', 'push' or 'copy'")
        self.exchange = exchange
        self.rows = M // self.world
        quantum = 8 << depth
        if self.rows % quantum or N % quantum or K % quantum:
            raise ValueError(f"rows per rank, N and K must be multiples of {quantum} at depth {depth}")
        while panels > 1 and (self.rows % panels or (self.rows // panels) % quantum):
            panels -= 1
        self.panels = panels
        self.prow = self.rows // panels
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.C = symm_mem.empty((M, N), dtype=dtype, device=self.device)
        self.hdl = symm_mem.rendezvous(self.C, self.group.group_name)
        self.peer_ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        es = self.C.element_size()
        div, P = 1 << depth, 7 ** depth
        self.P, self.Mb, self.Nb, self.Kb = P, self.prow // div, N // div, K // div
        self.sa = torch.empty(P * self.Mb * self.Kb, dtype=dtype, device=self.device)
        self.sb = torch.empty(P * self.Kb * self.Nb, dtype=dtype, device=self.device)
        self.mp = [torch.empty((P, self.Mb, self.Nb), dtype=dtype, device=self.device) for _ in range(min(2, panels))]
        # products on a high-priority stream, the NVLink-bound recombination on a low-priority one
        self.hi = torch.cuda.Stream(self.device, priority=-1)
        self.side = torch.cuda.Stream(self.device, priority=0)
        self.copy_streams = [torch.cuda.Stream(self.device) for _ in range(self.world)]
        self.ev_gemm = [torch.cuda.Event() for _ in range(panels)]
        self.ev_comb = [torch.cuda.Event() for _ in range(panels)]
        self._es = es

    def __call__(self, A_block: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
        import ctypes

        lib, ops = self._lib.load(), self._ops
        if A_block.shape != (self.rows, self.K) or B.shape != (self.K, self.N):
            raise ValueError("operand shapes do not match the plan")
        user = torch.cuda.current_stream(self.device)
        main = self.hi
        P, Mb, Nb, Kb = self.P, self.Mb, self.Nb, self.Kb
        self.hdl.barrier(channel=0)          # every rank is done with the previous contents of C
        main.wait_stream(user)
        first = None
        for i in range(self.panels):
            p0 = i * self.prow
            a_panel = A_block[p0:p0 + self.prow]
            c_rows = self.C[self.rank * self.rows + p0: self.rank * self.rows + p0 + self.prow]
            prob, a2, b2 = ops.make_problem(a_panel, B, c_rows, self.algo, self.depth)
            a_k, b_k = prob.a_major == self._lib.K_MAJOR, prob.b_major == self._lib.K_MAJOR
            with torch.cuda.stream(main):
                if first is None:
                    first = prob
                    self._lib.check(lib.b200s_preadd(ctypes.byref(prob), 1, b2.data_ptr(), self.sb.data_ptr(),
                                                     main.cuda_stream))
                self._lib.check(lib.b200s_preadd(ctypes.byref(prob), 0, a2.data_ptr(), self.sa.data_ptr(),
                                                 main.cuda_stream))
                sa = self.sa.view(P, Mb, Kb) if a_k else self.sa.view(P, Kb, Mb).transpose(1, 2)
                sb = self.sb.view(P, Nb, Kb).transpose(1, 2) if b_k else self.sb.view(P, Kb, Nb)
                mp = self.mp[i % len(self.mp)]
                if i >= len(self.mp):
                    main.wait_event(self.ev_comb[i - len(self.mp)])   # that recombination still reads this buffer
                ops.matmul_out(sa, sb, mp, algo="dense")
                self.ev_gemm[i].record(main)
            with torch.cuda.stream(self.side):
                self.side.wait_event(self.ev_gemm[i])
                row0 = self.rank * self.rows + p0
                if self.exchange == "store":
                    # one kernel: recombine and store every vector into all ranks' C over NVLink
                    dst = (ctypes.c_void_p * self.world)(*[ptr + row0 * self.N * self._es for ptr in self.peer_ptrs])
                    self._lib.check(lib.b200s_combine_peers(ctypes.byref(prob), mp.data_ptr(), dst, self.world,
                                                            self.side.cuda_stream))
                    self.ev_comb[i].record(self.side)
                elif self.exchange == "push":
                    # recombine into the local C at full occupancy, then a small-footprint kernel that
                    # fits beside the next panel's GEMM CTAs stores the rows into the peers' C
                    self._lib.check(lib.b200s_combine(ctypes.byref(prob), mp.data_ptr(), c_rows.data_ptr(),
                                                      self.side.cuda_stream))
                    self.ev_comb[i].record(self.side)
                    if self.world > 1:
                        peers = [ptr + row0 * self.N * self._es for r, ptr in enumerate(self.peer_ptrs) if r != self.rank]
                        dst = (ctypes.c_void_p * len(peers))(*peers)
                        self._lib.check(lib.b200s_push_rows(c_rows.data_ptr(), dst, len(peers),
                                                            self.prow * self.N * self._es, self.side.cuda_stream))
                else:
                    # recombine into the local C, then let the copy engines push the finished rows to
                    # the peers: no SM is held while the bytes cross NVLink
                    self._lib.check(lib.b200s_combine(ctypes.byref(prob), mp.data_ptr(), c_rows.data_ptr(),
                                                      self.side.cuda_stream))
                    self.ev_comb[i].record(self.side)
                    for r in range(self.world):
                        if r != self.rank:
                            # one stream per peer, so the transfers to different peers run side by side
                            cs = self.copy_streams[r]
                            cs.wait_event(self.ev_comb[i])
                            with torch.cuda.stream(cs):
                                peer_rows = self.hdl.get_buffer(r, (self.prow, self.N), self.dtype, row0 * self.N)
                                peer_rows.copy_(c_rows, non_blocking=True)
        user.wait_stream(main)
        user.wait_stream(self.side)
        if self.exchange == "copy":
            for cs in self.copy_streams:
                user.wait_stream(cs)
        for t in (A_block, B):
            t.record_stream(main)
        self.hdl.barrier(channel=1)          # every rank's stores have been issued and completed
        return self.C

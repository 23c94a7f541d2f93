"""Row-sharded matrix product over the GPUs of one node.

A is split into contiguous row blocks, one per rank; B is replicated; every rank runs the whole
product pipeline of libb200s.so on its (M/P) x K block. Two exchanges of the row blocks of C exist:
``sharded_matmul`` gathers them with an all-gather (NCCL over NVLink on GPUs; row panels let the
gather of panel i overlap the product of panel i+1), ``PeerShardedMatmul`` stores every finished tile
into all ranks' copies of C from the product kernels themselves. The reference has no multi-GPU
product; this is the partition its multi-GPU configuration names (M = N = K = 32768 over 1/2/4/8 GPUs).
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
        # reused by the later ones of the same extent (b_blocks_ready). The buffer is sized from the
        # very problem every call will pose (all keyword arguments included), and the blocks count as
        # ready only when the previous call really used this buffer for the same B and extent.
        state = {"key": None, "ws": matmul_kwargs.pop("workspace", None)}
        names = ("algo", "depth", "beta", "prod_dtype", "precision", "tile_variant", "pipeline", "b_blocks_ready", "fuse")
        defaults = ("auto", -1, 0, None, None, 0, 0, False, 0)

        def matmul_fn(a, b):
            c = torch.empty((a.shape[0], b.shape[-1]), dtype=a.dtype, device=a.device)
            args = [matmul_kwargs.get(n, d) for n, d in zip(names, defaults)]
            p, _, _ = ops.make_problem(a, b, c, *args)
            need = ops.workspace_bytes(p)
            if need and (state["ws"] is None or state["ws"].numel() * state["ws"].element_size() < need):
                state["ws"], state["key"] = torch.empty(need, dtype=torch.uint8, device=a.device), None
            key = (a.shape[0], b.data_ptr(), need)
            ready = need > 0 and state["key"] == key
            kw = {k: v for k, v in matmul_kwargs.items() if k != "b_blocks_ready"}
            ops.matmul_out(a, b, c, b_blocks_ready=ready, workspace=state["ws"], **kw)
            state["key"] = key
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


def balanced_row_counts(M: int, seconds_per_rank, rows_per_rank, quantum: int = 256):
    """Rows for every rank in proportion to the speed it showed (rows_per_rank[r] rows took
    seconds_per_rank[r]), in multiples of ``quantum``, adding up to M; at least one quantum each.
    A strong-scaling step ends with the slowest GPU, and the GPUs of a box differ under a power cap."""
    world = len(seconds_per_rank)
    if world != len(rows_per_rank) or M % quantum or M // quantum < world:
        raise ValueError("cannot split M into quanta over the ranks")
    speed = [max(r, 1) / max(t, 1e-9) for r, t in zip(rows_per_rank, seconds_per_rank)]
    units = M // quantum
    ideal = [units * v / sum(speed) for v in speed]
    counts = [max(1, int(x)) for x in ideal]
    # hand the remaining quanta to the ranks furthest below their share (largest remainder)
    while sum(counts) < units:
        r = max(range(world), key=lambda i: ideal[i] - counts[i])
        counts[r] += 1
    while sum(counts) > units:
        r = max((i for i in range(world) if counts[i] > 1), key=lambda i: counts[i] - ideal[i])
        counts[r] -= 1
    return [c * quantum for c in counts]


class PeerShardedMatmul:
    """Row-sharded C = A @ B whose exchange rides on the product kernels.

    Every rank holds a full-size C in symmetric memory (``torch.distributed._symmetric_memory``:
    each rank's buffer is mapped into every other rank's address space). A rank forms its row block
    of the product panel by panel through ``b200s_matmul_peers``: a dense panel stores each finished
    tile into all ranks' C straight from the GEMM's TMA-store epilogue, a Strassen panel does the same
    from its recombination kernel - plain stores over NVLink, tile by tile, no all-gather pass and no
    staging copy; every load reads local memory. ``exchange="multicast"`` (dense panels, NVLS systems)
    stores each tile once to the allocation's multicast address and lets the NVSwitch replicate it,
    so a rank sends its rows once instead of once per peer. Alternatives kept beside it, all with the
    same result bits: ``"senders"`` (``push_sms`` CTAs of the dense product kernel multiply nothing and
    send finished blocks of columns of C while the others multiply), ``"overlap"`` (row panels; a
    small kernel on a side stream sends panel i from ``push_sms`` SMs while panel i+1 is multiplied on
    the others), ``"push"`` / ``"copy"`` (the panel goes into the local C first, then a copy kernel or
    the copy engines send the finished rows).

    ``row_counts`` gives the ranks row blocks of unequal height (the same list on every rank;
    ``balanced_row_counts`` derives one from measured speeds); rank r then owns rows
    ``row_starts[r] : row_starts[r] + row_counts[r]`` of A and C.

    Algorithm and depth of a panel come from the library's tuner table for the per-rank shape unless
    given (at eight ranks a 4096 x 32768 x 32768 panel is a dense product: with B replicated its
    operand sums would be repeated on every rank).

    Two device-side barriers per call order the ranks (``b200s_peer_barrier`` over a symmetric pad of
    counters): nobody overwrites a peer's C before that peer has entered the call, nobody returns
    before all stores have landed. The barriers are bounded: a peer that never arrives costs
    ``barrier_ms`` and shows up in ``check()`` / ``ops.device_status()`` as a timeout, the GPU is not
    left spinning.

    Build it once per shape (allocation and rendezvous are collective and slow), then call it with
    this rank's row block of A and the whole B. The result tensor is reused by every call.
    """

    def __init__(self, M: int, N: int, K: int, dtype=torch.bfloat16, group=None, algo: str = "auto",
                 depth: int = -1, panels: int = 1, device=None, exchange: str = "auto", barrier_ms: float = 2000.0,
                 push_sms: int = 8, row_counts=None):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib, ops

        self._lib, self._ops = _lib, ops
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one node)")
        # Rows of A (and of C) per rank: equal blocks unless the caller hands out others, for instance
        # fewer rows to GPUs that measured slower (balanced_row_counts); every rank must pass the same list.
        if row_counts is None:
            if M % self.world:
                raise ValueError("M must be a multiple of the number of ranks")
            row_counts = [M // self.world] * self.world
        row_counts = [int(r) for r in row_counts]
        if len(row_counts) != self.world or sum(row_counts) != M or min(row_counts) <= 0:
            raise ValueError("row_counts must give every rank a positive number of rows adding up to M")
        self.row_counts = row_counts
        self.row_starts = [sum(row_counts[:r]) for r in range(self.world)]
        if exchange not in ("auto", "store", "multicast", "senders", "copy", "push", "overlap"):
            raise ValueError("exchange must be 'auto', 'store', 'multicast', 'senders', 'overlap', 'push' or 'copy'")
        # 'senders': as 'auto', but push_sms CTAs of the product kernel do the remote stores, block of
        # columns by block of columns as C gets finished, instead of the epilogue warps of all CTAs
        self.sender_sms = 0
        if exchange == "senders":
            self.sender_sms, exchange = int(push_sms), "auto"
        if exchange == "overlap" and panels < 2:
            panels = 4                       # the last panel's transfer is the part that is not hidden
        self.M, self.N, self.K, self.dtype = M, N, K, dtype
        self.exchange = exchange
        self.rows = self.row_counts[self.rank]
        self.row_start = self.row_starts[self.rank]
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        if algo == "auto" and self.world >= 4:
            # The tuner table is measured on one GPU, where a Strassen block is a few per cent ahead of
            # a dense one at these shapes; sharded, its exchange (the recombination kernel's stores)
            # runs after the products while a dense block's exchange runs under them. Measured at
            # 32768^3: 8 ranks 7.4 ms dense against 9.7 ms two-level; 2 ranks 27.0 against 25.1.
            algo, depth = "dense", 0
        # what the library would run for one panel (its tuner table, or the caller's choice) decides
        # how many panels fit: fewer when the rows of a panel do not split as the depth needs
        while True:
            prow = self.rows // panels
            if self.rows % panels == 0:
                prob = _lib.Problem()
                prob.M, prob.N, prob.K, prob.batch = prow, N, K, 1
                prob.lda, prob.ldb, prob.ldc = K, N, N
                prob.a_major, prob.b_major = _lib.K_MAJOR, _lib.MN_MAJOR
                prob.in_dtype = prob.out_dtype = ops._DTYPE[dtype]
                prob.algo = ops._ALGO[algo]
                prob.depth, prob.prod_dtype, prob.pipeline, prob.fuse = int(depth), -1, 2, 2
                try:
                    a_res, d_res = ops.resolve(prob)
                    break
                except ValueError:
                    pass
            if panels == 1:
                raise ValueError(f"rows per rank ({self.rows}), N and K do not fit algo {algo!r} at depth {depth}")
            panels -= 1
        self.panels, self.prow = panels, self.rows // panels
        self.algo = {_lib.ALGO_DENSE: "dense", _lib.ALGO_CLASSIC: "classic", _lib.ALGO_WINOGRAD: "winograd"}[a_res]
        self.depth = d_res
        if self.depth > 2:
            raise ValueError("a panel runs dense or as one pipeline of up to two levels")
        if (N * torch.empty((), dtype=dtype).element_size()) % 16:
            raise ValueError("rows of C must be a multiple of 16 bytes long")
        self.C = symm_mem.empty((M, N), dtype=dtype, device=self.device)
        self.hdl = symm_mem.rendezvous(self.C, self.group.group_name)
        self.peer_ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.multicast_ptr = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        if exchange in ("auto", "multicast"):
            # multicast stores where the NVSwitch offers them and the panel is a dense product (a
            # Strassen panel's exchange lives in its recombination kernel); peer stores otherwise.
            # Measured at 8 GPUs, 4096 x 32768 x 32768 per rank: 7.4 ms a step against 8.5 ms.
            usable = self.multicast_ptr != 0 and self.depth == 0 and self.world > 1
            self.exchange = exchange = "multicast" if usable else "store"
        self.pad = symm_mem.empty((64,), dtype=torch.int32, device=self.device)
        self.pad.zero_()
        torch.cuda.synchronize(self.device)
        pad_hdl = symm_mem.rendezvous(self.pad, self.group.group_name)
        dist.barrier(self.group)          # every pad is zero before the first device-side barrier
        self._pads = (ctypes.c_void_p * self.world)(*[int(p) for p in pad_hdl.buffer_ptrs])
        self._epoch = 0
        self._limit_ns = int(barrier_ms * 1e6)
        self._es = self.C.element_size()
        self._ws = None
        self.copy_streams = [torch.cuda.Stream(self.device) for _ in range(self.world)] if exchange == "copy" else []
        self.push_stream = torch.cuda.Stream(self.device, priority=-1) if exchange == "overlap" else None
        self.push_sms = push_sms
        self.ev_panel = [torch.cuda.Event() for _ in range(panels)]

    def _barrier(self, stream):
        self._epoch += 1
        self._lib.check(self._lib.load().b200s_peer_barrier(self._pads, self.rank, self.world, self._epoch,
                                                            self._limit_ns, stream.cuda_stream))

    def panel_product(self, a_panel: torch.Tensor, B: torch.Tensor, algo=None, depth=None) -> torch.Tensor:
        """The product of one row panel as this plan computes it (or as another rank's plan does, given
        its algorithm and depth), into fresh local memory: the same kernels and arithmetic as the
        exchanged panel, for checking what arrived bit for bit."""
        return self._ops.matmul(a_panel, B, algo=self.algo if algo is None else algo,
                                depth=self.depth if depth is None else depth, pipeline=2, fuse=2)

    def _overlapped(self, A_block: torch.Tensor, B: torch.Tensor, stream) -> torch.Tensor:
        """Row panels one after the other into this rank's own rows of C, each on all SMs but
        ``push_sms``; as soon as a panel is done a small kernel on the push stream sends its rows to
        every rank (one multicast store per 16 bytes where the switch offers it, else one store per
        peer) on the SMs the next panel's product leaves free. Only the last panel's transfer is not
        hidden behind a product."""
        import ctypes

        lib, ops = self._lib.load(), self._ops
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        before = lib.b200s_set_product_sms(max(2, sms - self.push_sms))
        try:
            for i in range(self.panels):
                p0 = i * self.prow
                row0 = self.row_start + p0
                c_rows = self.C[row0: row0 + self.prow]
                prob, a2, b2 = ops.make_problem(A_block[p0:p0 + self.prow], B, c_rows, self.algo, self.depth, pipeline=2,
                                                fuse=2, b_blocks_ready=i > 0 and self.depth > 0)
                need = ops.workspace_bytes(prob)
                if need and (self._ws is None or self._ws.numel() < need):
                    if i > 0:
                        raise RuntimeError("scratch of a later panel larger than the first panel's")
                    self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
                self._lib.check(lib.b200s_matmul(ctypes.byref(prob), a2.data_ptr(), b2.data_ptr(), c_rows.data_ptr(),
                                                 self._ws.data_ptr() if need else None, need, stream.cuda_stream))
                if self.world == 1:
                    continue
                self.ev_panel[i].record(stream)
                self.push_stream.wait_event(self.ev_panel[i])
                offset = row0 * self.N * self._es
                nbytes = self.prow * self.N * self._es
                blocks = self.push_sms if i + 1 < self.panels else sms     # nothing runs beside the last transfer
                if self.multicast_ptr:
                    rc = lib.b200s_push_panel(c_rows.data_ptr(), None, 0, self.multicast_ptr + offset, nbytes,
                                              blocks, self.push_stream.cuda_stream)
                else:
                    peers = [self.peer_ptrs[(self.rank + k) % self.world] + offset for k in range(1, self.world)]
                    dst = (ctypes.c_void_p * len(peers))(*peers)
                    rc = lib.b200s_push_panel(c_rows.data_ptr(), dst, len(peers), None, nbytes, blocks,
                                              self.push_stream.cuda_stream)
                self._lib.check(rc)
        finally:
            lib.b200s_set_product_sms(before)
        if self.push_stream is not None:
            stream.wait_stream(self.push_stream)
        self._barrier(stream)                # every rank's rows have been sent and have landed
        return self.C

    def check(self) -> None:
        """Synchronises and raises if a device-side wait (a barrier, a kernel role) gave up."""
        status, detail = self._ops.device_status(self.device)
        if status != 0:
            raise self._lib.B200SError(status, f"{self._lib.status_string(status)} (waiter {detail})")

    def __call__(self, A_block: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
        import ctypes

        lib, ops = self._lib.load(), self._ops
        if A_block.shape != (self.rows, self.K) or B.shape != (self.K, self.N):
            raise ValueError("operand shapes do not match the plan")
        stream = torch.cuda.current_stream(self.device)
        self._barrier(stream)                # every rank is done with the previous contents of C
        if self.exchange == "overlap":
            return self._overlapped(A_block, B, stream)
        senders_before = lib.b200s_set_sender_sms(self.sender_sms) if self.sender_sms else 0
        try:
            self._panels(A_block, B, stream, lib, ops)
        finally:
            if self.sender_sms:
                lib.b200s_set_sender_sms(senders_before)
        for cs in self.copy_streams:
            stream.wait_stream(cs)
        self._barrier(stream)                # every rank's stores have been issued and completed
        return self.C

    def _panels(self, A_block, B, stream, lib, ops):
        import ctypes

        for i in range(self.panels):
            p0 = i * self.prow
            a_panel = A_block[p0:p0 + self.prow]
            row0 = self.row_start + p0
            c_rows = self.C[row0: row0 + self.prow]
            prob, a2, b2 = ops.make_problem(a_panel, B, c_rows, self.algo, self.depth, pipeline=2, fuse=2,
                                            b_blocks_ready=i > 0 and self.depth > 0)
            need = ops.workspace_bytes(prob)
            if need and (self._ws is None or self._ws.numel() < need):
                if i > 0:
                    raise RuntimeError("scratch of a later panel larger than the first panel's")
                self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
            ws_ptr = self._ws.data_ptr() if need else None
            if self.exchange == "multicast":
                self._lib.check(lib.b200s_matmul_multicast(ctypes.byref(prob), a2.data_ptr(), b2.data_ptr(),
                                                           c_rows.data_ptr(), self.multicast_ptr + row0 * self.N * self._es,
                                                           ws_ptr, need, stream.cuda_stream))
                continue
            if self.exchange == "store":
                # this rank's own copy first (the kernel writes it by TMA), then the peers, each rank
                # starting with its right-hand neighbour so that at any moment the ranks write to
                # different peers instead of all to the same one
                order = [(self.rank + k) % self.world for k in range(self.world)]
                dst = (ctypes.c_void_p * self.world)(*[self.peer_ptrs[r] + row0 * self.N * self._es for r in order])
                self._lib.check(lib.b200s_matmul_peers(ctypes.byref(prob), a2.data_ptr(), b2.data_ptr(), dst, self.world,
                                                       ws_ptr, need, stream.cuda_stream))
                continue
            self._lib.check(lib.b200s_matmul(ctypes.byref(prob), a2.data_ptr(), b2.data_ptr(), c_rows.data_ptr(), ws_ptr,
                                             need, stream.cuda_stream))
            if self.world == 1:
                continue
            nbytes = self.prow * self.N * self._es
            if self.exchange == "push":
                peers = [ptr + row0 * self.N * self._es for r, ptr in enumerate(self.peer_ptrs) if r != self.rank]
                dst = (ctypes.c_void_p * len(peers))(*peers)
                self._lib.check(lib.b200s_push_rows(c_rows.data_ptr(), dst, len(peers), nbytes, stream.cuda_stream))
            else:
                self.ev_panel[i].record(stream)
                for r in range(self.world):
                    if r != self.rank:
                        cs = self.copy_streams[r]     # one stream per peer: the transfers run side by side
                        cs.wait_event(self.ev_panel[i])
                        with torch.cuda.stream(cs):
                            peer_rows = self.hdl.get_buffer(r, (self.prow, self.N), self.dtype, row0 * self.N)
                            peer_rows.copy_(c_rows, non_blocking=True)

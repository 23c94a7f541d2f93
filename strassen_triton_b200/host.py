"""Products whose operands and result live in host memory.

The reference's functions take the tensors wherever they are; its profiling script creates the
operands on the GPU before it times anything (main_profiling.py:119-124). A caller whose matrices sit in host
memory pays the PCIe link for both operands on the way in and for the result on the way out. Done
one after the other (copy A, copy B, multiply, copy C) the link idles during the product and the GPU
idles during the copies. ``HostStreamedMatmul`` streams instead:

* B goes to the device first, A follows in row panels on a copy stream;
* every panel is multiplied as soon as it has arrived (B's operand blocks are formed by the first
  panel and reused by all later panels of the same height);
* its rows of C travel back on a second copy stream, in the other direction of the link, while the
  next panel is being multiplied and the one after that is still arriving.

The step then costs the inbound transfer plus the tail of the last panel instead of the sum of
everything. The arithmetic of a panel is that of ``ops.matmul`` on the same rows: the result is
bit-identical to multiplying the row panels one by one.
"""
from __future__ import annotations

from typing import Optional

import torch

from .sharded import panel_bounds


class HostStreamedMatmul:
    """C = A @ B for A (M x K), B (K x N) and C (M x N) in host memory, on one GPU.

    Build it once per shape (it owns the device buffers: B, two panels of A, two panels of C and the
    scratch of one panel product), then call it with the host tensors. Pinned host memory is what
    lets the three streams overlap; pageable tensors work, but their copies block the host.
    """

    PANEL_QUANTUM = 256   # rows: whole tiles of the product kernel, and blocks that split two levels deep

    def __init__(self, M: int, N: int, K: int, dtype=torch.bfloat16, algo: str = "auto", depth: int = -1,
                 panels: int = 8, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("HostStreamedMatmul needs a CUDA device: the product has no CPU path")
        from . import ops

        self._ops = ops
        self.M, self.N, self.K, self.dtype = int(M), int(N), int(K), dtype
        self.algo, self.depth = algo, int(depth)
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.bounds = panel_bounds(self.M, panels, self.PANEL_QUANTUM)
        rows = max(p1 - p0 for p0, p1 in self.bounds)
        with torch.cuda.device(self.device):
            self.B_dev = torch.empty((self.K, self.N), dtype=dtype, device=self.device)
            self.A_buf = [torch.empty((rows, self.K), dtype=dtype, device=self.device) for _ in range(2)]
            self.C_buf = [torch.empty((rows, self.N), dtype=dtype, device=self.device) for _ in range(2)]
            p, _, _ = ops.make_problem(self.A_buf[0], self.B_dev, self.C_buf[0], algo, self.depth, pipeline=2, fuse=2)
            need = ops.workspace_bytes(p)
            self.ws = torch.empty(max(need, 16), dtype=torch.uint8, device=self.device)
            self.s_in = torch.cuda.Stream(self.device)
            self.s_out = torch.cuda.Stream(self.device)
            n = len(self.bounds)
            self.e_in = [torch.cuda.Event() for _ in range(n)]
            self.e_comp = [torch.cuda.Event() for _ in range(n)]
            self.e_out = [torch.cuda.Event() for _ in range(n)]
            self.e_b = torch.cuda.Event()
        self.h2d_bytes = (self.M * self.K + self.K * self.N) * self.A_buf[0].element_size()
        self.d2h_bytes = self.M * self.N * self.A_buf[0].element_size()

    def _check(self, t: torch.Tensor, shape, what: str):
        if t.is_cuda:
            raise ValueError(f"{what} must live in host memory (use ops.matmul for device tensors)")
        if tuple(t.shape) != tuple(shape) or t.dtype != self.dtype:
            raise ValueError(f"{what} must be {tuple(shape)} of {self.dtype}, got {tuple(t.shape)} of {t.dtype}")
        if t.stride(-1) != 1:
            raise ValueError(f"{what} must be row-major")

    def __call__(self, A_host: torch.Tensor, B_host: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Enqueues the whole product and returns ``out`` (allocated pinned when not given). The result
        is complete once the current stream has finished (``torch.cuda.current_stream().synchronize()``)."""
        self._check(A_host, (self.M, self.K), "A")
        self._check(B_host, (self.K, self.N), "B")
        if out is None:
            out = torch.empty((self.M, self.N), dtype=self.dtype, pin_memory=True)
        self._check(out, (self.M, self.N), "out")
        ops = self._ops
        with torch.cuda.device(self.device):
            cur = torch.cuda.current_stream(self.device)
            # whatever the current stream still does with the buffers of an earlier call comes first
            self.s_in.wait_stream(cur)
            self.s_out.wait_stream(cur)
            with torch.cuda.stream(self.s_in):
                self.B_dev.copy_(B_host, non_blocking=True)
                self.e_b.record(self.s_in)
            rows0 = self.bounds[0][1] - self.bounds[0][0]
            for i, (p0, p1) in enumerate(self.bounds):
                j, rows = i % 2, p1 - p0
                with torch.cuda.stream(self.s_in):
                    if i >= 2:
                        self.s_in.wait_event(self.e_comp[i - 2])       # the product that read this buffer is done
                    self.A_buf[j][:rows].copy_(A_host[p0:p1], non_blocking=True)
                    self.e_in[i].record(self.s_in)
                if i == 0:
                    cur.wait_event(self.e_b)
                cur.wait_event(self.e_in[i])
                if i >= 2:
                    cur.wait_event(self.e_out[i - 2])                  # these rows of C have left the buffer
                ops.matmul_out(self.A_buf[j][:rows], self.B_dev, self.C_buf[j][:rows], algo=self.algo, depth=self.depth,
                               pipeline=2, fuse=2, b_blocks_ready=i > 0 and rows == rows0, workspace=self.ws)
                self.e_comp[i].record(cur)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(self.e_comp[i])
                    out[p0:p1].copy_(self.C_buf[j][:rows], non_blocking=True)
                    self.e_out[i].record(self.s_out)
            cur.wait_stream(self.s_out)
        return out


_plans = {}


def matmul_from_host(A_host: torch.Tensor, B_host: torch.Tensor, out: Optional[torch.Tensor] = None, *,
                     algo: str = "auto", depth: int = -1, panels: int = 8, device=None) -> torch.Tensor:
    """A @ B for host tensors through a cached ``HostStreamedMatmul`` of their shape; synchronises
    before it returns, so ``out`` is ready to read."""
    if A_host.dim() != 2 or B_host.dim() != 2 or A_host.shape[1] != B_host.shape[0]:
        raise ValueError("A (M x K) and B (K x N) must be 2-D with matching inner extents")
    dev = torch.device(device if device is not None else (torch.cuda.current_device() if torch.cuda.is_available() else "cpu"))
    key = (A_host.shape[0], B_host.shape[1], A_host.shape[1], A_host.dtype, algo, int(depth), int(panels), str(dev))
    plan = _plans.get(key)
    if plan is None:
        plan = _plans[key] = HostStreamedMatmul(A_host.shape[0], B_host.shape[1], A_host.shape[1], A_host.dtype,
                                                algo=algo, depth=depth, panels=panels, device=device)
    out = plan(A_host, B_host, out)
    torch.cuda.current_stream(plan.device).synchronize()
    return out

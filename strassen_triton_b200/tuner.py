"""Measured algorithm/depth table (stands where the reference has ``triton.autotune`` config lists
keyed on (M, N, K), strassen.py:9-30,93-114,218-236, and a hand-chosen ``depth=``).

``sweep`` times dense / classic / Winograd at depths 0..2, each Strassen candidate under both
schedules (separate passes, fused kernel), for a list of shapes on the current GPU and records the
fastest choice per shape in the library's process-wide table; ``save`` / ``load`` persist it. ``load_default`` reads ``tuner_table.txt`` beside this file when it exists; without a
table the library uses its built-in size thresholds.
"""
from __future__ import annotations

import os
from typing import Iterable, Optional, Tuple

import torch

from . import _lib, ops

DEFAULT_TABLE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tuner_table.txt")
_ALGO_NAME = {_lib.ALGO_DENSE: "dense", _lib.ALGO_CLASSIC: "classic", _lib.ALGO_WINOGRAD: "winograd"}
_DT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.FP16, torch.float32: _lib.FP32}


def _time(fn, reps: int) -> float:
    """Milliseconds per call over `reps` back-to-back calls (CUDA events around the whole run), best
    of three such runs after warm-up: the regime of a training loop or of bench.py, where host-side
    launch work is hidden behind the previous call."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / reps)
    return best


_SCHEDULES = {2: "separate", 3: "fused"}      # b200s_problem.fuse values the sweep tries


def sweep(shapes: Iterable[Tuple[int, int, int]], dtype=torch.bfloat16, reps: int = 5, algos=("classic", "winograd"),
          verbose: bool = True):
    """Measure every candidate for each (M, N, K) and record the fastest. Candidates: the dense
    product, and each Strassen algorithm at depth 1 and 2 under both schedules (separate passes, and
    the fused kernel with the last quadrant recombined after it). Returns the rows."""
    lib = _lib.load()
    rows = []
    for M, N, K in shapes:
        A = torch.randn(M, K, device="cuda").to(dtype)
        B = torch.randn(K, N, device="cuda").to(dtype)
        C = torch.empty(M, N, device="cuda", dtype=dtype)
        cands = [("dense", 0, 0)]
        for d in (1, 2):
            if all(v % (8 << d) == 0 for v in (M, N, K)):
                cands += [(a, d, f) for a in algos for f in _SCHEDULES]
        timings = {}
        for algo, d, fuse in cands:
            p, _, _ = ops.make_problem(A, B, C, algo, d, fuse=fuse, pipeline=2 if fuse == 2 else 0)
            ws = torch.empty(max(ops.workspace_bytes(p), 1), dtype=torch.uint8, device="cuda")
            timings[(algo, d, fuse)] = _time(lambda: ops.matmul_out(A, B, C, algo=algo, depth=d, fuse=fuse,
                                                                    pipeline=2 if fuse == 2 else 0, workspace=ws), reps)
        (algo, d, fuse), ms = min(timings.items(), key=lambda kv: kv[1])
        _lib.check(lib.b200s_tuner_record_schedule(M, N, K, _DT[dtype], ops._ALGO[algo], d, fuse))
        rows.append((M, N, K, algo, d, fuse, ms, timings))
        if verbose:
            print(f"{M}x{N}x{K}: best {algo} depth {d} {_SCHEDULES.get(fuse, '')} {ms:.3f} ms  " +
                  " ".join(f"{a}/d{dd}/{_SCHEDULES.get(ff, '-')}={t:.3f}"
                           for (a, dd, ff), t in sorted(timings.items(), key=lambda kv: kv[1])))
    return rows


def save(path: str = DEFAULT_TABLE) -> None:
    _lib.check(_lib.load().b200s_tuner_save(path.encode()))


def load(path: str = DEFAULT_TABLE) -> None:
    _lib.check(_lib.load().b200s_tuner_load(path.encode()))


def load_default() -> bool:
    """Load the table shipped beside this module; a missing or corrupt file leaves the built-in
    thresholds in force."""
    if not os.path.exists(DEFAULT_TABLE):
        return False
    return _lib.load().b200s_tuner_load(DEFAULT_TABLE.encode()) == _lib.OK


def lookup(M: int, N: int, K: int, dtype=torch.bfloat16) -> Tuple[str, int]:
    import ctypes

    a, d = ctypes.c_int32(0), ctypes.c_int32(0)
    _lib.check(_lib.load().b200s_tuner_lookup(M, N, K, _DT[dtype], ctypes.byref(a), ctypes.byref(d)))
    return _ALGO_NAME[a.value], d.value

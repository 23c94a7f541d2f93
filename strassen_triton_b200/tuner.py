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


def _time(fn, seconds: float) -> float:
    """Milliseconds per call in the sustained regime: back-to-back calls for `seconds`, mean over the
    second half of the run. A B200 runs a dense product against its power limit, and the first few
    tens of milliseconds after an idle gap are faster than anything a training loop or a serving
    process will see; a table measured there would pick schedules that lose under load."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    events = [torch.cuda.Event(enable_timing=True)]
    events[0].record()
    import time

    t0 = time.time()
    while True:
        for _ in range(5):
            fn()
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        events.append(e)
        if len(events) > 3:
            events[-3].synchronize()
        if time.time() - t0 >= seconds:
            break
    torch.cuda.synchronize()
    per = [events[i].elapsed_time(events[i + 1]) / 5 for i in range(len(events) - 1)]
    tail = per[len(per) // 2:]
    return sum(tail) / len(tail)


_SCHEDULES = {2: "separate", 3: "fused"}      # b200s_problem.fuse values the sweep tries
TIE = 1.01                                    # candidates within 1 % of the fastest count as tied


def _pick(timings):
    """The fastest candidate, except that among candidates within TIE of it the plainer one wins:
    dense before Strassen (better accuracy), classic before Winograd (better accuracy), separate
    passes before the fused kernel (one schedule fewer to reason about)."""
    best = min(timings.values())
    tied = [k for k, t in timings.items() if t <= TIE * best]
    rank = lambda k: (k[0] != "dense", k[2] == 3, k[0] != "classic", k[1])  # noqa: E731
    k = min(tied, key=rank)
    return k, timings[k]


def sweep(shapes: Iterable[Tuple[int, int, int]], dtype=torch.bfloat16, seconds: float = 0.6,
          algos=("classic", "winograd"), verbose: bool = True):
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
                                                                    pipeline=2 if fuse == 2 else 0, workspace=ws), seconds)
        (algo, d, fuse), ms = _pick(timings)
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


# Shapes of the shipped table: cubes around the crossover, the GPT-2-124M Linear shapes, and the
# per-rank blocks of the row-sharded 32768^3 product at 8, 4, 2 and 1 ranks.
DEFAULT_SHAPES = [(2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (8192, 768, 3072), (8192, 3072, 768),
                  (8192, 2304, 768), (12288, 12288, 12288), (16384, 16384, 16384), (4096, 32768, 32768),
                  (8192, 32768, 32768), (16384, 32768, 32768), (32768, 32768, 32768)]


def main():
    """Regenerates the shipped table on the current GPU: ``python -m strassen_triton_b200.tuner [path]``."""
    import sys

    path = sys.argv[1] if len(sys.argv) > 1 else DEFAULT_TABLE
    _lib.check(_lib.load().b200s_tuner_clear())
    sweep(DEFAULT_SHAPES, torch.bfloat16)
    sweep([(4096, 4096, 4096), (8192, 8192, 8192), (16384, 16384, 16384)], torch.float16, algos=("classic",))
    save(path)
    print(f"saved {path}")


if __name__ == "__main__":
    main()

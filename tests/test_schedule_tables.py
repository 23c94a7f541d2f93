"""The coefficient tables compiled into the CUDA kernels (csrc/schedule.h) are the same tables the
oracle's model uses: schedule.h is plain C++ on the host side, so it is compiled with g++ into a
small program that prints every entry at one and two levels."""
import os
import shutil
import subprocess

import pytest

from oracle import strassen_oracle as so

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r"""
#include <cstdio>
#include "schedule.h"
using namespace b200s::sched;
int main() {
  for (int algo = 0; algo < 2; ++algo)
    for (int depth = 1; depth <= 2; ++depth) {
      const int np = ipow(7, depth), nq = ipow(4, depth);
      for (int side = 0; side < 2; ++side)
        for (int p = 0; p < np; ++p) {
          for (int q = 0; q < nq; ++q) std::printf("%d ", uv(algo, side, depth, p, q));
          std::printf("\n");
        }
      for (int r = 0; r < nq; ++r) {
        for (int p = 0; p < np; ++p) std::printf("%d ", w(algo, depth, r, p));
        std::printf("\n");
      }
      for (int q = 0; q < nq; ++q) std::printf("%d %d ", block_row(depth, q), block_col(depth, q));
      std::printf("\n");
    }
  return 0;
}
"""


def test_kernel_tables_match_oracle_tables(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no host C++ compiler")
    src = tmp_path / "tables.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "tables"
    subprocess.run([gxx, "-std=c++17", "-I", os.path.join(ROOT, "strassen_triton_b200", "csrc"), str(src), "-o", str(exe)],
                   check=True)
    lines = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.strip().splitlines()
    it = iter([[int(x) for x in ln.split()] for ln in lines])
    for algo in ("classic", "winograd"):
        for depth in (1, 2):
            U, V, W = so.tables(algo, depth)
            for table in (U, V):
                for row in table:
                    assert next(it) == row
            for row in W:
                assert next(it) == row
            pos = next(it)
            # quadrant index -> (block row, block column): the same nesting the oracle's _blocks uses
            n = 2 ** depth
            want = []
            for q in range(4 ** depth):
                if depth == 1:
                    want += [q >> 1, q & 1]
                else:
                    q1, q2 = divmod(q, 4)
                    want += [2 * (q1 >> 1) + (q2 >> 1), 2 * (q1 & 1) + (q2 & 1)]
            assert pos == want and max(pos) == n - 1

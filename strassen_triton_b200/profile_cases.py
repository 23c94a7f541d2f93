"""Runs one kernel of the pipeline a few times on synthetic data, for profiling one kernel at a
time (for example under ``ncu -k regex:<kernel> -c 1``).

    python -m strassen_triton_b200.profile_cases gemm_grouped [products] [n]   # batch of n^3 bf16 products
    python -m strassen_triton_b200.profile_cases dense [n]                     # one n^3 bf16 product
    python -m strassen_triton_b200.profile_cases preadd [n]                    # depth-2 operand sums of an n x n A
    python -m strassen_triton_b200.profile_cases combine [n]                   # depth-2 recombination into n x n C
"""
import ctypes
import sys

import torch

from . import _lib, ops


def main(argv):
    what = argv[0] if argv else "gemm_grouped"
    lib = _lib.load()
    if what == "gemm_grouped":
        nb = int(argv[1]) if len(argv) > 1 else 14
        n = int(argv[2]) if len(argv) > 2 else 4096
        A = torch.randn(nb, n, n, device="cuda").bfloat16()
        B = torch.randn(nb, n, n, device="cuda").bfloat16()
        C = torch.empty_like(A)
        for _ in range(5):
            ops.matmul_out(A, B, C, algo="dense")
    elif what == "dense":
        n = int(argv[1]) if len(argv) > 1 else 8192
        A = torch.randn(n, n, device="cuda").bfloat16()
        B = torch.randn(n, n, device="cuda").bfloat16().t()
        C = torch.empty(n, n, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            ops.matmul_out(A, B, C, algo="dense")
    elif what in ("preadd", "combine"):
        n = int(argv[1]) if len(argv) > 1 else 16384
        A = (torch.rand(n, n, device="cuda") * 2 - 1).bfloat16()
        C = torch.empty(n, n, device="cuda", dtype=torch.bfloat16)
        p, _, _ = ops.make_problem(A, A, C, "classic", 2)
        m = n // 4
        blocks = torch.randn(49, m, m, device="cuda").bfloat16()
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            if what == "preadd":
                _lib.check(lib.b200s_preadd(ctypes.byref(p), 0, A.data_ptr(), blocks.data_ptr(), stream))
            else:
                _lib.check(lib.b200s_combine(ctypes.byref(p), blocks.data_ptr(), C.data_ptr(), stream))
    else:
        raise SystemExit(__doc__)
    torch.cuda.synchronize()
    print("ok", ops.device_status())


if __name__ == "__main__":
    main(sys.argv[1:])

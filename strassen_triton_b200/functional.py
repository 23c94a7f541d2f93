"""The reference's matmul entry points (same names, argument order, return / in-place
behaviour and exception types), routed to libb200s.so.

Reference functions mirrored here:
  strassen.py:66-88      run_matmul_fp32_accum(A, B, C, BLOCK_SIZE=32)         C += A.B, dense
  strassen.py:195-213    run_strassen(A, B, C, BLOCK_SIZE=32)                  C += A.B, one level
  strassen.py:674-693    run_strassen2(A, B, C, BLOCK_SIZE=64)                 C += A.B, two levels
  strassen_2_layer.py:7  run_strassen_2_layer_fp32_accum(A, B, C, BLOCK_SIZE=64)
  strassen_no_tuning.py:536  run_winograd_strassen(A, B, C, BLOCK_SIZE=32)
  strassen.py:697-740    _strassen_base(A, B)
  strassen.py:742-812    strassen_matmul_two_layers(A, B)
  fixed_strassen[_fp32_agg].py:12-126  _strassen_base / strassen_matmul_n_layers(A, B, n_depth, base_dtype)

The reference's two-level and Winograd Triton kernels compute wrong values (block-indexing and
formula errors); the functions of those names here compute the correct product.
"""
from __future__ import annotations

import torch

from . import ops

MAX_DEPTH = 4  # levels the CUDA library accepts; deeper requests run four levels


def _accumulate(A, B, C, algo, depth):
    """Shared body of the run_* launchers: C += A.B, returns None, 2-D or 3-D operands."""
    if A.dim() == 3:
        # strassen.py:67-77: batch on the first axis, no shape assertion in the reference
        ops.matmul_out(A, B, C, algo=algo, depth=depth, beta=1)
        return
    M, K = A.shape
    _, N = B.shape
    assert K == B.shape[0] and A.shape[0] == M and B.shape[1] == N  # strassen.py:81
    ops.matmul_out(A, B, C, algo=algo, depth=depth, beta=1)


def _depth_that_fits(A, B, depth):
    """The run_* kernels of the reference mask ragged tiles, so any size is accepted; here sizes
    that do not split into 2^depth blocks of whole 16-byte vectors use fewer levels."""
    M, K, N = A.shape[-2], A.shape[-1], B.shape[-1]
    while depth > 0 and any(x % (8 << depth) for x in (M, N, K)):
        depth -= 1
    return depth


def run_matmul_fp32_accum(A, B, C, BLOCK_SIZE=32):
    _accumulate(A, B, C, "dense", 0)


def run_strassen(A, B, C, BLOCK_SIZE=32):
    d = _depth_that_fits(A, B, 1)
    _accumulate(A, B, C, "classic" if d else "dense", d)


def run_strassen2(A, B, C, BLOCK_SIZE=64):
    d = _depth_that_fits(A, B, 2)
    _accumulate(A, B, C, "classic" if d else "dense", d)


def run_strassen_2_layer_fp32_accum(A, B, C, BLOCK_SIZE=64):
    M, N = C.shape  # strassen_2_layer.py:8-10
    K = A.shape[1]
    assert K == B.shape[0] and A.shape[0] == M and B.shape[1] == N
    d = _depth_that_fits(A, B, 2)
    ops.matmul_out(A, B, C, algo="classic" if d else "dense", depth=d, beta=1)


def run_winograd_strassen(A, B, C, BLOCK_SIZE=32, **kwargs):
    d = _depth_that_fits(A, B, 1)
    _accumulate(A, B, C, "winograd" if d else "dense", d)


def strassen_base_same_dtype(A, B, algo="classic"):
    """strassen.py:697-740 / fixed_strassen.py:12-57: one level, result in the input dtype;
    n <= 16 is a plain product."""
    if A.shape[0] <= 16:
        return ops.matmul(A, B, algo="dense")
    d = _depth_that_fits(A, B, 1)
    return ops.matmul(A, B, algo=algo if d else "dense", depth=d)


def strassen_matmul_two_layers(A, B, algo="classic"):
    """strassen.py:742-812, including its argument checks."""
    n = A.shape[0]
    if n != B.shape[0] or A.shape[1] != B.shape[0] or A.shape[0] != A.shape[1]:
        raise ValueError("Input matrices must be square and have the same dimensions.")
    if n % 4 != 0:
        raise ValueError("Matrix size must be divisible by 4 for two Strassen layers.")
    if n <= 0:
        raise ValueError("Matrix size must be positive.")
    d = _depth_that_fits(A, B, 2)
    return ops.matmul(A, B, algo=algo if d else "dense", depth=d)


def strassen_n_layers(A, B, n_depth=2, base_dtype=None, algo="classic", prod_dtype=None):
    """strassen_matmul_n_layers of fixed_strassen_fp32_agg.py:59-125 (``base_dtype`` given: operands
    and result in ``base_dtype``, sums in fp32) and of fixed_strassen.py:60-126 (``base_dtype``
    None: everything in the input dtype)."""
    if base_dtype is not None and A.dtype != base_dtype:
        A = A.to(base_dtype)
    if base_dtype is not None and B.dtype != base_dtype:
        B = B.to(base_dtype)
    if A.shape[0] <= 16:
        return ops.matmul(A, B, algo="dense")
    d = _depth_that_fits(A, B, min(int(n_depth), MAX_DEPTH))
    return ops.matmul(A, B, algo=algo if d else "dense", depth=d, prod_dtype=prod_dtype)

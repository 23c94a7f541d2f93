"""Drop-in for the reference module ``fixed_strassen_fp32_agg`` (fixed_strassen_fp32_agg.py):
products in ``base_dtype``, quadrant sums in fp32, result in ``base_dtype`` (default fp32, as
there)."""
import torch

from strassen_triton_b200 import functional as _f
from strassen_triton_b200.linear import LinearStrassen  # noqa: F401

agg_dtype = torch.float32


def _strassen_base(A: torch.Tensor, B: torch.Tensor, base_dtype=torch.float32) -> torch.Tensor:
    return _f.strassen_n_layers(A, B, 1, base_dtype)


def strassen_matmul_n_layers(A: torch.Tensor, B: torch.Tensor, n_depth: int = 2,
                             base_dtype=torch.float32) -> torch.Tensor:
    return _f.strassen_n_layers(A, B, n_depth, base_dtype)

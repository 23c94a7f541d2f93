"""B200-native Strassen / Strassen-Winograd matrix multiplication (sm_100a CUDA behind a C ABI).

`strassen_triton_b200.ops.matmul` is the tensor-level entry; the modules `strassen`,
`strassen_2_layer`, `fixed_strassen`, `fixed_strassen_fp32_agg` and `model.layers` at the
repository root keep the reference project's names and signatures on top of it.
"""
from . import _lib  # noqa: F401
from .ops import device_status, matmul, matmul_autograd, matmul_out  # noqa: F401

__all__ = ["matmul", "matmul_out", "matmul_autograd", "device_status"]

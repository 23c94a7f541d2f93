"""Drop-in for the reference module ``strassen`` (strassen.py): same callables, backed by the
sm_100a CUDA library instead of Triton kernels and torch.mm."""
from strassen_triton_b200.functional import (  # noqa: F401
    run_matmul_fp32_accum,
    run_strassen,
    run_strassen2,
    run_winograd_strassen,
    strassen_matmul_two_layers,
)
from strassen_triton_b200.functional import strassen_base_same_dtype as _strassen_base  # noqa: F401

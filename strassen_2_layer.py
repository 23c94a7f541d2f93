"""Drop-in for the reference module ``strassen_2_layer`` (strassen_2_layer.py:7-15)."""
from strassen_triton_b200.functional import run_strassen_2_layer_fp32_accum  # noqa: F401

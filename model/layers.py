"""Drop-in for the Strassen parts of the reference module ``model.layers``
(model/layers.py:232-300). The attention / rotary / feed-forward classes of that file are plain
PyTorch model code outside the matmul path and are not provided."""
from strassen_triton_b200.linear import LinearStrassen, replace_linear_with_strassen  # noqa: F401

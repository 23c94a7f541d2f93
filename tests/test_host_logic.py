"""Host-side decisions that need no GPU: depth fitting, precision resolution, panel planning."""
import pytest
import torch

from strassen_triton_b200 import functional, ops


def test_depth_that_fits_lowers_depth_until_blocks_are_whole_vectors():
    A = torch.empty(1024, 1024)
    assert functional._depth_that_fits(A, A, 2) == 2
    assert functional._depth_that_fits(A, A, 4) == 4             # 1024 = 8 * 2^7
    odd = torch.empty(48, 48)                                    # 48 = 16 * 3: one level only
    assert functional._depth_that_fits(odd, odd, 2) == 1
    assert functional._depth_that_fits(torch.empty(100, 64), torch.empty(64, 64), 2) == 0
    assert functional._depth_that_fits(torch.empty(3, 64, 64), torch.empty(3, 64, 64), 2) == 2   # batched


def test_precision_follows_torch_switch():
    old = torch.backends.cuda.matmul.allow_tf32
    try:
        torch.backends.cuda.matmul.allow_tf32 = True
        assert ops.resolve_precision(None) == "tf32"
        torch.backends.cuda.matmul.allow_tf32 = False
        assert ops.resolve_precision(None) == "3xtf32"
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    assert ops.resolve_precision("tf32") == "tf32" and ops.resolve_precision("3xtf32") == "3xtf32"
    with pytest.raises(ValueError):
        ops.resolve_precision("fp64")


def test_problem_fields_from_tensors():
    from strassen_triton_b200 import _lib

    A = torch.zeros(3, 64, 128, dtype=torch.float16)
    B = torch.zeros(3, 128, 32, dtype=torch.float16)
    C = torch.zeros(3, 64, 32, dtype=torch.float32)
    p, _, _ = ops.make_problem(A, B, C, "winograd", 1, beta=1, prod_dtype=torch.float32, pipeline=2, b_blocks_ready=True)
    assert (p.M, p.N, p.K, p.batch) == (64, 32, 128, 3)
    assert (p.strideA, p.strideB, p.strideC) == (64 * 128, 128 * 32, 64 * 32)
    assert p.in_dtype == _lib.FP16 and p.out_dtype == _lib.FP32 and p.prod_dtype == _lib.FP32
    assert p.algo == _lib.ALGO_WINOGRAD and p.depth == 1 and p.beta == 1 and p.pipeline == 2 and p.b_blocks_ready == 1
    with pytest.raises(TypeError):
        ops.make_problem(A, B.double(), C)
    with pytest.raises(ValueError):
        ops.make_problem(A, B[0], C)
    with pytest.raises(AssertionError):
        ops.make_problem(A, torch.zeros(3, 64, 32, dtype=torch.float16), C)


def test_struct_layout_matches_header():
    """The ctypes mirror has one field per member of struct b200s_problem, in order."""
    import os
    import re

    from strassen_triton_b200 import _lib

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "include", "b200s.h")).read()
    body = text[text.index("typedef struct b200s_problem {"):text.index("} b200s_problem;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for decl in re.findall(r"(int64_t|int32_t)\s+([^;]+);", body):
        names += [n.strip() for n in decl[1].split(",")]
    assert names == [f[0] for f in _lib.Problem._fields_]

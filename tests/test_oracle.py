"""The CPU oracle against the reference's own outputs (tests/golden/reference_outputs.npz, made by
tests/golden/make_golden.py from the reference project) and against fp64."""
import os

import numpy as np
import pytest
import torch

from oracle import strassen_oracle as so
from tests.golden.make_golden import CASES, make_inputs

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz")

# How each golden case maps to an oracle call.
ORACLE_CALL = {
    ("fixed_strassen_fp32_agg", "_strassen_base"): lambda A, B, kw: so.one_level(A, B, kw.get("base_dtype", torch.float32), True),
    ("fixed_strassen_fp32_agg", "strassen_matmul_n_layers"): lambda A, B, kw: so.n_layers(
        A, B, kw.get("n_depth", 2), kw.get("base_dtype", torch.float32), True, False),
    ("fixed_strassen", "_strassen_base"): lambda A, B, kw: so.one_level(A, B, None, False),
    ("fixed_strassen", "strassen_matmul_n_layers"): lambda A, B, kw: so.n_layers(A, B, kw.get("n_depth", 2), None, False),
    ("strassen", "_strassen_base"): lambda A, B, kw: so.one_level(A, B, None, False),
    ("strassen", "strassen_matmul_two_layers"): lambda A, B, kw: so.n_layers(A, B, 2, None, False),
}


def _from_numpy(arr, dtype_name):
    if "bfloat16" in dtype_name:
        return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
    if "float16" in dtype_name:
        return torch.from_numpy(arr.view(np.int16).copy()).view(torch.float16)
    return torch.from_numpy(arr.copy())


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_oracle_matches_reference_outputs(case):
    name, mod, fn, kwargs, seed, n, dtype, dist = case
    data = np.load(GOLDEN)
    want = _from_numpy(data[name], str(data[name + "__dtype"]))
    A, B = make_inputs(seed, n, dtype, dist)
    got = ORACLE_CALL[(mod, fn)](A, B, kwargs)
    assert got.dtype == want.dtype and got.shape == want.shape
    if torch.equal(got, want):
        return
    # A different host CPU may order torch.mm's fp32 accumulation differently; allow only that.
    d = (got.double() - want.double()).norm() / want.double().norm()
    assert d < 5e-4, f"{name}: oracle differs from the reference output by rel-Fro {d:.3e}"


@pytest.mark.parametrize("algo", ["classic", "winograd"])
@pytest.mark.parametrize("depth", [1, 2])
def test_tables_are_exact_bilinear_algorithms(algo, depth):
    """The coefficient tables multiply matrices exactly (fp64 blocks, error at rounding level)."""
    g = torch.Generator().manual_seed(7)
    A = torch.randn(24, 40, generator=g, dtype=torch.float64)
    B = torch.randn(40, 16, generator=g, dtype=torch.float64)
    C = so.library_model(A, B, depth, algo)
    assert (C - A @ B).abs().max() < 1e-12


def test_table_sparsity():
    U, V, W = so.tables("classic", 1)
    assert sum(map(abs, sum(U, []))) == 12 and sum(map(abs, sum(V, []))) == 12 and sum(map(abs, sum(W, []))) == 12
    U2, V2, W2 = so.tables("classic", 2)
    assert len(U2) == 49 and len(U2[0]) == 16 and len(W2) == 16 and len(W2[0]) == 49
    assert sum(map(abs, sum(U2, []))) == 144
    raw = [p for p in range(49) if sum(map(abs, U2[p])) == 1]
    assert len(raw) == 4  # four of the 49 A operands are single raw blocks


def test_winograd_recursion_matches_fp64():
    g = torch.Generator().manual_seed(3)
    A = torch.randn(64, 64, generator=g)
    B = torch.randn(64, 64, generator=g)
    for d in (1, 2):
        C = so.winograd_levels(A, B, d, torch.float32)  # sums are made in fp32 by design
        assert so.errors_vs_fp64(C, A, B)[1] < 1e-5


def test_small_matrices_short_circuit_to_mm():
    """fixed_strassen_fp32_agg.py:19-20: n <= 16 is torch.mm in the input dtype."""
    A, B = make_inputs(4, 16, torch.float32, "normal")
    assert torch.equal(so.one_level(A, B), torch.mm(A, B))


def test_as_shipped_depth2_runs_inner_level_in_fp32():
    """The sub-calls drop base_dtype (fixed_strassen_fp32_agg.py:99-113): as shipped, depth 2 has
    the error of a one-level bf16 scheme; with base_dtype forwarded it is clearly larger."""
    A, B = make_inputs(0, 256, torch.bfloat16, "uniform")
    shipped = so.n_layers(A, B, 2, torch.bfloat16, True, False)
    intended = so.n_layers(A, B, 2, torch.bfloat16, True, True)
    one = so.n_layers(A, B, 1, torch.bfloat16, True)
    e_shipped = so.errors_vs_fp64(shipped, A, B)[1]
    e_intended = so.errors_vs_fp64(intended, A, B)[1]
    e_one = so.errors_vs_fp64(one, A, B)[1]
    assert abs(e_shipped - e_one) / e_one < 0.3
    assert e_intended > 1.5 * e_shipped


def test_library_model_error_is_below_reference_at_equal_depth():
    """The rounding points the CUDA library uses are no worse than the reference's genuine bf16
    paths at the same depth (fixed_strassen, and fp32-agg with base_dtype forwarded)."""
    A, B = make_inputs(0, 256, torch.bfloat16, "uniform")
    for d in (1, 2):
        e_lib = so.errors_vs_fp64(so.library_model(A, B, d, "classic"), A, B)[1]
        e_plain = so.errors_vs_fp64(so.n_layers(A, B, d, None, False), A, B)[1]
        e_agg = so.errors_vs_fp64(so.n_layers(A, B, d, torch.bfloat16, True, True), A, B)[1]
        assert e_lib <= 1.05 * e_plain and e_lib <= 1.05 * e_agg, (d, e_lib, e_plain, e_agg)


def test_rectangular_restatement():
    g = torch.Generator().manual_seed(5)
    A = torch.randn(96, 160, generator=g)
    B = torch.randn(160, 64, generator=g)
    C = so.n_layers(A, B, 2, torch.float32, True, True)
    assert so.errors_vs_fp64(C, A, B)[1] < 1e-5


def test_recombine_is_the_table_walk_of_the_model():
    """recombine() on exact products gives A @ B: the tables close (U, V, W of both algorithms, one
    and two levels), and it is the same sum library_model forms."""
    import torch

    from oracle import strassen_oracle as so

    g = torch.Generator().manual_seed(3)
    A = torch.randint(-3, 4, (16, 8), generator=g).double()
    B = torch.randint(-3, 4, (8, 12), generator=g).double()
    for algo in ("classic", "winograd"):
        for depth in (1, 2):
            U, V, _ = so.tables(algo, depth)
            ab, bb = so._blocks(A, depth), so._blocks(B, depth)
            prods = [so._signed_sum(U[p], ab) @ so._signed_sum(V[p], bb) for p in range(7 ** depth)]
            assert torch.equal(so.recombine(prods, depth, algo), A @ B)
    import pytest
    with pytest.raises(ValueError):
        so.recombine([A] * 3, 1)

"""The reference-named Python surface without a GPU: names, signatures, argument checks and the
loud refusal of CPU tensors (there is no CPU compute path)."""
import inspect

import pytest
import torch
import torch.nn as nn


def test_reference_module_names_and_callables():
    import fixed_strassen
    import fixed_strassen_fp32_agg
    import model.layers
    import strassen
    import strassen_2_layer

    for fn in ("run_matmul_fp32_accum", "run_strassen", "run_strassen2", "run_winograd_strassen",
               "_strassen_base", "strassen_matmul_two_layers"):
        assert callable(getattr(strassen, fn))
    assert callable(strassen_2_layer.run_strassen_2_layer_fp32_accum)
    for mod in (fixed_strassen, fixed_strassen_fp32_agg):
        assert callable(mod._strassen_base) and callable(mod.strassen_matmul_n_layers)
        assert issubclass(mod.LinearStrassen, nn.Linear)
    assert fixed_strassen_fp32_agg.agg_dtype == torch.float32
    assert callable(model.layers.replace_linear_with_strassen)


def test_signatures_follow_the_reference():
    import fixed_strassen_fp32_agg as agg
    import strassen
    import strassen_2_layer

    assert list(inspect.signature(strassen.run_strassen).parameters) == ["A", "B", "C", "BLOCK_SIZE"]
    assert inspect.signature(strassen.run_strassen2).parameters["BLOCK_SIZE"].default == 64
    assert inspect.signature(strassen_2_layer.run_strassen_2_layer_fp32_accum).parameters["BLOCK_SIZE"].default == 64
    sig = inspect.signature(agg.strassen_matmul_n_layers)
    assert list(sig.parameters) == ["A", "B", "n_depth", "base_dtype"]
    assert sig.parameters["n_depth"].default == 2 and sig.parameters["base_dtype"].default == torch.float32
    sig = inspect.signature(agg.LinearStrassen.__init__)
    assert list(sig.parameters)[1:7] == ["in_features", "out_features", "bias", "dtype", "depth", "device"]
    assert sig.parameters["depth"].default == 1 and sig.parameters["device"].default == "cuda"


def test_two_layers_argument_checks_match_reference():
    """strassen.py:757-762 raises ValueError for non-square or n % 4 != 0 before any compute."""
    import strassen

    with pytest.raises(ValueError):
        strassen.strassen_matmul_two_layers(torch.zeros(8, 4), torch.zeros(4, 8))
    with pytest.raises(ValueError):
        strassen.strassen_matmul_two_layers(torch.zeros(6, 6), torch.zeros(6, 6))


def test_run_launchers_assert_on_shape_mismatch():
    """strassen.py:81,208,688: AssertionError on inconsistent 2-D shapes."""
    import strassen

    A, B, C = torch.zeros(8, 8), torch.zeros(16, 8), torch.zeros(8, 8)
    for fn in (strassen.run_strassen, strassen.run_strassen2, strassen.run_matmul_fp32_accum,
               strassen.run_winograd_strassen):
        with pytest.raises(AssertionError):
            fn(A, B, C)


def test_cpu_tensors_are_refused_loudly():
    import fixed_strassen_fp32_agg as agg
    import strassen

    A = torch.randn(64, 64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        agg.strassen_matmul_n_layers(A, A, 2, torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        strassen.run_strassen(A, A, torch.zeros(64, 64))


def test_linear_strassen_is_an_ordinary_linear_on_the_outside():
    from model.layers import LinearStrassen, replace_linear_with_strassen

    layer = LinearStrassen(64, 64, bias=True, dtype=torch.float32, depth=2, device="cpu")
    assert isinstance(layer, nn.Linear) and layer.depth == 2
    assert set(dict(layer.named_parameters())) == {"weight", "bias"}
    assert layer.weight.shape == (64, 64)
    rect = LinearStrassen(64, 256, bias=False, device="cpu")
    assert rect.weight.shape == (256, 64) and rect.bias is None
    # main_profiling.py:51 spelling: (features, bias, dtype, depth, device)
    sq = LinearStrassen(128, False, torch.float32, 1, "cpu")
    assert sq.weight.shape == (128, 128) and sq.bias is None
    with pytest.raises(RuntimeError, match="no CPU path"):
        layer(torch.randn(4, 64))

    net = nn.Sequential(nn.Linear(128, 128), nn.ReLU(), nn.Linear(128, 32), nn.Sequential(nn.Linear(256, 256)))
    w0 = net[0].weight.detach().clone()
    replace_linear_with_strassen(net, min_size=128, depth=1)
    assert isinstance(net[0], LinearStrassen) and torch.equal(net[0].weight, w0)
    assert not isinstance(net[2], LinearStrassen)          # not square
    assert isinstance(net[3][0], LinearStrassen)           # recursion into children


def test_operand_layout_detection():
    """Transposed views (weight.T) are passed by strides, not copied."""
    from strassen_triton_b200 import _lib, ops

    A = torch.zeros(64, 128, dtype=torch.bfloat16)
    W = torch.zeros(256, 128, dtype=torch.bfloat16)
    C = torch.zeros(64, 256, dtype=torch.bfloat16)
    p, A2, B2 = ops.make_problem(A, W.t(), C)
    assert (p.M, p.N, p.K) == (64, 256, 128)
    assert p.a_major == _lib.K_MAJOR and p.b_major == _lib.K_MAJOR and p.ldb == 128
    assert B2.data_ptr() == W.data_ptr()
    p, _, B2 = ops.make_problem(A, W.t().contiguous(), C)
    assert p.b_major == _lib.MN_MAJOR and p.ldb == 256
    p, A2, _ = ops.make_problem(torch.zeros(128, 64, dtype=torch.bfloat16).t(), W.t(), C)
    assert p.a_major == _lib.MN_MAJOR and p.lda == 64
    # a slice with an odd row pitch needs one copy
    odd = torch.zeros(64, 133, dtype=torch.bfloat16)[:, :128]
    p, A2, _ = ops.make_problem(odd, W.t(), C)
    assert A2.data_ptr() != odd.data_ptr() and p.lda == 128

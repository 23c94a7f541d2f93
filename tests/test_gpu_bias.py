"""The bias of a Linear layer added inside the product (b200s_matmul_bias): in the GEMM epilogue for a
dense product, in the recombination kernel for a Strassen one, always in fp32 before the single
rounding to the output dtype (model/layers.py:271-272 adds it in a separate pass)."""
import pytest
import torch

from tests.conftest import seeded_pair

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_library):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from strassen_triton_b200 import ops as _ops

    return _ops


def rel(x, ref):
    return ((x.double() - ref.double()).norm() / ref.double().norm()).item()


@pytest.mark.parametrize("tile_variant", [1, 2, 3])
@pytest.mark.parametrize("shape", [(300, 264, 200), (512, 1024, 256), (129, 520, 72)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_dense_epilogue_bias(ops, tile_variant, shape, out_dtype):
    M, N, K = shape
    A, B = seeded_pair(M + N + K, (M, K), (K, N))
    bias = torch.linspace(-3, 3, N)
    Ag, Bg = A.bfloat16().cuda(), B.bfloat16().cuda()
    C = ops.matmul(Ag, Bg, algo="dense", tile_variant=tile_variant, out_dtype=out_dtype, bias=bias.cuda())
    ref = Ag.double().cpu() @ Bg.double().cpu() + bias.to(out_dtype).double()
    assert rel(C.cpu(), ref) < (2e-6 if out_dtype == torch.float32 else 3e-3)
    # the bias really is per column: subtracting it leaves the plain product
    plain = ops.matmul(Ag, Bg, algo="dense", tile_variant=tile_variant, out_dtype=torch.float32)
    if out_dtype == torch.float32:
        assert (C - plain - bias.cuda()).abs().max().item() < 1e-4
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("algo,depth", [("classic", 1), ("classic", 2), ("winograd", 2)])
def test_strassen_recombination_bias(ops, algo, depth):
    M, N, K = 512, 768, 256
    A, B = seeded_pair(9, (M, K), (K, N), dist="uniform")
    bias = torch.randn(N, generator=torch.Generator().manual_seed(1))
    Ag, Bg = A.bfloat16().cuda(), B.bfloat16().cuda()
    C = ops.matmul(Ag, Bg, algo=algo, depth=depth, out_dtype=torch.float32, bias=bias.cuda())
    plain = ops.matmul(Ag, Bg, algo=algo, depth=depth, out_dtype=torch.float32, pipeline=2, fuse=2)
    assert (C - plain - bias.cuda()).abs().max().item() < 1e-4      # same sums, plus the bias, in fp32
    Cb = ops.matmul(Ag, Bg, algo=algo, depth=depth, bias=bias.cuda())
    assert rel(Cb.cpu(), plain.cpu() + bias) < 4e-3
    assert ops.device_status() == (0, 0)


def test_linear_bias_gradients(ops):
    from model.layers import LinearStrassen

    torch.manual_seed(0)
    layer = LinearStrassen(256, 384, bias=True, dtype=torch.bfloat16, depth=1, device="cuda")
    x = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = layer(x)
    g = torch.randn_like(y)
    y.backward(g)
    xd, wd, bd = x.detach().double(), layer.weight.detach().double(), layer.bias.detach().double()
    assert rel(y, xd @ wd.t() + bd) < 1.5e-2
    assert rel(layer.bias.grad, g.double().sum(0)) < 1e-2
    assert rel(x.grad, g.double() @ wd) < 1.5e-2
    assert rel(layer.weight.grad, g.double().t() @ xd) < 1.5e-2

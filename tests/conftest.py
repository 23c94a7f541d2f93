import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The oracle calls torch.mm eagerly; never let dynamo wrap anything in the tests.
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def built_library():
    """Path of libb200s.so, building it first if nvcc is available and it is stale."""
    from strassen_triton_b200 import build as _build

    return _build.build()


def seeded_pair(seed, shape_a, shape_b, dist="normal", scale=None):
    """A then B from one CPU generator, fp32: the input convention of every comparison here."""
    import torch

    g = torch.Generator("cpu").manual_seed(seed)
    if dist == "uniform":
        A = 2 * torch.rand(shape_a, generator=g) - 1
        B = 2 * torch.rand(shape_b, generator=g) - 1
    else:
        A = torch.randn(shape_a, generator=g)
        B = torch.randn(shape_b, generator=g)
    if scale is not None:
        A, B = A * scale, B * scale
    return A, B

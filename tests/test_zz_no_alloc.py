"""b200s_matmul_static: the product for callers that cannot allocate device memory.

Some users of this library run where allocation is not an option: a control loop that is forbidden
to touch an allocator once it is running, or a guest inside a host application that keeps all device
memory to itself. For them the library carries its Strassen scratch inside its own image. This test
drives that entry point through the C ABI, twice in a row with different inputs (the second call
finds the first call's blocks still in the shared array), and compares each result with what the
ordinary entry point computes from a caller-provided workspace: the two run the same kernels in the
same order, so the results must be bit-identical, and both must sit within the usual bound of the
oracle's model. It also checks that an over-sized problem is refused before anything is launched.

The file name sorts last on purpose: a run that stops at the first failure has then already been
through every other test.
"""
import ctypes

import pytest
import torch

from oracle import strassen_oracle as so
from tests.conftest import seeded_pair

pytestmark = pytest.mark.gpu


def test_static_scratch_product_matches_workspace_product(built_library):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from strassen_triton_b200 import _lib, ops

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, algo, depth, shape) in enumerate([(101, "classic", 2, (512, 768, 1024)),
                                                       (202, "winograd", 1, (1024, 512, 512))]):
        M, N, K = shape
        A, B = seeded_pair(seed, (M, K), (K, N), dist="uniform")
        A, B = A.bfloat16().cuda(), B.bfloat16().cuda()
        want = ops.matmul(A, B, algo=algo, depth=depth, pipeline=2)          # caller-provided workspace
        C = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        p, A2, B2 = ops.make_problem(A, B, C, algo, depth)
        launches = lib.b200s_launch_count()
        rc = lib.b200s_matmul_static(ctypes.byref(p), A2.data_ptr(), B2.data_ptr(), C.data_ptr(), stream)
        assert rc == 0, _lib.status_string(rc)
        assert lib.b200s_launch_count() - launches == 4                        # pre-add A, pre-add B, GEMM, combine
        torch.cuda.synchronize()
        assert torch.equal(C, want), f"call {call}: static-scratch result differs from the workspace result"
        model = so.library_model(A.cpu(), B.cpu(), depth, algo)
        d = ((C.cpu().double() - model.double()).norm() / model.double().norm()).item()
        assert d < 1e-3, d                                                     # the tolerance of the parity tests


def test_static_scratch_rejects_what_does_not_fit(built_library):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from strassen_triton_b200 import _lib, ops

    lib = _lib.load()
    n = 4096                                   # depth 2 needs 3 * 49 * 1024^2 * 2 bytes = 294 MiB > 64 MiB
    A = torch.zeros(n, n, device="cuda", dtype=torch.bfloat16)
    C = torch.zeros(n, n, device="cuda", dtype=torch.bfloat16)
    p, _, _ = ops.make_problem(A, A, C, "classic", 2)
    launches = lib.b200s_launch_count()
    rc = lib.b200s_matmul_static(ctypes.byref(p), A.data_ptr(), A.data_ptr(), C.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_TOO_LARGE
    assert "capacity" in _lib.status_string(rc)
    assert lib.b200s_launch_count() == launches
    assert lib.b200s_matmul_static(None, A.data_ptr(), A.data_ptr(), C.data_ptr(), None) == _lib.ERR_NULL_POINTER


CHILD = r"""
import ctypes, sys, torch
sys.path.insert(0, %r)
from strassen_triton_b200 import _lib, ops
lib = _lib.load()
dev = torch.device("cuda")
stream = torch.cuda.current_stream().cuda_stream
g = torch.Generator(device="cuda").manual_seed(7)
M, N, K = 512, 768, 1024
A = (torch.rand(M, K, device=dev, generator=g) * 2 - 1).bfloat16()
B = (torch.rand(K, N, device=dev, generator=g) * 2 - 1).bfloat16()
A2 = (torch.rand(M, K, device=dev, generator=g) * 2 - 1).bfloat16()
C = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
C2 = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
p, a, b = ops.make_problem(A, B, C, "classic", 2)
# the very first product of this process goes through the static entry: nothing of the ordinary
# path (workspace, status words, tuner) has been set up for it
assert lib.b200s_matmul_static(ctypes.byref(p), a.data_ptr(), b.data_ptr(), C.data_ptr(), stream) == 0
st, detail = ctypes.c_int32(-1), ctypes.c_int32(-1)
assert lib.b200s_static_status(stream, ctypes.byref(st), ctypes.byref(detail)) == 0
torch.cuda.synchronize()          # the first call loaded the kernels and with them the scratch array
free0, _ = torch.cuda.mem_get_info()
held0 = torch.cuda.memory_reserved()
for _ in range(3):
    assert lib.b200s_matmul_static(ctypes.byref(p), A2.data_ptr(), b.data_ptr(), C2.data_ptr(), stream) == 0
assert lib.b200s_static_status(stream, ctypes.byref(st), ctypes.byref(detail)) == 0
torch.cuda.synchronize()
free1, _ = torch.cuda.mem_get_info()
assert (st.value, detail.value) == (0, 0), (st.value, detail.value)
assert free1 == free0, (free0, free1)                     # the driver handed out no device memory
assert torch.cuda.memory_reserved() == held0
want = ops.matmul(A, B, algo="classic", depth=2, pipeline=2)
want2 = ops.matmul(A2, B, algo="classic", depth=2, pipeline=2)
assert torch.equal(C, want) and torch.equal(C2, want2)
print("static ok", free0)
"""


def test_static_entry_first_in_a_fresh_process_takes_no_device_memory(built_library):
    """In a process of its own the static entry is the first thing the library does; once the first
    call has loaded the kernels, further calls leave the device's free memory exactly as it was."""
    import os
    import subprocess
    import sys

    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TORCHDYNAMO_DISABLE="1")
    out = subprocess.run([sys.executable, "-c", CHILD % root], cwd=root, env=env, capture_output=True, text=True,
                         timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    assert "static ok" in out.stdout

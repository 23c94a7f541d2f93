"""The recombination pass on its own (b200s_combine): position-wise, so independent of how the
product data is cut into rows.

The same 49 product blocks are handed to the library twice: as blocks of Mb x Nb and, reinterpreted,
as blocks of 2Mb x Nb/2. Corresponding positions must come out bit for bit the same (one thread owns
one position; nothing may depend on where a row ends), and both must agree with the fp64
recombination by the oracle's tables. Wide block rows, many blocks per SM and both `C =` and `C +=`
are covered. The additions are those of fixed_strassen_fp32_agg.py:47-56 and :115-123."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib(built_library):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from strassen_triton_b200 import _lib

    return _lib


def _combine(lib, blocks, Mb, Nb, algo, out_dtype, beta, c0):
    """C (4Mb x 4Nb) from 49 product blocks viewed as Mb x Nb, through b200s_combine."""
    from strassen_triton_b200 import ops

    C = c0.clone() if c0 is not None else torch.zeros(4 * Mb, 4 * Nb, device="cuda", dtype=out_dtype)
    dummy = torch.empty(4 * Mb, 64, device="cuda", dtype=blocks.dtype)   # shapes only: M from A, N from B
    dummy_b = torch.empty(64, 4 * Nb, device="cuda", dtype=blocks.dtype)
    p, _, _ = ops.make_problem(dummy, dummy_b, C, algo, 2, beta=beta)
    lib.check(lib.load().b200s_combine(ctypes.byref(p), blocks.data_ptr(), C.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert ops.device_status() == (0, 0)
    return C


def _as_halved_rows(C, Mb, Nb):
    """C of the Mb x Nb problem rearranged to where the 2Mb x Nb/2 problem puts the same positions."""
    h = Nb // 2
    out = torch.empty(8 * Mb, 4 * h, device=C.device, dtype=C.dtype)
    for br in range(4):
        for bc in range(4):
            blk = C[br * Mb:(br + 1) * Mb, bc * Nb:(bc + 1) * Nb]
            out[br * 2 * Mb:(br + 1) * 2 * Mb, bc * h:(bc + 1) * h] = blk.reshape(2 * Mb, h)
    return out


@pytest.mark.parametrize("algo", ["classic", "winograd"])
@pytest.mark.parametrize("prod_dtype,out_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16),
                                                  (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("Mb,Nb", [(8, 1024), (40, 2048), (296, 1024)])
@pytest.mark.parametrize("beta", [0, 1])
def test_recombination_is_position_wise(lib, algo, prod_dtype, out_dtype, Mb, Nb, beta):
    g = torch.Generator(device="cuda").manual_seed(Mb * 7 + Nb)
    blocks = torch.randn(49, Mb, Nb, device="cuda", generator=g).to(prod_dtype)
    c0 = torch.randn(4 * Mb, 4 * Nb, device="cuda", generator=g).to(out_dtype) if beta else None
    wide = _combine(lib, blocks, Mb, Nb, algo, out_dtype, beta, c0)
    c0_tall = _as_halved_rows(c0, Mb, Nb) if beta else None
    tall = _combine(lib, blocks, 2 * Mb, Nb // 2, algo, out_dtype, beta, c0_tall)
    assert torch.equal(_as_halved_rows(wide, Mb, Nb), tall)
    # and the sums are the right ones: fp64 recombination of the same blocks
    from oracle import strassen_oracle as so

    want = so.recombine([blocks[i].double().cpu() for i in range(49)], 2, algo)
    if beta:
        want = want + c0.double().cpu()
    err = ((wide.double().cpu() - want).norm() / want.norm()).item()
    assert err < {torch.bfloat16: 4e-3, torch.float16: 6e-4, torch.float32: 1e-6}[out_dtype], err


def test_recombination_large_and_repeatable(lib):
    """A size of many waves of blocks; a repeat gives the same bits."""
    Mb, Nb = 1024, 2048
    g = torch.Generator(device="cuda").manual_seed(5)
    blocks = torch.randn(49, Mb, Nb, device="cuda", generator=g).bfloat16()
    wide = _combine(lib, blocks, Mb, Nb, "classic", torch.bfloat16, 0, None)
    tall = _combine(lib, blocks, 2 * Mb, Nb // 2, "classic", torch.bfloat16, 0, None)
    assert torch.equal(_as_halved_rows(wide, Mb, Nb), tall)
    again = _combine(lib, blocks, Mb, Nb, "classic", torch.bfloat16, 0, None)
    assert torch.equal(again, wide)

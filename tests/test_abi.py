"""The C-ABI library on a machine without a GPU: it loads, exports every symbol the header
declares, validates arguments and runs the tuner table. No kernel is launched here."""
import ctypes
import os
import re

import pytest

from strassen_triton_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib(built_library):
    return _lib.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "b200s.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200s_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/b200s.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes prototypes and header disagree"


def test_version_and_status_strings(lib):
    assert lib.b200s_version() >= 100
    for code in range(0, -14, -1):
        assert _lib.status_string(code) != "unknown status"
    assert _lib.status_string(-99) == "unknown status"


def problem(**kw):
    p = _lib.Problem()
    p.M = p.N = p.K = 1024
    p.batch = 1
    p.lda = p.ldb = p.ldc = 1024
    p.a_major, p.b_major = _lib.K_MAJOR, _lib.MN_MAJOR
    p.in_dtype = p.out_dtype = _lib.BF16
    p.algo, p.depth, p.prod_dtype = _lib.ALGO_CLASSIC, 2, -1
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def ws_bytes(lib, p):
    n = ctypes.c_size_t(0)
    rc = lib.b200s_workspace_bytes(ctypes.byref(p), ctypes.byref(n))
    return rc, n.value


FLAGS = 256   # counters of the fused schedule, at the end of every one- or two-level scratch


def test_workspace_layout(lib):
    rc, n = ws_bytes(lib, problem())
    blk = 256 * 256 * 2
    assert rc == 0 and n == 3 * 49 * blk + FLAGS
    rc, n = ws_bytes(lib, problem(depth=1))
    assert rc == 0 and n == 3 * 7 * 512 * 512 * 2 + FLAGS
    rc, n = ws_bytes(lib, problem(depth=1, prod_dtype=_lib.FP32))
    assert rc == 0 and n == 2 * 7 * 512 * 512 * 2 + 7 * 512 * 512 * 4 + FLAGS
    rc, n = ws_bytes(lib, problem(algo=_lib.ALGO_DENSE))
    assert rc == 0 and n == 0
    # three levels: one outer level (7 blocks of 512^2 per side and 7 products) around a two-level 512^3 product
    rc, n = ws_bytes(lib, problem(depth=3))
    assert rc == 0 and n == 3 * 7 * 512 * 512 * 2 + 3 * 49 * 128 * 128 * 2 + FLAGS


@pytest.mark.parametrize("kw,status", [
    (dict(M=0), _lib.ERR_BAD_SHAPE),
    (dict(M=1000), _lib.ERR_BAD_SHAPE),            # 1000 is not a multiple of 4 * 8
    (dict(in_dtype=7), _lib.ERR_BAD_DTYPE),
    (dict(algo=9), _lib.ERR_BAD_ALGO),
    (dict(depth=5), _lib.ERR_BAD_DEPTH),
    (dict(lda=512), _lib.ERR_BAD_STRIDE),
    (dict(beta=2), _lib.ERR_BAD_SHAPE),
])
def test_bad_arguments_are_rejected_on_the_host(lib, kw, status):
    rc, _ = ws_bytes(lib, problem(**kw))
    assert rc == status
    # the compute entry refuses the same problem before touching any device
    rc = lib.b200s_matmul(ctypes.byref(problem(**kw)), 16, 16, 16, 16, 1 << 40, None)
    assert rc == status


def test_null_pointers(lib):
    n = ctypes.c_size_t(0)
    assert lib.b200s_workspace_bytes(None, ctypes.byref(n)) == _lib.ERR_NULL_POINTER
    assert lib.b200s_matmul(ctypes.byref(problem()), None, 16, 16, 16, 0, None) == _lib.ERR_NULL_POINTER
    assert lib.b200s_matmul(ctypes.byref(problem()), 16, 16, 16, None, 0, None) == _lib.ERR_NULL_POINTER


def test_workspace_too_small_and_misaligned(lib):
    p = problem()
    assert lib.b200s_matmul(ctypes.byref(p), 16, 16, 16, 256, 1024, None) == _lib.ERR_WORKSPACE_TOO_SMALL
    assert lib.b200s_matmul(ctypes.byref(p), 16, 16, 16, 8, 1 << 40, None) == _lib.ERR_BAD_ALIGNMENT


def test_check_maps_status_to_reference_exception_types(lib):
    with pytest.raises(ValueError):
        _lib.check(_lib.ERR_BAD_SHAPE)
    with pytest.raises(_lib.B200SError):
        _lib.check(_lib.ERR_WORKSPACE_TOO_SMALL)
    _lib.check(0)


def lookup(lib, M, N, K, dt=_lib.BF16):
    a, d = ctypes.c_int32(-5), ctypes.c_int32(-5)
    assert lib.b200s_tuner_lookup(M, N, K, dt, ctypes.byref(a), ctypes.byref(d)) == 0
    return a.value, d.value


def test_tuner_table(lib, tmp_path):
    lib.b200s_tuner_clear()
    # built-in choice: dense for small problems
    assert lookup(lib, 768, 3072, 8192) == (_lib.ALGO_DENSE, 0)
    assert lib.b200s_tuner_record(4096, 4096, 4096, _lib.BF16, _lib.ALGO_DENSE, 0) == 0
    assert lib.b200s_tuner_record(16384, 16384, 16384, _lib.BF16, _lib.ALGO_CLASSIC, 2) == 0
    assert lib.b200s_tuner_record(8192, 8192, 8192, _lib.BF16, _lib.ALGO_WINOGRAD, 1) == 0
    assert lookup(lib, 16384, 16384, 16384) == (_lib.ALGO_CLASSIC, 2)
    assert lookup(lib, 15000, 16384, 16000) == (_lib.ALGO_CLASSIC, 2)   # nearest bucket
    assert lookup(lib, 3000, 4096, 5000) == (_lib.ALGO_DENSE, 0)
    assert lookup(lib, 8192, 8192, 8192) == (_lib.ALGO_WINOGRAD, 1)
    # other dtypes have no entries: built-in choice
    assert lookup(lib, 1024, 1024, 1024, _lib.FP32) == (_lib.ALGO_DENSE, 0)
    assert lib.b200s_tuner_record(0, 1, 1, _lib.BF16, _lib.ALGO_DENSE, 0) == _lib.ERR_BAD_SHAPE
    path = str(tmp_path / "table.txt").encode()
    assert lib.b200s_tuner_save(path) == 0
    lib.b200s_tuner_clear()
    assert lib.b200s_tuner_load(path) == 0
    assert lookup(lib, 8192, 8192, 8192) == (_lib.ALGO_WINOGRAD, 1)
    # resolution through the table, clamped to what the extents allow
    a, d = ctypes.c_int32(0), ctypes.c_int32(0)
    p = problem(M=16384, N=16384, K=16384, lda=16384, ldb=16384, ldc=16384, algo=_lib.ALGO_AUTO, depth=-1)
    assert lib.b200s_resolve(ctypes.byref(p), ctypes.byref(a), ctypes.byref(d)) == 0
    assert (a.value, d.value) == (_lib.ALGO_CLASSIC, 2)
    p = problem(M=16400, N=16400, K=16400, lda=16400, ldb=16400, ldc=16400, algo=_lib.ALGO_AUTO, depth=-1)
    assert lib.b200s_resolve(ctypes.byref(p), ctypes.byref(a), ctypes.byref(d)) == 0
    assert (a.value, d.value) == (_lib.ALGO_CLASSIC, 1)   # 16400 = 16 * 1025: one level only
    lib.b200s_tuner_clear()


def test_corrupt_or_missing_table_leaves_state_untouched(lib, tmp_path):
    lib.b200s_tuner_clear()
    lib.b200s_tuner_record(8192, 8192, 8192, _lib.BF16, _lib.ALGO_CLASSIC, 1)
    bad = tmp_path / "bad.txt"
    bad.write_text("8192 8192 8192 0 2 1\nthis is not a table line\n")
    assert lib.b200s_tuner_load(str(bad).encode()) == _lib.ERR_TUNER_IO
    assert lib.b200s_tuner_load(str(tmp_path / "missing.txt").encode()) == _lib.ERR_TUNER_IO
    assert lookup(lib, 8192, 8192, 8192) == (_lib.ALGO_CLASSIC, 1)
    lib.b200s_tuner_clear()


def test_launch_count_starts_at_zero_without_a_gpu(lib):
    assert lib.b200s_launch_count() >= 0


def test_tuner_table_carries_the_schedule(lib, tmp_path):
    lib.b200s_tuner_clear()
    a, d, f = ctypes.c_int32(0), ctypes.c_int32(0), ctypes.c_int32(9)
    assert lib.b200s_tuner_lookup_schedule(16384, 16384, 16384, _lib.BF16, ctypes.byref(a), ctypes.byref(d),
                                           ctypes.byref(f)) == 0
    assert f.value == 0                                           # nothing recorded: the built-in rule applies
    assert lib.b200s_tuner_record_schedule(16384, 16384, 16384, _lib.BF16, _lib.ALGO_CLASSIC, 2, 3) == 0
    assert lib.b200s_tuner_record_schedule(4096, 4096, 4096, _lib.BF16, _lib.ALGO_DENSE, 0, 3) == 0
    assert lib.b200s_tuner_record_schedule(8192, 8192, 8192, _lib.BF16, _lib.ALGO_CLASSIC, 1, 7) == _lib.ERR_BAD_SHAPE
    old = tmp_path / "six_columns.txt"
    old.write_text("# M N K in_dtype algo depth\n8192 8192 8192 0 3 1\n")
    new = str(tmp_path / "seven.txt").encode()
    assert lib.b200s_tuner_save(new) == 0
    lib.b200s_tuner_clear()
    assert lib.b200s_tuner_load(new) == 0
    for shape, want in (((16384, 16384, 16384), (_lib.ALGO_CLASSIC, 2, 3)), ((4096, 4096, 4096), (_lib.ALGO_DENSE, 0, 0))):
        assert lib.b200s_tuner_lookup_schedule(*shape, _lib.BF16, ctypes.byref(a), ctypes.byref(d), ctypes.byref(f)) == 0
        assert (a.value, d.value, f.value) == want                # a dense entry has no schedule
    assert lib.b200s_tuner_load(str(old).encode()) == 0           # tables without the column still load
    assert lib.b200s_tuner_lookup_schedule(8192, 8192, 8192, _lib.BF16, ctypes.byref(a), ctypes.byref(d),
                                           ctypes.byref(f)) == 0
    assert (a.value, d.value, f.value) == (_lib.ALGO_WINOGRAD, 1, 0)
    lib.b200s_tuner_clear()


def test_new_entry_points_validate_before_touching_a_device(lib):
    p = problem()
    assert lib.b200s_matmul_bias(ctypes.byref(p), 16, 16, None, 16, 256, 1 << 30, None) == _lib.ERR_NULL_POINTER
    assert lib.b200s_matmul_peers(ctypes.byref(p), 16, 16, None, 2, 256, 1 << 30, None) == _lib.ERR_NULL_POINTER
    dst = (ctypes.c_void_p * 2)(16, 32)
    assert lib.b200s_matmul_peers(ctypes.byref(p), 16, 16, dst, 9, 256, 1 << 30, None) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_matmul_peers(ctypes.byref(problem(beta=1)), 16, 16, dst, 2, 256, 1 << 30, None) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_matmul_multicast(ctypes.byref(p), 16, 16, 16, None, 256, 1 << 30, None) == _lib.ERR_NULL_POINTER
    # the multicast store lives in the dense epilogue: a Strassen problem is refused
    assert lib.b200s_matmul_multicast(ctypes.byref(p), 16, 16, 16, 32, 256, 1 << 30, None) == _lib.ERR_BAD_ALGO
    assert lib.b200s_peer_barrier(None, 0, 2, 1, 1000, None) == _lib.ERR_NULL_POINTER
    assert lib.b200s_peer_barrier(dst, 2, 2, 1, 1000, None) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_peer_barrier(dst, 0, 2, 1, 0, None) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_wait_probe(0, None) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_profile_begin(0) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_profile_end(None, None) == _lib.ERR_NULL_POINTER
    assert lib.b200s_workspace_bytes(ctypes.byref(problem(fuse=4)), ctypes.byref(ctypes.c_size_t(0))) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_push_panel(None, dst, 2, None, 256, 8, None) == _lib.ERR_NULL_POINTER
    assert lib.b200s_push_panel(16, None, 0, None, 256, 8, None) == _lib.ERR_NULL_POINTER      # neither peers nor multicast
    assert lib.b200s_push_panel(16, dst, 2, None, 250, 8, None) == _lib.ERR_BAD_SHAPE         # not whole 16-byte vectors
    assert lib.b200s_push_panel(16, dst, 2, None, 256, 0, None) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_push_panel(16, dst, 9, None, 256, 8, None) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_push_panel(24, None, 0, 32, 256, 8, None) == _lib.ERR_BAD_ALIGNMENT
    assert lib.b200s_set_product_sms(-1) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_set_product_sms(140) == 0 and lib.b200s_set_product_sms(0) == 140        # returns the previous setting
    assert lib.b200s_set_sender_sms(-2) == _lib.ERR_BAD_SHAPE and lib.b200s_set_sender_sms(66) == _lib.ERR_BAD_SHAPE
    assert lib.b200s_set_sender_sms(8) == 0 and lib.b200s_set_sender_sms(0) == 8


def test_fused_schedule_keeps_its_counters_at_the_end_of_the_scratch(lib):
    """Every one- or two-level scratch ends with the 256 bytes of counters the fused kernel's CTAs
    share, whatever schedule a call ends up using; the schedule itself does not change the size."""
    sizes = {ws_bytes(lib, problem(fuse=f))[1] for f in (0, 1, 2, 3)}
    assert len(sizes) == 1 and sizes.pop() == 3 * 49 * 256 * 256 * 2 + FLAGS

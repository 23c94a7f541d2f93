"""Tensor-level entry to libb200s.so: `matmul(A, B, ...)` on CUDA tensors, and the autograd
function every reference-named module in this repository routes through.

torch is plumbing here (device memory, streams, autograd bookkeeping); all arithmetic runs in
the CUDA library through its C ABI.
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import Optional

import torch

from . import _lib

_DTYPE = {torch.bfloat16: _lib.BF16, torch.float16: _lib.FP16, torch.float32: _lib.FP32}
_ALGO = {"auto": _lib.ALGO_AUTO, "dense": _lib.ALGO_DENSE, "classic": _lib.ALGO_CLASSIC,
         "strassen": _lib.ALGO_CLASSIC, "winograd": _lib.ALGO_WINOGRAD}


def resolve_precision(precision):
    """How fp32 operands reach the tensor cores: "tf32" (one pass) or "3xtf32" (hi/lo split, three
    passes, fp32-level accuracy). ``None`` follows ``torch.backends.cuda.matmul.allow_tf32``, the
    switch the reference's scripts set (main_profiling.py:31-34): TF32 when it is on, else the
    three-pass mode, as torch.mm would then compute in full fp32."""
    if precision is None:
        return "tf32" if torch.backends.cuda.matmul.allow_tf32 else "3xtf32"
    if precision not in ("tf32", "3xtf32"):
        raise ValueError("precision must be 'tf32', '3xtf32' or None")
    return precision


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"expected a torch.Tensor, got {type(t).__name__}")
        if not t.is_cuda:
            raise RuntimeError("b200s kernels run on CUDA tensors only; there is no CPU path "
                               f"(got a tensor on {t.device})")


def _operand(t: torch.Tensor):
    """(tensor, major_is_inner, ld, batch_stride) for a 2-D or 3-D operand, copying only when
    neither of the last two dimensions has unit stride or the strides break 16-byte alignment."""
    es = t.element_size()

    def ok(x):
        r, c = x.shape[-2], x.shape[-1]
        sr, sc = x.stride(-2), x.stride(-1)
        bs = x.stride(0) if x.dim() == 3 else 0
        if (x.data_ptr() % 16) or (bs * es) % 16:
            return None
        if sc == 1 and (sr * es) % 16 == 0 and sr >= c:
            return (True, sr, bs)       # rows x cols with cols contiguous
        if sr == 1 and (sc * es) % 16 == 0 and sc >= r:
            return (False, sc, bs)      # columns contiguous: a transposed view
        return None

    got = ok(t)
    if got is None:
        t = t.contiguous()
        got = ok(t)
        if got is None:
            raise ValueError("operand rows must be a multiple of 16 bytes long "
                             f"(shape {tuple(t.shape)}, dtype {t.dtype})")
    return (t,) + got


def make_problem(A, B, C, algo="auto", depth=-1, beta=0, prod_dtype=None, precision=None,
                 tile_variant=0, pipeline=0, b_blocks_ready=False, fuse=0):
    """Fill a ``b200s_problem`` for C (+)= A @ B. Returns (problem, A', B') where A'/B' are the
    tensors whose pointers must be passed (copies only when the strides force one)."""
    if A.dim() != B.dim() or A.dim() not in (2, 3):
        raise ValueError("A and B must both be 2-D, or both 3-D (batched)")
    if A.dtype != B.dtype or A.dtype not in _DTYPE:
        raise TypeError(f"unsupported operand dtypes {A.dtype}, {B.dtype}")
    if C.dtype not in _DTYPE:
        raise TypeError(f"unsupported output dtype {C.dtype}")
    M, K = A.shape[-2], A.shape[-1]
    K2, N = B.shape[-2], B.shape[-1]
    assert K == K2 and C.shape[-2] == M and C.shape[-1] == N, "shape mismatch"
    batch = A.shape[0] if A.dim() == 3 else 1
    if A.dim() == 3:
        assert B.shape[0] == batch and C.shape[0] == batch, "batch mismatch"
    if C.stride(-1) != 1:
        raise ValueError("C must be row-major (unit stride in its last dimension)")
    A2, a_inner, lda, sa = _operand(A)
    B2, b_inner, ldb, sb = _operand(B)
    p = _lib.Problem()
    p.M, p.N, p.K, p.batch = M, N, K, batch
    p.lda, p.ldb, p.ldc = lda, ldb, C.stride(-2)
    p.strideA, p.strideB = sa, sb
    p.strideC = C.stride(0) if C.dim() == 3 else 0
    # A is M x K: inner-contiguous means K-major. B is K x N: inner-contiguous means N-major.
    p.a_major = _lib.K_MAJOR if a_inner else _lib.MN_MAJOR
    p.b_major = _lib.MN_MAJOR if b_inner else _lib.K_MAJOR
    p.in_dtype = _DTYPE[A.dtype]
    p.out_dtype = _DTYPE[C.dtype]
    p.algo = _ALGO[algo] if isinstance(algo, str) else int(algo)
    p.depth = int(depth)
    p.beta = int(beta)
    p.prod_dtype = -1 if prod_dtype is None else _DTYPE[prod_dtype]
    p.precision = _lib.PREC_3XTF32 if resolve_precision(precision) == "3xtf32" else _lib.PREC_TF32
    p.tile_variant = int(tile_variant)
    p.pipeline = int(pipeline)
    p.b_blocks_ready = 1 if b_blocks_ready else 0
    p.fuse = int(fuse)
    return p, A2, B2


def workspace_bytes(p: "_lib.Problem") -> int:
    n = ctypes.c_size_t(0)
    _lib.check(_lib.load().b200s_workspace_bytes(ctypes.byref(p), ctypes.byref(n)))
    return n.value


def resolve(p: "_lib.Problem"):
    a, d = ctypes.c_int32(0), ctypes.c_int32(0)
    _lib.check(_lib.load().b200s_resolve(ctypes.byref(p), ctypes.byref(a), ctypes.byref(d)))
    return a.value, d.value


def matmul_out(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, *, algo="auto", depth=-1, beta=0,
               prod_dtype=None, precision=None, tile_variant=0, pipeline=0, b_blocks_ready=False, fuse=0,
               workspace: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A @ B (beta=0) or C += A @ B (beta=1) on the current CUDA stream, plus ``bias`` (N elements
    of C's dtype, added to every row before the rounding) when given. Returns C."""
    _require_cuda(A, B, C)
    if bias is not None:
        _require_cuda(bias)
        if bias.dim() != 1 or bias.shape[0] != B.shape[-1] or A.dim() != 2:
            raise ValueError("bias must hold one element per column of a 2-D product")
        bias = bias.to(C.dtype).contiguous()
    lib = _lib.load()
    p, A2, B2 = make_problem(A, B, C, algo, depth, beta, prod_dtype, precision, tile_variant, pipeline, b_blocks_ready,
                             fuse)
    with torch.cuda.device(C.device):
        need = workspace_bytes(p)
        ws_ptr = None
        if need:
            if workspace is None or workspace.numel() * workspace.element_size() < need:
                workspace = torch.empty(need, dtype=torch.uint8, device=C.device)
            ws_ptr = workspace.data_ptr()
        stream = torch.cuda.current_stream(C.device).cuda_stream
        if bias is None:
            rc = lib.b200s_matmul(ctypes.byref(p), A2.data_ptr(), B2.data_ptr(), C.data_ptr(), ws_ptr,
                                  need if need else 0, stream)
        else:
            rc = lib.b200s_matmul_bias(ctypes.byref(p), A2.data_ptr(), B2.data_ptr(), bias.data_ptr(), C.data_ptr(),
                                       ws_ptr, need if need else 0, stream)
        _lib.check(rc)
        if workspace is not None:
            workspace.record_stream(torch.cuda.current_stream(C.device))
    return C


def matmul(A: torch.Tensor, B: torch.Tensor, *, algo="auto", depth=-1, out_dtype=None, prod_dtype=None,
           precision=None, tile_variant=0, pipeline=0, b_blocks_ready=False, fuse=0, workspace=None,
           bias=None) -> torch.Tensor:
    """A @ B (+ bias) as a new tensor of ``out_dtype`` (default: the operand dtype)."""
    _require_cuda(A, B)
    shape = (A.shape[-2], B.shape[-1]) if A.dim() == 2 else (A.shape[0], A.shape[-2], B.shape[-1])
    C = torch.empty(shape, dtype=out_dtype or A.dtype, device=A.device)
    return matmul_out(A, B, C, algo=algo, depth=depth, beta=0, prod_dtype=prod_dtype, precision=precision,
                      tile_variant=tile_variant, pipeline=pipeline, b_blocks_ready=b_blocks_ready, fuse=fuse,
                      workspace=workspace, bias=bias)


def device_status(device=None):
    """(status, detail) of the device status word; synchronises the current stream."""
    lib = _lib.load()
    s, d = ctypes.c_int32(0), ctypes.c_int32(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.b200s_device_status(stream, ctypes.byref(s), ctypes.byref(d)))
    return s.value, d.value


STAGES = ("operand_blocks_A", "operand_blocks_B", "products", "recombination")


@contextlib.contextmanager
def stage_timing(max_calls: int = 256):
    """Collect the library's per-stage event timing for the matmul calls made inside the block.
    Yields a dict that, after the block, holds the mean milliseconds of the four stages (keys
    ``STAGES``; in the fused schedule: the first group's blocks of A and of B, the fused kernel, the
    recombination left after it) and ``calls``, the number of calls measured."""
    lib = _lib.load()
    _lib.check(lib.b200s_profile_begin(int(max_calls)))
    out = {}
    try:
        yield out
    finally:
        ms = (ctypes.c_float * 4)()
        calls = ctypes.c_int32(0)
        _lib.check(lib.b200s_profile_end(ms, ctypes.byref(calls)))
        out.update({k: float(ms[i]) for i, k in enumerate(STAGES)})
        out["calls"] = calls.value


# ---- the differentiable product as a torch.library custom op ------------------------------------
# The reference wraps its layers and whole models in torch.compile (main_profiling.py:130-144,
# modded_nanogpt/data_dist_train_gpt2.py:721); its own matmuls are plain torch ops that dynamo traces
# through. A ctypes call cannot be traced, so the product is registered as an opaque operator with a
# shape-only (fake) implementation and an autograd formula: dynamo and AOT autograd then carry it
# through a compiled graph without a graph break, forward and backward.
_DT_NAME = {None: "", torch.bfloat16: "bf16", torch.float16: "fp16", torch.float32: "fp32"}
_NAME_DT = {v: k for k, v in _DT_NAME.items()}


@torch.library.custom_op("b200s::matmul", mutates_args=())
def _matmul_op(X: torch.Tensor, W: torch.Tensor, algo: str, depth: int, prod_dtype: str) -> torch.Tensor:
    return matmul(X, W, algo=algo, depth=depth, prod_dtype=_NAME_DT[prod_dtype])


@_matmul_op.register_fake
def _(X, W, algo, depth, prod_dtype):
    shape = (X.shape[-2], W.shape[-1]) if X.dim() == 2 else (X.shape[0], X.shape[-2], W.shape[-1])
    return X.new_empty(shape)


def _matmul_setup(ctx, inputs, output):
    X, W, algo, depth, prod_dtype = inputs
    ctx.save_for_backward(X, W)
    ctx.cfg = (algo, depth, prod_dtype)


def _matmul_backward(ctx, dY):
    """dX = dY @ W^T and dW = X^T @ dY through the same operator, with transposed views (no copies).
    The reference has no custom backward: autograd differentiates its slice/add/mm graph
    (fixed_strassen_fp32_agg.py:13-125), which computes these same two products."""
    X, W = ctx.saved_tensors
    algo, depth, prod_dtype = ctx.cfg
    dX = dW = None
    if dY.dtype != X.dtype:
        dY = dY.to(X.dtype)
    if ctx.needs_input_grad[0]:
        dX = _matmul_op(dY, W.transpose(-1, -2), algo, depth, prod_dtype)
    if ctx.needs_input_grad[1]:
        dW = _matmul_op(X.transpose(-1, -2), dY, algo, depth, prod_dtype)
    return dX, dW, None, None, None


_matmul_op.register_autograd(_matmul_backward, setup_context=_matmul_setup)


@torch.library.custom_op("b200s::linear", mutates_args=())
def _linear_op(X: torch.Tensor, W: torch.Tensor, bias: torch.Tensor, algo: str, depth: int) -> torch.Tensor:
    """X @ W + bias with the bias added in the product's epilogue (X 2-D, W given as weight.T)."""
    if depth > 2:      # the recursion above two levels has no epilogue of its own to carry the bias
        return matmul(X, W, algo=algo, depth=depth) + bias.to(X.dtype)
    return matmul(X, W, algo=algo, depth=depth, bias=bias)


@_linear_op.register_fake
def _(X, W, bias, algo, depth):
    return X.new_empty((X.shape[0], W.shape[1]))


def _linear_setup(ctx, inputs, output):
    X, W, bias, algo, depth = inputs
    ctx.save_for_backward(X, W)
    ctx.cfg = (algo, depth, bias.dtype)


def _linear_backward(ctx, dY):
    X, W = ctx.saved_tensors
    algo, depth, bias_dtype = ctx.cfg
    dX = dW = db = None
    if ctx.needs_input_grad[2]:
        db = dY.sum(0).to(bias_dtype)
    if dY.dtype != X.dtype:
        dY = dY.to(X.dtype)
    if ctx.needs_input_grad[0]:
        dX = _matmul_op(dY, W.transpose(-1, -2), algo, depth, "")
    if ctx.needs_input_grad[1]:
        dW = _matmul_op(X.transpose(-1, -2), dY, algo, depth, "")
    return dX, dW, db, None, None


_linear_op.register_autograd(_linear_backward, setup_context=_linear_setup)


def linear_autograd(X, W, bias, algo="auto", depth=-1):
    """Differentiable X @ W + bias (X 2-D, W = weight.T as a view), the bias fused into the epilogue."""
    _require_cuda(X, W, bias)
    return _linear_op(X, W, bias, algo, int(depth))


def matmul_autograd(X, W, algo="auto", depth=-1, prod_dtype=None):
    """Differentiable X @ W (2-D or batched 3-D operands); traceable by torch.compile."""
    _require_cuda(X, W)
    return _matmul_op(X, W, algo, int(depth), _DT_NAME[prod_dtype])

"""CPU restatement of the reference's torch-level Strassen recursion, used as the parity checker.

THIS IS TEST INFRASTRUCTURE, not a product path: only ``tests/``, ``__graft_entry__.smoke()`` and
the CPU-baseline / reference legs of ``bench.py`` may import it. The shipped library never does.

What it restates (file:line in vmad18/strassen-triton):

* ``one_level``        - ``_strassen_base``: fixed_strassen_fp32_agg.py:13-56 (fp32 aggregation),
                         fixed_strassen.py:12-57 and strassen.py:697-740 (same dtype throughout).
* ``n_layers``         - ``strassen_matmul_n_layers``: fixed_strassen_fp32_agg.py:59-125,
                         fixed_strassen.py:60-126; ``strassen_matmul_two_layers``: strassen.py:742-812.
* ``winograd_levels``  - the Strassen-Winograd schedule; the reference's Winograd kernels
                         (strassen_no_tuning.py:452-556) are not a valid bilinear algorithm, so this
                         follows the published schedule instead.
* ``library_model``    - the rounding points of libb200s.so itself (operand sums in fp32 from the
                         original blocks, one rounding; fp32 products; one recombination in fp32),
                         written with the same coefficient tables, for tight GPU comparisons.

The sub-products are ``torch.mm`` on CPU tensors, as in the reference; torch is a third-party
dependency the reference does not pin (this image: torch 2.11.0).

Parity pin: the reference itself was imported and run in the build container on seeded inputs;
its outputs are committed under ``tests/golden/`` with the generating script, and
``tests/test_oracle.py`` checks every function here against them. The reference has no golden
vectors or known-answer tests of its own.
"""
from __future__ import annotations

from typing import Optional

import torch

AGG = torch.float32  # fixed_strassen_fp32_agg.py:10


def _quad(X: torch.Tensor):
    """The four quadrants (11, 12, 21, 22); rows and columns are halved independently so that
    rectangular operands work. On square inputs this is the reference's A[:mid,:mid] etc."""
    r, c = X.shape[-2] // 2, X.shape[-1] // 2
    return X[..., :r, :c], X[..., :r, c:], X[..., r:, :c], X[..., r:, c:]


def _assemble(C11, C12, C21, C22):
    return torch.vstack([torch.hstack([C11, C12]), torch.hstack([C21, C22])])


def one_level(A: torch.Tensor, B: torch.Tensor, base_dtype=torch.float32, agg: bool = True,
              mm=torch.mm) -> torch.Tensor:
    """One Strassen level. ``agg=True`` follows fixed_strassen_fp32_agg.py:13-56: quadrants are
    widened to fp32, operand sums are rounded to ``base_dtype``, the seven ``torch.mm`` run in
    ``base_dtype``, the products are widened, summed in fp32 and rounded to ``base_dtype``.
    ``agg=False`` follows fixed_strassen.py:12-57: no casts, ``base_dtype`` ignored."""
    if A.shape[0] <= 16:  # fixed_strassen_fp32_agg.py:19-20
        return mm(A, B)
    if agg:
        a11, a12, a21, a22 = (q.to(AGG) for q in _quad(A))
        b11, b12, b21, b22 = (q.to(AGG) for q in _quad(B))
        lo = lambda t: t.to(base_dtype)
        up = lambda t: t.to(AGG)
    else:
        a11, a12, a21, a22 = _quad(A)
        b11, b12, b21, b22 = _quad(B)
        lo = up = lambda t: t
    m1 = up(mm(lo(a11 + a22), lo(b11 + b22)))
    m2 = up(mm(lo(a21 + a22), lo(b11)))
    m3 = up(mm(lo(a11), lo(b12 - b22)))
    m4 = up(mm(lo(a22), lo(b21 - b11)))
    m5 = up(mm(lo(a11 + a12), lo(b22)))
    m6 = up(mm(lo(a21 - a11), lo(b11 + b12)))
    m7 = up(mm(lo(a12 - a22), lo(b21 + b22)))
    c11 = lo(m1 + m4 - m5 + m7)
    c12 = lo(m3 + m5)
    c21 = lo(m2 + m4)
    c22 = lo(m1 - m2 + m3 + m6)
    return _assemble(c11, c12, c21, c22)


def n_layers(A: torch.Tensor, B: torch.Tensor, n_depth: int = 2, base_dtype=torch.float32, agg: bool = True,
             forward_base_dtype: bool = False, mm=torch.mm) -> torch.Tensor:
    """The recursive driver, fixed_strassen_fp32_agg.py:59-125 (``agg=True``) or
    fixed_strassen.py:60-126 / strassen.py:742-812 (``agg=False``).

    ``forward_base_dtype=False`` reproduces the reference as shipped: the seven sub-calls at
    fixed_strassen_fp32_agg.py:99-113 omit ``base_dtype``, so every level below the top runs in
    fp32. ``True`` is the evident intent (``base_dtype`` at every level)."""
    if n_depth == 1:
        return one_level(A, B, base_dtype, agg, mm)
    mid = A.shape[0] // 2
    if agg:
        a11, a12, a21, a22 = (q.to(AGG) for q in _quad(A))
        b11, b12, b21, b22 = (q.to(AGG) for q in _quad(B))
        lo = lambda t: t.to(base_dtype)
        up = lambda t: t.to(AGG)
    else:
        a11, a12, a21, a22 = _quad(A)
        b11, b12, b21, b22 = _quad(B)
        lo = up = lambda t: t
    s1, s2, s3, s4, s5 = lo(b12 - b22), lo(a11 + a12), lo(a21 + a22), lo(b21 - b11), lo(a11 + a22)
    s6, s7, s8, s9, s10 = lo(b11 + b22), lo(a12 - a22), lo(b21 + b22), lo(a21 - a11), lo(b11 + b12)
    inner_dtype = base_dtype if forward_base_dtype else torch.float32
    if mid == 2 or n_depth == 2:
        sub = lambda x, y: one_level(x, y, inner_dtype, agg, mm)
    else:
        sub = lambda x, y: n_layers(x, y, n_depth - 1, inner_dtype, agg, forward_base_dtype, mm)
    # The raw quadrants reach the sub-calls widened to fp32 in the agg variant (:100-104).
    m1 = up(sub(s5, s6))
    m2 = up(sub(s3, b11))
    m3 = up(sub(a11, s1))
    m4 = up(sub(a22, s4))
    m5 = up(sub(s2, b22))
    m6 = up(sub(s9, s10))
    m7 = up(sub(s7, s8))
    c11 = lo(m1 + m4 - m5 + m7)
    c12 = lo(m3 + m5)
    c21 = lo(m2 + m4)
    c22 = lo(m1 - m2 + m3 + m6)
    return _assemble(c11, c12, c21, c22)


def winograd_levels(A: torch.Tensor, B: torch.Tensor, depth: int = 1, base_dtype: Optional[torch.dtype] = None,
                    mm=torch.mm) -> torch.Tensor:
    """Strassen-Winograd, ``depth`` levels, with the reference's fp32-aggregation casts
    (operand sums in fp32 rounded to ``base_dtype``, products widened and summed in fp32)."""
    base_dtype = base_dtype or A.dtype
    if depth == 0:
        return mm(A.to(base_dtype), B.to(base_dtype))
    a11, a12, a21, a22 = (q.to(AGG) for q in _quad(A))
    b11, b12, b21, b22 = (q.to(AGG) for q in _quad(B))
    lo = lambda t: t.to(base_dtype)
    sub = lambda x, y: winograd_levels(lo(x), lo(y), depth - 1, base_dtype, mm).to(AGG)
    s1 = a21 + a22
    s2 = s1 - a11
    s3 = a11 - a21
    s4 = a12 - s2
    t1 = b12 - b11
    t2 = b22 - t1
    t3 = b22 - b12
    t4 = t2 - b21
    p1, p2, p3, p4 = sub(a11, b11), sub(a12, b21), sub(s4, b22), sub(a22, t4)
    p5, p6, p7 = sub(s1, t1), sub(s2, t2), sub(s3, t3)
    u2 = p1 + p6
    u3 = u2 + p7
    u4 = u2 + p5
    return _assemble(lo(p1 + p2), lo(u4 + p3), lo(u3 - p4), lo(u3 + p5))


# ---------------------------------------------------------------------------------------------
# Model of the library's own rounding points (same tables as strassen_triton_b200/csrc/schedule.h)
# ---------------------------------------------------------------------------------------------

_U = {
    "classic": [[1, 0, 0, 1], [0, 0, 1, 1], [1, 0, 0, 0], [0, 0, 0, 1], [1, 1, 0, 0], [-1, 0, 1, 0], [0, 1, 0, -1]],
    "winograd": [[1, 0, 0, 0], [0, 1, 0, 0], [1, 1, -1, -1], [0, 0, 0, 1], [0, 0, 1, 1], [-1, 0, 1, 1], [1, 0, -1, 0]],
}
_V = {
    "classic": [[1, 0, 0, 1], [1, 0, 0, 0], [0, 1, 0, -1], [-1, 0, 1, 0], [0, 0, 0, 1], [1, 1, 0, 0], [0, 0, 1, 1]],
    "winograd": [[1, 0, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1], [1, -1, -1, 1], [-1, 1, 0, 0], [1, -1, 0, 1], [0, -1, 0, 1]],
}
_W = {
    "classic": [[1, 0, 0, 1, -1, 0, 1], [0, 0, 1, 0, 1, 0, 0], [0, 1, 0, 1, 0, 0, 0], [1, -1, 1, 0, 0, 1, 0]],
    "winograd": [[1, 1, 0, 0, 0, 0, 0], [1, 0, 1, 0, 1, 1, 0], [1, 0, 0, -1, 0, 1, 1], [1, 0, 0, 0, 1, 1, 1]],
}


def tables(algo: str, depth: int):
    """(U, V, W) as nested lists for ``depth`` levels: Kronecker powers of the one-level tables,
    product index p = 7*p1 + p2, quadrant index q = 4*q1 + q2 (index 1 = outer level)."""
    U, V, W = _U[algo], _V[algo], _W[algo]
    for _ in range(depth - 1):
        U = [[a * b for a in ro for b in ri] for ro in _U[algo] for ri in U]
        V = [[a * b for a in ro for b in ri] for ro in _V[algo] for ri in V]
        W = [[a * b for a in ro for b in ri] for ro in _W[algo] for ri in W]
    return U, V, W


def _blocks(X: torch.Tensor, depth: int):
    """4^depth blocks in quadrant-index order q = 4*q1 + q2."""
    if depth == 0:
        return [X]
    out = []
    for q in _quad(X):
        out.extend(_blocks(q, depth - 1))
    return out


def _unblocks(blocks, depth: int):
    if depth == 0:
        return blocks[0]
    n = len(blocks) // 4
    qs = [_unblocks(blocks[i * n:(i + 1) * n], depth - 1) for i in range(4)]
    return _assemble(*qs)


def _signed_sum(coefs, blocks):
    acc = None
    for c, b in zip(coefs, blocks):
        if c == 0:
            continue
        if acc is None:
            acc = b if c > 0 else -b
        else:
            acc = acc + b if c > 0 else acc - b
    return acc


def recombine(products, depth: int, algo: str = "classic") -> torch.Tensor:
    """C from the 7^depth product blocks (index p = 7*p1 + p2) by the recombination table: the
    post-additions and quadrant assembly of fixed_strassen_fp32_agg.py:47-56 and :115-123, in the
    dtype of the blocks (pass fp64 blocks for a rounding-free reference)."""
    _, _, W = tables(algo, depth)
    blocks = list(products)
    if len(blocks) != 7 ** depth:
        raise ValueError(f"{7 ** depth} product blocks expected, got {len(blocks)}")
    return _unblocks([_signed_sum(W[r], blocks) for r in range(4 ** depth)], depth)


def library_model(A: torch.Tensor, B: torch.Tensor, depth: int, algo: str = "classic",
                  prod_dtype: Optional[torch.dtype] = None, out_dtype: Optional[torch.dtype] = None,
                  exact_products: bool = True) -> torch.Tensor:
    """What libb200s.so computes, restated on the CPU: operand blocks summed in fp32 from the
    original blocks and rounded once to the input dtype; products of the rounded operands (fp64
    when ``exact_products``, else fp32 ``torch.mm``) rounded to ``prod_dtype``; one fp32
    recombination over all levels, rounded once to ``out_dtype``."""
    in_dtype = A.dtype
    prod_dtype = prod_dtype or in_dtype
    out_dtype = out_dtype or in_dtype
    if depth == 0:
        C = (A.double() @ B.double()) if exact_products else torch.mm(A.float(), B.float())
        return C.to(out_dtype)
    U, V, W = tables(algo, depth)
    wide = torch.float64 if in_dtype == torch.float64 else torch.float32  # fp64 only to test the tables
    ab = [b.to(wide) for b in _blocks(A, depth)]
    bb = [b.to(wide) for b in _blocks(B, depth)]
    prods = []
    for p in range(7 ** depth):
        sa = _signed_sum(U[p], ab).to(in_dtype)
        sb = _signed_sum(V[p], bb).to(in_dtype)
        m = (sa.double() @ sb.double()) if exact_products else torch.mm(sa.float(), sb.float())
        prods.append(m.to(prod_dtype).to(wide))
    cb = [_signed_sum(W[r], prods).to(out_dtype) for r in range(4 ** depth)]
    return _unblocks(cb, depth)


def errors_vs_fp64(C: torch.Tensor, A: torch.Tensor, B: torch.Tensor):
    """(max-abs, relative Frobenius) error of C against A.double() @ B.double()."""
    ref = A.double() @ B.double()
    d = C.double() - ref
    return d.abs().max().item(), (d.norm() / ref.norm()).item()

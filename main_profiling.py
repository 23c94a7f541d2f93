"""Drop-in for the reference's README benchmark (``python main_profiling.py``,
main_profiling.py:94-302): ``LinearStrassen`` against ``nn.Linear`` for square layers of size N and
several depths, with the same columns - time of the standard layer, time of the Strassen layer,
speed-up, TFLOP/s by the standard count 2*N^3, max-abs difference and allclose - measured with CUDA
events after warm-up (the reference uses ``triton.testing.do_bench`` on ``torch.compile``d layers; no
compiler is involved here, ``nn.Linear`` is cuBLAS and ``LinearStrassen`` is this library). A third
timing column shows how the reference itself computes the layer on this GPU: the torch-level Strassen
recursion (slices, elementwise sums in fp32, ``torch.mm`` sub-products) of
fixed_strassen_fp32_agg.py:13-125, restated below as the baseline ``torch_strassen``.

    python main_profiling.py [--sizes 4096 8192 16384] [--depths 1 2] [--dtype bf16] [--reps 20]
"""
import argparse

import torch
import torch.nn as nn

from model.layers import LinearStrassen

USE_TF32 = True  # main_profiling.py:14
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def bench_ms(fn, warmup, reps):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[0], sum(times) / len(times)


def torch_strassen(A, B, depth, dtype):
    """Baseline only: Strassen as the reference runs it, with torch ops (eight quadrant views widened to
    fp32, ten sums rounded to `dtype`, seven torch.mm, eight fp32 sums, two concatenations per level)."""
    n = A.shape[0]
    if depth == 0 or n <= 16:
        return torch.mm(A.to(dtype), B.to(dtype))
    m = n // 2
    a11, a12, a21, a22 = (A[:m, :m].float(), A[:m, m:].float(), A[m:, :m].float(), A[m:, m:].float())
    b11, b12, b21, b22 = (B[:m, :m].float(), B[:m, m:].float(), B[m:, :m].float(), B[m:, m:].float())
    mul = lambda x, y: torch_strassen(x.to(dtype), y.to(dtype), depth - 1, dtype).float()  # noqa: E731
    m1 = mul(a11 + a22, b11 + b22)
    m2 = mul(a21 + a22, b11)
    m3 = mul(a11, b12 - b22)
    m4 = mul(a22, b21 - b11)
    m5 = mul(a11 + a12, b22)
    m6 = mul(a21 - a11, b11 + b12)
    m7 = mul(a12 - a22, b21 + b22)
    top = torch.cat((m1 + m4 - m5 + m7, m3 + m5), dim=1)
    bottom = torch.cat((m2 + m4, m1 - m2 + m3 + m6), dim=1)
    return torch.cat((top, bottom), dim=0).to(dtype)


def benchmark_linear_layers(N, depth, dtype, reps):
    """One row of the table: a D x D input through nn.Linear(D, D) and LinearStrassen(D, D, depth)."""
    std = nn.Linear(N, N, bias=False, device="cuda", dtype=dtype)
    strassen = LinearStrassen(N, N, bias=False, dtype=dtype, depth=depth, device="cuda")
    with torch.no_grad():
        strassen.weight.copy_(std.weight)
        x = torch.randn(N, N, device="cuda", dtype=dtype) / N ** 0.5
        y_std, y_str = std(x), strassen(x)
        max_diff = (y_std.float() - y_str.float()).abs().max().item()
        close = torch.allclose(y_std.float(), y_str.float(), rtol=5e-2, atol=5e-2 * y_std.float().abs().max().item())
        std_min, std_mean = bench_ms(lambda: std(x), 5, reps)
        str_min, str_mean = bench_ms(lambda: strassen(x), 5, reps)
        wt = std.weight.t()
        ref_min, ref_mean = bench_ms(lambda: torch_strassen(x, wt, depth, dtype), 2, max(3, reps // 4))
    flops = 2.0 * N ** 3
    return {"N": N, "depth": depth, "std_ms": std_mean, "strassen_ms": str_mean, "torch_strassen_ms": ref_mean,
            "speedup": std_mean / str_mean, "speedup_vs_torch_strassen": ref_mean / str_mean,
            "std_tflops": flops / std_min / 1e9, "strassen_tflops": flops / str_min / 1e9,
            "torch_strassen_tflops": flops / ref_min / 1e9, "max_abs_diff": max_diff, "allclose": close}


def profile_linear_layers(sizes, depths, dtype, reps):
    rows = []
    print(f"{'N':>6} {'depth':>5} {'std ms':>9} {'strassen ms':>12} {'torch-str ms':>13} {'speedup':>8} {'std TF/s':>9} "
          f"{'str TF/s':>9} {'t-str TF/s':>10} {'max|diff|':>10} allclose")
    for N in sizes:
        for depth in depths:
            if N % (8 << depth):
                continue
            r = benchmark_linear_layers(N, depth, dtype, reps)
            rows.append(r)
            print(f"{r['N']:6d} {r['depth']:5d} {r['std_ms']:9.3f} {r['strassen_ms']:12.3f} {r['torch_strassen_ms']:13.3f} "
                  f"{r['speedup']:8.3f} {r['std_tflops']:9.1f} {r['strassen_tflops']:9.1f} {r['torch_strassen_tflops']:10.1f} "
                  f"{r['max_abs_diff']:10.3e} {r['allclose']}")
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=int, nargs="+", default=[1024, 2048, 4096, 8192, 16384])
    ap.add_argument("--depths", type=int, nargs="+", default=[1, 2])
    ap.add_argument("--dtype", default="bf16", choices=sorted(DTYPES))
    ap.add_argument("--reps", type=int, default=20)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("main_profiling.py needs a CUDA device (the library has no CPU path)")
    torch.backends.cuda.matmul.allow_tf32 = USE_TF32   # main_profiling.py:31-34
    torch.backends.cudnn.allow_tf32 = USE_TF32
    profile_linear_layers(args.sizes, args.depths, DTYPES[args.dtype], args.reps)

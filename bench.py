#!/usr/bin/env python
"""Benchmark of the Strassen matmul path: effective TFLOP/s (2*M*N*K / t), bf16.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one full product C = A @ B through the library (two Strassen levels where the tuner
table picks them, bf16 operands, fp32 accumulation and aggregation, bf16 result).

* N = 1: M = N = K = 16384, inputs U(-1,1) from seed 0 (the configuration the headline metric is
  quoted on), algorithm classic / depth 2, schedule from the library's tuner table. ``value`` times
  K steps with the inputs resident in HBM; ``e2e`` times the same product with operands and result in
  pinned host memory through ``strassen_triton_b200.host.HostStreamedMatmul`` (B, then A in row panels,
  products and the way back of C overlapping the arrivals; all copies inside the timed region), and
  reports beside it the plain sequence copy, copy, ``strassen_matmul_n_layers``, copy. ``interleaved`` is the comparison with cuBLAS dense on the same GPU: three
  arms (separate passes, fused kernel, cuBLAS) take turns, every turn starts on a rested GPU and runs back to back for
  ``--seconds``; the first 20 calls of a turn are its "burst" figure, the last second its "sustained"
  one, each with the SM clock sampled during the turn. ``reference_gpu`` is the reference recursion
  (the oracle port) on CUDA tensors, i.e. the reference as it would run on this GPU with cuBLAS
  sub-products. ``stages_ms`` comes from the library's own stage events recorded during the K timed
  steps.
* N > 1 (launched by torch.distributed.run, one rank per GPU): M = N = K = 32768, A split into row
  blocks, B replicated; every rank runs the algorithm the tuner table picks for its block (a dense product at four ranks
  and more, where replicated operand sums no longer pay) and stores
  every finished tile into all ranks' C over NVLink from the product kernel itself (one NVLS multicast
  store per 16 bytes where the switch offers it and the block is a dense product, else one ordinary
  store per peer; no NCCL collective in the timed path; ``--exchange nccl`` gathers with an NCCL
  all-gather instead).
  Total work is fixed: scaling "strong". After the timed region every rank recomputes row panels that
  other ranks own and compares them bit for bit with what arrived (``verify``); a mismatch ends the
  run with a non-zero exit code. Then a GPT-2-124M FSDP train step with every Linear through the
  library is timed (``fsdp_step``) and checked against an nn.Linear twin (``fsdp_twin_ok``).
* ``--impl reference``: the reference's own recursion restated for the CPU (``oracle/``) on the host
  cores; ``config`` states the product it really multiplies and ``stands_for`` the workload it samples.
* ``--only CASE``: runs one kernel of the pipeline a few times on synthetic data and exits (for
  profiling one kernel under ncu): gemm_grouped, cublas_grouped, dense, preadd, combine, fused. ``--quick`` keeps only
  the timed steps and the end-to-end leg of the N = 1 run (for a launch list under ncu).

Prints one JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import torch  # noqa: E402

METRIC = "effective TFLOP/s (2MNK/t) bf16 Strassen"
UNIT = "TFLOP/s"

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the product kernel on a
# one-kernel ncu capture of 14 products of 4096^3; a full launch of the N = 1 workload runs 49 such
# products and its traffic grows in proportion.
GEMM_DRAM_BYTES_14_PRODUCTS = 1.334e9 + 0.447e9
E2E_PANELS = 16  # row panels of A in the end-to-end leg (host-resident operands streamed over PCIe)

GEMM_DRAM_SOURCE = ("ncu one-kernel capture, 14 products of 4096^3 (1.334 GB read + 0.447 GB written), "
                    "scaled by 49/14 to the 49 products of a launch")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks, power and throttle reasons every 20 ms, with host timestamps."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.rows = []      # (host time, sm MHz, max MHz, watts, set of active reasons)

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                row = (time.time(), float(parts[1]), float(parts[2]), float(parts[3]),
                       {n for n, v in zip(self.NAMES, parts[5:9]) if v.lower().startswith("active")})
            except ValueError:
                continue
            self.rows.append(row)

    def window(self, t0, t1):
        """Summary of the samples taken between two host times."""
        rows = [r for r in self.rows if t0 <= r[0] <= t1]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(r[1] for r in rows)
        reasons = set()
        for r in rows:
            reasons |= r[4]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(r[2] for r in rows),
                "power_w_max": max(r[3] for r in rows), "samples": len(rows), "reasons": sorted(reasons)}

    def stop(self):
        if self.proc is None:
            return
        time.sleep(0.1)
        self.proc.terminate()


def seeded_inputs(n_rows_a, n, dist, seed, device, row_offset=0, want_b=True):
    """A (rows [row_offset, row_offset + n_rows_a) of the full M x K matrix) and B (K x N), bf16.
    Generated on the device from seeded generators: synthetic data with the configuration's
    distribution (the parity tests use CPU-generated inputs; throughput does not depend on bits).
    The rows of A depend only on (seed, row_offset, n_rows_a), so any rank can regenerate any block."""
    g = torch.Generator(device=device).manual_seed(seed + 7919 * row_offset)
    gb = torch.Generator(device=device).manual_seed(seed + 1)
    B = None
    if dist == "uniform":
        A = torch.rand((n_rows_a, n), generator=g, device=device) * 2 - 1
        if want_b:
            B = torch.rand((n, n), generator=gb, device=device) * 2 - 1
    else:
        A = torch.randn((n_rows_a, n), generator=g, device=device) / n ** 0.5
        if want_b:
            B = torch.randn((n, n), generator=gb, device=device) / n ** 0.5
    return A.bfloat16(), (B.bfloat16() if want_b else None)


# ------------------------------------------------------------------------------------------------
# CPU legs (oracle port of the reference recursion)
# ------------------------------------------------------------------------------------------------

def cpu_reference_step(n, depth, A=None, B=None):
    from oracle import strassen_oracle as so

    if A is None:
        g = torch.Generator("cpu").manual_seed(0)
        A = (2 * torch.rand((n, n), generator=g) - 1).bfloat16()
        B = (2 * torch.rand((n, n), generator=g) - 1).bfloat16()
    t0 = time.perf_counter()
    # fixed_strassen_fp32_agg.strassen_matmul_n_layers as shipped (inner level in fp32)
    so.n_layers(A, B, depth, torch.bfloat16, True, False)
    return time.perf_counter() - t0, A, B


def cpu_baseline(budget_s=25.0):
    """The reference recursion (oracle port) on the host cores, on a bounded sample."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = 2048
    t, A, B = cpu_reference_step(n, 2)
    while n < 8192 and t * 8 * 2 < budget_s:
        n *= 2
        t, A, B = cpu_reference_step(n, 2)
    t2, _, _ = cpu_reference_step(n, 2, A, B)
    t = min(t, t2)
    return {"value": round(2 * n ** 3 / t / 1e12, 4), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"one {n}^3 two-level bf16 product (fp32 aggregation as shipped), min of 2 runs, "
                      f"{t * 1e3:.0f} ms; oracle/strassen_oracle.py through torch CPU"}


def run_reference_arm(args):
    """The reference recursion on the host cores. `config` carries the product that is really
    multiplied; when that is smaller than the workload of the GPU arm, `stands_for` names the latter."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    full = 16384 if args.gpus == 1 else 32768
    probe, _, _ = cpu_reference_step(2048, 2)
    n = full
    # keep the whole run within a few minutes: the cost grows with n^3
    while n > 2048 and probe * (n / 2048) ** 3 * (args.steps + args.warmup) > 240:
        n //= 2
    g = torch.Generator("cpu").manual_seed(0)
    A = (2 * torch.rand((n, n), generator=g) - 1).bfloat16()
    B = (2 * torch.rand((n, n), generator=g) - 1).bfloat16()
    for _ in range(args.warmup):
        cpu_reference_step(n, 2, A, B)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(n, 2, A, B)
    dt = time.perf_counter() - t0
    value = 2 * n ** 3 * args.steps / dt / 1e12
    sample = (f"each step one {n}^3 two-level bf16 product of the reference recursion (oracle port) on {cores} "
              "host threads")
    config = {"workload": f"two-level Strassen C=A.B, M=N=K={n}, bf16 inputs U(-1,1) seed 0, the reference recursion "
                          "(fixed_strassen_fp32_agg.strassen_matmul_n_layers as shipped) through torch on the host cores",
              "M": n, "N": n, "K": n, "depth": 2, "algo": "classic"}
    if n != full:
        config["stands_for"] = workload_config(args.gpus)["workload"]
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": round(value, 4), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    if n_gpus == 1:
        return {"workload": "two-level Strassen C=A.B, M=N=K=16384, bf16 inputs U(-1,1) seed 0, fp32 accumulation "
                            "and aggregation, bf16 output (the headline configuration)",
                "M": 16384, "N": 16384, "K": 16384, "depth": 2, "algo": "classic",
                "l2": "inputs (1.6 GB) exceed L2 (126 MB); no flush between steps"}
    return {"workload": f"row-sharded product, M=N=K=32768, bf16 inputs N(0,1)/sqrt(K), A in {n_gpus} row "
                        "blocks, B replicated, every rank ends with the whole C (the multi-GPU configuration); "
                        "per-rank algorithm from the tuner table (dense at 4 ranks and more)",
            "M": 32768, "N": 32768, "K": 32768, "parallelism": f"rowshard{n_gpus}",
            "l2": "inputs exceed L2 (126 MB); no flush between steps"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------

def timed(fn, steps, sync, barrier):
    """Run fn() `steps` times between barrier+synchronize on both sides; CUDA-event time in ms."""
    barrier()
    sync()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    sync()
    barrier()
    return e0.elapsed_time(e1)


def one_turn(fn, seconds, sampler, chunk=20):
    """One turn of an arm: back-to-back calls for `seconds` from a rested GPU, an event every `chunk`
    calls. Returns the ms per call of the first chunk (burst), of the last second (sustained) and the
    SM clock sampled during the turn."""
    torch.cuda.synchronize()
    time.sleep(0.5)
    events = [torch.cuda.Event(enable_timing=True)]
    t0 = time.time()
    events[0].record()
    while True:
        for _ in range(chunk):
            fn()
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        events.append(e)
        if len(events) > 3:
            events[-3].synchronize()        # at most two chunks queued ahead
        if time.time() - t0 >= seconds:
            break
    torch.cuda.synchronize()
    t1 = time.time()
    per_chunk = [events[i].elapsed_time(events[i + 1]) / chunk for i in range(len(events) - 1)]
    tail, acc = [], 0.0
    for ms in reversed(per_chunk):
        tail.append(ms)
        acc += ms * chunk
        if acc >= 1000.0:
            break
    clk = sampler.window(t0 + 0.2, t1) if sampler else {"sm_mhz": None}
    return {"burst_ms": per_chunk[0], "sustained_ms": sum(tail) / len(tail), "calls": chunk * len(per_chunk),
            "sm_mhz": clk.get("sm_mhz"), "reasons": clk.get("reasons", [])}


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2] if len(xs) % 2 else 0.5 * (xs[len(xs) // 2 - 1] + xs[len(xs) // 2])


def interleaved(arms, rounds, seconds, sampler, flops):
    """A B A B ... turns; per arm the list of burst and sustained figures and their medians."""
    out = {name: {"burst_ms": [], "sustained_ms": [], "sm_mhz": []} for name in arms}
    for _ in range(rounds):
        for name, fn in arms.items():
            r = one_turn(fn, seconds, sampler)
            out[name]["burst_ms"].append(round(r["burst_ms"], 4))
            out[name]["sustained_ms"].append(round(r["sustained_ms"], 4))
            out[name]["sm_mhz"].append(r["sm_mhz"])
    for name, d in out.items():
        d["burst_ms_median"] = round(median(d["burst_ms"]), 4)
        d["sustained_ms_median"] = round(median(d["sustained_ms"]), 4)
        d["burst_tflops"] = round(flops / (d["burst_ms_median"] * 1e-3) / 1e12, 1)
        d["sustained_tflops"] = round(flops / (d["sustained_ms_median"] * 1e-3) / 1e12, 1)
        mhz = [m for m in d["sm_mhz"] if m]
        if mhz:
            # clock-normalised cost: milliseconds x MHz of the sustained second
            d["sustained_ms_x_mhz"] = round(d["sustained_ms_median"] * median(mhz), 1)
    return out


def run_only(args):
    """One kernel of the pipeline a few times on synthetic data (for one-kernel profiling)."""
    from strassen_triton_b200 import _lib, ops

    lib = _lib.load()
    what, n, nb = args.only, args.n, args.products
    stream = torch.cuda.current_stream().cuda_stream
    if what == "gemm_grouped":
        A = torch.randn(nb, n, n, device="cuda").bfloat16()
        B = torch.randn(nb, n, n, device="cuda").bfloat16()
        C = torch.empty_like(A)
        for _ in range(args.steps):
            ops.matmul_out(A, B, C, algo="dense")
    elif what == "cublas_grouped":     # the same batch through cuBLAS (torch.bmm), for a side-by-side capture
        A = torch.randn(nb, n, n, device="cuda").bfloat16()
        B = torch.randn(nb, n, n, device="cuda").bfloat16()
        C = torch.empty_like(A)
        for _ in range(args.steps):
            torch.bmm(A, B, out=C)
    elif what == "dense":
        A = torch.randn(n, n, device="cuda").bfloat16()
        B = torch.randn(n, n, device="cuda").bfloat16()
        C = torch.empty(n, n, device="cuda", dtype=torch.bfloat16)
        for _ in range(args.steps):
            ops.matmul_out(A, B, C, algo="dense")
    elif what in ("preadd", "combine"):
        A = (torch.rand(n, n, device="cuda") * 2 - 1).bfloat16()
        C = torch.empty(n, n, device="cuda", dtype=torch.bfloat16)
        p, _, _ = ops.make_problem(A, A, C, "classic", 2)
        blocks = torch.randn(49, n // 4, n // 4, device="cuda").bfloat16()
        for _ in range(args.steps):
            if what == "preadd":
                _lib.check(lib.b200s_preadd(ctypes.byref(p), 0, A.data_ptr(), blocks.data_ptr(), stream))
            else:
                _lib.check(lib.b200s_combine(ctypes.byref(p), blocks.data_ptr(), C.data_ptr(), stream))
    elif what == "fused":
        A = (torch.rand(n, n, device="cuda") * 2 - 1).bfloat16()
        B = (torch.rand(n, n, device="cuda") * 2 - 1).bfloat16()
        C = torch.empty(n, n, device="cuda", dtype=torch.bfloat16)
        for _ in range(args.steps):
            ops.matmul_out(A, B, C, algo="classic", depth=2, fuse=3)
    else:
        raise SystemExit(f"unknown --only case {what!r}")
    torch.cuda.synchronize()
    print(json.dumps({"only": what, "n": n, "products": nb, "steps": args.steps, "device_status": ops.device_status()}))


def verify_sharded(plan, B, n, world, rank, dev, dist):
    """Every rank recomputes row panels that OTHER ranks own (A's rows are regenerable from the seed,
    B is replicated) with the same per-panel product, and compares them bit for bit with the rows that
    arrived in its copy of C; one panel is also checked against fp64 through a probe vector."""
    from strassen_triton_b200.sharded import row_block

    C = plan.C
    owners = sorted({(rank + 1) % world, (rank + world // 2) % world} - {rank})
    rows_checked, exact = 0, True
    probe_err = 0.0
    layout = [None] * world       # every rank's first row, rows, row panels and algorithm
    dist.all_gather_object(layout, (plan.row_start, plan.rows, plan.panels, plan.algo, plan.depth))
    for owner in owners:
        r0, rows_o, panels_o, algo_o, depth_o = layout[owner]
        r1, prow = r0 + rows_o, rows_o // panels_o
        A_owner, _ = seeded_inputs(r1 - r0, n, "normal", 0, dev, row_offset=r0, want_b=False)
        for pi in sorted({0, panels_o - 1}):
            p0 = pi * prow
            want = plan.panel_product(A_owner[p0:p0 + prow], B, algo_o, depth_o)
            got = C[r0 + p0: r0 + p0 + prow]
            exact = exact and bool(torch.equal(got, want))
            rows_checked += prow
            if owner == owners[0] and pi == 0:
                # C x = A (B x) in fp64 on the first rows of this panel
                x = torch.randn(n, 1, device=dev, dtype=torch.float64)
                k = min(prow, 2048)
                ref = A_owner[p0:p0 + k].double() @ _b_times_x(B, x)
                probe_err = ((got[:k].double() @ x - ref).norm() / ref.norm()).item()
        del A_owner
    flag = torch.tensor([1 if exact else 0, rows_checked], device=dev, dtype=torch.int64)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    err = torch.tensor([probe_err], device=dev, dtype=torch.float64)
    dist.all_reduce(err, op=dist.ReduceOp.MAX)
    return {"rows_checked_per_rank": int(flag[1].item()), "panels_of_ranks": "rank+1 and rank+world/2",
            "bit_exact": bool(flag[0].item()), "rel_fro_probe": round(err.item(), 6),
            "how": "rows stored by other ranks into this rank's C against the same panel product recomputed here"}


def _b_times_x(B, x):
    """B @ x in fp64 without holding all of B in fp64: slabs of 4096 rows at a time."""
    out = torch.empty(B.shape[0], 1, device=B.device, dtype=torch.float64)
    for i in range(0, B.shape[0], 4096):
        out[i:i + 4096] = B[i:i + 4096].double() @ x
    return out


def fsdp_leg(world, rank, dev, dist):
    """GPT-2-124M FSDP train step with every Linear through the library, and a two-layer twin check
    against nn.Linear (same weights, same tokens, one forward/backward under FSDP)."""
    from strassen_triton_b200 import _lib, fsdp_gpt2

    lib = _lib.load()
    torch.manual_seed(0)
    model = fsdp_gpt2.build(layers=12, seq=1024, depth=None, device="cuda", world=world)
    fsdp_gpt2.train_steps(model, 2, batch=8, seq=1024, rank=rank)
    torch.cuda.synchronize()
    dist.barrier()
    n0 = lib.b200s_launch_count()
    t0 = time.perf_counter()
    steps = 3
    losses = fsdp_gpt2.train_steps(model, steps, batch=8, seq=1024, rank=rank)
    torch.cuda.synchronize()
    dist.barrier()
    dt = (time.perf_counter() - t0) / steps
    launches = (lib.b200s_launch_count() - n0) // steps
    del model
    torch.cuda.empty_cache()
    twin_ok, twin = fsdp_gpt2.twin_check(world, rank)
    t = torch.tensor([dt], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = torch.tensor([1 if twin_ok else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    return {"ms": round(t.item() * 1e3, 2), "tokens_per_s": round(world * 8 * 1024 / t.item()),
            "library_launches_per_step": int(launches), "loss0": round(losses[0], 4),
            "model": "GPT-2-124M (12 layers, d 768, 12 heads, vocab 50257 padded to 50304, seq 1024, 8 seqs/GPU), "
                     "FSDP bf16 mixed precision, AdamW, random tokens", "twin": twin}, bool(ok.item())


def run_gpu_arm(args):
    import torch.distributed as dist

    from strassen_triton_b200 import _lib, ops
    from strassen_triton_b200.sharded import row_block, sharded_matmul
    import fixed_strassen_fp32_agg as api  # the reference-named public entry

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    sync = lambda: torch.cuda.synchronize(dev)  # noqa: E731
    lib = _lib.load()
    peaks = measured_peaks()
    depth = 2
    warmup = max(args.warmup, 3)
    plan = None

    if world == 1:
        n = 16384
        A, B = seeded_inputs(n, n, "uniform", 0, dev)
        C = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
        p, _, _ = ops.make_problem(A, B, C, "classic", depth)
        ws = torch.empty(ops.workspace_bytes(p), dtype=torch.uint8, device=dev)
        fuse = {"auto": 0, "fused_all": 1, "separate": 2, "fused": 3}[args.schedule]
        pipe = 2 if fuse == 2 else 0
        step = lambda: ops.matmul_out(A, B, C, algo="classic", depth=depth, fuse=fuse, pipeline=pipe,  # noqa: E731
                                      workspace=ws)
    else:
        n = 32768
        balance = None
        r0, r1 = row_block(n, world, rank)
        A, B = seeded_inputs(r1 - r0, n, "normal", 0, dev, row_offset=r0)
        if args.exchange.startswith("peer"):
            from strassen_triton_b200.sharded import PeerShardedMatmul, balanced_row_counts

            def make_plan(row_counts=None):
                return PeerShardedMatmul(n, n, n, torch.bfloat16, algo=args.algo, depth=-1 if args.algo == "auto" else depth,
                                         panels=args.panels, device=dev,
                                         exchange={"peer": "auto", "peer_store": "store", "peer_multicast": "multicast",
                                                   "peer_push": "push", "peer_copy": "copy", "peer_overlap": "overlap",
                                                   "peer_senders": "senders"}[args.exchange],
                                         push_sms=args.push_sms, row_counts=row_counts)

            plan = make_plan()
            C = plan.C
            step = lambda: plan(A, B)  # noqa: E731
            if args.balance:
                # The GPUs of a box differ in sustained speed under the power cap and the step ends with the
                # slowest: time every rank's own kernels on equal blocks, then hand out rows by speed.
                for _ in range(2):
                    step()
                torch.cuda.synchronize()
                with ops.stage_timing(16) as own:
                    for _ in range(3):
                        step()
                    torch.cuda.synchronize()
                own_ms = sum(own[k] for k in ops.STAGES) * max(own["calls"], 1) / 3.0
                mine = torch.tensor([own_ms], device=dev, dtype=torch.float64)
                everyone = [torch.zeros_like(mine) for _ in range(world)]
                dist.all_gather(everyone, mine)
                times_ms = [t.item() for t in everyone]
                counts = balanced_row_counts(n, times_ms, plan.row_counts)
                balance = {"own_kernel_ms_on_equal_blocks": [round(t, 3) for t in times_ms], "rows": counts}
                if counts != plan.row_counts:
                    del plan
                    plan = make_plan(counts)
                    C = plan.C
                    r0, r1 = plan.row_start, plan.row_start + plan.rows
                    A, _ = seeded_inputs(r1 - r0, n, "normal", 0, dev, row_offset=r0, want_b=False)
        else:
            C = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
            p, _, _ = ops.make_problem(A, B, C[r0:r1], args.algo, -1 if args.algo == "auto" else depth)
            ws = torch.empty(max(ops.workspace_bytes(p), 1), dtype=torch.uint8, device=dev)
            step = lambda: sharded_matmul(A, B, n, panels=args.panels, out=C, algo=args.algo,  # noqa: E731
                                          depth=-1 if args.algo == "auto" else depth, workspace=ws)
    flops = 2.0 * n ** 3

    for _ in range(warmup):
        step()
    sampler = ClockSampler(local).start() if rank == 0 else None
    launches0 = lib.b200s_launch_count()
    t_region0 = time.time()
    with ops.stage_timing(min(args.steps, 256)) as stages:
        ms = timed(step, args.steps, sync, barrier)
    t_region1 = time.time()
    launches = lib.b200s_launch_count() - launches0
    clocks = sampler.window(t_region0, t_region1) if sampler else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    status = ops.device_status(dev)
    if status != (0, 0):
        raise SystemExit(f"device status {status}: a kernel gave up on a bounded wait")
    value = flops * args.steps / (ms * 1e-3) / 1e12

    verify = None
    if plan is not None:
        verify = verify_sharded(plan, B, n, world, rank, dev, dist)
        if not verify["bit_exact"] or verify["rel_fro_probe"] > 2e-2:
            if rank == 0:
                print(json.dumps({"error": "the row-sharded product failed its verification", "verify": verify}), flush=True)
            dist.barrier()
            dist.destroy_process_group()
            raise SystemExit(3)

    # ---- end to end through the public API with host buffers ----
    hA = torch.empty(A.shape, dtype=A.dtype, pin_memory=True)
    hB = torch.empty(B.shape, dtype=B.dtype, pin_memory=True)
    hA.copy_(A)
    hB.copy_(B)
    e2e_sequential = None
    if world == 1:
        from strassen_triton_b200.host import HostStreamedMatmul

        hC = torch.empty((n, n), dtype=torch.bfloat16, pin_memory=True)

        def sequential_step():      # copy A, copy B, multiply, copy C, one after the other
            dA = hA.to(dev, non_blocking=True)
            dB = hB.to(dev, non_blocking=True)
            out = api.strassen_matmul_n_layers(dA, dB, depth, torch.bfloat16)
            hC.copy_(out, non_blocking=True)

        sequential_step()
        e2e_sequential = flops * 3 / (timed(sequential_step, 3, sync, barrier) * 1e-3) / 1e12
        streamed = HostStreamedMatmul(n, n, n, torch.bfloat16, algo="classic", depth=depth, panels=E2E_PANELS)

        def e2e_step():             # B, then A in row panels; products and C's way back overlap the arrivals
            streamed(hA, hB, hC)
    else:
        hC = torch.empty((r1 - r0, n), dtype=torch.bfloat16, pin_memory=True)    # r0, r1: this rank's rows

        def e2e_step():
            dA = hA.to(dev, non_blocking=True)
            dB = hB.to(dev, non_blocking=True)
            out = plan(dA, dB) if plan is not None else step_nccl(dA, dB)
            hC.copy_(out[r0:r1], non_blocking=True)

        def step_nccl(dA, dB):
            return sharded_matmul(dA, dB, n, panels=args.panels, out=C, algo=args.algo,
                                  depth=-1 if args.algo == "auto" else depth, workspace=ws)

    e2e_steps = max(1, min(args.steps, 5))
    e2e_step()
    ms_e2e = timed(e2e_step, e2e_steps, sync, barrier)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = t.item()
    e2e_value = flops * e2e_steps / (ms_e2e * 1e-3) / 1e12
    h2d = (hA.numel() + hB.numel()) * 2
    d2h = hC.numel() * 2
    del hA, hB, hC

    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world), "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "api": "strassen_triton_b200.host.HostStreamedMatmul" if world == 1
                    else ("strassen_triton_b200.sharded.PeerShardedMatmul" if plan is not None
                          else "strassen_triton_b200.sharded.sharded_matmul")},
            "gpu_launches": int(launches),
        }
        if e2e_sequential is not None:
            line["e2e"]["how"] = (f"pinned host operands streamed over PCIe: B, then A in {E2E_PANELS} row panels; each panel "
                                  "is multiplied (two levels, B's operand blocks reused) as it arrives and its rows of C go "
                                  "back while the next panel is multiplied")
            line["e2e"]["sequential_value"] = round(e2e_sequential, 2)
            line["e2e"]["sequential_api"] = ("fixed_strassen_fp32_agg.strassen_matmul_n_layers between plain copies "
                                             "(copy A, copy B, multiply, copy C, one after the other)")
    stage_names = ("operand_blocks_A", "operand_blocks_B", "products", "recombination")

    if world > 1:
        # per-rank stage times of rank 0's own block (library events during the timed steps); what is
        # left of a step is the two device-side barriers and launch gaps
        st = {k: round(stages[k], 4) for k in stage_names}
        if rank == 0:
            per_step = ms / args.steps
            line["config"]["exchange"] = (f"{plan.exchange}: stores from the product kernel into every rank's C (no "
                                          "collective in the timed path)" if plan is not None and plan.exchange in
                                          ("store", "multicast") else
                                          f"overlap: row panel i is sent by a kernel on {plan.push_sms} SMs while panel i+1 is "
                                          "multiplied on the others (no collective in the timed path)"
                                          if plan is not None and plan.exchange == "overlap" else args.exchange)
            if plan is not None and plan.sender_sms:
                line["config"]["exchange"] = (f"{plan.exchange} stores by {plan.sender_sms} sending CTAs of the product kernel, "
                                              "block of columns by block of columns as C gets finished (no collective in the "
                                              "timed path)")
            line["config"]["panels"] = plan.panels if plan is not None else args.panels
            if balance is not None:
                line["config"]["row_blocks"] = {"rows_per_rank": balance["rows"],
                                                "own_kernel_ms_on_equal_blocks": balance["own_kernel_ms_on_equal_blocks"],
                                                "how": "after 5 steps on equal blocks every rank's block is sized by the speed "
                                                       "its GPU showed, in units of 256 rows (the GPUs of a box differ under "
                                                       "the power cap, and a strong-scaling step ends with the slowest)"}
            if plan is not None:
                line["config"]["per_rank"] = {"algo": plan.algo, "depth": plan.depth,
                                              "shape": [plan.prow, n, n], "from": ("flag" if args.algo != "auto" else
                                                       "plan rule: dense at 4 ranks and more" if world >= 4 else "tuner table")}
            calls = max(stages["calls"], 1) / args.steps     # panels per step
            line["stages_ms"] = {"B_operand_blocks": round(st["operand_blocks_B"] * calls, 4),
                                 "A_operand_blocks": round(st["operand_blocks_A"] * calls, 4),
                                 "products": round(st["products"] * calls, 4),
                                 "recombination_and_exchange": round(st["recombination"] * calls, 4)}
            line["stages_ms"]["barriers_and_gaps"] = round(per_step - sum(line["stages_ms"].values()), 4)
            line["stages_ms"]["note"] = ("rank 0; a dense block has one stage, the product kernel, whose epilogue also "
                                         "performs the exchange")
            line["verify"] = verify
        if args.fsdp:
            fs, twin_ok = fsdp_leg(world, rank, dev, dist)
            if rank == 0:
                line["fsdp_step"] = fs
                line["fsdp_twin_ok"] = twin_ok
    elif args.quick:
        line["stages_ms"] = {k: round(stages[k], 4) for k in stage_names}
        line["note"] = "--quick: timed steps and end-to-end only (the short run behind the ncu launch list)"
    else:
        # ---- comparison with cuBLAS dense on the same GPU, interleaved ----
        dense = lambda: torch.mm(A, B, out=C)  # noqa: E731
        for _ in range(warmup):
            dense()
        prob = ops.make_problem(A, B, C, "classic", depth)[0]
        fuse_used = resolved_schedule(lib, prob, fuse)
        sep = lambda: ops.matmul_out(A, B, C, algo="classic", depth=depth, fuse=2, pipeline=2, workspace=ws)  # noqa: E731
        fus = lambda: ops.matmul_out(A, B, C, algo="classic", depth=depth, fuse=3, workspace=ws)  # noqa: E731
        inter = interleaved({"strassen_separate": sep, "strassen_fused": fus, "cublas_dense": dense}, args.rounds,
                            args.seconds, sampler, flops)
        mine = "strassen_fused" if "fused" in fuse_used else "strassen_separate"
        st, cu = inter[mine], inter["cublas_dense"]
        line["interleaved"] = {
            "protocol": f"{args.rounds} rounds of strassen_separate, strassen_fused, cublas_dense turns; a turn = 0.5 s rest, "
                        f"then back-to-back calls for {args.seconds} s; burst = first 20 calls, sustained = last second; "
                        "the SM clock is the median of the samples taken during the turn",
            "library_default": mine, **inter,
            "ratio_burst": round(cu["burst_ms_median"] / st["burst_ms_median"], 4),
            "ratio_sustained": round(cu["sustained_ms_median"] / st["sustained_ms_median"], 4),
            "ratios_by_schedule": {k: {"burst": round(cu["burst_ms_median"] / inter[k]["burst_ms_median"], 4),
                                       "sustained": round(cu["sustained_ms_median"] / inter[k]["sustained_ms_median"], 4)}
                                   for k in ("strassen_separate", "strassen_fused")}}
        line["cublas_dense"] = {"value": cu["burst_tflops"], "sustained_value": cu["sustained_tflops"], "unit": UNIT,
                                "ms_per_step": cu["burst_ms_median"],
                                "protocol": "median over the interleaved turns (see `interleaved`)"}

        # ---- the reference recursion on this GPU (oracle port on CUDA tensors, cuBLAS sub-products) ----
        from oracle import strassen_oracle as so

        ref_step = lambda: so.n_layers(A, B, depth, torch.bfloat16, True, False)  # noqa: E731
        for _ in range(2):
            ref_step()
        ms_ref = timed(ref_step, 5, sync, barrier) / 5
        line["reference_gpu"] = {"value": round(flops / (ms_ref * 1e-3) / 1e12, 2), "unit": UNIT,
                                 "ms_per_step": round(ms_ref, 3),
                                 "what": "the reference's torch recursion (fixed_strassen_fp32_agg.strassen_matmul_n_layers "
                                         "as shipped, restated in oracle/) on CUDA tensors: cuBLAS sub-products and "
                                         "eager elementwise passes, 5 steps"}
        del ref_step
        torch.cuda.empty_cache()

        # ---- roofline of the dominant kernel, from the stage events of the timed steps ----
        executed = (7.0 / 8.0) ** depth * flops
        t_prod = stages["products"] * 1e-3
        achieved = executed / t_prod / 1e12
        region_s = ms * 1e-3
        burst_region = region_s < 1.0
        peak = peaks["bf16_burst"] if burst_region else peaks["bf16_sustained"]
        line["config"]["schedule"] = fuse_used
        line["roofline"] = {
            "kernel": "gemm_kernel (grouped tcgen05 GEMM over the 49 sub-products of 4096^3"
                      + ("; fused form: its adder warps also form operand blocks and recombine C" if "fused" in fuse_used else "") + ")",
            "bound": "tensor", "achieved": round(achieved, 1), "peak": peak, "unit": UNIT,
            "frac": round(achieved / peak, 4),
            "peak_kind": f"cuBLAS bf16 {'burst' if burst_region else 'sustained'} rate, of {peaks['source']} "
                         f"(timed region {region_s:.2f} s)",
            "traffic": round(GEMM_DRAM_BYTES_14_PRODUCTS * 49 / 14), "traffic_source": GEMM_DRAM_SOURCE,
            "algorithmic_flops_per_launch": executed, "duration_ms": round(stages["products"], 4),
            "duration_source": f"library stage events over the {stages['calls']} timed steps"}
        hbm = peaks["hbm_gbs"]
        blk = (n // 4) ** 2 * 2
        line["stages_ms"] = {k: round(stages[k], 4) for k in stage_names}
        line["stages_ms"]["sum"] = round(sum(stages[k] for k in stage_names), 4)
        if "fused" not in fuse_used:
            pre_bytes = n * n * 2 + 49 * blk
            comb_bytes = 49 * blk + n * n * 2
            line["add_passes"] = {
                "preadd_A_gbs": round(pre_bytes / (stages["operand_blocks_A"] * 1e-3) / 1e9, 1),
                "preadd_B_gbs": round(pre_bytes / (stages["operand_blocks_B"] * 1e-3) / 1e9, 1),
                "combine_gbs": round(comb_bytes / (stages["recombination"] * 1e-3) / 1e9, 1),
                "hbm_peak_gbs": hbm, "peak_kind": f"copy bandwidth, of {peaks['source']}"}

        # ---- one GPU on the multi-GPU workload: the basis of T(1) / (P T(P)) ----
        del A, B, C, ws
        torch.cuda.empty_cache()
        n2 = 32768
        A2, B2 = seeded_inputs(n2, n2, "normal", 0, dev)
        C2 = torch.empty((n2, n2), dtype=torch.bfloat16, device=dev)
        p2, _, _ = ops.make_problem(A2, B2, C2, "auto", -1)
        ws2 = torch.empty(max(ops.workspace_bytes(p2), 1), dtype=torch.uint8, device=dev)
        big = lambda: ops.matmul_out(A2, B2, C2, algo="auto", depth=-1, workspace=ws2)  # noqa: E731
        for _ in range(3):
            big()
        line["t1_32768_ms"] = round(timed(big, 5, sync, barrier) / 5, 3)
        a32, d32 = ops.resolve(p2)
        line["t1_32768_algo"] = {"algo": {1: "dense", 2: "classic", 3: "winograd"}[a32], "depth": d32}
        del A2, B2, C2, ws2
        torch.cuda.empty_cache()
        line["cpu_baseline"] = cpu_baseline()
    if sampler:
        sampler.stop()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def resolved_schedule(lib, prob, fuse=0):
    """Name of the schedule the library runs for this problem (fuse 0: the one it picks itself)."""
    a, d, f = ctypes.c_int32(0), ctypes.c_int32(0), ctypes.c_int32(0)
    lib.b200s_tuner_lookup_schedule(prob.M, prob.N, prob.K, prob.in_dtype, ctypes.byref(a), ctypes.byref(d), ctypes.byref(f))
    if fuse == 0:
        fuse = f.value if f.value else 2
    return {1: "fused (one persistent kernel)", 2: "separate passes (pre-add A, pre-add B, grouped GEMM, recombination)",
            3: "fused kernel, last quadrant of C recombined by a full-width launch after it"}[fuse]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rounds", type=int, default=5, help="N = 1: rounds of the interleaved comparison with cuBLAS")
    ap.add_argument("--seconds", type=float, default=2.0, help="N = 1: length of one turn of an arm")
    ap.add_argument("--schedule", default="auto", choices=["auto", "separate", "fused", "fused_all"],
                    help="N = 1: schedule of the Strassen passes ('auto' = the library's tuner table)")
    ap.add_argument("--panels", type=int, default=1, help="row panels per rank (N > 1)")
    ap.add_argument("--algo", default="auto", choices=["auto", "dense", "classic", "winograd"],
                    help="N > 1: per-rank algorithm ('auto' = the library's tuner table; dense at 4 ranks and more)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "peer_store", "peer_multicast", "peer_senders", "peer_overlap", "peer_push", "peer_copy", "nccl"],
                    help="N > 1: 'peer' = the product kernel stores into every rank's C over NVLink (NVLS multicast "
                         "stores for dense blocks where available, plain peer stores otherwise); 'nccl' = all-gather of "
                         "the row blocks")
    ap.add_argument("--push-sms", type=int, default=8, help="N > 1, --exchange peer_overlap: SMs left to the kernel that sends "
                                                            "a finished row panel while the next one is multiplied")
    ap.add_argument("--balance", type=int, default=0, help="N > 1, peer exchanges: 1 = after a few steps on equal row blocks, "
                                                            "size every rank's block by the speed its GPU showed (0 = equal blocks; "
                                                            "measured: the GPUs' order changes from run to run and nothing is gained)")
    ap.add_argument("--fsdp", type=int, default=1, help="N > 1: also time the FSDP GPT-2 step (0 = skip)")
    ap.add_argument("--quick", action="store_true", help="N = 1: skip the comparison arms (for a launch list under ncu)")
    ap.add_argument("--only", default=None, help="run one kernel a few times and exit: gemm_grouped, cublas_grouped, "
                                                 "dense, preadd, combine, fused")
    ap.add_argument("--n", type=int, default=4096, help="--only: matrix extent")
    ap.add_argument("--products", type=int, default=14, help="--only gemm_grouped: products in the batch")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU path exists for the b200 arm)")
    if args.only:
        run_only(args)
        return
    run_gpu_arm(args)


if __name__ == "__main__":
    main()

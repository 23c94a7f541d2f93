#!/usr/bin/env python
"""Benchmark of the Strassen matmul path: effective TFLOP/s (2*M*N*K / t), bf16.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one full product C = A @ B through the library's public entry
(``fixed_strassen_fp32_agg.strassen_matmul_n_layers`` semantics: two Strassen levels, bf16
operands, fp32 accumulation and aggregation, bf16 result).

* N = 1: M = N = K = 16384, inputs U(-1,1) from seed 0 (the configuration the headline metric is
  quoted on). Inputs are resident in HBM for ``value``; ``e2e`` times the same call with pinned host
  buffers, the host->device copies of A and B and the device->host copy of C inside the timed region.
* N > 1 (launched by torch.distributed.run, one rank per GPU): M = N = K = 32768, A split into
  row blocks, B replicated, all-gather of C (NCCL). Total work is fixed: scaling "strong".
* ``--impl reference``: the reference's own recursion restated for the CPU (``oracle/``), on the host
  cores, each step a bounded sample (an 8192^3 two-level product) of the same workload.

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

# DRAM bytes (read + write) of one launch of the grouped GEMM kernel on the N=1 workload, from
# the ncu launch list summarised in profiles/bench_16384_depth2_launch_list.md.
GEMM_DRAM_TRAFFIC_BYTES = 9.58e9


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 50 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, smax, power, reasons = [], [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(smax), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def seeded_inputs(n_rows_a, n, dist, seed, device, row_offset=0, total_rows=None):
    """A (rows [row_offset, row_offset + n_rows_a) of the full M x K matrix) and B (K x N), bf16.
    Generated on the device from seeded generators: synthetic data with the configuration's
    distribution (the parity tests use CPU-generated inputs; throughput does not depend on bits)."""
    g = torch.Generator(device=device).manual_seed(seed + 7919 * row_offset)
    gb = torch.Generator(device=device).manual_seed(seed + 1)
    if dist == "uniform":
        A = torch.rand((n_rows_a, n), generator=g, device=device) * 2 - 1
        B = torch.rand((n, n), generator=gb, device=device) * 2 - 1
    else:
        A = torch.randn((n_rows_a, n), generator=g, device=device) / n ** 0.5
        B = torch.randn((n, n), generator=gb, device=device) / n ** 0.5
    return A.bfloat16(), B.bfloat16()


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
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = 8192
    probe, A, B = cpu_reference_step(2048, 2)
    # keep the whole run within a few minutes on slow hosts
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
    sample = f"each step one {n}^3 two-level bf16 product of the reference recursion (oracle port) on {cores} host threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
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
    return {"workload": f"row-sharded two-level Strassen, M=N=K=32768, bf16 inputs N(0,1)/sqrt(K), A in {n_gpus} row "
                        "blocks, B replicated, every rank ends with the whole C (the multi-GPU configuration)",
            "M": 32768, "N": 32768, "K": 32768, "depth": 2, "algo": "classic", "parallelism": f"rowshard{n_gpus}",
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


def stage_breakdown(ops, _lib, A, B, C, depth, steps):
    """Average duration of each kernel of the pipeline, driven through the stand-alone C-ABI
    passes with CUDA events between them on the launching stream."""
    lib = _lib.load()
    p, A2, B2 = ops.make_problem(A, B, C, "classic", depth)
    need = ops.workspace_bytes(p)
    ws = torch.empty(need, dtype=torch.uint8, device=A.device)
    M, N, K = p.M, p.N, p.K
    div, np_ = 1 << depth, 7 ** depth
    Mb, Nb, Kb = M // div, N // div, K // div
    sa = ws[: np_ * Mb * Kb * 2].view(torch.bfloat16).view(np_, Mb, Kb)
    off = (np_ * Mb * Kb * 2 + 255) // 256 * 256
    sb = ws[off: off + np_ * Kb * Nb * 2].view(torch.bfloat16).view(np_, Kb, Nb)
    off2 = off + (np_ * Kb * Nb * 2 + 255) // 256 * 256
    mp = ws[off2: off2 + np_ * Mb * Nb * 2].view(torch.bfloat16).view(np_, Mb, Nb)
    stream = torch.cuda.current_stream().cuda_stream
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(steps)]
    for s in range(steps):
        ev[s][0].record()
        _lib.check(lib.b200s_preadd(ctypes.byref(p), 0, A2.data_ptr(), sa.data_ptr(), stream))
        ev[s][1].record()
        _lib.check(lib.b200s_preadd(ctypes.byref(p), 1, B2.data_ptr(), sb.data_ptr(), stream))
        ev[s][2].record()
        ops.matmul_out(sa, sb, mp, algo="dense")
        ev[s][3].record()
        _lib.check(lib.b200s_combine(ctypes.byref(p), mp.data_ptr(), C.data_ptr(), stream))
        ev[s][4].record()
    torch.cuda.synchronize()
    names = ["preadd_A", "preadd_B", "gemm_grouped", "combine"]
    return {n: sum(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(steps)) / steps for i, n in enumerate(names)}


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

    if world == 1:
        n = 16384
        A, B = seeded_inputs(n, n, "uniform", 0, dev)
        C = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
        p, _, _ = ops.make_problem(A, B, C, "classic", depth)
        ws = torch.empty(ops.workspace_bytes(p), dtype=torch.uint8, device=dev)
        step = lambda: ops.matmul_out(A, B, C, algo="classic", depth=depth, workspace=ws)  # noqa: E731
        flops = 2.0 * n ** 3
    else:
        n = 32768
        r0, r1 = row_block(n, world, rank)
        A, B = seeded_inputs(r1 - r0, n, "normal", 0, dev, row_offset=r0)
        C = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
        p, _, _ = ops.make_problem(A, B, C[r0:r1], "classic", depth)
        ws = torch.empty(ops.workspace_bytes(p), dtype=torch.uint8, device=dev)
        if args.exchange.startswith("peer"):
            from strassen_triton_b200.sharded import PeerShardedMatmul

            del C, ws
            plan = PeerShardedMatmul(n, n, n, torch.bfloat16, algo="classic", depth=depth, panels=args.panels,
                                     device=dev, exchange={"peer": "store", "peer_push": "push", "peer_copy": "copy"}[args.exchange])
            C = plan.C
            step = lambda: plan(A, B)  # noqa: E731
        else:
            step = lambda: sharded_matmul(A, B, n, panels=args.panels, out=C, algo="classic", depth=depth,  # noqa: E731
                                          workspace=ws)
        flops = 2.0 * n ** 3

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = lib.b200s_launch_count()
    ms = timed(step, args.steps, sync, barrier)
    launches = lib.b200s_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    status = ops.device_status(dev)
    if status != (0, 0):
        raise SystemExit(f"device status {status}: a kernel gave up on a bounded wait")
    value = flops * args.steps / (ms * 1e-3) / 1e12

    # ---- end to end through the reference-named API with host buffers ----
    hA = torch.empty(A.shape, dtype=A.dtype, pin_memory=True)
    hB = torch.empty(B.shape, dtype=B.dtype, pin_memory=True)
    hA.copy_(A)
    hB.copy_(B)
    if world == 1:
        hC = torch.empty((n, n), dtype=torch.bfloat16, pin_memory=True)

        def e2e_step():
            dA = hA.to(dev, non_blocking=True)
            dB = hB.to(dev, non_blocking=True)
            out = api.strassen_matmul_n_layers(dA, dB, depth, torch.bfloat16)
            hC.copy_(out, non_blocking=True)
    else:
        r0, r1 = row_block(n, world, rank)
        hC = torch.empty((r1 - r0, n), dtype=torch.bfloat16, pin_memory=True)

        def e2e_step():
            dA = hA.to(dev, non_blocking=True)
            dB = hB.to(dev, non_blocking=True)
            if args.exchange.startswith("peer"):
                out = plan(dA, dB)
            else:
                out = sharded_matmul(dA, dB, n, panels=args.panels, out=C, algo="classic", depth=depth, workspace=ws)
            hC.copy_(out[r0:r1], non_blocking=True)

    e2e_steps = max(1, min(args.steps, 5))
    e2e_step()
    ms_e2e = timed(e2e_step, e2e_steps, sync, barrier)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = t.item()
    e2e_value = flops * e2e_steps / (ms_e2e * 1e-3) / 1e12
    ms_dense = None
    if world == 1:
        # cuBLAS dense bf16 on the same GPU and inputs, same timing protocol as `value`
        dense = lambda: torch.mm(A, B, out=C)  # noqa: E731
        for _ in range(max(args.warmup, 3)):
            dense()
        ms_dense = timed(dense, args.steps, sync, barrier) / args.steps
    h2d = (hA.numel() + hB.numel()) * 2
    d2h = hC.numel() * 2

    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world), "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "api": "fixed_strassen_fp32_agg.strassen_matmul_n_layers" if world == 1
                    else ("strassen_triton_b200.sharded.PeerShardedMatmul" if args.exchange != "nccl"
                          else "strassen_triton_b200.sharded.sharded_matmul")},
            "gpu_launches": int(launches),
        }
        if world > 1:
            line["config"]["exchange"] = args.exchange
            line["config"]["panels"] = args.panels
        if world == 1:
            # per-kernel durations and the roofline of the dominant kernel (the grouped GEMM)
            stages = stage_breakdown(ops, _lib, A, B, C, depth, args.steps)
            t_gemm = stages["gemm_grouped"] * 1e-3
            executed = (7.0 / 8.0) ** depth * flops
            achieved = executed / t_gemm / 1e12
            peak = peaks["bf16_sustained"]
            line["roofline"] = {
                "kernel": "gemm_kernel (grouped tcgen05 GEMM, 49 sub-products of 4096^3)", "bound": "tensor",
                "achieved": round(achieved, 1), "peak": peak, "unit": UNIT, "frac": round(achieved / peak, 4),
                "peak_kind": f"cuBLAS bf16 sustained, of {peaks['source']} (burst {peaks['bf16_burst']})",
                "traffic": GEMM_DRAM_TRAFFIC_BYTES, "algorithmic_flops_per_launch": executed,
                "duration_ms": round(stages["gemm_grouped"], 4)}
            hbm = peaks["hbm_gbs"]
            es = 2
            blk = (n // 4) ** 2 * es
            pre_bytes = n * n * es + 49 * blk
            comb_bytes = 49 * blk + n * n * es
            line["stages_ms"] = {k: round(v, 4) for k, v in stages.items()}
            line["add_passes"] = {
                "preadd_A_gbs": round(pre_bytes / (stages["preadd_A"] * 1e-3) / 1e9, 1),
                "preadd_B_gbs": round(pre_bytes / (stages["preadd_B"] * 1e-3) / 1e9, 1),
                "combine_gbs": round(comb_bytes / (stages["combine"] * 1e-3) / 1e9, 1),
                "hbm_peak_gbs": hbm, "peak_kind": f"copy bandwidth, of {peaks['source']}"}
            line["cublas_dense"] = {"value": round(flops / (ms_dense * 1e-3) / 1e12, 2), "unit": UNIT,
                                    "ms_per_step": round(ms_dense, 4),
                                    "protocol": "same steps and warm-up as `value`, started after the PCIe-bound "
                                                "end-to-end phase so that both start on an equally rested GPU"}
            line["cpu_baseline"] = cpu_baseline()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--panels", type=int, default=1, help="row panels per rank for exchange/compute overlap (N > 1)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "peer_push", "peer_copy", "nccl"],
                    help="N > 1: 'peer' = recombination kernel stores into every rank's C over NVLink; "
                         "'nccl' = all-gather of the row blocks")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU path exists for the b200 arm)")
    run_gpu_arm(args)


if __name__ == "__main__":
    main()

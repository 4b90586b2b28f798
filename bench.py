#!/usr/bin/env python
"""Benchmark of the two hot paths on B200.

``python bench.py --gpus N --steps K --warmup W`` times the bf16 GEMM
16384 x 16384 x 16384 (entries N(0,1)/sqrt(K), seed 1; under torchrun B is split
by N-column blocks across the ranks, no collective) and prints ONE JSON line.
A step is one launch of the GEMM over the rank's shard. The same line carries
cuBLASLt on the same operands, flash-attention forward (non-causal,
B=16 H=16 S=4096 D=128, seed 3; planes split across ranks), the end-to-end
figure through the host-buffer C-ABI call, the tensor-core roofline of the
GEMM kernel, and the CPU baseline (the oracle port on the host cores).

``--impl reference`` times the reference's CPU path (the oracle port of its
CPU GEMM reference) on the host cores, on a bounded slab per step.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N = K = 16384
GEMM_SEED = 1
FLASH = dict(batch=16, heads=16, seq=4096, head_dim=128, seed=3, causal=False)
FLASH_CAUSAL = dict(batch=4, heads=32, seq=16384, head_dim=128, seed=4, causal=True)
WORKLOAD = "gemm_bf16_16384x16384x16384_normal_over_sqrtK_seed1"
METRIC = "bf16_gemm_tflops_16384"
#: 4 Mi rows x 128 bf16 = 1 GiB in and 1 GiB out per launch, far larger than the L2.
ROW_KERNEL_ROWS = 4 * 1024 * 1024
ROW_KERNEL_SEED = 5


def env_int(name: str, default: int) -> int:
    return int(os.environ.get(name, default))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            data = json.load(handle)
        return dict(burst=float(data["bf16_tflops"]), sustained=float(data["bf16_tflops_sustained"]),
                    hbm=float(data["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.process = None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
        return self

    def __exit__(self, *exc):
        self.samples = []
        if self.process is None:
            return
        self.process.terminate()
        try:
            out, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            out, _ = self.process.communicate()
        for line in out.splitlines():
            fields = [f.strip() for f in line.split(",")]
            if len(fields) >= 9:
                self.samples.append(fields)

    def summary(self):
        clocks, reasons, sm_max, power = [], set(), None, []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for fields in getattr(self, "samples", []):
            try:
                clocks.append(float(fields[1]))
                sm_max = float(fields[2])
                power.append(float(fields[3]))
            except ValueError:
                continue
            for name, value in zip(names, fields[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c, p in zip(clocks, power) if p > 300.0] or clocks
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": sm_max,
                "reasons": sorted(reasons), "samples": len(clocks),
                "power_w_max": max(power) if power else None}


# ------------------------------------------------------------------ reference arm / CPU baseline

def cpu_gemm_rate(a_words, b_words, rows: int):
    """Time the oracle's GEMM over `rows` rows of C (full N, full K); returns (TFLOP/s, seconds)."""
    import oracle

    start = time.perf_counter()
    oracle.gemm_rows(a_words, b_words, 0, rows)
    elapsed = time.perf_counter() - start
    return 2.0 * rows * b_words.shape[0] * b_words.shape[1] / elapsed / 1e12, elapsed


def host_operands(rows: int):
    """Seeded N(0,1)/sqrt(K) bf16 operands on the host: `rows` rows of A and all of B, as bf16 words."""
    import numpy as np
    import torch

    generator = torch.Generator(device="cpu").manual_seed(GEMM_SEED)
    a = (torch.randn((rows, K), generator=generator) / math.sqrt(K)).to(torch.bfloat16)
    b = (torch.randn((N, K), generator=generator) / math.sqrt(K)).to(torch.bfloat16)
    words = lambda t: t.view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    return words(a), words(b)


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    import oracle

    oracle.use_all_cores()
    a_words, b_words = host_operands(256)
    probe_rate, _ = cpu_gemm_rate(a_words, b_words, 8)
    budget = 120.0 / max(1, args.steps + args.warmup)
    rows = int(max(1, min(256, probe_rate * 1e12 * budget / (2.0 * N * K))))
    for _ in range(args.warmup):
        cpu_gemm_rate(a_words, b_words, rows)
    start = time.perf_counter()
    for _ in range(args.steps):
        oracle.gemm_rows(a_words, b_words, 0, rows)
    elapsed = time.perf_counter() - start
    value = 2.0 * rows * N * K * args.steps / elapsed / 1e12
    sample = f"{rows} rows of C x full N={N} x full K={K} per step (of {M} rows)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": oracle.threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference is Rust + cuda-oxide and cannot be built here; this is the C port of its CPU "
                "GEMM reference (oracle/fk_oracle.c) on all host threads",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ our arm

def time_steps(fn, steps: int, warmup: int, barrier):
    """W untimed steps, then K steps between CUDA events on the current stream; returns seconds."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(stop) / 1e3


def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    from ferro_kittens_b200 import flash_forward, gemm, shard
    from ferro_kittens_b200._lib import check, library
    from ferro_kittens_b200.build import build_cublaslt

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(seconds: float) -> float:
        if world == 1:
            return seconds
        value = torch.tensor([seconds], dtype=torch.float64, device=device)
        dist.all_reduce(value, op=dist.ReduceOp.MAX)
        return float(value.item())

    peaks = measured_peaks()
    stream = torch.cuda.current_stream().cuda_stream

    # ---- operands: every rank derives the same A and B from the seed, then keeps its B shard
    generator = torch.Generator(device=device).manual_seed(GEMM_SEED)
    a = (torch.randn((M, K), generator=generator, device=device) / math.sqrt(K)).to(torch.bfloat16)
    b_full = (torch.randn((N, K), generator=generator, device=device) / math.sqrt(K)).to(torch.bfloat16)
    n0, n1 = shard.gemm_columns(N, world, rank)
    b = b_full[n0:n1].contiguous()
    # The end-to-end leg starts from host buffers, where the upload is the cost: it cuts C into a grid of
    # blocks (fewest bytes uploaded per rank) instead of column blocks alone; keep that block of B on the host.
    e_r0, e_r1, e_c0, e_c1 = shard.gemm_block(M, N, world, rank)
    host_b = b_full[e_c0:e_c1].cpu().pin_memory()
    del b_full
    n_local = n1 - n0
    c = torch.empty((M, n_local), dtype=torch.bfloat16, device=device)
    status = gemm.new_status(device)
    a_map, b_map, c_map = gemm.maps(a, b, c)

    def step():
        gemm.launch(a_map, b_map, c_map, M, n_local, K, args.group, status)

    # ---- verify before timing: our C against cuBLASLt's on the same operands
    cublaslt = ctypes.CDLL(str(build_cublaslt()))
    cublaslt.fkb_gemm.argtypes = [ctypes.c_void_p] * 4
    cublaslt.fkb_last_error.restype = ctypes.c_char_p
    if cublaslt.fkb_prepare(M, n_local, K) != 0:
        raise RuntimeError(cublaslt.fkb_last_error().decode())
    c_ref = torch.empty_like(c)

    def cublaslt_step():
        if cublaslt.fkb_gemm(a.data_ptr(), b.data_ptr(), c_ref.data_ptr(), stream) != 0:
            raise RuntimeError(cublaslt.fkb_last_error().decode())

    step()
    gemm.check_status(status)
    cublaslt_step()
    torch.cuda.synchronize()
    worst = (c.float() - c_ref.float()).abs().max().item()
    scale = c_ref.float().abs().max().item()
    if not worst <= 2 ** -7 * scale:
        raise RuntimeError(f"GEMM disagrees with cuBLASLt: max |diff| {worst} against max |c| {scale}")

    # ---- the timed region: K launches, device-timed, max over ranks. cuBLASLt is timed the same way
    # immediately before and after, so that neither side owns the cooler chip.
    with ClockSampler(local_rank) as sampler:
        cublaslt_before = max_over_ranks(time_steps(cublaslt_step, args.steps, args.warmup, barrier))
        seconds = max_over_ranks(time_steps(step, args.steps, args.warmup, barrier))
        cublaslt_after = max_over_ranks(time_steps(cublaslt_step, args.steps, args.warmup, barrier))
    gemm.check_status(status)
    clocks = sampler.summary()
    flops_total = 2.0 * M * N * K
    value = flops_total * args.steps / seconds / 1e12
    per_launch_s = seconds / args.steps
    achieved = 2.0 * M * n_local * K / per_launch_s / 1e12  # this rank's kernel
    long_region = seconds > 2.0
    peak = peaks["sustained"] if long_region else peaks["burst"]
    cublaslt_seconds = 0.5 * (cublaslt_before + cublaslt_after)
    cublaslt_value = flops_total * args.steps / cublaslt_seconds / 1e12

    # ---- flash-attention forward, planes split across ranks
    planes_total = FLASH["batch"] * FLASH["heads"]
    p0, p1 = shard.planes(planes_total, world, rank)
    generator = torch.Generator(device=device).manual_seed(FLASH["seed"])
    qkv = [torch.randn((planes_total, FLASH["seq"], 128), generator=generator, device=device)
           .to(torch.bfloat16)[p0:p1].contiguous() for _ in range(3)]
    flash_status = gemm.new_status(device)
    out = torch.empty_like(qkv[0])
    lse = torch.empty((p1 - p0, FLASH["seq"]), dtype=torch.float32, device=device)

    def flash_step():
        check(library().fk_flash_fwd(qkv[0].data_ptr(), qkv[1].data_ptr(), qkv[2].data_ptr(), out.data_ptr(),
                                     None, lse.data_ptr(), p1 - p0, FLASH["seq"], 128 ** -0.5,
                                     int(FLASH["causal"]), stream, flash_status.data_ptr()))

    flash_step()
    gemm.check_status(flash_status)
    reference = torch.nn.functional.scaled_dot_product_attention(
        qkv[0][:2].unsqueeze(0), qkv[1][:2].unsqueeze(0), qkv[2][:2].unsqueeze(0))[0]
    flash_error = (out[:2].float() - reference.float()).abs().max().item()
    if not flash_error <= 2e-2:
        raise RuntimeError(f"flash forward disagrees with torch SDPA: max |diff| {flash_error}")
    flash_seconds = max_over_ranks(time_steps(flash_step, args.steps, args.warmup, barrier))
    flash_flops = 4.0 * planes_total * FLASH["seq"] ** 2 * 128
    flash_value = flash_flops * args.steps / flash_seconds / 1e12

    # ---- its backward on the same shard: dQ, dK, dV from the forward's O and LSE
    d_out = torch.randn(qkv[0].shape, generator=generator, device=device).to(torch.bfloat16)
    grads = [torch.empty_like(qkv[0]) for _ in range(3)]
    workspace = torch.empty(library().fk_flash_bwd_workspace_bytes(p1 - p0, FLASH["seq"]) // 4,
                            dtype=torch.float32, device=device)

    def flash_bwd_step():
        check(library().fk_flash_bwd(qkv[0].data_ptr(), qkv[1].data_ptr(), qkv[2].data_ptr(), out.data_ptr(),
                                     d_out.data_ptr(), lse.data_ptr(), grads[0].data_ptr(), grads[1].data_ptr(),
                                     grads[2].data_ptr(), workspace.data_ptr(), p1 - p0, FLASH["seq"], 128 ** -0.5,
                                     int(FLASH["causal"]), stream, flash_status.data_ptr()))

    flash_bwd_step()
    gemm.check_status(flash_status)
    leaves = [t[:1].float().requires_grad_() for t in qkv]
    torch.nn.functional.scaled_dot_product_attention(*[t.unsqueeze(0) for t in leaves]).backward(
        d_out[:1].float().unsqueeze(0))
    bwd_error = max(((g[:1].float() - leaf.grad).abs().max() / leaf.grad.abs().max()).item()
                    for g, leaf in zip(grads, leaves))
    if not bwd_error <= 2e-2:
        raise RuntimeError(f"flash backward disagrees with fp32 autograd: {bwd_error} of the largest gradient")
    bwd_seconds = max_over_ranks(time_steps(flash_bwd_step, args.steps, args.warmup, barrier))
    bwd_value = 2.5 * flash_flops * args.steps / bwd_seconds / 1e12
    del qkv, out, lse, d_out, grads, workspace, leaves

    # ---- the causal long-sequence forward (the sharded attention configuration), planes split across ranks
    causal_planes = FLASH_CAUSAL["batch"] * FLASH_CAUSAL["heads"]
    c0, c1 = shard.planes(causal_planes, world, rank)
    generator = torch.Generator(device=device).manual_seed(FLASH_CAUSAL["seed"])
    qkv = [torch.randn((causal_planes, FLASH_CAUSAL["seq"], 128), generator=generator, device=device)
           .to(torch.bfloat16)[c0:c1].contiguous() for _ in range(3)]
    out = torch.empty_like(qkv[0])
    lse = torch.empty((c1 - c0, FLASH_CAUSAL["seq"]), dtype=torch.float32, device=device)

    def causal_step():
        check(library().fk_flash_fwd(qkv[0].data_ptr(), qkv[1].data_ptr(), qkv[2].data_ptr(), out.data_ptr(),
                                     None, lse.data_ptr(), c1 - c0, FLASH_CAUSAL["seq"], 128 ** -0.5, 1, stream,
                                     flash_status.data_ptr()))

    causal_step()
    gemm.check_status(flash_status)
    reference = torch.nn.functional.scaled_dot_product_attention(
        qkv[0][:1].unsqueeze(0), qkv[1][:1].unsqueeze(0), qkv[2][:1].unsqueeze(0), is_causal=True)[0]
    causal_error = (out[:1].float() - reference.float()).abs().max().item()
    if not causal_error <= 2e-2:
        raise RuntimeError(f"causal flash forward disagrees with torch SDPA: max |diff| {causal_error}")
    causal_seconds = max_over_ranks(time_steps(causal_step, args.steps, args.warmup, barrier))
    # useful flops: key blocks above the diagonal are neither computed nor counted
    causal_flops = 4.0 * causal_planes * 128 * FLASH_CAUSAL["seq"] * (FLASH_CAUSAL["seq"] + 1) / 2
    causal_value = causal_flops * args.steps / causal_seconds / 1e12
    del qkv, out, lse, reference

    # ---- the row kernels either side of the two contractions: rows split across ranks, HBM roofline
    from ferro_kittens_b200 import rows as row_kernels

    rows_total = ROW_KERNEL_ROWS
    r0, r1 = shard.row_tiles(rows_total, world, rank)
    generator = torch.Generator(device=device).manual_seed(ROW_KERNEL_SEED)
    activations = (torch.randn((r1 - r0, 128), generator=generator, device=device) * 2).to(torch.bfloat16)
    normalised = torch.empty_like(activations)
    ones = torch.ones(128, dtype=torch.bfloat16, device=device)
    zeros = torch.zeros(128, dtype=torch.bfloat16, device=device)
    row_status = gemm.new_status(device)
    row_results = {}
    for name, call in (("softmax_rows", lambda: row_kernels.softmax_rows(activations, out=normalised, status=row_status)),
                       ("layernorm_rows", lambda: row_kernels.layernorm_rows(activations, ones, zeros, 1e-5,
                                                                              out=normalised, status=row_status)),
                       ("groupnorm_tile", lambda: row_kernels.groupnorm_tile(activations, 1e-5, out=normalised,
                                                                             status=row_status))):
        call()
        gemm.check_status(row_status)
        if name == "softmax_rows":
            drift = (normalised[:4096].float().sum(dim=1) - 1).abs().max().item()
        elif name == "layernorm_rows":
            drift = normalised[:4096].float().mean(dim=1).abs().max().item()
        else:
            drift = abs(normalised[:128].float().mean().item())
        if not drift <= 2e-2:
            raise RuntimeError(f"{name} fails its row property: {drift}")
        row_seconds = max_over_ranks(time_steps(call, args.steps, args.warmup, barrier))
        gbs = 4.0 * rows_total * 128 * args.steps / row_seconds / 1e9
        row_results[name] = {"value": gbs, "unit": "GB/s", "ms_per_step": row_seconds / args.steps * 1e3,
                             "frac_of_measured_hbm": gbs / world / peaks["hbm"]}
    del activations, normalised

    # ---- end to end: host buffers through the C-ABI call, copies inside the timed region
    e2e_steps = 3
    e_m, e_n = e_r1 - e_r0, e_c1 - e_c0
    host_a = torch.empty((e_m, K), dtype=torch.bfloat16).pin_memory()
    host_c = torch.empty((e_m, e_n), dtype=torch.bfloat16).pin_memory()
    host_a.copy_(a[e_r0:e_r1])
    torch.cuda.synchronize()
    gemm.run_host(host_a, host_b, host_c, e_m, e_n, K, args.group)  # warm: allocates the staging buffers
    barrier()
    start = time.perf_counter()
    for _ in range(e2e_steps):
        gemm.run_host(host_a, host_b, host_c, e_m, e_n, K, args.group)
    e2e_seconds = max_over_ranks(time.perf_counter() - start)
    expected_block = gemm.run(a[e_r0:e_r1].contiguous(), host_b.to(device))
    if not torch.equal(host_c, expected_block.cpu()):
        raise RuntimeError("the host-buffer entry point returned a different C")
    del expected_block
    e2e_value = flops_total * e2e_steps / e2e_seconds / 1e12
    h2d = (e_m * K + e_n * K) * 2
    d2h = e_m * e_n * 2
    e2e_grid = shard.gemm_grid(M, N, world)

    # ---- CPU baseline: the oracle port on the host cores, rank 0 of a single-GPU run only
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        import oracle

        oracle.use_all_cores()
        a_words = host_a[:2048].view(torch.int16).numpy().view(np.uint16)
        b_words = host_b.view(torch.int16).numpy().view(np.uint16)
        probe_rate, _ = cpu_gemm_rate(a_words, b_words, 8)
        rows = int(max(8, min(2048, probe_rate * 1e12 * 15.0 / (2.0 * N * K))))
        rate, elapsed = cpu_gemm_rate(a_words, b_words, rows)
        cpu_baseline = {"value": rate, "unit": "TFLOP/s", "cores": oracle.threads(), "kind": "port",
                        "sample": f"{rows} rows of C x full N={N} x full K={K} in {elapsed:.1f} s "
                                  f"(of {M} rows; whole problem extrapolates to {2.0 * M * N * K / rate / 1e12:.0f} s)"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per_launch_s * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "m": M, "n": N, "k": K, "group": args.group,
                       "sharding": f"B split by N-column blocks over {world} rank(s), {n_local} columns each; "
                                   "A replicated; no collective",
                       "l2": "inputs (A 512 MiB + B shard) larger than the 126 MB L2; no flush between steps"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         # dram__bytes_read + write of one launch of this kernel on the full 16384^3 shape
                         # (one ncu capture of four metrics at group 8; see profiles/), scaled by the rank's share of N.
                         "traffic": (7.35e9 + 0.591e9) * n_local / N, "traffic_unit": "bytes/launch",
                         "algorithmic_flops_per_launch": 2.0 * M * n_local * K,
                         "peak_source": f"{peaks['source']} ({'sustained' if long_region else 'burst'} cuBLAS bf16)",
                         "frac_of_nominal_2250": achieved / 2250.0},
            "cublaslt": {"value": cublaslt_value, "unit": "TFLOP/s", "ratio_ours_over_cublaslt": value / cublaslt_value,
                         "before": flops_total * args.steps / cublaslt_before / 1e12,
                         "after": flops_total * args.steps / cublaslt_after / 1e12,
                         "max_abs_diff_vs_ours": worst},
            "flash_fwd": {"config": {k: v for k, v in FLASH.items()}, "value": flash_value, "unit": "TFLOP/s",
                          "ms_per_step": flash_seconds / args.steps * 1e3,
                          "frac_of_measured_peak": flash_value / world / peaks["burst"],
                          "frac_of_nominal_2250": flash_value / world / 2250.0,
                          "max_abs_diff_vs_sdpa": flash_error},
            "flash_fwd_causal": {"config": {k: v for k, v in FLASH_CAUSAL.items()}, "value": causal_value,
                                 "unit": "TFLOP/s", "flops_counted": "4 * planes * 128 * seq * (seq + 1) / 2",
                                 "ms_per_step": causal_seconds / args.steps * 1e3,
                                 "frac_of_measured_peak": causal_value / world / peaks["burst"],
                                 "max_abs_diff_vs_sdpa": causal_error},
            "flash_bwd": {"config": {k: v for k, v in FLASH.items()}, "value": bwd_value, "unit": "TFLOP/s",
                          "flops_counted": "10 * planes * seq^2 * 128 (five tile products; seven are executed)",
                          "ms_per_step": bwd_seconds / args.steps * 1e3,
                          "frac_of_measured_peak": bwd_value / world / peaks["burst"],
                          "max_error_over_max_gradient_vs_fp32_autograd": bwd_error},
            "row_kernels": {"config": {"rows": rows_total, "columns": 128, "seed": ROW_KERNEL_SEED,
                                       "bytes_per_element": 4, "sharding": f"rows over {world} rank(s)"},
                            "peak": peaks["hbm"], "peak_unit": "GB/s", "peak_source": peaks["source"], **row_results},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "call": "fk_gemm_bf16_host",
                    "blocks_of_c": f"{e2e_grid[0]} x {e2e_grid[1]} (one per rank)"},
            "gpu_launches": args.steps,
            "clocks": clocks,
        }
        if cpu_baseline:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_only(args, local_rank: int) -> None:
    """One kernel alone on a chosen size: the command an ncu capture wraps."""
    import torch

    from ferro_kittens_b200 import gemm
    from ferro_kittens_b200._lib import check, library

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    stream = torch.cuda.current_stream().cuda_stream
    status = gemm.new_status(device)
    if args.only == "gemm":
        m, n, k = args.m, args.n, args.k
        generator = torch.Generator(device=device).manual_seed(GEMM_SEED)
        a = (torch.randn((m, k), generator=generator, device=device) / math.sqrt(k)).to(torch.bfloat16)
        b = (torch.randn((n, k), generator=generator, device=device) / math.sqrt(k)).to(torch.bfloat16)
        c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        a_map, b_map, c_map = gemm.maps(a, b, c)
        fn = lambda: gemm.launch(a_map, b_map, c_map, m, n, k, args.group, status)  # noqa: E731
        flops = 2.0 * m * n * k
        name = f"gemm_bf16_{m}x{n}x{k}"
    elif args.only in ("softmax", "layernorm", "groupnorm"):
        from ferro_kittens_b200 import rows as row_kernels

        generator = torch.Generator(device=device).manual_seed(ROW_KERNEL_SEED)
        x = (torch.randn((args.rows, 128), generator=generator, device=device) * 2).to(torch.bfloat16)
        y = torch.empty_like(x)
        ones = torch.ones(128, dtype=torch.bfloat16, device=device)
        zeros = torch.zeros(128, dtype=torch.bfloat16, device=device)
        fn = {"softmax": lambda: row_kernels.softmax_rows(x, out=y, status=status),
              "layernorm": lambda: row_kernels.layernorm_rows(x, ones, zeros, 1e-5, out=y, status=status),
              "groupnorm": lambda: row_kernels.groupnorm_tile(x, 1e-5, out=y, status=status)}[args.only]
        seconds = time_steps(fn, args.steps, args.warmup, lambda: None)
        gemm.check_status(status)
        print(json.dumps({"only": f"{args.only}_rows{args.rows}", "steps": args.steps,
                          "ms_per_step": seconds / args.steps * 1e3,
                          "gbs": 4.0 * args.rows * 128 * args.steps / seconds / 1e9}), flush=True)
        return
    elif args.only == "flash_bwd":
        from ferro_kittens_b200 import flash_backward, flash_forward

        planes, seq = args.planes, args.seq
        generator = torch.Generator(device=device).manual_seed(FLASH["seed"])
        q, kk, v, d_out = (torch.randn((planes, seq, 128), generator=generator, device=device).to(torch.bfloat16)
                           for _ in range(4))
        out, lse = flash_forward.run(q, kk, v, causal=args.causal, status=status)
        workspace = torch.empty(2 * planes * seq, dtype=torch.float32, device=device)
        fn = lambda: flash_backward.run(q, kk, v, out, d_out, lse, causal=args.causal, status=status,  # noqa: E731
                                        workspace=workspace)
        flops = 10.0 * planes * seq * seq * 128 * (0.5 if args.causal else 1.0)
        name = f"flash_bwd_planes{planes}_seq{seq}_{'causal' if args.causal else 'full'}"
    else:
        planes, seq = args.planes, args.seq
        generator = torch.Generator(device=device).manual_seed(FLASH["seed"])
        q, kk, v = (torch.randn((planes, seq, 128), generator=generator, device=device).to(torch.bfloat16)
                    for _ in range(3))
        out = torch.empty_like(q)
        lse = torch.empty((planes, seq), dtype=torch.float32, device=device)
        fn = lambda: check(library().fk_flash_fwd(  # noqa: E731
            q.data_ptr(), kk.data_ptr(), v.data_ptr(), out.data_ptr(), None, lse.data_ptr(), planes, seq,
            128 ** -0.5, int(args.causal), stream, status.data_ptr()))
        flops = 4.0 * planes * seq * seq * 128 * (0.5 if args.causal else 1.0)
        name = f"flash_fwd_planes{planes}_seq{seq}_{'causal' if args.causal else 'full'}"
    seconds = time_steps(fn, args.steps, args.warmup, lambda: None)
    gemm.check_status(status)
    line = {"only": name, "steps": args.steps, "ms_per_step": seconds / args.steps * 1e3,
            "tflops": flops * args.steps / seconds / 1e12}
    if args.only == "gemm" and args.beside_library:
        # The library's kernel for the same product, launched the same number of times, so that a
        # launch list of this command holds both.
        out = torch.empty((args.m, args.n), dtype=torch.bfloat16, device=device)
        library_seconds = time_steps(lambda: torch.matmul(a, b.T, out=out), args.steps, args.warmup, lambda: None)
        line["library_ms_per_step"] = library_seconds / args.steps * 1e3
    print(json.dumps(line), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--only", choices=["gemm", "flash", "flash_bwd", "softmax", "layernorm", "groupnorm"],
                        help="run one kernel alone (for profiling)")
    parser.add_argument("--rows", type=int, default=1 << 20, help="rows of 128 columns for the row kernels")
    parser.add_argument("--beside-library", action="store_true",
                        help="with --only gemm: also launch torch.matmul (cuBLAS) on the same operands")
    parser.add_argument("--m", type=int, default=8192)
    parser.add_argument("--n", type=int, default=8192)
    parser.add_argument("--k", type=int, default=8192)
    parser.add_argument("--planes", type=int, default=32)
    parser.add_argument("--seq", type=int, default=4096)
    parser.add_argument("--causal", action="store_true")
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--group", type=int, default=8)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank, local_rank, world = env_int("RANK", 0), env_int("LOCAL_RANK", 0), env_int("WORLD_SIZE", 1)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.only:
        run_only(args, local_rank)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the two hot paths on B200.

``python bench.py --gpus N --steps K --warmup W`` times the bf16 GEMM
16384 x 16384 x 16384 (entries N(0,1)/sqrt(K), seed 1; under torchrun B is split
by N-column blocks across the ranks, no collective) and prints ONE JSON line.
A step is one launch of the GEMM over the rank's shard. Every block of the line is
read twice, on the first K steps after the warm-up and on K steps after the device
has run that kernel back to back for ``--settle`` seconds (the figure reported: the
board is at its power limit within tens of milliseconds, so only settled regions
compare across rank counts), with the reference clock's per-launch columns (min,
median, max, spread, drift) beside it. The same line carries cuBLASLt on the same
operands (alone and interleaved launch by launch), the sharded 8192 x 28672 x 8192
GEMM, flash-attention forward (non-causal B=16 H=16 S=4096 and causal B=4 H=32
S=16384, D=128; planes split across ranks) and backward, the row kernels, the
end-to-end figure from host buffers, the tensor-core roofline of the GEMM kernel,
and the CPU baseline (the oracle port on the host cores).

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
C2 = dict(m=M, n=N, k=K, seed=GEMM_SEED, scale=1.0 / 128.0, entries="N(0,1) / sqrt(K)")
C3 = dict(m=8192, n=28672, k=8192, seed=2, scale=0.02, entries="N(0, 0.02)")
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


# ------------------------------------------------------------------ operands

#: tensor ids of the counter-based generator, per configuration
A_ID, B_ID = 0, 1


def gemm_operand(config: dict, which: str, row0: int, rows: int, device):
    """Rows [row0, row0 + rows) of A ([M, K]) or of the K-major B ([N, K]) of a GEMM configuration."""
    from ferro_kittens_b200 import seeded

    return seeded.bf16_rows("normal", config["seed"], A_ID if which == "a" else B_ID, row0, rows, config["k"],
                            config["scale"], device=device)


def attention_operands(config: dict, plane0: int, planes: int, device):
    """Q, K, V of planes [plane0, plane0 + planes): [planes, seq, 128] bf16, N(0, 1)."""
    from ferro_kittens_b200 import seeded

    seq = config["seq"]
    return [seeded.bf16_rows("normal", config["seed"], tensor, plane0 * seq, planes * seq, 128, 1.0, device=device)
            .view(planes, seq, 128) for tensor in range(3)]


# ------------------------------------------------------------------ reference arm / CPU baseline

def cpu_gemm_rate(a_words, b_words, rows: int):
    """Time the oracle's GEMM over `rows` rows of C (full N, full K); returns (TFLOP/s, seconds)."""
    import oracle

    start = time.perf_counter()
    oracle.gemm_rows(a_words, b_words, 0, rows)
    elapsed = time.perf_counter() - start
    return 2.0 * rows * b_words.shape[0] * b_words.shape[1] / elapsed / 1e12, elapsed


def words(tensor):
    """bf16 torch tensor on the host -> numpy uint16 view."""
    import numpy as np
    import torch

    return tensor.view(torch.int16).numpy().view(np.uint16)


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    import oracle

    oracle.use_all_cores()
    # The same words the GPU arm derives: the generator is a function of (seed, tensor, index).
    a_words = words(gemm_operand(C2, "a", 0, 256, "cpu"))
    b_words = words(gemm_operand(C2, "b", 0, N, "cpu"))
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


# ------------------------------------------------------------------ the clock

def launch_stats(milliseconds, flops):
    """The reference clock's columns (examples/src/bench.rs:67-105) over per-launch device times
    kept in launch order: min, median, max, spread = max / min - 1, drift = mean of the second
    half over mean of the first half - 1."""
    ordered = sorted(milliseconds)
    half = len(milliseconds) // 2
    mean = lambda xs: sum(xs) / len(xs)  # noqa: E731
    drift = mean(milliseconds[half:]) / mean(milliseconds[:half]) - 1.0 if half else 0.0
    out = {"launches": len(milliseconds), "min_ms": ordered[0], "median_ms": ordered[len(ordered) // 2],
           "max_ms": ordered[-1], "spread": ordered[-1] / ordered[0] - 1.0, "drift": drift}
    if flops:
        out["tflops_at_min"] = flops / ordered[0] / 1e9
        out["tflops_at_median"] = flops / out["median_ms"] / 1e9
    return out


class Clock:
    """W warm-up steps, then EXACTLY K steps between CUDA events with a barrier and a synchronize on
    both sides, max over ranks -- taken twice: on the first K steps after the warm-up and again
    once the device has run this kernel back to back for `settle` seconds, so that every block of
    the line, at every rank count, is read in the same power state (the board reaches its power
    limit within tens of milliseconds of dense work). The settled region also carries one event
    pair per launch."""

    def __init__(self, steps, warmup, barrier, max_over_ranks, settle=0.5):
        self.steps, self.warmup, self.barrier, self.max_over_ranks, self.settle = steps, warmup, barrier, max_over_ranks, settle

    def region(self, fn, per_launch: bool):
        import torch

        torch.cuda.synchronize()
        self.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        marks = []
        start.record()
        for _ in range(self.steps):
            if per_launch:
                before, after = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                before.record()
                fn()
                after.record()
                marks.append((before, after))
            else:
                fn()
        stop.record()
        torch.cuda.synchronize()
        self.barrier()
        return start.elapsed_time(stop) / 1e3, [b.elapsed_time(a) for b, a in marks]

    def measure(self, fn, flops_per_step=None):
        """Returns {"first_s", "seconds" (settled K steps, max over ranks), "conditioning_launches", "launch": stats}."""
        import torch

        for _ in range(self.warmup):
            fn()
        first = self.max_over_ranks(self.region(fn, False)[0])
        # keep the device on this kernel until `settle` seconds have gone by; same count on every rank
        extra = max(0, int(math.ceil((self.settle - first) / max(first / self.steps, 1e-9))))
        extra = min(extra, 200_000)
        for index in range(extra):
            fn()
            if index % 256 == 255:
                torch.cuda.synchronize()  # bound the queue depth
        seconds, per_launch = self.region(fn, True)
        return {"first_s": first, "seconds": self.max_over_ranks(seconds), "conditioning_launches": extra,
                "launch": launch_stats(per_launch, flops_per_step)}


def interleaved(fns: dict, pairs: int):
    """A B A B ... with an event pair around every launch: both sides see the same thermal history.
    Returns per-name lists of device milliseconds in launch order."""
    import torch

    for fn in fns.values():
        fn()
    torch.cuda.synchronize()
    marks = {name: [] for name in fns}
    for _ in range(pairs):
        for name, fn in fns.items():
            before, after = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            before.record()
            fn()
            after.record()
            marks[name].append((before, after))
    torch.cuda.synchronize()
    return {name: [b.elapsed_time(a) for b, a in pairs_] for name, pairs_ in marks.items()}


# ------------------------------------------------------------------ our arm

def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    from ferro_kittens_b200 import gemm, shard
    from ferro_kittens_b200._lib import check, library
    from ferro_kittens_b200.build import build_cublaslt

    asked_group = args.group
    args.group = args.group or gemm.GROUP

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
    clock = Clock(args.steps, args.warmup, barrier, max_over_ranks, args.settle)
    cublaslt = ctypes.CDLL(str(build_cublaslt()))
    cublaslt.fkb_gemm.argtypes = [ctypes.c_void_p] * 4
    cublaslt.fkb_last_error.restype = ctypes.c_char_p

    def gemm_block(config: dict, sampled: bool):
        """One GEMM configuration on this rank's shard: verify against cuBLASLt, time ours (settled K
        steps), cuBLASLt the same way, then the two interleaved launch by launch."""
        m, n, k = config["m"], config["n"], config["k"]
        n0, n1 = shard.gemm_columns(n, world, rank)
        n_local = n1 - n0
        a = gemm_operand(config, "a", 0, m, device)          # replicated
        b = gemm_operand(config, "b", n0, n_local, device)    # this rank's rows of the K-major B only
        c = torch.empty((m, n_local), dtype=torch.bfloat16, device=device)
        c_ref = torch.empty_like(c)
        status = gemm.new_status(device)
        # maps built once, as the reference's `run` does, to the item width this shard's waves want
        maps = gemm.TiledMaps(a, b, c)
        group = asked_group or gemm.group_for(m, n_local, device)
        if cublaslt.fkb_prepare(m, n_local, k) != 0:
            raise RuntimeError(cublaslt.fkb_last_error().decode())

        def step():
            gemm.launch_tiled(maps, m, n_local, k, group, status)

        def library_step():
            if cublaslt.fkb_gemm(a.data_ptr(), b.data_ptr(), c_ref.data_ptr(), stream) != 0:
                raise RuntimeError(cublaslt.fkb_last_error().decode())

        # a tripwire before timing (the parity gates against the oracle are the -m gpu tests)
        step()
        gemm.check_status(status)
        library_step()
        torch.cuda.synchronize()
        worst = (c.float() - c_ref.float()).abs().max().item()
        scale = c_ref.float().abs().max().item()
        if not worst <= 2 ** -7 * scale:
            raise RuntimeError(f"GEMM disagrees with cuBLASLt: max |diff| {worst} against max |c| {scale}")

        flops_total, flops_rank = 2.0 * m * n * k, 2.0 * m * n_local * k
        with ClockSampler(local_rank) as ours_clocks:
            ours = clock.measure(step, flops_rank)
        gemm.check_status(status)
        with ClockSampler(local_rank) as library_clocks:
            theirs = clock.measure(library_step, flops_rank)
        pairs = interleaved({"ours": step, "cublaslt": library_step}, max(10, args.steps))
        side = {name: launch_stats(ms, flops_rank) for name, ms in pairs.items()}
        gemm.check_status(status)

        def with_cycles(result, sampler):
            clocks = sampler.summary()
            out = {"value": flops_total * args.steps / result["seconds"] / 1e12, "unit": "TFLOP/s",
                   "first_region_value": flops_total * args.steps / result["first_s"] / 1e12,
                   "ms_per_step": result["seconds"] / args.steps * 1e3, "launch": result["launch"],
                   "sm_mhz": clocks["sm_mhz"], "power_w_max": clocks["power_w_max"], "reasons": clocks["reasons"]}
            if clocks["sm_mhz"]:
                out["cycles_per_launch_at_median"] = result["launch"]["median_ms"] * clocks["sm_mhz"] * 1e3
            return out, clocks

        ours_out, ours_summary = with_cycles(ours, ours_clocks)
        theirs_out, _ = with_cycles(theirs, library_clocks)
        achieved = flops_rank / (ours["seconds"] / args.steps) / 1e12
        result = {
            "config": {"m": m, "n": n, "k": k, "seed": config["seed"], "entries": config["entries"],
                       "columns_per_rank": n_local, "item_columns": maps.columns, "group": group},
            "ours": ours_out, "cublaslt_alone": theirs_out,
            "interleaved": {"pairs": max(10, args.steps), "ours": side["ours"], "cublaslt": side["cublaslt"],
                            "ratio_ours_over_cublaslt_at_median": side["cublaslt"]["median_ms"] / side["ours"]["median_ms"],
                            "ratio_ours_over_cublaslt_at_min": side["cublaslt"]["min_ms"] / side["ours"]["min_ms"]},
            "ratio_ours_over_cublaslt_alone": ours_out["value"] / theirs_out["value"],
            "achieved_per_gpu": achieved, "max_abs_diff_vs_cublaslt": worst,
        }
        return result, (a, b, c, n0, n1, ours, ours_summary)

    # ---- C2, the headline
    c2, (a, b, c, n0, n1, c2_timing, clocks) = gemm_block(C2, True)
    n_local = n1 - n0
    seconds = c2_timing["seconds"]
    flops_total = 2.0 * M * N * K
    value = flops_total * args.steps / seconds / 1e12
    per_launch_s = seconds / args.steps
    achieved = c2["achieved_per_gpu"]
    sustained = (c2_timing["first_s"] + seconds + c2_timing["conditioning_launches"] * per_launch_s) > 0.4
    peak = peaks["sustained"] if sustained else peaks["burst"]

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region. One rank:
    # the C-ABI host entry. Several: every rank uploads its share of A's rows and its block of B, the
    # ranks complete A in their own memory over NVLink, block by block (staging, outside the kernels).
    e2e_steps = max(args.steps, 10)
    a0, a1 = shard.a_rows(M, world, rank)
    host_a = a[a0:a1].cpu().pin_memory()
    host_b = b.cpu().pin_memory()
    host_c = torch.empty((M, n_local), dtype=torch.bfloat16).pin_memory()
    if world == 1:
        def e2e_step():
            gemm.run_host(host_a, host_b, host_c, M, n_local, K, args.group)
        h2d, d2h = (M * K + n_local * K) * 2, M * n_local * 2
        e2e_call = "fk_gemm_bf16_host"
    else:
        plan = gemm.ShardedHostGemm(M, n_local, K, world, rank, device, args.group, blocks=args.gather_blocks)
        def e2e_step():
            plan.run(host_a, host_b, host_c)
        h2d, d2h = plan.bytes_per_step()
        e2e_call = "ShardedHostGemm.run (fk_gemm_bf16 per gathered block of A's rows)"
    e2e_step()  # warm: allocates the staging buffers, opens the NCCL channels
    e2e_step()
    torch.cuda.synchronize()
    barrier()
    start = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_seconds = max_over_ranks(time.perf_counter() - start)
    if not torch.equal(host_c, c.cpu()):
        raise RuntimeError("the host-buffer path returned a different C")
    e2e_value = flops_total * e2e_steps / e2e_seconds / 1e12

    # ---- CPU baseline: the oracle port on the host cores, rank 0 of a single-GPU run only
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        import oracle

        oracle.use_all_cores()
        a_words, b_words = words(host_a[:2048]), words(host_b)
        probe_rate, _ = cpu_gemm_rate(a_words, b_words, 8)
        rows = int(max(8, min(2048, probe_rate * 1e12 * 15.0 / (2.0 * N * K))))
        rate, elapsed = cpu_gemm_rate(a_words, b_words, rows)
        cpu_baseline = {"value": rate, "unit": "TFLOP/s", "cores": oracle.threads(), "kind": "port",
                        "sample": f"{rows} rows of C x full N={N} x full K={K} in {elapsed:.1f} s "
                                  f"(of {M} rows; whole problem extrapolates to {2.0 * M * N * K / rate / 1e12:.0f} s)"}
    del a, b, c, host_a, host_b, host_c
    if world > 1:
        del plan
    torch.cuda.empty_cache()

    # ---- C3, the sharded MLP up-projection shape
    c3, _ = gemm_block(C3, False)
    del _
    torch.cuda.empty_cache()

    # ---- flash-attention forward (C4), its backward, and the causal long-sequence forward (C5)
    flash_status = gemm.new_status(device)

    def attention_block(config: dict, backward: bool):
        planes_total = config["batch"] * config["heads"]
        p0, p1 = shard.planes(planes_total, world, rank)
        seq, causal = config["seq"], int(config["causal"])
        qkv = attention_operands(config, p0, p1 - p0, device)
        out = torch.empty_like(qkv[0])
        lse = torch.empty((p1 - p0, seq), dtype=torch.float32, device=device)

        def forward_step():
            check(library().fk_flash_fwd(qkv[0].data_ptr(), qkv[1].data_ptr(), qkv[2].data_ptr(), out.data_ptr(),
                                         None, lse.data_ptr(), p1 - p0, seq, 128 ** -0.5, causal, stream,
                                         flash_status.data_ptr()))

        forward_step()
        gemm.check_status(flash_status)
        reference = torch.nn.functional.scaled_dot_product_attention(
            qkv[0][:1].unsqueeze(0), qkv[1][:1].unsqueeze(0), qkv[2][:1].unsqueeze(0), is_causal=bool(causal))[0]
        error = (out[:1].float() - reference.float()).abs().max().item()
        if not error <= 2e-2:
            raise RuntimeError(f"flash forward disagrees with torch SDPA: max |diff| {error}")
        flops = 4.0 * planes_total * 128 * (seq * (seq + 1) / 2 if causal else seq * seq)
        flops_rank = flops * (p1 - p0) / planes_total
        timing = clock.measure(forward_step, flops_rank)
        gemm.check_status(flash_status)
        forward = {"config": dict(config), "value": flops * args.steps / timing["seconds"] / 1e12, "unit": "TFLOP/s",
                   "first_region_value": flops * args.steps / timing["first_s"] / 1e12,
                   "ms_per_step": timing["seconds"] / args.steps * 1e3, "launch": timing["launch"],
                   "max_abs_diff_vs_sdpa": error}
        forward["frac_of_measured_peak"] = forward["value"] / world / peaks["burst"]
        forward["frac_of_measured_sustained_peak"] = forward["value"] / world / peaks["sustained"]
        forward["frac_of_nominal_2250"] = forward["value"] / world / 2250.0
        if causal:
            forward["flops_counted"] = "4 * planes * 128 * seq * (seq + 1) / 2 (blocks above the diagonal are neither computed nor counted)"
        if not backward:
            return forward, None
        generator = torch.Generator(device=device).manual_seed(config["seed"] + 100 + rank)
        d_out = torch.randn(qkv[0].shape, generator=generator, device=device).to(torch.bfloat16)
        grads = [torch.empty_like(qkv[0]) for _ in range(3)]
        workspace = torch.empty(library().fk_flash_bwd_workspace_bytes(p1 - p0, seq) // 4, dtype=torch.float32,
                                device=device)

        def backward_step():
            check(library().fk_flash_bwd(qkv[0].data_ptr(), qkv[1].data_ptr(), qkv[2].data_ptr(), out.data_ptr(),
                                         d_out.data_ptr(), lse.data_ptr(), grads[0].data_ptr(), grads[1].data_ptr(),
                                         grads[2].data_ptr(), workspace.data_ptr(), p1 - p0, seq, 128 ** -0.5, causal,
                                         stream, flash_status.data_ptr()))

        backward_step()
        gemm.check_status(flash_status)
        leaves = [t[:1].float().requires_grad_() for t in qkv]
        torch.nn.functional.scaled_dot_product_attention(*[t.unsqueeze(0) for t in leaves]).backward(
            d_out[:1].float().unsqueeze(0))
        bwd_error = max(((g[:1].float() - leaf.grad).abs().max() / leaf.grad.abs().max()).item()
                        for g, leaf in zip(grads, leaves))
        if not bwd_error <= 2e-2:
            raise RuntimeError(f"flash backward disagrees with fp32 autograd: {bwd_error} of the largest gradient")
        timing = clock.measure(backward_step, 2.5 * flops_rank)
        gemm.check_status(flash_status)
        back = {"config": dict(config), "value": 2.5 * flops * args.steps / timing["seconds"] / 1e12, "unit": "TFLOP/s",
                "first_region_value": 2.5 * flops * args.steps / timing["first_s"] / 1e12,
                "flops_counted": "10 * planes * seq^2 * 128 (five tile products; seven are executed)",
                "ms_per_step": timing["seconds"] / args.steps * 1e3, "launch": timing["launch"],
                "max_error_over_max_gradient_vs_fp32_autograd": bwd_error}
        back["frac_of_measured_peak"] = back["value"] / world / peaks["burst"]
        return forward, back

    flash_fwd, flash_bwd = attention_block(FLASH, True)
    torch.cuda.empty_cache()
    flash_causal, _ = attention_block(FLASH_CAUSAL, False)
    torch.cuda.empty_cache()

    # ---- the row kernels either side of the two contractions: rows split across ranks, HBM roofline
    from ferro_kittens_b200 import rows as row_kernels
    from ferro_kittens_b200 import seeded

    rows_total = ROW_KERNEL_ROWS
    r0, r1 = shard.row_tiles(rows_total, world, rank)
    activations = seeded.bf16_rows("normal", ROW_KERNEL_SEED, 0, r0, r1 - r0, 128, 2.0, device=device, chunk_rows=1 << 17)
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
            off = (normalised[:4096].float().sum(dim=1) - 1).abs().max().item()
        elif name == "layernorm_rows":
            off = normalised[:4096].float().mean(dim=1).abs().max().item()
        else:
            off = abs(normalised[:128].float().mean().item())
        if not off <= 2e-2:
            raise RuntimeError(f"{name} fails its row property: {off}")
        timing = clock.measure(call)
        gbs = 4.0 * rows_total * 128 * args.steps / timing["seconds"] / 1e9
        row_results[name] = {"value": gbs, "unit": "GB/s", "ms_per_step": timing["seconds"] / args.steps * 1e3,
                             "launch": timing["launch"], "frac_of_measured_hbm": gbs / world / peaks["hbm"]}
    del activations, normalised

    if rank == 0:
        ratio = c2["interleaved"]["ratio_ours_over_cublaslt_at_median"]
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per_launch_s * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "m": M, "n": N, "k": K, "group": c2["config"]["group"],
                       "sharding": f"B split by N-column blocks over {world} rank(s), {n_local} columns each; "
                                   "A replicated; no collective",
                       "l2": "inputs (A 512 MiB + B shard) larger than the 126 MB L2; no flush between steps",
                       "generator": "counter-based (seed, tensor, index) -> Irwin-Hall(12) normal x 1/sqrt(K), bf16; "
                                    "every rank derives only its own shard",
                       "timed_region": f"the {args.steps} steps after {args.warmup} warm-up steps and "
                                       f"{c2_timing['conditioning_launches']} further back-to-back launches "
                                       f"(>= {args.settle} s on this kernel: the power-limited state)"},
            "first_region_value": c2["ours"]["first_region_value"],
            "launch": c2["ours"]["launch"],
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         # dram__bytes_read + write of one launch of this kernel on the full 16384^3 shape,
                         # the mean of six launches in one ncu capture at traversal width 6, scaled by the rank's share of N
                         "traffic": (8.11e9 + 0.669e9) * n_local / N, "traffic_unit": "bytes/launch",
                         "algorithmic_flops_per_launch": 2.0 * M * n_local * K,
                         "peak_source": f"{peaks['source']} ({'sustained' if sustained else 'burst'} cuBLAS bf16)",
                         "frac_of_measured_burst": achieved / peaks["burst"],
                         "frac_of_nominal_2250": achieved / 2250.0},
            "cublaslt": {"value": c2["cublaslt_alone"]["value"], "unit": "TFLOP/s",
                         "ratio_ours_over_cublaslt": ratio,
                         "ratio_definition": "median device time of cuBLASLt over ours, launches interleaved A B A B",
                         "ratio_at_min": c2["interleaved"]["ratio_ours_over_cublaslt_at_min"],
                         "ratio_of_settled_blocks": c2["ratio_ours_over_cublaslt_alone"],
                         "interleaved": c2["interleaved"], "ours_alone": c2["ours"], "cublaslt_alone": c2["cublaslt_alone"],
                         "max_abs_diff_vs_ours": c2["max_abs_diff_vs_cublaslt"]},
            "gemm_8192x28672x8192": {**c3, "value": c3["ours"]["value"], "unit": "TFLOP/s",
                                     "frac_of_measured_sustained_peak": c3["achieved_per_gpu"] / peaks["sustained"],
                                     "ratio_ours_over_cublaslt": c3["interleaved"]["ratio_ours_over_cublaslt_at_median"]},
            "flash_fwd": flash_fwd,
            "flash_fwd_causal": flash_causal,
            "flash_bwd": flash_bwd,
            "row_kernels": {"config": {"rows": rows_total, "columns": 128, "seed": ROW_KERNEL_SEED,
                                       "bytes_per_element": 4, "sharding": f"rows over {world} rank(s)"},
                            "peak": peaks["hbm"], "peak_unit": "GB/s", "peak_source": peaks["source"], **row_results},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_seconds / e2e_steps * 1e3, "call": e2e_call,
                    "blocks_of_c": f"1 x {world} (column blocks of B; A uploaded once across the ranks and "
                                   "completed in each GPU's memory by all-gather)" if world > 1 else "1 x 1"},
            "gpu_launches": args.steps,
            "clocks": clocks,
        }
        if cpu_baseline:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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


def run_only(args, local_rank: int) -> None:
    """One kernel alone on a chosen size: the command an ncu capture wraps."""
    import torch

    from ferro_kittens_b200 import gemm
    from ferro_kittens_b200._lib import check, library

    asked_group = args.group
    args.group = args.group or gemm.GROUP
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
        maps = gemm.TiledMaps(a, b, c, columns=args.item_columns or None)
        flags = (gemm.TILE_WIDE if args.item_columns else 0) | {"": 0, "feed": gemm.ORDER_FEED, "static": gemm.ORDER_STATIC}[args.order]
        group = asked_group or gemm.group_for(m, n, device)
        fn = lambda: gemm.launch_tiled(maps, m, n, k, group, status, flags=flags)  # noqa: E731
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
    if args.only == "gemm":
        line["item_columns"] = maps.columns
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
    parser.add_argument("--item-columns", type=int, default=0, choices=[0, 256, 224, 192],
                        help="with --only gemm: force the wide kernel with items this many columns wide (0: the launch chooses)")
    parser.add_argument("--order", default="", choices=["", "feed", "static"],
                        help="with --only gemm: how the wide kernel's clusters get their items (default: the launch chooses)")
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
    parser.add_argument("--group", type=int, default=0, help="traversal width of the GEMM's item walk (0: the library's default)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--settle", type=float, default=0.5,
                        help="seconds of back-to-back launches before the timed K steps of every block")
    parser.add_argument("--gather-blocks", type=int, default=4,
                        help="row blocks per rank of the all-gathered A in the multi-GPU host-buffer leg")
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

#!/usr/bin/env python
"""Benchmark of the znn MatMul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--n 8192] [--impl reference]

A "step" is one pass of the reference's MatMul operator over one batch of
synthetic N(0,1) operands: forward C = A.B (src/autodiff.zig:110-133) and the two
backward products dA += dC.B^T, dB += A^T.dC (:593-641), all through znn_sgemm,
the cblas_sgemm boundary.  The metric is fp32-accurate GEMM TFLOP/s = 3*2*n^3 / t.

N > 1 (launched by torchrun, one rank per GPU): the sweep has no exchange step,
so every rank runs an independent replica ("replicas only"); the value is the sum
over ranks divided by the slowest rank's time.

--impl reference times the reference's CPU path for the same step: the oracle's
restatement of the MatMul arms with cblas_sgemm bound to the host OpenBLAS (all
host threads), on a bounded sample size.

The default run (--workload all) prints ONE JSON line: the MatMul step (value, roofline of the tensor-core kernel,
e2e through znn_matmul_host_fwd_bwd with pinned host tensors, cpu_baseline, clocks) with a "gpt" object inside
(GPT training step of the workload definition, tokens/s).  Other workloads, one JSON line each:
  --workload matmul | gpt   one of the two parts alone (used for profiler captures)
  --workload attention      the fused causal-attention kernels at the sizes of configs 5 and 4 (--small: one size, few launches)
  --workload conv           the Conv2D entry points at the padded CNN's layer shapes, both paths (--small: few launches)
  --workload cnn_dp         the padded CNN step, global batch 256 split over the ranks (data parallel, strong scaling)
  --workload sweep          every shape of the MatMul sweep, forward and both backward products
  --workload configs        MLP / CNN / transformer-block / greedy-decode configurations
  --workload rowops         HBM bandwidth of the row-wise kernels
  --workload shape --shape M,N,K,ta,tb,batch [--path P]   one (batched) product, for small-case captures
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fp32_accurate_gemm_tflops"
UNIT = "TFLOP/s"


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def wait_first_sample(self, limit_s=5.0):
        """nvidia-smi needs a moment to start; a short timed region would otherwise end before its first line."""
        t_end = time.time() + limit_s
        while self.proc and not self.lines and time.time() < t_end:
            time.sleep(0.01)

    def stop(self, window=None):
        """window = (t0, t1) host times of the timed region: only samples inside it count; where the region was
        shorter than two sampling periods, the samples of the warm-up (the same work) are used and the result says so."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        scope, lines = "whole run", [ln for _, ln in self.lines]
        if window:
            inside = [ln for t, ln in self.lines if window[0] <= t <= window[1]]
            scope, lines = ("timed region", inside) if len(inside) >= 2 else ("warm-up and timed region", lines)
        sm, mx, power, reasons = [], [], [], set()
        for ln in lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "sampled_over": scope,
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU side
def cpu_step(zo, A, B, dC, Cm, dA, dB, n):
    zo.sgemm(111, 111, n, n, n, 1.0, A, n, B, n, 0.0, Cm, n)
    zo.sgemm(111, 112, n, n, n, 1.0, dC, n, B, n, 1.0, dA, n)
    zo.sgemm(112, 111, n, n, n, 1.0, A, n, dC, n, 1.0, dB, n)


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def set_blas_threads(info, n):
    """The CPU arm uses every host core whatever OMP_NUM_THREADS the launcher exported (torchrun sets it to 1)."""
    h = info.get("handle")
    for sym in ("scipy_openblas_set_num_threads", "openblas_set_num_threads", "goto_set_num_threads"):
        if h is not None and hasattr(h, sym):
            getattr(h, sym)(C.c_int(n))
            for gsym in ("scipy_openblas_get_num_threads", "openblas_get_num_threads"):
                if hasattr(h, gsym):
                    return int(getattr(h, gsym)())
            return n
    return info.get("threads") or 1


def cpu_measure(steps, warmup, n=8192, budget_s=25.0, with_naive=True):
    """Times the oracle's MatMul step (forward + dA + dB at size n, the GPU arm's own workload) on the host cores.
    The sample is bounded in the number of steps, never in n: after the first step the step count is cut so that the
    run fits budget_s."""
    import numpy as np
    from oracle import zo
    zo.build()
    ptr, info = zo.find_host_cblas()
    out = {"kind": "port", "unit": UNIT}
    r = np.random.default_rng(0)
    naive = None
    if with_naive:
        # the reference's Linux code path: the naive loops of src/cblas.zig:37-96, one thread
        m = 768
        A, B = r.standard_normal((m, m), np.float32), r.standard_normal((m, m), np.float32)
        Cm = np.zeros((m, m), np.float32)
        zo.bind_sgemm(None)
        t0 = time.perf_counter()
        zo.sgemm(111, 111, m, m, m, 1.0, A, m, B, m, 0.0, Cm, m)
        naive = 2.0 * m ** 3 / (time.perf_counter() - t0) / 1e12
        out["naive_fallback_1thread_tflops"] = naive
        out["naive_sample"] = f"{m}^3 forward product, 1 thread (src/cblas.zig:37-96 restated)"
    if ptr is None:
        out.update({"value": naive, "cores": 1, "sample": out.get("naive_sample", ""), "blas": "none found", "n": 768})
        return out
    zo.bind_sgemm(ptr)
    cores = set_blas_threads(info, host_cores())
    A, B, dC = (r.standard_normal((n, n), np.float32) for _ in range(3))
    Cm, dA, dB = (np.zeros((n, n), np.float32) for _ in range(3))
    t0 = time.perf_counter()
    cpu_step(zo, A, B, dC, Cm, dA, dB, n)              # first step: untimed warm-up, and the measure for the cut
    t_first = time.perf_counter() - t0
    warm_run = 1
    max_total = max(2, int(budget_s / max(t_first, 1e-3)))
    while warm_run < warmup and warm_run + 1 < max_total:
        cpu_step(zo, A, B, dC, Cm, dA, dB, n)
        warm_run += 1
    steps_run = max(1, min(steps, max_total - warm_run))
    t0 = time.perf_counter()
    for _ in range(steps_run):
        cpu_step(zo, A, B, dC, Cm, dA, dB, n)
    dt = time.perf_counter() - t0
    zo.bind_sgemm(None)
    out.update({"value": 6.0 * n ** 3 * steps_run / dt / 1e12, "cores": int(cores), "ms_per_step": dt / steps_run * 1e3,
                "sample": f"{steps_run} timed steps (of {steps} asked; {warm_run} warm-up) of fwd+dA+dB at n={n}, the GPU arm's own "
                          f"size; cblas_sgemm = {os.path.basename(info['path'])} with {cores} threads on {host_cores()} host cores",
                "n": n, "steps_run": steps_run, "warmup_run": warm_run})
    return out


def gpt_cpu_measure(V, T, D, H, B, n_layer_full):
    """One training step of the GPT configuration on the CPU oracle (literal reference op sequence, cblas_sgemm bound to
    the host OpenBLAS with all cores, everything else the restated scalar loops on one thread).  Bounded sample: ONE
    layer at full width, context and vocabulary; the full model's time is that of the sample scaled by the flop ratio."""
    import numpy as np
    from oracle import models, zo
    ptr, info = zo.find_host_cblas()
    if ptr is None:
        return {"kind": "port", "unavailable": "no host CBLAS found for the oracle"}
    zo.bind_sgemm(ptr)
    cores = set_blas_threads(info, host_cores())
    cfg = {"vocab_size": V, "block_size": T, "n_embd": D, "n_head": H, "n_layer": 1}
    P0 = models.init_params("gpt", cfg, seed=1, scheme="n002")
    r = np.random.default_rng(2)
    x = r.integers(0, V, (B, T)).astype(np.float32)
    t = r.integers(0, V, B * T).astype(np.int32)
    tr = models.OracleTrainer("gpt", P0, cfg, lr=0.01, momentum=0.9)
    t0 = time.perf_counter()
    tr.step(x, t)
    dt = time.perf_counter() - t0
    zo.bind_sgemm(None)
    layer = 3 * 2.0 * B * T * (4 * D * D + 8 * D * D + 2 * T * D)     # projections, FFN, attention (full square)
    head = 3 * 2.0 * B * T * D * V
    ratio = (n_layer_full * layer + head) / (layer + head)
    return {"kind": "port", "unit": "tokens/s", "cores": int(cores), "value": B * T / (dt * ratio),
            "sample_tokens_per_s": B * T / dt, "sample_s": dt,
            "sample": f"one training step of a 1-layer model at full width (d_model {D}, context {T}, vocab {V}, batch {B}); "
                      f"value = the sample's rate divided by the flop ratio {ratio:.2f} of the {n_layer_full}-layer model; "
                      f"sgemm = OpenBLAS with {cores} threads, other ops scalar on one thread"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    t_wall = time.perf_counter()
    res = cpu_measure(steps, warmup, n=args.n, budget_s=150.0, with_naive=True)
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": res.get("steps_run", steps), "warmup": res.get("warmup_run", warmup), "steps_asked": steps,
        "ms_per_step": res.get("ms_per_step"), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"matmul_sweep_square_{args.n}_fwd_dA_dB", "M": res.get("n"), "N": res.get("n"), "K": res.get("n"),
                   "note": "CPU path of the reference restated in C (oracle port; the reference is Zig and cannot be built "
                           "here), cblas_sgemm bound to the host OpenBLAS with every host core"},
        "cpu_baseline": {k: res[k] for k in res if k in ("value", "unit", "cores", "kind", "sample",
                                                         "naive_fallback_1thread_tflops", "naive_sample")},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t_wall,
    }
    print(json.dumps(line), flush=True)
    return 0


# --------------------------------------------------------------------------- GPU side
def run_gpu(args):
    import torch
    import torch.distributed as dist
    from znn_b200._lib import lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the znn_b200 hot path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = lib()
    L.call("znn_init", local)
    # a non-default stream, so that torch's events and the shim's kernels share it
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    L.call("znn_set_stream", stream.cuda_stream)

    if args.workload == "shape":
        if rank == 0:
            print(json.dumps({"metric": "gemm_shape_tflops", "n_gpus": 1, "data": "synthetic",
                              "product": shape_part(args, L, torch, stream)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0
    if args.workload == "sweep":
        if rank == 0:
            print(json.dumps({"metric": "fp32_accurate_gemm_tflops_per_shape", "unit": "TFLOP/s", "n_gpus": 1,
                              "data": "synthetic", "sweep": sweep_part(args, L, torch, stream)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0
    if args.workload == "rowops":
        if rank == 0:
            print(json.dumps({"metric": "rowop_hbm_bandwidth", "n_gpus": 1, "data": "synthetic",
                              "rowops": rowops_part(args, L, torch, stream)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0
    if args.workload == "configs":
        if rank == 0:
            print(json.dumps({"metric": "config_timings", "n_gpus": 1, "data": "synthetic",
                              "configs": configs_part(args, L, torch, stream)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0
    if args.workload in ("attention", "conv"):
        part = attention_part(args, L, torch, stream) if args.workload == "attention" else conv_part(args, L, torch, stream)
        if rank == 0:
            print(json.dumps({"metric": args.workload + "_kernels", "n_gpus": 1, "data": "synthetic", "dtype": "f32 (3xTF32)",
                              args.workload: part}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0
    if args.workload == "cnn_dp":       # the data-parallel CNN step alone
        cnn = cnn_dp_part(args, L, torch, dist, stream, world, rank)
        if rank == 0:
            cnn.update({"higher_is_better": True, "vs_baseline": None, "dtype": "f32", "data": "synthetic"})
            print(json.dumps(cnn), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0
    if args.workload == "gpt":          # the GPT training step alone (used for profiling captures)
        gpt = gpt_part(args, L, torch, dist, stream, world, rank, local)
        if rank == 0:
            gpt.update({"higher_is_better": True, "vs_baseline": None, "dtype": "f32 (3xTF32 GEMMs)", "data": "synthetic"})
            print(json.dumps(gpt), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0

    n = args.n
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    A = torch.randn((n, n), device="cuda", generator=g, dtype=torch.float32)
    B = torch.randn((n, n), device="cuda", generator=g, dtype=torch.float32)
    dC = torch.randn((n, n), device="cuda", generator=g, dtype=torch.float32)
    Cm = torch.empty((n, n), device="cuda", dtype=torch.float32)
    dA = torch.zeros((n, n), device="cuda", dtype=torch.float32)
    dB = torch.zeros((n, n), device="cuda", dtype=torch.float32)
    L.call("znn_gemm_workspace_reserve", 4 * 2 * n * n * 4 + (1 << 20))

    def step():
        L.call("znn_sgemm", 101, 111, 111, n, n, n, 1.0, A.data_ptr(), n, B.data_ptr(), n, 0.0, Cm.data_ptr(), n)
        L.call("znn_sgemm", 101, 111, 112, n, n, n, 1.0, dC.data_ptr(), n, B.data_ptr(), n, 1.0, dA.data_ptr(), n)
        L.call("znn_sgemm", 101, 112, 111, n, n, n, 1.0, A.data_ptr(), n, dC.data_ptr(), n, 1.0, dB.data_ptr(), n)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        sampler.wait_first_sample()
    for _ in range(warmup):
        step()
    barrier()
    cnt = C.c_longlong(0)
    L.call("znn_launch_count", C.byref(cnt), 1)
    L.call("znn_gemm_profile", 1)
    t_host0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop((t_host0, time.time())) if rank == 0 else None
    L.call("znn_launch_count", C.byref(cnt), 1)
    launches = cnt.value
    kms, kl, kfl = C.c_double(0), C.c_longlong(0), C.c_double(0)
    L.call("znn_gemm_profile_read", C.byref(kms), C.byref(kl), C.byref(kfl))
    L.call("znn_gemm_profile", 0)
    last_path = L.dll.znn_gemm_last_path()
    st = C.c_int(0)
    L.call("znn_device_status", C.byref(st), 1)
    if st.value:
        raise SystemExit(f"device status word {st.value}: a bounded device-side wait expired; the run is invalid")
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    flops_step = 6.0 * n ** 3
    value = world * flops_step * steps / (ms_max * 1e-3) / 1e12

    # ---- end to end: host tensors in, host tensors out, ONE call of the host-operand entry point.
    # The shim pipelines the three uploads, the three products and the three downloads by panels.
    hA, hB, hdC = (torch.empty((n, n), dtype=torch.float32).pin_memory() for _ in range(3))
    hC, hdA, hdB = (torch.empty((n, n), dtype=torch.float32).pin_memory() for _ in range(3))
    hA.copy_(A)
    hB.copy_(B)
    hdC.copy_(dC)
    nbytes = n * n * 4

    def e2e_step():
        # gradients start from zero (after zeroGrad), so accumulate = 0 writes them without uploading zeros
        L.call("znn_matmul_host_fwd_bwd", hA.data_ptr(), hB.data_ptr(), hdC.data_ptr(), hC.data_ptr(),
               hdA.data_ptr(), hdB.data_ptr(), n, n, n, 0, 0)

    for _ in range(2):
        e2e_step()
    barrier()
    e2e_steps = steps    # the same count as the device-resident figure
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()       # returns when its results are in host memory
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = world * flops_step * e2e_steps / (float(t.item()) * 1e-3) / 1e12
    # spot check of the pipelined results against the device-resident products of the same inputs
    L.call("znn_sgemm", 101, 111, 111, n, n, n, 1.0, A.data_ptr(), n, B.data_ptr(), n, 0.0, Cm.data_ptr(), n)
    torch.cuda.synchronize()
    sl = slice(n - 256, n)
    ref_rows = Cm[sl].cpu()
    e2e_check = float((hC[sl] - ref_rows).norm() / ref_rows.norm())
    if not e2e_check <= 1e-5:
        raise SystemExit(f"end-to-end result differs from the device-resident product: {e2e_check}")

    tf32_live = None
    if rank == 0 and world == 1:
        # context only: the library TF32 GEMM rate on this GPU right now (one pass, not 3xTF32)
        torch.backends.cuda.matmul.allow_tf32 = True
        for _ in range(3):
            torch.matmul(A, B, out=Cm)
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(5):
            e0.record(stream)
            torch.matmul(A, B, out=Cm)
            e1.record(stream)
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        tf32_live = 2.0 * n ** 3 / (best * 1e-3) / 1e12
        torch.backends.cuda.matmul.allow_tf32 = False

    gpt = sweep = configs = cnn = None
    if args.workload == "all":
        gpt = gpt_part(args, L, torch, dist, stream, world, rank, local)
        cnn = cnn_dp_part(args, L, torch, dist, stream, world, rank)
        if world == 1:
            # the other shapes and configurations of the workload definition, compact, in the same record
            peaks_now, _ = read_peaks()
            sweep = sweep_compact(sweep_part(args, L, torch, stream), peaks_now)
            configs = configs_compact(configs_part(args, L, torch, stream), peaks_now)

    if rank == 0:
        peaks, peaks_kind = read_peaks()
        # 3xTF32 ceiling: the TF32 dense rate is half the bf16 rate on this part, and each algorithmic flop costs
        # three tensor-core passes.  The timed region lasts a fraction of a second, so the denominator is the BURST
        # measured bf16 rate; the fraction of the sustained (seconds-long, power-capped) rate is given beside it.
        peak = peaks["bf16_tflops"] / 2.0 / 3.0
        peak_sustained = peaks["bf16_tflops_sustained"] / 2.0 / 3.0
        achieved = (kfl.value / (kms.value * 1e-3) / 1e12) if kms.value > 0 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_max / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 (3xTF32 split, fp32 accumulate)", "data": "synthetic",
            "config": {"workload": f"matmul_sweep_square_{n}_fwd_dA_dB", "M": n, "N": n, "K": n,
                       "flops_per_step": flops_step, "l2": "inputs (3 x %d MB) exceed the 126 MB L2" % (nbytes >> 20),
                       "parallelism": "replicas only" if world > 1 else "single GPU"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": UNIT,
                         "frac": (achieved / peak) if achieved else None,
                         "traffic": 2.714e9 if (n == 8192 and last_path == 4) else None,
                         "traffic_source": "DRAM bytes per launch from a one-pass ncu capture of this workload (committed "
                                           "summary); not measured in this run",
                         "algorithmic_bytes_per_launch": (3 + 4 + 4) * nbytes / 3.0,
                         "kernel": ("gemm3x_direct_kernel<256,*,*> (operands read in place)" if last_path == 4
                                    else "gemm3x_tf32_kernel<256,2> (pre-split operand planes)"),
                         "launches": kl.value,
                         "avg_launch_ms": (kms.value / kl.value) if kl.value else None,
                         "peak_source": f"{peaks_kind}: bf16 burst {peaks['bf16_tflops']} TF/s / 2 (tf32) / 3 (passes)",
                         "peak_sustained": peak_sustained,
                         "frac_of_sustained_peak": (achieved / peak_sustained) if achieved else None,
                         "cublas_tf32_live_tflops": tf32_live,
                         "frac_of_live_cublas_tf32_third": (achieved / (tf32_live / 3.0)) if (achieved and tf32_live) else None},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 3 * nbytes, "d2h_bytes_per_step": 3 * nbytes,
                    "steps": e2e_steps, "call": "znn_matmul_host_fwd_bwd (pinned host tensors; copies and panels pipelined)"},
            "gpu_launches": launches, "clocks": clocks,
        }
        if gpt is not None:
            line["gpt"] = gpt
        if cnn is not None:
            line["cnn"] = cnn
        if sweep is not None:
            line["sweep"] = sweep
        if configs is not None:
            line["configs"] = configs
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = {k: v for k, v in cpu_measure(3, 1, n=n, budget_s=20.0).items()
                                    if k not in ("n", "steps_run", "warmup_run")}
            if gpt is not None:
                gpt["cpu_baseline"] = gpt_cpu_measure(8192, 1024, 768, 12, 8, 6)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def dp_init(L, torch, dist, world, rank):
    """One NCCL communicator per rank for the shim's gradient exchange; the 128-byte id travels over torch.distributed."""
    if world <= 1:
        return
    uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        buf = C.create_string_buffer(128)
        L.call("znn_dp_unique_id", buf)
        uid.copy_(torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8))
    dist.broadcast(uid, src=0)
    torch.cuda.synchronize()
    L.call("znn_dp_init", world, rank, bytes(uid.cpu().numpy().tobytes()))


def param_checksum(m):
    """A position-sensitive checksum of every parameter's bit pattern (below 2^52, so that it survives a float64)."""
    import numpy as np
    P = m.get_params()
    h = 0
    for name in sorted(P):
        a = np.ascontiguousarray(P[name]).view(np.uint32).astype(np.uint64)
        h = (h * 1000003 + int(a.sum() % (1 << 61)) + int((a[::7] * np.uint64(2654435761)).sum() % (1 << 61))) % (1 << 61)
    return h % (1 << 52)


def cnn_dp_part(args, L, torch, dist, stream, world, rank):
    """Config 3 data parallel (strong scaling): the padded CNN (1->32->64 3x3 pad 1, 3136->128->10) on a GLOBAL batch of
    256 images split evenly over the ranks, gradients summed by NCCL and applied with 1/world.  Self-check printed with
    the numbers: replicas bit-identical after the timed steps, and the loss of the first five steps equal (1e-4) to the
    same model trained on the whole batch by one GPU."""
    import numpy as np
    from znn_b200.models import Model
    G = 256
    if G % world:
        return {"unavailable": f"global batch {G} does not split over {world} ranks"}
    Bper = G // world
    r = np.random.default_rng(5)                          # the same on every rank
    steps_check = 5
    X = (r.integers(0, 256, (steps_check, G, 784)).astype(np.float32) / np.float32(255.0))
    Y = r.integers(0, 10, (steps_check, G)).astype(np.int32)

    def fresh():
        m = Model("cnn_padded", (), arena_bytes=2 << 30)
        rr = np.random.default_rng(6)
        P = {}
        for name, shape, _, fan_in in m.params:
            P[name] = ((rr.standard_normal(shape, np.float32) * np.float32((2.0 / fan_in) ** 0.5)) if fan_in
                       else np.zeros(shape, np.float32))
        m.set_params(P)
        m.set_option("lr", 0.01)
        m.set_option("momentum", 0.9)
        return m

    dp_init(L, torch, dist, world, rank)
    m = fresh()
    sl = slice(rank * Bper, (rank + 1) * Bper)
    dp_losses = []
    for s in range(steps_check):
        local = m.train_step(X[s, sl], Y[s, sl])
        t = torch.tensor([local], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t)
        dp_losses.append(float(t.item()) / world)
    dx, dt = torch.from_numpy(X[0, sl].copy()).cuda(), torch.from_numpy(Y[0, sl].copy()).cuda()
    steps, warmup = 100, 10
    for _ in range(warmup):
        m.train_step_device(dx.data_ptr(), dt.data_ptr(), Bper)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        m.train_step_device(dx.data_ptr(), dt.data_ptr(), Bper)
    e1.record(stream)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    h = torch.tensor([float(param_checksum(m))], device="cuda", dtype=torch.float64)
    lo, hi = h.clone(), h.clone()
    if world > 1:
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    identical = bool(lo.item() == hi.item())
    m.close()
    if world > 1:
        L.call("znn_dp_finalize")
    m1 = fresh()                                          # the same five steps on the whole batch, one GPU, no exchange
    single = [m1.train_step(X[s], Y[s]) for s in range(steps_check)]
    m1.close()
    worst = max(abs(a - b) / abs(b) for a, b in zip(dp_losses, single))
    if not identical or worst > 1e-4:
        raise SystemExit(f"CNN data-parallel parity check failed: replicas identical {identical}, loss rel diff {worst:.3e}")
    return {"metric": "cnn_train_images_per_s", "value": G * steps / (ms * 1e-3), "unit": "images/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "scaling": "strong",
            "config": {"workload": "cnn_padded_train_step", "global_batch": G, "per_gpu_batch": Bper, "parallelism": f"dp{world}",
                       "optimizer": "SGD momentum 0.9"},
            "dp_parity": {"replicas_bit_identical": identical, "loss_max_rel_diff_vs_single_gpu": worst, "steps": steps_check,
                          "bar": 1e-4, "passed": True}}


def sweep_compact(rows, peaks):
    """One entry per sweep shape: microseconds and TFLOP/s of the three products, and the fraction of the bound that
    applies: the 3xTF32 tensor ceiling (burst) for the square shapes, the HBM time of the operands for the skinny ones."""
    ceiling = peaks["bf16_tflops"] / 2.0 / 3.0
    out = {}
    for row in rows:
        M, N, K = row["M"], row["N"], row["K"]
        hbm_us = row["operand_MB"] * 1e6 / (peaks["hbm_gbs"] * 1e9) * 1e6
        skinny = min(M, N) <= 64
        e = {}
        for k in ("fwd_NN", "dA_NT", "dB_TN"):
            e[k] = {"us": round(row[k]["us"], 1), "tflops": round(row[k]["tflops"], 1),
                    "frac": round((hbm_us / row[k]["us"]) if skinny else (row[k]["tflops"] / ceiling), 3)}
        e["bound"] = ("hbm: operand bytes / measured copy bandwidth" if skinny else
                      ("tensor (3xTF32 burst ceiling); launch-bound below 1024^3" if max(M, N, K) < 1024 else "tensor (3xTF32 burst ceiling)"))
        e["l2_resident"] = row["l2_resident"]
        out[f"{M}x{N}x{K}"] = e
    return out


def configs_compact(cfgs, peaks):
    ceiling = peaks["bf16_tflops"] / 2.0 / 3.0
    out = {}
    for k, v in cfgs.items():
        if "us_per_step" in v:
            out[k] = {"us_per_step": round(v["us_per_step"], 1), "cuda_graph_us_per_step": round(v["cuda_graph_us_per_step"], 1),
                      "e2e_us_per_step": round(v["e2e_us_per_step"], 1), "bound": v.get("bound", "launch-bound")}
            if "tflops" in v:
                out[k]["tflops"] = round(v["tflops"], 2)
        elif "ms_fwd_bwd" in v:
            out[k] = {"ms_fwd_bwd": round(v["ms_fwd_bwd"], 3), "tflops": round(v["tflops"], 1),
                      "frac": round(v["tflops"] / ceiling, 3), "bound": "tensor (3xTF32 burst ceiling)",
                      "ms_fwd_bwd_incl_host_copies": round(v["ms_fwd_bwd_incl_host_copies"], 2)}
        elif "tokens_per_s" in v:
            out[k] = {kk: v[kk] for kk in v if kk != "note"}
            out[k]["bound"] = "launch-bound (about 200 launches per position, batch 64)"
        else:
            out[k] = {kk: (round(vv, 1) if isinstance(vv, float) else vv) for kk, vv in v.items() if kk != "note"}
    return out


def gpt_part(args, L, torch, dist, stream, world, rank, local):
    """GPT training step of examples/transformer_gpt.zig at the workload definition's size (vocab 8192, 6 layers,
    d_model 768, 12 heads, FFN 3072, context 1024, per-GPU batch 8), data parallel over the ranks: every rank
    trains on its own 8 x 1024 tokens, gradients are summed by NCCL (overlapped with backward) and applied with
    1/world.  Returns tokens/s over all ranks (weak scaling)."""
    import numpy as np
    from znn_b200.models import Model

    V, T, D, H, NL, B = 8192, 1024, 768, 12, 6, 8
    dp_init(L, torch, dist, world, rank)
    m = Model("gpt", (V, T, D, H, NL), arena_bytes=30 << 30)
    r = np.random.default_rng(42)                       # the same seed on every rank: identical replicas
    P = {}
    for name, shape, _, fan_in in m.params:
        if fan_in:
            P[name] = (r.standard_normal(shape, np.float32) * np.float32(0.02))
        else:
            P[name] = np.ones(shape, np.float32) if "ln_" in name else np.zeros(shape, np.float32)
    m.set_params(P)
    del P
    m.set_option("lr", 0.01)
    m.set_option("momentum", 0.9)
    if os.environ.get("ZNN_BENCH_FUSED_EPILOGUE"):      # A/B of the epilogue forms (bit mask, see znn_host.h)
        m.set_option("fused_epilogue", int(os.environ["ZNN_BENCH_FUSED_EPILOGUE"]))
    if args.dp_bucket_mb > 0:
        m.set_option("dp_bucket_floats", args.dp_bucket_mb * (1 << 20) // 4)
    rr = np.random.default_rng(1000 + rank)             # each rank its own shard of the global batch
    ids = rr.integers(0, V, (B, T)).astype(np.float32)
    tgt = np.concatenate([ids[:, 1:], rr.integers(0, V, (B, 1))], axis=1).astype(np.int32)
    d_ids = torch.from_numpy(ids).cuda()
    d_tgt = torch.from_numpy(tgt).cuda()
    steps, warmup = max(1, min(args.steps, 20)), 3

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        m.train_step_device(d_ids.data_ptr(), d_tgt.data_ptr(), B, T)
    barrier()
    cnt = C.c_longlong(0)
    L.call("znn_launch_count", C.byref(cnt), 1)
    L.call("znn_gemm_profile", 1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        m.train_step_device(d_ids.data_ptr(), d_tgt.data_ptr(), B, T)
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    L.call("znn_launch_count", C.byref(cnt), 1)
    kms, kl, kfl = C.c_double(0), C.c_longlong(0), C.c_double(0)
    L.call("znn_gemm_profile_read", C.byref(kms), C.byref(kl), C.byref(kfl))
    L.call("znn_gemm_profile", 0)
    eager_ms = ms
    replayed = False
    if world == 1 and not os.environ.get("ZNN_BENCH_NO_GRAPH"):
        # One GPU: the step uploads nothing, so it is captured once into a CUDA graph and replayed (the same kernels in
        # the same order, bit-identical results: tests/test_gpu_models.py); the eager figure above stays in the line.
        m.set_option("cuda_graph", 1)
        for _ in range(warmup + 2):              # eager sizing step, capture, replays
            m.train_step_device(d_ids.data_ptr(), d_tgt.data_ptr(), B, T)
        barrier()
        replayed = m.graph_replays() > 0
        if replayed:
            e0.record(stream)
            for _ in range(steps):
                m.train_step_device(d_ids.data_ptr(), d_tgt.data_ptr(), B, T)
            e1.record(stream)
            barrier()
            ms = float(e0.elapsed_time(e1))
        m.set_option("cuda_graph", 0)
    # end to end: token ids and targets from host memory every step, loss read back every step
    loss = m.train_step(ids, tgt, seq=T)
    barrier()
    e2e_steps = steps            # the same count as the device-resident figure: both see the same clock behaviour
    e0.record(stream)
    for _ in range(e2e_steps):
        loss = m.train_step(ids, tgt, seq=T)
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    st = C.c_int(0)
    L.call("znn_device_status", C.byref(st), 1)
    if st.value:
        rec = (C.c_int * 16)()
        L.call("znn_gemm_wait_record", rec)
        raise SystemExit(f"device status word {st.value} during the GPT step; the run is invalid; first expired wait: {list(rec)}")
    out = {
        "metric": "gpt_train_tokens_per_s", "value": world * B * T * steps / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "scaling": "weak",
        "config": {"workload": "gpt_train_step", "vocab": V, "n_layer": NL, "d_model": D, "n_head": H, "ffn": 4 * D,
                   "context": T, "per_gpu_batch": B, "global_batch": B * world, "head": "untied Linear with bias",
                   "norm": "RMSNorm", "optimizer": "SGD momentum 0.9", "parallelism": f"dp{world}",
                   "params": sum(int(np.prod(sh)) for _, sh, _, _ in m.params)},
        "e2e": {"value": world * B * T * e2e_steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": ids.nbytes + tgt.nbytes, "d2h_bytes_per_step": 4, "steps": e2e_steps},
        "gpu_launches": cnt.value, "tape_ops": m.last_step_ops(), "last_loss": loss,
        "cuda_graph_replay": replayed, "eager_ms_per_step": eager_ms / steps,
        "launch_note": ("kernels of the eager pass of the same steps; the timed steps replay the same kernels from one "
                        "captured graph" if replayed else "kernels launched in the timed steps"),
        "arena_high_water_gb": m.arena_high_water() / 2 ** 30,
        "tensor_core_gemm": {"launches": kl.value, "kernel_ms_per_step": kms.value / steps,
                             "tflops": (kfl.value / (kms.value * 1e-3) / 1e12) if kms.value > 0 else None,
                             "share_of_step": (kms.value / ms) if ms > 0 else None},
        "model_flops_per_token": 349e6,
    }
    if world > 1:
        out["dp_parity"] = dp_parity_check(L, torch, dist, m, world, rank)
    m.close()
    if world > 1:
        L.call("znn_dp_finalize")
        out["dp_parity"].update(dp_small_model_check(L, torch, dist, world, rank, phase="single", carry=out["dp_parity"]))
    return out


def dp_parity_check(L, torch, dist, m, world, rank):
    """Self-check of the data-parallel run, printed with the numbers: (1) after the timed steps every rank must hold
    bit-identical parameters (same initial replica, same summed gradients, same update): a checksum of the parameter
    slab is min- and max-reduced over the ranks; (2) a small GPT trained for a few steps with the batch sharded over
    the ranks must follow the loss of the same model trained on the whole batch by one GPU (second half of the check
    runs after the communicator is gone: dp_small_model_check(phase='single'))."""
    h = param_checksum(m)
    t = torch.tensor([float(h % (1 << 52))], device="cuda", dtype=torch.float64)
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    res = {"replicas_bit_identical": bool(lo.item() == hi.item()), "param_checksum": int(lo.item())}
    if not res["replicas_bit_identical"]:
        raise SystemExit("data-parallel parity check failed: the ranks' parameter replicas differ after the timed steps")
    res.update(dp_small_model_check(L, torch, dist, world, rank, phase="dp"))
    return res


def dp_small_model_check(L, torch, dist, world, rank, phase, carry=None):
    import numpy as np
    from znn_b200.models import Model
    V, T, D, H, NL, Bper, steps = 96, 128, 128, 2, 2, 2, 5
    dims = (V, T, D, H, NL)
    r = np.random.default_rng(7)                         # the same on every rank
    Bg = Bper * world
    ids = r.integers(0, V, (steps, Bg, T)).astype(np.float32)
    tgt = r.integers(0, V, (steps, Bg, T)).astype(np.int32)
    m = Model("gpt", dims, arena_bytes=1 << 30)
    P = {}
    for name, shape, _, fan_in in m.params:
        P[name] = (r.standard_normal(shape, np.float32) * np.float32(0.05)) if fan_in else (
            np.ones(shape, np.float32) if "ln_" in name else np.zeros(shape, np.float32))
    m.set_params(P)
    m.set_option("lr", 0.05)
    m.set_option("momentum", 0.9)
    if phase == "dp":
        losses = []
        for s in range(steps):
            sl = slice(rank * Bper, (rank + 1) * Bper)
            local = m.train_step(ids[s, sl], tgt[s, sl], seq=T)
            t = torch.tensor([local], device="cuda", dtype=torch.float64)
            dist.all_reduce(t)                           # mean of equal shards' mean losses = the global mean loss
            losses.append(float(t.item()) / world)
        Pf = m.get_params()
        m.close()
        return {"small_gpt_dp_losses": losses, "_small_params": Pf}
    losses = [m.train_step(ids[s], tgt[s], seq=T) for s in range(steps)]
    Pf = m.get_params()
    m.close()
    dp_losses, dp_params = carry["small_gpt_dp_losses"], carry.pop("_small_params")
    worst = max(abs(a - b) / abs(b) for a, b in zip(dp_losses, losses))
    scale = max(float(np.abs(v).max()) for v in Pf.values())
    perr = max(float(np.abs(Pf[k] - dp_params[k]).max()) for k in Pf) / scale
    ok = worst <= 1e-4 and perr <= 1e-4
    if not ok:
        raise SystemExit(f"data-parallel parity check failed: loss rel {worst:.3e}, params {perr:.3e} of scale")
    return {"small_gpt_single_gpu_losses": losses, "small_gpt_loss_max_rel_diff": worst,
            "small_gpt_param_max_diff_of_scale": perr, "small_gpt_config": {"vocab": V, "context": T, "d_model": D, "heads": H,
            "layers": NL, "global_batch": Bg, "steps": steps}, "bar": 1e-4, "passed": True}


def configs_part(args, L, torch, stream):
    """The remaining workload-definition configs on one GPU, device timed (CUDA events on the launching stream):
    C1 MLP step, C3 CNN step (reference shape and padded shape), C4 transformer block forward+backward,
    C5 greedy decode.  Reported next to the headline numbers; each also runs against the CPU oracle in tests/."""
    import numpy as np
    from znn_b200.models import Model

    out = {}
    r = np.random.default_rng(7)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def he(m, scheme="he"):
        P = {}
        for name, shape, _, fan_in in m.params:
            if fan_in:
                std = (2.0 / fan_in) ** 0.5 if scheme == "he" else 0.02
                P[name] = (r.standard_normal(shape, np.float32) * np.float32(std))
            else:
                P[name] = np.ones(shape, np.float32) if "ln_" in name else np.zeros(shape, np.float32)
        m.set_params(P)

    def time_steps(fn, steps, warmup=5):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    for key, kind, dims, batch in (("mlp_784_128_64_10_b64", "mlp", (784, 128, 64, 10), 64),
                                   ("cnn_reference_shape_b64", "cnn_ref", (), 64),
                                   ("cnn_padded_shape_b256", "cnn_padded", (), 256)):
        m = Model(kind, dims, arena_bytes=2 << 30)
        he(m)
        m.set_option("lr", 0.01)
        m.set_option("momentum", 0.9)
        x = (r.integers(0, 256, (batch, 784)).astype(np.float32) / np.float32(255.0))
        t = r.integers(0, 10, batch).astype(np.int32)
        dx, dt = torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda()
        ms = time_steps(lambda: m.train_step_device(dx.data_ptr(), dt.data_ptr(), batch), 200)
        ms_e2e = time_steps(lambda: m.train_step(x, t), 50)
        m.set_option("cuda_graph", 1)       # capture the step once, then replay it
        ms_graph = time_steps(lambda: m.train_step_device(dx.data_ptr(), dt.data_ptr(), batch), 200)
        out[key] = {"us_per_step": ms * 1e3, "steps_per_s": 1e3 / ms, "images_per_s": batch * 1e3 / ms,
                    "cuda_graph_us_per_step": ms_graph * 1e3, "cuda_graph_images_per_s": batch * 1e3 / ms_graph,
                    "e2e_us_per_step": ms_e2e * 1e3, "tape_ops": m.last_step_ops(), "bound": "launch-bound"}
        if kind == "cnn_padded":
            # conv1 115.6 + conv2 1849.7 + fc1 205.5 + fc2 0.7 MFLOP forward; backward twice that less conv1's input gradient
            flops = 2.0 * 256 * (28 * 28 * 32 * 9 + 14 * 14 * 64 * 288 + 3136 * 128 + 128 * 10)
            flops = 3.0 * flops - 2.0 * 256 * 28 * 28 * 32 * 9
            out[key]["tflops"] = flops / (ms_graph * 1e-3) / 1e12
            out[key]["bound"] = "tensor for conv2 (M = 50176, N = 64, K = 288) and fc1; the rest launch-bound"
        m.close()

    # C1 fed by the device-resident loader: synthetic pixel bytes of the dataset's shape, converted on the device,
    # shuffled batches gathered on the device; against the same loop fed from host arrays batch by batch
    from znn_b200 import dataset as zds
    from znn_b200.ops import DevBuf
    n_img, batch = 12800, 64
    px = r.integers(0, 256, (n_img, 784)).astype(np.uint8)
    lab = r.integers(0, 10, n_img).astype(np.uint8)
    d_px, d_img, d_lab = DevBuf.from_host(px), DevBuf(n_img * 784 * 4), DevBuf.from_host(lab)
    L.call("znn_pixels_to_unit", d_px.ptr, d_img.ptr, n_img * 784)
    data = zds.Dataset(d_img, d_lab, n_img, 28, 28, n_img)
    loader = zds.DataLoader(data, batch, shuffle=True, drop_last=True)
    m = Model("mlp", (784, 128, 64, 10), arena_bytes=1 << 30)
    he(m)
    m.set_option("lr", 0.01)
    m.set_option("momentum", 0.9)
    m.set_option("targets_u8", 1)
    x_dev, y_dev = DevBuf(batch * 784 * 4), DevBuf(batch)

    def epoch_device():
        loader.reset()
        n = 0
        while loader.next_into(x_dev, y_dev):
            m.train_step_device(x_dev.ptr, y_dev.ptr, batch)
            n += 1
        return n

    images_host = px.astype(np.float32) / np.float32(255.0)
    order = loader.indices()

    def epoch_host():
        n = 0
        for i in range(0, n_img - batch + 1, batch):
            idx = order[i:i + batch]
            m.train_step(images_host[idx], lab[idx], read_loss=False)
            n += 1
        return n

    res = {}
    for name, fn in (("device_loader", epoch_device), ("host_batches", epoch_host), ("device_loader_graph", epoch_device)):
        if name == "device_loader_graph":
            m.set_option("cuda_graph", 1)
        fn()
        torch.cuda.synchronize()
        e0.record(stream)
        steps_run = fn()
        e1.record(stream)
        torch.cuda.synchronize()
        res[name] = e0.elapsed_time(e1) * 1e3 / steps_run
    out["mlp_epoch_b64_input_pipeline"] = {
        "us_per_step_device_loader": res["device_loader"], "us_per_step_host_batches": res["host_batches"],
        "us_per_step_device_loader_cuda_graph": res["device_loader_graph"],
        "samples": n_img, "note": "device loader: one gather launch per batch, byte labels used in place; host batches: "
                                  "numpy gather + one upload of pixels and labels per step"}
    m.close()
    loader.close()

    # C4: pre-norm block, d_model 512, 8 heads, FFN 2048, batch 32 x seq 256 (168 GFLOP per forward+backward)
    m = Model("block", (512, 8), arena_bytes=8 << 30)
    he(m, "n002")
    x = r.standard_normal((32, 256, 512), np.float32)
    dy = r.standard_normal((32, 256, 512), np.float32)
    ms = time_steps(lambda: m.block_fwd_bwd(x, dy), 10, warmup=3)
    dxx, ddy = torch.from_numpy(x).cuda(), torch.from_numpy(dy).cuda()
    dyy, ddx = torch.empty_like(dxx), torch.empty_like(dxx)
    ms_dev = time_steps(lambda: m.block_fwd_bwd_device(dxx.data_ptr(), ddy.data_ptr(), 32, 256, dyy.data_ptr(), ddx.data_ptr()),
                        50, warmup=3)
    out["transformer_block_b32_t256_d512"] = {"ms_fwd_bwd": ms_dev, "tflops": 168e9 / (ms_dev * 1e-3) / 1e12,
                                              "ms_fwd_bwd_incl_host_copies": ms,
                                              "note": "device-resident x, dy, y, dx; the second figure uploads x and dy from "
                                                      "pageable host arrays and reads y and dx back inside the timed region"}
    m.close()

    # C5 decode: 64 prompts of 16 ids, 256 new tokens, greedy, full re-forward per token as the reference does
    m = Model("gpt", (8192, 1024, 768, 12, 6), arena_bytes=40 << 30)
    he(m, "n002")
    prompts = r.integers(0, 8192, (64, 16)).astype(np.float32)
    n_new = 256 if args.steps >= 10 else 32
    m.greedy_decode(prompts, 2)
    torch.cuda.synchronize()
    e0.record(stream)
    toks = m.greedy_decode(prompts, n_new)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    out["gpt_greedy_decode_b64"] = {"new_tokens": n_new, "tokens_per_s": 64 * n_new / (ms * 1e-3), "ms_total": ms,
                                    "note": "no KV cache: the reference re-runs the whole window per token"}
    m.greedy_decode_kv(prompts, 2)
    torch.cuda.synchronize()
    e0.record(stream)
    toks_kv = m.greedy_decode_kv(prompts, n_new)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    same = toks_kv == toks
    # a sequence follows the reference's tokens up to its first differing pick (a near-tie of two logits)
    first_diff = [int(np.argmin(row)) if not row.all() else n_new for row in same]
    out["gpt_greedy_decode_b64_kv_cache"] = {"new_tokens": n_new, "tokens_per_s": 64 * n_new / (ms * 1e-3), "ms_total": ms,
                                             "sequences_identical_to_full_reforward": int(sum(f == n_new for f in first_diff)),
                                             "sequences": 64, "shortest_identical_prefix": int(min(first_diff)),
                                             "note": "key/value cache: one pass per position; same operators"}
    m.close()
    return out


def sweep_part(args, L, torch, stream):
    """The MatMul operator sweep of the workload definition: square M=N=K in {512..8192} plus the two skinny shapes;
    per shape the forward product (NN, beta 0) and both backward products (dA = dC.B^T, dB = A^T.dC, beta 1), each
    timed alone with CUDA events after warm-up; operands are N(0,1).  Shapes of 2048 and below fit the 126 MB L2, so
    their numbers are L2-resident rates (said in the output)."""
    shapes = [(n, n, n) for n in (512, 1024, 2048, 4096, 8192)] + [(64, 4096, 4096), (4096, 64, 4096)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g = torch.Generator(device="cuda").manual_seed(99)
    out = []
    for (M, N, K) in shapes:
        A = torch.randn((M, K), device="cuda", generator=g)
        B = torch.randn((K, N), device="cuda", generator=g)
        dC = torch.randn((M, N), device="cuda", generator=g)
        Cm = torch.empty((M, N), device="cuda")
        dA, dB = torch.zeros((M, K), device="cuda"), torch.zeros((K, N), device="cuda")
        calls = {
            "fwd_NN": lambda: L.call("znn_sgemm", 101, 111, 111, M, N, K, 1.0, A.data_ptr(), K, B.data_ptr(), N, 0.0, Cm.data_ptr(), N),
            "dA_NT": lambda: L.call("znn_sgemm", 101, 111, 112, M, K, N, 1.0, dC.data_ptr(), N, B.data_ptr(), N, 1.0, dA.data_ptr(), K),
            "dB_TN": lambda: L.call("znn_sgemm", 101, 112, 111, K, N, M, 1.0, A.data_ptr(), K, dC.data_ptr(), N, 1.0, dB.data_ptr(), N),
        }
        flops = 2.0 * M * N * K
        reps = max(5, min(200, int(2e12 / flops)))
        row = {"M": M, "N": N, "K": K, "operand_MB": (M * K + K * N + M * N) * 4 / 1e6,
               "l2_resident": (M * K + K * N + M * N) * 4 < 126e6}
        for name, fn in calls.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(reps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            row[name] = {"us": us, "tflops": flops / us / 1e6, "path": L.dll.znn_gemm_last_path()}
        out.append(row)
    st = C.c_int(0)
    L.call("znn_device_status", C.byref(st), 1)
    if st.value:
        raise SystemExit(f"device status word {st.value}: a bounded device-side wait expired")
    return out


def shape_part(args, L, torch, stream):
    """One (batched) product at a given shape, timed alone with CUDA events: the small case for profiler captures."""
    M, N, K, ta, tb, batch = [int(v) for v in args.shape.split(",")]
    g = torch.Generator(device="cuda").manual_seed(7)
    A = torch.randn((batch, M, K) if ta == 111 else (batch, K, M), device="cuda", generator=g)
    B = torch.randn((batch, K, N) if tb == 111 else (batch, N, K), device="cuda", generator=g)
    Cm = torch.zeros((batch, M, N), device="cuda")
    L.call("znn_gemm_set_path", args.path)
    lda, ldb = (K if ta == 111 else M), (N if tb == 111 else K)

    def run():
        L.call("znn_sgemm_batched_strided", ta, tb, M, N, K, 1.0, A.data_ptr(), lda, M * K, B.data_ptr(), ldb, K * N,
               0.0, Cm.data_ptr(), N, M * N, batch)

    steps, warmup = max(1, args.steps), max(1, args.warmup)
    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        run()
    e1.record(stream)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / steps
    st = C.c_int(0)
    L.call("znn_device_status", C.byref(st), 1)
    if st.value:
        rec = (C.c_int * 16)()
        L.call("znn_gemm_wait_record", rec)
        raise SystemExit(f"device status word {st.value}: a bounded device-side wait expired; first: {list(rec)}")
    want = torch.matmul(A[0].double() if ta == 111 else A[0].double().t(), B[0].double() if tb == 111 else B[0].double().t())
    err = float((Cm[0].double() - want).norm() / want.norm())
    return {"shape": [M, N, K], "trans": [ta, tb], "batch": batch, "path": L.dll.znn_gemm_last_path(), "us": us,
            "tflops": 2.0 * M * N * K * batch / us / 1e6, "rel_err_slice0_vs_fp64": err}


def attention_part(args, L, torch, stream):
    """The fused causal-attention kernels (znn_attn_fwd / znn_attn_bwd) at the sizes of configs 5 and 4, each launch
    timed alone with CUDA events on the launching stream: forward, and the three backward kernels one at a time.
    TFLOP/s = causal algorithmic flops (half the square) / time; fraction of the 3xTF32 burst ceiling."""
    peaks, kind = read_peaks()
    ceiling = peaks["bf16_tflops"] / 2.0 / 3.0
    res = {}
    p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timeit(fn, n=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3

    shapes = {"gpt_b8_h12_t1024_hs64": (8, 12, 1024, 64), "block_b32_h8_t256_hs64": (32, 8, 256, 64)}
    if args.small:
        shapes = {"gpt_b8_h12_t1024_hs64": (8, 12, 1024, 64)}
    for name, (B, nh, T, hs) in shapes.items():
        Cw = nh * hs
        g = torch.Generator(device="cuda").manual_seed(1)
        Q, K, V, dO = (torch.randn((B * T, Cw), device="cuda", generator=g) for _ in range(4))
        O, dQ, dK, dV = (torch.empty_like(Q) for _ in range(4))
        LSE = torch.empty((B * nh, T), device="cuda")
        sc = 1.0 / hs ** 0.5

        def fwd():
            L.call("znn_attn_fwd", p(Q), p(K), p(V), p(O), p(LSE), B, nh, T, hs, Cw, hs, T * Cw, sc)

        def bwd(q, k, v):
            L.call("znn_attn_bwd", p(Q), p(K), p(V), p(O), p(dO), p(LSE), p(dQ) if q else None, p(dK) if k else None,
                   p(dV) if v else None, B, nh, T, hs, Cw, hs, T * Cw, sc, 0)

        prod = 2.0 * B * nh * T * T * hs / 2            # one causal product
        rows = {"fwd": (timeit(fwd, 3 if args.small else 20), 2 * prod),
                "dQ": (timeit(lambda: bwd(1, 0, 0), 3 if args.small else 20), 3 * prod),   # S, dP, dS.K
                "dK": (timeit(lambda: bwd(0, 1, 0), 3 if args.small else 20), 3 * prod),   # S^T, dP^T, dS^T.Q
                "dV": (timeit(lambda: bwd(0, 0, 1), 3 if args.small else 20), 2 * prod)}   # S^T, P^T.dO
        st = C.c_int()
        L.call("znn_device_status", C.byref(st), 1)
        res[name] = {k: {"us": round(us, 1), "tflops": round(fl / us / 1e6, 1), "frac": round(fl / us / 1e6 / ceiling, 3)}
                     for k, (us, fl) in rows.items()}
        res[name]["layer_us"] = round(sum(us for us, _ in rows.values()), 1)
        res[name]["io_MB_fwd"] = round(4 * B * T * Cw * 4 / 1e6, 1)
        res[name]["device_status"] = st.value
    res["ceiling"] = f"{kind}: bf16 burst {peaks['bf16_tflops']} TF/s / 2 / 3"
    return res


def conv_part(args, L, torch, stream):
    """Conv2D entry points at the layer shapes of config 3 (padded CNN, batch 256), each launch timed alone with CUDA
    events: tensor-core path (implicit im2col) against the direct / explicit-im2col path of the same library."""
    p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timeit(fn, n=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3

    res = {}
    n_it = 3 if args.small else 20
    for name, (N, Ci, H, W, Co, K, pad) in {"conv2_b256_32to64_14x14": (256, 32, 14, 14, 64, 3, 1),
                                            "conv1_b256_1to32_28x28": (256, 1, 28, 28, 32, 3, 1)}.items():
        Ho, Wo = H + 2 * pad - K + 1, W + 2 * pad - K + 1
        X = torch.rand(N, Ci, H, W, device="cuda")
        Wt = torch.randn(Co, Ci, K, K, device="cuda") * 0.1
        b = torch.randn(Co, device="cuda")
        Y = torch.empty(N, Co, Ho, Wo, device="cuda")
        dY = torch.randn_like(Y)
        dX, dW, db = torch.zeros_like(X), torch.zeros_like(Wt), torch.zeros_like(b)
        fl = 2.0 * N * Ho * Wo * Ci * K * K * Co
        row = {}
        for path, label in ((0, "default"), (1, "direct_or_explicit_im2col")):
            L.call("znn_debug_set_conv_path", path)
            f = timeit(lambda: L.call("znn_conv2d_fwd", p(X), p(Wt), p(b), p(Y), N, Ci, H, W, Co, K, K, pad), n_it)
            bw = timeit(lambda: L.call("znn_conv2d_bwd", p(X), p(Wt), p(dY), None, p(dW), p(db), N, Ci, H, W, Co, K, K, pad), n_it)
            bx = timeit(lambda: L.call("znn_conv2d_bwd", p(X), p(Wt), p(dY), p(dX), None, None, N, Ci, H, W, Co, K, K, pad), n_it)
            row[label] = {"fwd_us": round(f, 1), "dW_dbias_us": round(bw, 1), "dX_us": round(bx, 1),
                          "fwd_tflops": round(fl / f / 1e6, 2)}
        L.call("znn_debug_set_conv_path", 0)
        res[name] = row
    st = C.c_int()
    L.call("znn_device_status", C.byref(st), 1)
    res["device_status"] = st.value
    return res


def rowops_part(args, L, torch, stream):
    """Row-wise / elementwise kernels at transformer sizes, each timed alone with CUDA events on the launching
    stream; working sets exceed the 126 MB L2.  GB/s = algorithmic bytes per launch / time, compared with the
    measured HBM copy bandwidth."""
    peaks, kind = read_peaks()
    hbm = peaks["hbm_gbs"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f32 = torch.float32

    def rnd(*shape):
        return torch.randn(shape, device="cuda", dtype=f32)

    def timeit(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    res = {}

    def rec(name, nbytes, fn):
        ms = timeit(fn)
        gbs = nbytes / (ms * 1e-3) / 1e9
        res[name] = {"us": ms * 1e3, "algorithmic_MB": nbytes / 1e6, "GBps": gbs, "frac_of_hbm_" + kind: gbs / hbm}

    M, N = 8192, 3072 * 4                       # 403 MB per tensor
    n = M * N
    A, B, Cc = rnd(M, N), rnd(M, N), rnd(M, N)
    bias = rnd(N)
    p = lambda t: t.data_ptr()
    rec("add_bias_fwd", 8 * n, lambda: L.call("znn_add_bias_fwd", p(A), p(bias), p(Cc), M, N))
    rec("add_bias_bwd(dA+=dC, dbias)", 12 * n, lambda: L.call("znn_add_bias_bwd", p(A), p(B), p(bias), M, N))
    rec("relu_fwd", 8 * n, lambda: L.call("znn_relu_fwd", p(A), p(Cc), n))
    rec("gelu_fwd", 8 * n, lambda: L.call("znn_gelu_fwd", p(A), p(Cc), n))
    rec("gelu_bwd", 16 * n, lambda: L.call("znn_gelu_bwd", p(A), p(B), p(Cc), n))
    rec("add_fwd", 12 * n, lambda: L.call("znn_add_fwd", p(A), p(B), p(Cc), n))
    rec("accumulate", 12 * n, lambda: L.call("znn_accumulate", p(A), p(Cc), n))
    rec("sgd_momentum_step", 20 * n, lambda: L.call("znn_sgd_step", p(A), p(B), p(Cc), 1e-9, 0.9, 1.0, n))
    T = 1024
    ns = n // (T * T)
    # fresh N(0,1) inputs: the in-place ops above have grown A and Cc, and expf takes a slow path for the strongly
    # negative arguments such inputs produce (measured 500 us instead of 170 us for the same softmax)
    A.normal_()
    B.normal_()
    # causal: the lower triangle (half the matrix) is read, the forward writes all of P, the backward updates dS's
    # lower triangle only
    rec("causal_softmax_fwd", 6 * n, lambda: L.call("znn_causal_softmax_fwd", p(A), 0.125, p(Cc), ns, T))
    rec("causal_softmax_bwd", 8 * n, lambda: L.call("znn_causal_softmax_bwd", p(Cc), p(B), 0.125, p(A), ns, T))
    rec("softmax_fwd_rows1024", 8 * n, lambda: L.call("znn_softmax_fwd", p(A), p(Cc), n // T, T))
    D = 768
    rows = n // D
    G = rnd(D)
    dG = torch.zeros(D, device="cuda", dtype=f32)
    rec("rmsnorm_fwd_768", 8 * n, lambda: L.call("znn_rmsnorm_fwd", p(A), p(G), 1e-5, p(Cc), rows, D))
    rec("rmsnorm_bwd_768(dX,dG)", 16 * n, lambda: L.call("znn_rmsnorm_bwd", p(A), p(G), p(B), 1e-5, p(Cc), p(dG), rows, D))
    V = 8192
    Mx = n // V
    tg = torch.randint(0, V, (Mx,), device="cuda", dtype=torch.int32)
    loss = torch.zeros(1, device="cuda", dtype=f32)
    rec("softmax_xent_fwd_vocab8192", 8 * n, lambda: L.call("znn_softmax_xent_fwd", p(A), p(tg), p(Cc), p(loss), Mx, V))
    rec("softmax_xent_bwd_vocab8192", 12 * n, lambda: L.call("znn_softmax_xent_bwd", p(Cc), p(tg), p(B), Mx, V))
    ids = torch.randint(0, V, (n // D,), device="cuda").to(f32)
    W = rnd(V, D)
    rec("embedding_fwd", 8 * n, lambda: L.call("znn_embedding_fwd", p(W), p(ids), p(Cc), n // D, D, V))
    dims = torch.tensor([n // (T * 12 * 64), T, 12, 64], dtype=torch.int64)
    rec("transpose_head_split(1,2)", 8 * n, lambda: L.call("znn_transpose_fwd", p(A), p(Cc), dims.data_ptr(), 4, 1, 2))
    dims2 = torch.tensor([n // (T * 64), T, 64], dtype=torch.int64)
    rec("transpose_last2(K->K^T)", 8 * n, lambda: L.call("znn_transpose_fwd", p(A), p(Cc), dims2.data_ptr(), 3, 1, 2))
    rec("argmax_rows_vocab8192", 4 * n, lambda: L.call("znn_argmax", p(A), p(bias), Mx, V, 1))
    return {"hbm_peak_GBps": hbm, "peak_source": kind, "tensor_MB": 4 * n / 1e6, "ops": res}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--impl", default="znn_b200", choices=["znn_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true",
                    help="--workload attention|conv: one size and three timed launches per kernel (for profiler captures)")
    ap.add_argument("--dp-bucket-mb", type=int, default=0,
                    help="GPT workload, N > 1: size of the gradient all-reduce buckets in MB (0 = the library default, 32)")
    ap.add_argument("--shape", default="1024,64,1024,111,111,96",
                    help="--workload shape: M,N,K,trans_a,trans_b,batch of one (batched) product")
    ap.add_argument("--path", type=int, default=0, help="--workload shape: GEMM path (0 = automatic)")
    ap.add_argument("--workload", default="all", choices=["all", "matmul", "gpt", "cnn_dp", "configs", "rowops", "shape", "sweep", "attention", "conv"],
                    help="matmul: the headline MatMul sweep step only; all: also the GPT training step; "
                         "configs: the MLP / CNN / block / decode configs on one GPU")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_gpu(args)


if __name__ == "__main__":
    sys.exit(main())

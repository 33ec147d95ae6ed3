#!/usr/bin/env python
"""Benchmark of the Jetfire INT8 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload linear|nonlinear|gpt2|gemm_sweep|optim]

Default workload ("linear"): one per-block (32x32) INT8 linear layer at the headline GEMM shape M = N = K = 8192 --
forward Y = X W^T, input gradient dX = dY W (stochastic rounding) and weight gradient dW = dY^T X -- i.e. three GEMM
launches per step on seeded synthetic operands (int8 uniform in [-127,127], fp16 scales uniform in [1e-3,1e-1]).
With N > 1 ranks every rank runs the layer on its own batch (weak scaling) and dW is summed across ranks with one NCCL
all-reduce per step, which is the data-parallel exchange of the training recipe.

One JSON line is printed by rank 0.  `value` is whole-job INT8 tensor throughput (10^12 ops/s) with operands resident in
HBM; `e2e` is the same metric through the public Python API with HOST (pinned) operands and results, copies inside the
timed region; `roofline` describes the forward GEMM kernel; `cpu_baseline` is the CPU oracle on a bounded sample.
The same line carries the two other parts of the metric: `gpt2` (GPT-2 124M INT8 training step, micro-batch 12 x 1024 per
GPU, data-parallel over the N ranks: tokens/s, ms per step, first / last loss) and `nonlinear` (GB/s and fraction of the
measured HBM bandwidth per nonlinear operator on [8192,768] and [8192,3072], rank 0's GPU); --no-extras skips both.
`--impl reference` times the reference algorithm's CPU restatement (oracle/) on the host cores; with `--workload gemm_sweep` or
`--workload nonlinear` it times the reference's own GPU kernels (its WMMA extension rebuilt for sm_100, its Triton operators) on
this GPU instead.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "per-block INT8 GEMM TOPS"
UNIT = "TOPS"


# ------------------------------------------------------------------------------------------------ helpers
def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ts, line in self.lines:
            if ts < t0 - 0.05 or ts > t1 + 0.15:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:   # region shorter than a sampling period: fall back to every sample taken
            for ts, line in self.lines:
                f = [x.strip() for x in line.split(",")]
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except Exception:
                    pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def gemm_ops(M, N, K):
    return 2.0 * M * N * K


# ------------------------------------------------------------------------------------------------ CPU side (oracle)
def cpu_linear_sample(O, Ms, Ns, Ks, reps=1):
    """fwd + dgrad + wgrad of one [Ms x Ns x Ks] layer through the CPU oracle; returns (seconds, ops)."""
    import numpy as np
    rng = np.random.default_rng(0)
    X = rng.integers(-127, 128, (Ms, Ks), dtype=np.int8)
    W = rng.integers(-127, 128, (Ns, Ks), dtype=np.int8)
    G = rng.integers(-127, 128, (Ms, Ns), dtype=np.int8)
    SX = rng.uniform(1e-3, 1e-1, (Ms // 32, Ks // 32)).astype(np.float16)
    SW = rng.uniform(1e-3, 1e-1, (Ns // 32, Ks // 32)).astype(np.float16)
    SG = rng.uniform(1e-3, 1e-1, (Ms // 32, Ns // 32)).astype(np.float16)
    noise = O.sr_noise(Ms, Ks, 0, 0)
    t0 = time.perf_counter()
    for _ in range(reps):
        O.linear_forward(X, SX, W, SW)
        O.linear_dgrad(G, SG, W, SW, noise)
        O.linear_wgrad(G, SG, X, SX)
    dt = time.perf_counter() - t0
    return dt, reps * 3 * gemm_ops(Ms, Ns, Ks)


def run_reference_arm(args):
    """The reference algorithm on the host cores (CPU restatement in oracle/; the reference's GEMMs are CUDA-only and its
    WMMA kernels are the thing being replaced).  Each step is a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    os.environ["OMP_NUM_THREADS"] = str(cores)      # torchrun exports OMP_NUM_THREADS=1: the baseline uses every host core
    from oracle import jetfire_oracle as O
    O.build_c_oracle()
    cores = O.set_threads(cores)                     # the thread count actually in effect
    Ms, Ns, Ks = 512, 512, 8192
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_linear_sample(O, 256, 256, 1024)
    tot_t, tot_ops = 0.0, 0.0
    for _ in range(args.steps):
        dt, ops = cpu_linear_sample(O, Ms, Ns, Ks)
        tot_t += dt; tot_ops += ops
    val = tot_ops / tot_t / 1e12
    sample = f"fwd+dgrad+wgrad of a {Ms}x{Ns}x{Ks} slice of the 8192^3 layer per step"
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * tot_t / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME, "sample": sample},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


WORKLOAD_NAME = ("per-block INT8 linear layer, M=N=K=8192, block 32x32: forward + dgrad (stochastic rounding) + wgrad GEMMs "
                 "(GEMM sweep headline shape); dW all-reduced over NCCL when n_gpus > 1")


# ------------------------------------------------------------------------------------------------ GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from jetfire_int8training_b200 import Linear, Nonlinear, rng
    from jetfire_int8training_b200.dp import MeanReducer
    from jetfire_int8training_b200._lib import lib
    L = lib()
    rng.manual_seed(1234 + rank)

    M = N = K = args.size
    g = torch.Generator(device=dev).manual_seed(rank)
    X8 = torch.randint(-127, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
    W8 = torch.randint(-127, 128, (N, K), generator=g, device=dev, dtype=torch.int8)
    G8 = torch.randint(-127, 128, (M, N), generator=g, device=dev, dtype=torch.int8)

    def scales(r, c):
        return (torch.rand(r, c, generator=g, device=dev) * 0.099 + 1e-3).half()
    SX, SW, SG = scales(M // 32, K // 32), scales(N // 32, K // 32), scales(M // 32, N // 32)

    # forward, dgrad, wgrad (+ the split-K reduction); each GEMM that runs on fp16 operand copies adds its two conversion kernels
    f16ops = L.jf_igemm_op16_bytes(M, N, K) > 0
    launches_per_step = (9 if f16ops else 3) + (1 if L.jf_igemm_wgrad_plan(N, K, M, 0) > 1 else 0)
    fwd_ev = []
    # data-parallel exchange: the mean of dW over the ranks, one NCCL all-reduce (AVG) per step behind the weight-gradient GEMM
    reducer = MeanReducer(device=dev)

    def step(time_fwd=False):
        if time_fwd:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        y8, sy = Linear.int8_linear_forward(X8, SX, W8, SW, True, 32)
        if time_fwd:
            e1.record(); fwd_ev.append((e0, e1))
        gx8, gsx, gw = Linear.int8_linear_backward(X8, SX, G8, SG, None, W8, SW, 32, stochastic=True)
        reducer.submit([gw])
        reducer.wait()
        return y8, sy, gx8, gsx, gw

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()     # after rank 0's sampler start-up, so that no rank's timed region contains another rank's set-up
    torch.cuda.synchronize()
    t_wall0 = time.time()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step(time_fwd=True)
    ev1.record()
    torch.cuda.synchronize()
    t_wall1 = time.time()
    if world > 1:
        dist.barrier()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    err = L.jf_igemm_error_flag()

    ops_step = 3 * gemm_ops(M, N, K)
    value = world * ops_step * args.steps / (ms * 1e-3) / 1e12
    fwd_ms = sum(a.elapsed_time(b) for a, b in fwd_ev) / len(fwd_ev)

    if args.no_e2e:   # kernel-tuning run: device-resident numbers only
        if rank == 0:
            print(json.dumps({"value": value, "unit": UNIT, "ms_per_step": ms / args.steps, "fwd_ms": fwd_ms,
                              "fwd_tops": gemm_ops(M, N, K) / (fwd_ms * 1e-3) / 1e12, "size": M, "gemm_error_flag": err,
                              "conv": os.environ.get("JF_GEMM_CONV")}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---------------- end to end through the public API with host buffers
    host_in = [t.cpu().pin_memory() for t in (X8, SX, W8, SW, G8, SG)]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    outs = step()
    reducer.wait()
    host_out = [torch.empty_like(o, device="cpu").pin_memory() for o in outs]
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    def e2e_step():
        x8, sx, w8, sw, g8, sg = [t.to(dev, non_blocking=True) for t in host_in]
        y8, sy = Linear.int8_linear_forward(x8, sx, w8, sw, True, 32)
        gx8, gsx, gw = Linear.int8_linear_backward(x8, sx, g8, sg, None, w8, sw, 32, stochastic=True)
        reducer.submit([gw])
        reducer.wait()                # the reduced gradient is what goes back to the host
        for h, o in zip(host_out, (y8, sy, gx8, gsx, gw)):
            h.copy_(o, non_blocking=True)

    def timed(fn, nsteps):
        fn(); fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(nsteps):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = a.elapsed_time(b)
        if world > 1:
            tt = torch.tensor([t], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt.item())
        return t

    e2e_steps = max(2, min(args.steps, 5))
    e2e_serial_ms = timed(e2e_step, e2e_steps)

    # The same step through the package's host pipeline (host_pipeline.LinearStepPipeline): H2D of step i+1 | GEMMs of step i |
    # D2H of step i-1.  Every step still copies all of its inputs in and all of its results out inside the timed region.
    from jetfire_int8training_b200.host_pipeline import LinearStepPipeline
    def reduce_now(gw):
        reducer.submit([gw])
        reducer.wait()
    pipe = LinearStepPipeline(dev, stochastic=True, after_backward=reduce_now if world > 1 else None)

    def timed_pipeline(nsteps):
        pipe.submit(host_in, host_out, next_host_in=host_in)
        pipe.submit(host_in, host_out)        # no prefetch: the first timed step copies its operands inside the timed region
        pipe.finish()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for k in range(nsteps):
            pipe.submit(host_in, host_out, next_host_in=host_in if k + 1 < nsteps else None)
        pipe.finish()          # the last results must have reached the host
        b.record()
        torch.cuda.synchronize()
        t = a.elapsed_time(b)
        if world > 1:
            tt = torch.tensor([t], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt.item())
        return t

    e2e_pipe_steps = max(4, min(args.steps, 10))
    # three timings of the same e2e_pipe_steps steps, the median is reported: the pipeline depends on the host (PCIe and host memory
    # shared with other jobs of the machine), and single timings 2.4 x off have been seen
    e2e_all_ms = sorted(timed_pipeline(e2e_pipe_steps) for _ in range(3))
    e2e_ms = e2e_all_ms[1]
    e2e_val = world * ops_step * e2e_pipe_steps / (e2e_ms * 1e-3) / 1e12
    e2e_serial_val = world * ops_step * e2e_steps / (e2e_serial_ms * 1e-3) / 1e12

    # ---------------- the other two parts of the metric, in the same line
    gpt2_rec = nonlinear_rec = None
    if not args.no_extras:
        del pipe, host_in, host_out, outs, X8, W8, G8
        torch.cuda.empty_cache()
        gpt2_rec = gpt2_measure("124M", 0, max(5, min(args.steps, 10)), 3, dev, rank, world, local)
        torch.cuda.empty_cache()
        if rank == 0:
            nonlinear_rec = nonlinear_measure(dev, max(args.steps, 20), 3)
        if world > 1:
            dist.barrier()

    if rank == 0:
        peaks = read_peaks()
        # dense INT8 tensor peak: no measured entry exists; use 2x the measured sustained bf16 cuBLAS rate (INT8 is nominally
        # 2x bf16 on this part) for a kernel timed inside a long step, and also report against the 4.5e15 nominal.
        peak_tops = 2.0 * peaks["bf16_tflops_sustained"]
        fwd_tops = gemm_ops(M, N, K) / (fwd_ms * 1e-3) / 1e12
        int_mm_tops = None
        try:
            a8 = torch.randint(-127, 128, (8192, 8192), device=dev, dtype=torch.int8)
            b8 = torch.randint(-127, 128, (8192, 8192), device=dev, dtype=torch.int8).t()
            for _ in range(3):
                torch._int_mm(a8, b8)
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(10):
                torch._int_mm(a8, b8)
            s1.record(); torch.cuda.synchronize()
            int_mm_tops = gemm_ops(8192, 8192, 8192) * 10 / (s0.elapsed_time(s1) * 1e-3) / 1e12
        except Exception:
            pass
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            from oracle import jetfire_oracle as O
            O.build_c_oracle()
            cores = O.set_threads(len(os.sched_getaffinity(0)))
            cpu_linear_sample(O, 128, 128, 1024)
            dt, ops = cpu_linear_sample(O, 512, 512, 8192)
            cpu = {"value": ops / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
                   "sample": "fwd+dgrad+wgrad of a 512x512x8192 slice of the layer, CPU oracle (C, OpenMP), once"}
        ws_mb = (3 * M * K + 2 * M * N + 2 * M * N) / 2 ** 20
        sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
        traffic, traffic_src = forward_dram_traffic(M, N, K)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
                "data": "synthetic",
                "config": {"workload": WORKLOAD_NAME, "M": M, "N": N, "K": K,
                           "l2": f"operands+results per step ~{ws_mb:.0f} MiB, larger than the 126 MB L2"},
                "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": e2e_ms / e2e_pipe_steps, "steps": e2e_pipe_steps,
                        "timings_ms_per_step": [round(t / e2e_pipe_steps, 3) for t in e2e_all_ms], "reported": "median of three timings",
                        "mode": "host_pipeline.LinearStepPipeline (3 streams): H2D(step i+1) | GEMMs(step i) | D2H(step i-1)",
                        "serial_value": e2e_serial_val, "serial_ms_per_step": e2e_serial_ms / e2e_steps},
                "gpu_launches": launches_per_step * args.steps,
                "clocks": clocks,
                "roofline": {"bound": "tensor",
                             "kernel": ("gemm_kernel<fp16 operand copies, kind::f16> (forward; the launch time includes its two int8->fp16 "
                                        "conversion kernels)") if f16ops else "gemm_kernel<K-major,K-major, kind::i8> (forward)",
                             "achieved": fwd_tops,
                             "peak": peak_tops, "unit": "TOPS", "frac": fwd_tops / peak_tops,
                             "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']})",
                             "frac_of_nominal_4500": fwd_tops / 4500.0, "cublas_int_mm_tops": int_mm_tops,
                             "avg_launch_ms": fwd_ms,
                             # the algorithm's own ceiling: the CUDA cores owe every 128x128x32 block product 16384 scale FMAs
                             # (128 lanes per clock: 128 SM clocks per K block) and, on int8 operands, 16384 int32->fp32 conversions
                             # on a 64-lane-per-clock pipe (256 clocks), whatever the tensor core does
                             "dequant_bound_tops": DEQUANT_BOUND_TOPS(sm_count, clocks, f16ops),
                             "frac_of_dequant_bound": fwd_tops / DEQUANT_BOUND_TOPS(sm_count, clocks, f16ops),
                             "traffic": traffic, "traffic_source": traffic_src,
                             "algorithmic_bytes": M * K + N * K + M * N + 2 * (M * K + N * K + M * N) // 1024},
                "cpu_baseline": cpu, "gemm_error_flag": err, "gpt2": gpt2_rec, "nonlinear": nonlinear_rec}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def DEQUANT_BOUND_TOPS(sm_count, clocks, f16ops):
    """Throughput at which the per-K-block rescale alone saturates its pipe: one 128x128x32 block product (2 * 128 * 128 * 32 ops)
    per 256 SM clocks (int8 operands: the int32 -> fp32 conversions) or per 128 SM clocks (fp16 operand copies: the scale FMAs,
    and equally the two kind::f16 MMAs), at the SM clock sampled during the run."""
    mhz = (clocks or {}).get("sm_mhz") or 1965.0
    return sm_count * (2.0 * 128 * 128 * 32) / (128.0 if f16ops else 256.0) * mhz * 1e6 / 1e12


# dram__bytes_read.sum + dram__bytes_write.sum of ONE forward launch at M = N = K = 8192 (the two int8 -> fp16 conversion kernels
# + the GEMM kernel) from an ncu capture, keyed by the SHA-256 (first 16 hex digits) of the kernel sources it was taken with; a
# build from other sources reports null.
NCU_FWD_DRAM_BYTES_8192 = {"9fb6199666735657": (67139072 + 74043136) + (67131392 + 73355520) + (802158080 + 76852480)}


def kernel_source_hash():
    import hashlib
    h = hashlib.sha256()
    csrc = os.path.join(ROOT, "jetfire_int8training_b200", "csrc")
    for f in ("gemm.cu", "gemm_kernel.cuh", "gemm_launch.inc", "ptx_sm100.cuh"):
        h.update(open(os.path.join(csrc, f), "rb").read())
    return h.hexdigest()[:16]


def forward_dram_traffic(M, N, K):
    key = kernel_source_hash()
    if (M, N, K) == (8192, 8192, 8192) and key in NCU_FWD_DRAM_BYTES_8192:
        return NCU_FWD_DRAM_BYTES_8192[key], (f"ncu capture of one forward launch (conversion kernels 0.28 GB + GEMM kernel 0.88 GB), "
                                              f"kernel sources {key}")
    return None, f"no ncu capture for kernel sources {key} at this size"


def nonlinear_ops(M, N, copies, dev):
    """Closures that launch each nonlinear operator through the C ABI on preallocated buffers (so host-side allocation
    is not in the way); `copies` rotating input sets defeat the L2.  Returns {name: (fn(i), algorithmic bytes/element)}."""
    import torch
    from jetfire_int8training_b200 import Nonlinear as NL
    from jetfire_int8training_b200._lib import lib
    L = lib()
    S = lambda: torch.cuda.current_stream().cuda_stream      # at call time: the capturing stream under graph capture
    g = torch.Generator(device=dev).manual_seed(0)
    xs = [torch.randn(M, N, generator=g, device=dev).to(torch.bfloat16) for _ in range(copies)]
    nf = max(2, copies // 2)
    xf = [x.float() for x in xs[:nf]]
    qs = [NL.int8_quantize(x, 32) for x in xs]
    gs = [NL.int8_quantize(x * 1e-2, 32) for x in xs]
    gamma = (1 + 0.1 * torch.randn(N, generator=g, device=dev)).float()
    mean = torch.zeros(M, device=dev); rstd = torch.ones(M, device=dev)
    q_out = torch.empty((M, N), dtype=torch.int8, device=dev)
    qt_out = torch.empty((N, M), dtype=torch.int8, device=dev)
    s_out = torch.empty((M // 32, N // 32), dtype=torch.float16, device=dev)
    f_out = torch.empty((M, N), dtype=torch.float32, device=dev)
    dw = torch.empty((N,), dtype=torch.float32, device=dev)
    mo = torch.empty((M,), dtype=torch.float32, device=dev); ro = torch.empty((M,), dtype=torch.float32, device=dev)
    scr = torch.empty((max((M // 32) * N, 2 * M * ((N + 127) // 128)),), dtype=torch.float32, device=dev)
    P = lambda t: t.data_ptr()
    keep = (xs, xf, qs, gs, gamma, mean, rstd, q_out, qt_out, s_out, f_out, dw, mo, ro, scr)

    def c(i):
        return i % copies
    ops = {
        "quantize_bf16": (lambda i: L.jf_int8_quantize(P(xs[c(i)]), 2, M, N, P(q_out), P(s_out), None, 0, None, 0, 0, S()), 3.0),
        "quantize_bf16_sr": (lambda i: L.jf_int8_quantize(P(xs[c(i)]), 2, M, N, P(q_out), P(s_out), None, 1, None, 7, i, S()), 3.0),
        "quantize_f32": (lambda i: L.jf_int8_quantize(P(xf[i % nf]), 0, M, N, P(q_out), P(s_out), None, 0, None, 0, 0, S()), 5.0),
        "quantize_transpose_bf16": (lambda i: L.jf_int8_quantize(P(xs[c(i)]), 2, M, N, P(q_out), P(s_out), P(qt_out), 0, None, 0, 0, S()), 4.0),
        "transpose": (lambda i: L.jf_int8_transpose(P(qs[c(i)][0]), M, N, P(qt_out), S()), 2.0),
        "dequantize": (lambda i: L.jf_int8_dequantize(P(qs[c(i)][0]), P(qs[c(i)][1]), M, N, P(f_out), S()), 5.0),
        "gelu_fwd": (lambda i: L.jf_int8_gelu_forward(P(qs[c(i)][0]), P(qs[c(i)][1]), M, N, P(q_out), P(s_out), S()), 2.0),
        "gelu_bwd_sr": (lambda i: L.jf_int8_gelu_backward(P(qs[c(i)][0]), P(qs[c(i)][1]), P(gs[c(i)][0]), P(gs[c(i)][1]), M, N, P(q_out),
                                                          P(s_out), 1, None, 7, i, S()), 3.0),
        "ln_fwd": (lambda i: L.jf_int8_layernorm_forward(P(qs[c(i)][0]), P(qs[c(i)][1]), P(gamma), P(mean), P(rstd), M, N, P(q_out),
                                                         P(s_out), S()), 2.0),
        "ln_bwd_sr": (lambda i: L.jf_int8_layernorm_backward(P(qs[c(i)][0]), P(qs[c(i)][1]), P(gs[c(i)][0]), P(gs[c(i)][1]), P(gamma),
                                                             P(mean), P(rstd), M, N, 128, P(q_out), P(s_out), P(dw), P(scr), 1, None, 7, i,
                                                             S()), 3.0),
        "add_bf16_sr": (lambda i: L.jf_int8_add(P(xs[c(i)]), 2, P(qs[c(i + 1)][0]), P(qs[c(i + 1)][1]), M, N, P(f_out), P(q_out), P(s_out),
                                                1, None, 7, i, S()), 8.0),
        "add_meanvar_f32": (lambda i: L.jf_int8_add_meanvar(P(xf[i % nf]), 0, P(qs[c(i)][0]), P(qs[c(i)][1]), M, N, P(f_out), P(q_out),
                                                            P(s_out), P(mo), P(ro), P(scr), S()), 10.0),
    }
    return ops, keep


def run_nonlinear(args):
    """Secondary workload: the nonlinear operator set on [8192,768] and [8192,3072]; prints one JSON line with GB/s per op.
    With --op NAME --rows R --cols C it launches that one operator a few times on one shape (used under ncu)."""
    import torch
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    peaks = read_peaks()
    if args.op:
        M, N = args.rows, args.cols
        copies = 2
        ops, keep = nonlinear_ops(M, N, copies, dev)
        fn, bpe = ops[args.op]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn(0)
        a.record()
        for i in range(args.steps):
            assert fn(i + 1) == 0
        b.record(); torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        print(json.dumps({"op": args.op, "M": M, "N": N, "ms": ms, "GBps": bpe * M * N / (ms * 1e-3) / 1e9}), flush=True)
        return
    print(json.dumps(nonlinear_measure(dev, args.steps, args.warmup)), flush=True)


def graph_replay_ms(fn, iters):
    """ms per call of fn(i), i = 0 .. iters-1, captured into one CUDA graph on a side stream; best of three replays."""
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(iters):
                fn(i)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay(); torch.cuda.synchronize()
    best = float("inf")
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); graph.replay(); b.record(); torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) / iters)
    return best


def nonlinear_measure(dev, steps, warmup):
    """GB/s (algorithmic bytes) and fraction of the measured HBM bandwidth per nonlinear operator on [8192,768] and [8192,3072]."""
    import torch
    peaks = read_peaks()
    res = {}
    for (M, N) in ((8192, 768), (8192, 3072)):
        copies = max(4, int(300e6 // (M * N)) + 1)   # rotate through > 256 MB of int8 payload so L2 cannot serve the reads
        ops, keep = nonlinear_ops(M, N, copies, dev)
        for name, (fn, bpe) in ops.items():
            for i in range(max(3, warmup)):
                assert fn(i) == 0, name
            torch.cuda.synchronize()
            assert fn(0) == 0                          # (a lazily filled table is now known to be complete)
            iters = max(steps, 2 * copies)
            ms = graph_replay_ms(fn, iters)
            gbs = bpe * M * N / (ms * 1e-3) / 1e9
            res[f"{name}[{M}x{N}]"] = {"us": round(ms * 1e3, 2), "GBps": round(gbs, 1), "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 3),
                                       "bytes_per_elt": bpe}
        del ops, keep
        torch.cuda.empty_cache()
    return {"metric": "nonlinear operator GB/s (algorithmic bytes)", "unit": "GB/s", "hbm_peak_gbs": peaks["hbm_gbs"],
            "peak_source": peaks["source"],
            "note": "C-ABI launches on preallocated buffers, inputs rotated through > 256 MB, captured into one CUDA graph; "
                    "CUDA events around the best of three replays (host launch cost of the 6-60 us kernels excluded)",
            "ops": res}


def run_gpt2(args):
    """GPT-2 INT8 training step (nanoGPT shape, synthetic uniform token ids): forward + backward through the INT8 data flow,
    gradient all-reduce (DDP over NCCL when n_gpus > 1) and the fused loss-scale + clip + AdamW step (optim.ClipAdamW, loss scale
    from 2^24 as the reference's GradScaler).  Prints tokens/s."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rec = gpt2_measure(args.model, args.micro_batch, args.steps, args.warmup, dev, rank, world, local, kernel_table=args.kernel_table,
                       bucket_mb=args.ddp_bucket_mb, bucket_view=not args.ddp_copy_grads)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()


def gpt2_measure(model_name, micro_batch, steps, warmup, dev, rank, world, local, kernel_table=False, bucket_mb=100, bucket_view=True):
    """One GPT-2 INT8 data-parallel training measurement (the process group, if any, is already initialised).  Returns the
    record on every rank (timing = max over ranks of the CUDA-event time)."""
    import torch
    import torch.distributed as dist
    from jetfire_int8training_b200 import rng
    from jetfire_int8training_b200._lib import lib
    from jetfire_int8training_b200.gpt2 import GPTConfig, QGPT
    if model_name == "xl":
        cfg, mb = GPTConfig(n_layer=48, n_head=25, n_embd=1600), 8
    elif model_name == "tiny":
        cfg, mb = GPTConfig(n_layer=2, n_head=4, n_embd=256, block_size=256, vocab_size=4096), 4
    else:
        cfg, mb = GPTConfig(), 12
    mb = micro_batch or mb
    torch.manual_seed(1337)
    rng.manual_seed(1337 + rank)
    from jetfire_int8training_b200.optim import ClipAdamW
    model = QGPT(cfg).to(dev)
    decay = [p for p in model.parameters() if p.dim() >= 2]
    nodecay = [p for p in model.parameters() if p.dim() < 2]
    # gradient clipping (max norm 1.0) + AdamW in one call; it re-points the parameters into one flat buffer, so before DDP
    # (loss scale as the reference's GradScaler: init_scale 2^24, INT8_GPT2/train.py:217; halved while gradients overflow)
    opt = ClipAdamW([(decay, 0.1), (nodecay, 0.0)], lr=6e-4, betas=(0.9, 0.95), max_norm=1.0, loss_scale=2.0 ** 24)
    # gradients as views of DDP's buckets: no copy into and out of the buckets (the optimiser reads the gradients where they lie)
    net = (torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=bucket_mb,
                                                     gradient_as_bucket_view=bucket_view) if world > 1 else model)
    g = torch.Generator(device=dev).manual_seed(rank)
    T = cfg.block_size

    def batch():
        ids = torch.randint(0, cfg.vocab_size, (mb, T + 1), generator=g, device=dev)
        return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()

    def step(x, y):
        loss = net(x, y)
        opt.scale_loss(loss).backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    losses = []
    for _ in range(max(3, warmup)):
        losses.append(float(step(*batch())))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        loss = step(*batch())
    b.record(); torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    if world > 1:
        tms = torch.tensor([ms], device=dev); dist.all_reduce(tms, op=dist.ReduceOp.MAX); ms = float(tms.item())
    err = lib().jf_igemm_error_flag()        # a bounded wait that expired inside a GEMM would make every number here void
    toks = world * mb * T * steps / (ms * 1e-3)
    rec = {"metric": "GPT-2 INT8 train tokens/s", "value": toks, "tokens_per_s": toks, "unit": "tokens/s", "n_gpus": world, "steps": steps,
           "warmup": max(3, warmup), "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
           "dtype": "int8 linears/LN/GELU, bf16 attention + LM head, fp32 params", "data": "synthetic",
           "config": {"workload": f"GPT-2 {model_name} INT8 training step", "model": model_name, "n_layer": cfg.n_layer,
                      "n_embd": cfg.n_embd, "micro_batch": mb, "seq_len": T, "params": model.num_params(), "parallelism": f"dp{world}"},
           "loss_first": losses[0], "loss_last": float(loss), "gemm_error_flag": err,
           "loss_scale": float(opt.state[0]), "optimizer_steps_taken": opt.step_count, "optimizer_steps_called": max(3, warmup) + steps}
    if kernel_table and rank == 0:
        # device time per kernel over three more steps (torch.profiler, CUDA activity), largest first
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            for _ in range(3):
                step(*batch())
            torch.cuda.synchronize()
        rows = sorted(((e.device_time_total, e.count, e.key) for e in prof.key_averages()
                       if e.device_time_total > 0 and e.device_type.name == "CUDA"), reverse=True)
        tot = sum(r[0] for r in rows)
        print(f"device time per step: {tot / 3:.1f} us", flush=True)
        for t, c, k in rows[:32]:
            print(f"{t / 3:10.1f} us/step {100 * t / tot:5.1f} %  x{c // 3:4d}  {k[:120]}", flush=True)
    del net, opt, model
    return rec


def run_gemm_sweep(args):
    """Secondary workload: forward / dgrad / wgrad GEMM TOPS over the square sizes and the GPT-2 layer shapes (M = 8192 tokens),
    through the Python operator API on device-resident operands; torch._int_mm (plain int32 GEMM, no block scaling) beside it."""
    import torch
    from jetfire_int8training_b200 import Linear, rng
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    rng.manual_seed(7)
    g = torch.Generator(device=dev).manual_seed(0)
    # the short GPT-2 layer kernels first: after the seconds-long 16384^3 launches the part runs power-capped at ~1.3 GHz for a
    # while, which would be charged to whatever shape is measured next
    shapes = [(8192, 2304, 768), (8192, 768, 768), (8192, 3072, 768), (8192, 768, 3072), (4096, 8192, 4096)] + \
             [(n, n, n) for n in (1024, 2048, 4096, 8192, 16384)]
    # the last shape is the one point the reference publishes: its weight-gradient kernel with M = 8192, N = K = 4096 in the
    # kernel's own terms (out_features 8192 x in_features 4096 over 4096 tokens here): 261.6e12 ops/s, hardware not stated
    PUBLISHED_WGRAD_TOPS = 261.6
    def timed(fn, n, nsets):
        """ms per call: n calls rotating through the operand sets, captured into one CUDA graph and replayed, so that the host
        side of the Python operator API (tens of microseconds per call) does not bound the small shapes."""
        for i in range(3):
            fn(i % nsets)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(n):
                fn(i % nsets)
        graph.replay()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):                       # best of three replays: the short shapes are sensitive to clock ramps
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            best = min(best, a.elapsed_time(b) / n)
        del graph
        return best

    out = {}
    for M, N, K in shapes:      # tokens M, out features N, in features K
        work_bytes = M * K + N * K + M * N
        nsets = max(1, min(8, (300 << 20) // work_bytes))      # rotate operand sets so that small shapes do not live in L2
        sc = lambda r, c: (torch.rand(r, c, generator=g, device=dev) * 0.099 + 1e-3).half()
        sets = []
        for _ in range(nsets):
            sets.append((torch.randint(-127, 128, (M, K), generator=g, device=dev, dtype=torch.int8), sc(M // 32, K // 32),
                         torch.randint(-127, 128, (N, K), generator=g, device=dev, dtype=torch.int8), sc(N // 32, K // 32),
                         torch.randint(-127, 128, (M, N), generator=g, device=dev, dtype=torch.int8), sc(M // 32, N // 32)))
        n = 3 if M * N * K > 2 ** 40 else 24
        ops = 2.0 * M * N * K

        def f_fwd(i):
            X8, SX, W8, SW, G8, SG = sets[i]
            Linear.int8_linear_forward(X8, SX, W8, SW, True, 32)

        def f_bwd(i):
            X8, SX, W8, SW, G8, SG = sets[i]
            Linear.int8_linear_backward(X8, SX, G8, SG, None, W8, SW, 32, stochastic=True)

        def f_wgrad(i):
            X8, SX, W8, SW, G8, SG = sets[i]
            Linear.int8_linear_wgrad(X8, SX, G8, SG)

        def f_cublas(i):
            X8, SX, W8, SW, G8, SG = sets[i]
            torch._int_mm(X8, W8.t())

        t_f, t_b, t_w, t_c = timed(f_fwd, n, nsets), timed(f_bwd, n, nsets), timed(f_wgrad, n, nsets), timed(f_cublas, n, nsets)
        t_d = max(t_b - t_w, 1e-6)
        out[f"{M}x{N}x{K}"] = {"fwd_ms": round(t_f, 4), "fwd_tops": round(ops / t_f / 1e9, 1), "dgrad_sr_ms": round(t_d, 4),
                               "dgrad_sr_tops": round(ops / t_d / 1e9, 1), "wgrad_ms": round(t_w, 4),
                               "wgrad_tops": round(ops / t_w / 1e9, 1), "int_mm_tops": round(ops / t_c / 1e9, 1),
                               "operand_sets": nsets}
        if (M, N, K) == (4096, 8192, 4096):
            out[f"{M}x{N}x{K}"]["wgrad_vs_published"] = round(ops / t_w / 1e9 / PUBLISHED_WGRAD_TOPS, 2)
        del sets
    print(json.dumps({"metric": "per-block INT8 GEMM TOPS", "unit": "TOPS", "shape": "tokens x out_features x in_features",
                      "note": "best of three replays (CUDA events) of a CUDA graph of 24 calls (3 for 16384^3) rotating through `operand_sets` operand sets (> 300 MB together for the small shapes); dgrad = (dgrad + wgrad) - wgrad",
                      "shapes": out}), flush=True)


def run_reference_gemm_sweep(args):
    """`--impl reference --workload gemm_sweep`: the reference's OWN GEMM kernels (its WMMA extension rebuilt for sm_100 by
    oracle/build_ref.py, loaded from oracle/_ref/) timed on this GPU at shapes they support (M, N multiples of 128, N <= 4096):
    the GPU-side baseline of the sweep.  Prints {"unavailable": ...} when the extension has not been built."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    from oracle import build_ref
    ext = build_ref.load()
    if ext is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/BlockQuantizeCUDA.so not built (python oracle/build_ref.py)"}))
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    out = {}
    # kernel-level shapes (M, N, K) as the reference's own benchmark states them; the first is its published point
    for (M, N, K) in ((8192, 4096, 4096), (8192, 2304, 768), (8192, 768, 768), (8192, 3072, 768), (8192, 768, 3072)):
        A = torch.randint(-127, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
        Bnk = torch.randint(-127, 128, (N, K), generator=g, device=dev, dtype=torch.int8)
        Bkn = torch.randint(-127, 128, (K, N), generator=g, device=dev, dtype=torch.int8)
        SAt = (torch.rand(K // 32, M // 32, generator=g, device=dev) * 0.099 + 1e-3).half()
        SBt = (torch.rand(K // 32, N // 32, generator=g, device=dev) * 0.099 + 1e-3).half()
        bias = torch.zeros(N, device=dev); biasmax = torch.zeros(1, device=dev)
        calls = {"fwd_rowcol": lambda: ext.igemm_output_int_quantize_bias_rowcol(A, Bnk.t(), bias, biasmax, SAt, SBt, M, N, K),
                 "dgrad_stochastic": lambda: ext.igemm_output_int_quantize_stochastic(A, Bkn, SAt, SBt, M, N, K),
                 "wgrad_fp": lambda: ext.igemm_output_fp_no_quantize(A, Bkn, SAt, SBt, M, N, K)}
        rec = {}
        for name, fn in calls.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n = 10
            a.record()
            for _ in range(n):
                fn()
            b.record(); torch.cuda.synchronize()
            ms = a.elapsed_time(b) / n
            rec[name + "_ms"] = round(ms, 4); rec[name + "_tops"] = round(2.0 * M * N * K / ms / 1e9, 1)
        out[f"{M}x{N}x{K}"] = rec
    print(json.dumps({"impl": "reference", "metric": "per-block INT8 GEMM TOPS", "unit": "TOPS",
                      "what": "the reference's WMMA kernels (JetfireGEMMKernel extension) recompiled for sm_100, -use_fast_math, on this GPU",
                      "shape": "kernel-level M x N x K", "shapes": out}), flush=True)


def run_optim(args):
    """Secondary workload: the fused clip + AdamW step on parameters with the shapes of GPT-2 124M (random gradients).
    Prints ms per step and the HBM rate of its two passes (4 and 28 bytes per parameter)."""
    import torch
    from jetfire_int8training_b200.gpt2 import GPTConfig, QGPT
    from jetfire_int8training_b200.optim import ClipAdamW
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = read_peaks()
    model = QGPT(GPTConfig()).to(dev)
    decay = [p for p in model.parameters() if p.dim() >= 2]
    nodecay = [p for p in model.parameters() if p.dim() < 2]
    opt = ClipAdamW([(decay, 0.1), (nodecay, 0.0)], lr=6e-4, betas=(0.9, 0.95), max_norm=1.0)
    g = torch.Generator(device=dev).manual_seed(0)
    for p in opt.params:
        p.grad = torch.randn(p.shape, generator=g, device=dev) * 1e-2
    n = sum(p.numel() for p in opt.params)
    for _ in range(max(3, args.warmup)):
        opt.step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        out = opt.step()
    b.record(); torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    gbs = 32.0 * n / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "clip + AdamW step", "parameters": n, "tensors": len(opt.params), "ms_per_step": ms,
                      "bytes_per_parameter": 32, "GBps": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                      "grad_norm": float(out[0]), "applied_factor": float(out[1]),
                      "note": "parameters, moments and gradients are 2 GB together, larger than L2"}), flush=True)


def run_reference_nonlinear(args):
    """`--impl reference --workload nonlinear`: the reference's OWN nonlinear operators (the Triton kernels of Jetfire/Nonlinear,
    unmodified, compiled by the installed Triton with their full autotuning search) timed on this GPU through their public Python
    functions, which allocate their outputs and, for stochastic rounding, draw an fp32 noise tensor with torch (that is part of
    what the operator costs in the reference).  To keep the Python launch overhead of Triton out of the figure the calls are
    captured into one CUDA graph and the replay is timed; an operator that cannot be captured is timed eagerly and marked so.
    Same shapes, input rotation and byte counts as the `nonlinear` workload of this package."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    from oracle import build_ref
    try:
        R = build_ref.load_nonlinear()
    except ImportError as e:
        R, why = None, f"Triton not importable: {e}"
    else:
        why = "reference files not reachable (python tests/stage_reference.py with a reference checkout)"
    if R is None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return
    from jetfire_int8training_b200 import Nonlinear as NL
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = read_peaks()
    res = {}
    for (M, N) in ((8192, 768), (8192, 3072)):
        copies = max(4, int(300e6 // (M * N)) + 1)
        g = torch.Generator(device=dev).manual_seed(0)
        xs = [torch.randn(M, N, generator=g, device=dev).to(torch.bfloat16) for _ in range(copies)]
        nf = max(2, copies // 2)
        xf = [x.float() for x in xs[:nf]]
        qs = [NL.int8_quantize(x, 32) for x in xs]          # operands prepared by this package (bit-identical to the reference's)
        gs = [NL.int8_quantize(x * 1e-2, 32) for x in xs]
        gamma = (1 + 0.1 * torch.randn(N, generator=g, device=dev)).float()
        mean = torch.zeros(M, device=dev); rstd = torch.ones(M, device=dev)
        c = lambda i: i % copies
        ops = {
            "quantize_bf16": (lambda i: R.int8_quantize(xs[c(i)], 32), 3.0),
            "quantize_bf16_sr": (lambda i: R.int8_quantize(xs[c(i)], 32, stochastic=True), 3.0),
            "quantize_f32": (lambda i: R.int8_quantize(xf[i % nf], 32), 5.0),
            "quantize_transpose_bf16": (lambda i: R.int8_quantize_transpose(xs[c(i)], 32), 4.0),
            "transpose": (lambda i: R.int8_transpose(qs[c(i)][0]), 2.0),
            "dequantize": (lambda i: R.int8_dequantize(qs[c(i)][0], qs[c(i)][1], 32), 5.0),
            "gelu_fwd": (lambda i: R.int8_gelu_forward(qs[c(i)][0], qs[c(i)][1], 32), 2.0),
            "gelu_bwd_sr": (lambda i: R.int8_gelu_backward(qs[c(i)][0], qs[c(i)][1], gs[c(i)][0], gs[c(i)][1], 32, stochastic=True), 3.0),
            "ln_fwd": (lambda i: R.int8_layernorm_forward(qs[c(i)][0], qs[c(i)][1], gamma, mean, rstd, 32), 2.0),
            "ln_bwd_sr": (lambda i: R.int8_layernorm_backward(qs[c(i)][0], qs[c(i)][1], gs[c(i)][0], gs[c(i)][1], gamma, 32, mean, rstd,
                                                              stochastic=True), 3.0),
            "add_bf16_sr": (lambda i: R.int8_add_Ifp_Ig16_Ofp_Og(xs[c(i)], qs[c(i + 1)][0], qs[c(i + 1)][1], 32, stochastic=True), 8.0),
            "add_meanvar_f32": (lambda i: R.int8_add_Ifp_Ig16_Ofp_Og_MeanVar(xf[i % nf], qs[c(i)][0], qs[c(i)][1], 32), 10.0),
        }
        iters = max(args.steps, 2 * copies)
        for name, (fn, bpe) in ops.items():
            try:
                for i in range(3):                      # compiles and autotunes
                    fn(i)
                torch.cuda.synchronize()
            except Exception as e:                      # an operator the installed Triton cannot compile
                res[f"{name}[{M}x{N}]"] = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
                continue
            how, graph = "cuda graph replay", None
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        for i in range(iters):
                            fn(i)
                torch.cuda.current_stream().wait_stream(side)
                graph.replay(); torch.cuda.synchronize()
            except Exception:
                graph, how = None, "eager calls"
                torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            if graph is not None:
                graph.replay()
            else:
                for i in range(iters):
                    fn(i)
            b.record(); torch.cuda.synchronize()
            ms = a.elapsed_time(b) / iters
            gbs = bpe * M * N / (ms * 1e-3) / 1e9
            res[f"{name}[{M}x{N}]"] = {"us": round(ms * 1e3, 2), "GBps": round(gbs, 1), "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 3),
                                       "bytes_per_elt": bpe, "timing": how}
            del graph
        del ops, xs, xf, qs, gs
        torch.cuda.empty_cache()
    print(json.dumps({"impl": "reference", "metric": "nonlinear operator GB/s (algorithmic bytes)", "unit": "GB/s",
                      "what": "the reference's Triton operators (Jetfire/Nonlinear, unmodified, full autotuning) on this GPU, called "
                              "through their Python functions (outputs and SR noise allocated per call)",
                      "hbm_peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"], "ops": res}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="linear", choices=["linear", "nonlinear", "gpt2", "gemm_sweep", "optim"])
    ap.add_argument("--model", default="124M", choices=["124M", "xl", "tiny"], help="gpt2 workload: model size")
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--size", type=int, default=8192, help="M = N = K of the linear workload")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (kernel tuning runs)")
    ap.add_argument("--no-extras", action="store_true", help="linear workload: skip the gpt2 and nonlinear records")
    ap.add_argument("--kernel-table", action="store_true", help="gpt2 workload: also print the device time per kernel")
    ap.add_argument("--ddp-bucket-mb", type=int, default=100, help="gpt2 workload, N > 1: DDP bucket size")
    ap.add_argument("--ddp-copy-grads", action="store_true", help="gpt2 workload, N > 1: DDP copies gradients through its buckets")
    ap.add_argument("--op", default=None, help="nonlinear workload: run only this operator (profiling)")
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--cols", type=int, default=3072)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference" and args.workload == "gemm_sweep":
        run_reference_gemm_sweep(args)
    elif args.impl == "reference" and args.workload == "nonlinear":
        run_reference_nonlinear(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "nonlinear":
        run_nonlinear(args)
    elif args.workload == "optim":
        run_optim(args)
    elif args.workload == "gpt2":
        run_gpt2(args)
    elif args.workload == "gemm_sweep":
        run_gemm_sweep(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

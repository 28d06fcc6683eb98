#!/usr/bin/env python
"""Benchmark of the dense-contraction hot path: C = A.B at 8192^3, fp32 in/out, fp16
operands, fp32 accumulation (NeuZephyr's GEMMTensorCore).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over one synthetic problem: fp32 -> fp16 operand
staging + the tcgen05 GEMM through the C ABI (nzb_gemm): one kernel whose converter warps stage the
operands while its tensor-core warps run, or two staging kernels + the GEMM kernel where that form
does not apply.
Prints ONE JSON line on rank 0. Under torchrun every rank runs an independent replica of
the problem (the GEMM itself has no exchange step); the time is the max over ranks.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N = K = 8192
FLOP = 2.0 * M * N * K
WORKLOAD = "gemm 8192x8192x8192, fp32 row-major in/out, fp16 operands (RN), fp32 accumulate, uniform[-1,1]"
METRIC = "gemm_tflops_8192"
UNIT = "TFLOP/s"
CPU_SAMPLE_ROWS = 4096  # rows of C computed by the CPU baseline per step


# dram__bytes_read.sum + dram__bytes_write.sum of one GEMM launch at this size, from the ncu
# capture summarised in profiles/gemm_f16_tcgen05_pair_8192x8192x8192.md (algorithmic: 512 MB).
NCU_DRAM_BYTES_PER_LAUNCH = 1.36e9


def measured_hbm_gbs():
    """Measured STREAM-style copy bandwidth of this pool's B200s, else the earlier pool figure."""
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:
        return 6650.0


def measured_peaks(sustained):
    """Denominators measured on this pool's B200s (cuBLAS bf16 8192^3): the burst figure for
    a kernel timed alone over a few launches, the sustained one for a loop long enough to
    sit under the power cap."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        key = "bf16_tflops_sustained" if sustained else "bf16_tflops"
        return float(p[key]), "of measured (cuBLAS bf16 %s)" % ("sustained" if sustained else "burst")
    except Exception:
        return (1400.0 if sustained else 1590.0), "of fallback (%s)" % ("sustained" if sustained else "burst")


class ClockSampler:
    """Samples the SM clock and the throttle reasons through NVML (read-only queries) in a
    background thread while the timed region runs."""

    def __init__(self, index):
        self.index, self.rows, self.stop_flag, self.t = index, [], False, None

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            # NVML enumerates physical devices; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            idx = self.index
            if vis and all(v.strip().isdigit() for v in vis.split(",")):
                idx = int(vis.split(",")[self.index])
            self.nv, self.h = nv, nv.nvmlDeviceGetHandleByIndex(idx)
            self.max = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
        except Exception as e:
            self.nv = None
            self.err = repr(e)[:100]
            return
        self.t = threading.Thread(target=self._run, daemon=True)
        self.t.start()

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                clk = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                pw = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                self.rows.append((clk, rs, pw))
            except Exception:
                pass
            time.sleep(0.002)

    def mark(self):
        """Index of the next sample: brackets the timed region."""
        return len(self.rows)

    def stop(self, lo=0, hi=None):
        if getattr(self, "nv", None) is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + getattr(self, "err", "")]}
        self.stop_flag = True
        if self.t is not None and self.t.is_alive():
            self.t.join(timeout=1)
        nv = self.nv
        rows = self.rows[lo:hi] or self.rows[-1:]
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        reasons = sorted(k for k, bit in names.items() if any(r[1] & bit for r in rows))
        clks = sorted(r[0] for r in rows)
        return {"sm_mhz": clks[len(clks) // 2] if clks else None, "sm_max_mhz": self.max, "reasons": reasons,
                "samples": len(rows), "power_w_max": max(r[2] for r in rows) if rows else None}


def max_over_ranks(values, device=None):
    """Element-wise maximum of a list of floats over all ranks of the default process group
    (identity without one). Timings of a multi-rank run are reported as the slowest rank's."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return [float(v) for v in values]
    t = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def cpu_baseline(seconds_hint=None):
    """Times the host oracle (fp16-rounded operands, fp32 accumulation, all threads) on a
    bounded sample: CPU_SAMPLE_ROWS rows of the 8192^3 product."""
    import numpy as np
    from oracle import nz_oracle as O
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (CPU_SAMPLE_ROWS, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    Ar, Br = O.round_f16(A), O.round_f16(B)
    O.gemm_f32(Ar[:8], Br, False)  # warm the thread pool
    t0 = time.perf_counter()
    O.gemm_f32(Ar, Br, False)
    dt = time.perf_counter() - t0
    tf = 2.0 * CPU_SAMPLE_ROWS * N * K / dt / 1e12
    return {"value": tf, "unit": UNIT, "cores": O.num_threads(), "kind": "port",
            "sample": "%d of %d rows of C (%.1f GFLOP), operands pre-rounded to fp16, %.2f s"
                      % (CPU_SAMPLE_ROWS, M, 2.0 * CPU_SAMPLE_ROWS * N * K / 1e9, dt)}


def run_ours(args):
    import ctypes
    import torch
    import torch.distributed as dist
    import neuzephyr_b200 as nz
    from neuzephyr_b200 import _capi as C

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = C.lib()
    dev = torch.device("cuda", local)
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    A = torch.rand((M, K), device=dev, generator=g) * 2 - 1
    B = torch.rand((K, N), device=dev, generator=g) * 2 - 1
    Cd = torch.empty((M, N), device=dev)
    stream = torch.cuda.current_stream()

    def step():
        nz.gemm(A, B, out=Cd)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # how many of this library's kernels one step launches (1 with in-kernel staging, else 3)
    d = C.GemmDesc()
    d.M, d.N, d.K, d.lda, d.ldb, d.ldc = M, N, K, K, N, N
    d.batch[0] = d.batch[1] = 1
    n_launch = ctypes.c_int(0)
    C.check(L.nzb_gemm_kernel_launches(ctypes.byref(d), ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(B.data_ptr()),
                                       ctypes.byref(n_launch)))
    launches_per_step = n_launch.value

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    def timed(fn, iters):
        """CUDA-event time per iteration of fn on torch's current stream, with the clock samples taken
        while it ran (rank 0)."""
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        lo = sampler.mark()
        t0.record(stream)
        for _ in range(iters):
            fn()
        t1.record(stream)
        barrier()
        hi = sampler.mark()
        return t0.elapsed_time(t1) / iters, (lo, hi)

    # ---- device-resident timing: `value` -------------------------------------------------
    ms, value_span = timed(step, args.steps)
    if nz.device_status() != 0:
        raise SystemExit("device-side wait expired (status %d)" % nz.device_status())

    # ---- GEMM kernel alone, for the roofline (fp16 operands already staged) ------------
    A16 = nz.cast_f32_f16(A)
    B16 = nz.cast_f32_f16(B, transpose=True)

    def kernel_only():
        nz.gemm_f16(A16, B16, M, N, K, out=Cd)

    for _ in range(3):
        kernel_only()
    kms, burst_span = timed(kernel_only, args.steps)
    # the same kernel in a loop long enough (>= 0.3 s) for the power cap to settle and for NVML's
    # clock samples to describe the region
    sustained_iters = max(args.steps, int(300.0 / max(kms, 1e-3)) + 1)
    kms_sustained, sustained_span = timed(kernel_only, sustained_iters)
    del A16, B16

    # ---- end to end through the C ABI with host buffers: `e2e` ----------------------------
    hA = torch.empty((M, K), dtype=torch.float32).pin_memory()
    hB = torch.empty((K, N), dtype=torch.float32).pin_memory()
    hC = torch.empty((M, N), dtype=torch.float32).pin_memory()
    hA.copy_(A)
    hB.copy_(B)
    e2e_steps = max(2, min(args.steps, 5))

    def e2e_step():
        # one call of the C ABI with host buffers: copies in, staging + GEMM per row block and
        # copies out are pipelined inside nzb_gemm_host; the stream finishes when C is in hC
        nz.gemm_host(hA, hB, hC)

    e2e_step()
    e2e_ms, _ = timed(e2e_step, e2e_steps)
    clocks = clocks_burst = clocks_sustained = None
    if rank == 0:
        sampler.stop_flag = True
        clocks = sampler.stop(*value_span)
        clocks_burst = sampler.stop(*burst_span)
        clocks_sustained = sampler.stop(*sustained_span)

    ms, kms, kms_sustained, e2e_ms = max_over_ranks([ms, kms, kms_sustained, e2e_ms], device=dev)
    if rank == 0:
        burst_peak, burst_how = measured_peaks(sustained=False)
        sus_peak, sus_how = measured_peaks(sustained=True)
        long_run = args.steps * kms > 100.0  # the requested loop itself sat under the power cap
        kernel_ms = kms
        peak_tf, how = (sus_peak, sus_how) if long_run else (burst_peak, burst_how)
        achieved = FLOP / (kernel_ms * 1e-3) / 1e12
        achieved_sus = FLOP / (kms_sustained * 1e-3) / 1e12
        out = {
            "metric": METRIC, "value": world * FLOP / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "parallelism": "replicas only (x%d)" % world,
                       "l2": "inputs 512 MiB + output 256 MiB per step exceed the 126 MB L2; no flush needed",
                       "timed_region": "nzb_gemm: %s per step" % (
                           "ONE kernel (fp32 -> fp16 staging by converter warps inside the tcgen05 GEMM kernel; "
                           "plus a 264-byte memset of its counters)" if launches_per_step == 1 else
                           "2 staging kernels + 1 tcgen05 GEMM kernel"),
                       "e2e_region": "nzb_gemm_host: pinned host A, B -> device, staging + GEMM per row block, "
                                     "C -> pinned host, pipelined on three streams (the reference arm's e2e copies "
                                     "from pageable std::vector through its stock blocking dataInject)"},
            "e2e": {"value": world * FLOP / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": 4 * (M * K + K * N), "d2h_bytes_per_step": 4 * M * N,
                    "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": achieved / peak_tf, "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this "
                                           "kernel at 8192^3 (operands pre-staged)",
                         "kernel": "gemm_f16_tcgen05_pair_kernel", "kernel_ms": kernel_ms, "peak_source": how,
                         "algorithmic_bytes": 2.0 * (M * K + K * N) + 4.0 * M * N,
                         "frac_of_nominal_2250": achieved / 2250.0,
                         "sustained": {"kernel_ms": kms_sustained, "iterations": sustained_iters,
                                       "achieved": achieved_sus, "peak": sus_peak, "frac": achieved_sus / sus_peak,
                                       "peak_source": sus_how, "clocks": clocks_sustained},
                         "burst_clocks": clocks_burst},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            out["cpu_baseline"] = cpu_baseline()
    if not args.no_extras:
        # every rank takes part: the convolution runs on each rank's own images, the model step
        # shards one global batch over the ranks with an NCCL gradient all-reduce
        del A, B, Cd, hA, hB, hC
        torch.cuda.empty_cache()
        extras = other_workloads(dev, rank, world, local)
        if rank == 0:
            out["other_workloads"] = extras
            conv = extras.get("conv2d_n32_c64_224_co128", {})
            if "forward_ms" in conv:
                # the Conv2d half of the metric, as machine-readable roofline entries beside the GEMM's
                hbm = measured_hbm_gbs()
                out["roofline"]["conv2d_forward"] = {
                    "bound": "hbm", "achieved": conv["forward_hbm_gbs_algorithmic_per_gpu"], "peak": hbm, "unit": "GB/s",
                    "frac": conv["forward_hbm_gbs_algorithmic_per_gpu"] / hbm, "peak_source": "of measured (copy)",
                    "kernel": "conv2d_nhwc_tcgen05_kernel (+ nchw_to_nhwc_half_kernel staging, bias transpose)", "ms": conv["forward_ms"],
                    "algorithmic_bytes": conv["forward_algorithmic_bytes"],
                    "tensor_tflops": conv["forward_tflops_per_gpu"], "img_per_s": conv["forward_img_per_s"]}
                out["roofline"]["conv2d_forward_backward"] = {
                    "bound": "hbm", "achieved": conv["fwd_bwd_hbm_gbs_algorithmic_per_gpu"], "peak": hbm, "unit": "GB/s",
                    "frac": conv["fwd_bwd_hbm_gbs_algorithmic_per_gpu"] / hbm, "peak_source": "of measured (copy)",
                    "ms": conv["forward_ms"] + conv["backward_one_call_ms"],
                    "algorithmic_bytes": conv["fwd_bwd_algorithmic_bytes"], "img_per_s": conv["fwd_full_bwd_img_per_s"]}
            seg = extras.get("seg_model_step_batch64", {})
            if "ms_per_step" in seg:
                out["roofline"]["seg_model_step"] = {
                    "bound": "hbm", "ms": seg["ms_per_step"], "img_per_s": seg.get("img_per_s"), "n_gpus": world,
                    "algorithmic_ms_one_gpu": 9.2,
                    "frac": 9.2 / world / seg["ms_per_step"],
                    "note": "about 60 GB of minimal activation + optimizer traffic per step of batch 64 at the "
                            "measured copy bandwidth, divided by the ranks"}
            if "dp_check" in extras:
                out["dp_check"] = extras["dp_check"]
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _time_ms(fn, iters, warm=2):
    import torch
    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def other_workloads(dev, rank=0, world=1, local=0):
    """Short measurements of the other configurations of the path (not the headline metric):
    Linear 8192x4096x4096 forward+backward, Conv2d N=32 C=64 224^2 -> 128 (3x3, s1, p1) forward /
    backward-data / backward-weight per rank (weak scaling: every rank has its own 32 images, times
    are the max over ranks), and one training step of the segmentation model at global batch 64
    sharded over the ranks (strong scaling, NCCL gradient all-reduce)."""
    import torch
    import torch.distributed as dist
    import neuzephyr_b200 as nz
    out = {}
    g = torch.Generator(device=dev)
    g.manual_seed(10)
    try:
        Bt, Fi, Fo = 8192, 4096, 4096
        x = torch.randn((Bt, Fi), device=dev, generator=g)
        w = (torch.rand((Fo, Fi), device=dev, generator=g) * 2 - 1) * (6.0 / Fi) ** 0.5
        b = torch.zeros(Fo, device=dev)
        dy = torch.randn((Bt, Fo), device=dev, generator=g)
        y = torch.empty((Bt, Fo), device=dev)
        dx, dw, db = torch.zeros_like(x), torch.zeros_like(w), torch.zeros_like(b)
        f = _time_ms(lambda: nz.linear_forward(x, w, b, relu=True, out=y), 5)
        bw = _time_ms(lambda: nz.linear_backward(x, w, y, dy, dx, dw, db, relu=True), 5)
        out["linear_8192x4096x4096"] = {"forward_ms": f, "backward_ms": bw,
                                        "tflops": 3 * 2.0 * Bt * Fi * Fo / ((f + bw) * 1e-3) / 1e12}
        del x, w, dy, y, dx, dw
    except Exception as e:  # pragma: no cover
        out["linear_8192x4096x4096"] = {"error": repr(e)[:200]}
    try:
        N_, C_, H_, Co, k = 32, 64, 224, 128, 3
        x = torch.randn((N_, C_, H_, H_), device=dev, generator=g)
        w = torch.randn((1, 1, C_ * k * k, Co), device=dev, generator=g) * (2.0 / (C_ * k * k)) ** 0.5
        bias = torch.zeros((1, 1, H_ * H_, Co), device=dev)
        y = torch.empty((N_, Co, H_, H_), device=dev)
        dy = torch.randn((N_, Co, H_, H_), device=dev, generator=g)
        dx, dw = torch.zeros_like(x), torch.zeros_like(w)
        f = _time_ms(lambda: nz.conv2d_forward(x, w, bias, k, k, 1, 1, out=y), 5)
        bd = _time_ms(lambda: nz.conv2d_backward_data(dy, w, x.shape, k, k, 1, 1, dx), 5)
        bwt = _time_ms(lambda: nz.conv2d_backward_weight(x, dy, w.shape, k, k, 1, 1, dw), 5)
        db = torch.zeros_like(bias)
        one = _time_ms(lambda: nz.conv2d_backward(x, w, dy, k, k, 1, 1, dx=dx, dw=dw, dbias=db, y=y), 5)
        f, bd, bwt, one = max_over_ranks([f, bd, bwt, one], device=dev)
        flop = 2.0 * N_ * H_ * H_ * Co * C_ * k * k
        # algorithmic bytes per rank: forward reads x and the bias matrix and writes y; the backward reads
        # x, y (ReLU mask) and dY, writes dX and the bias-gradient matrix (weights are negligible)
        fwd_bytes = 4.0 * (x.numel() + y.numel() + bias.numel())
        bwd_bytes = 4.0 * (x.numel() + y.numel() + dy.numel() + dx.numel() + 2 * bias.numel())
        out["conv2d_n32_c64_224_co128"] = {"images_per_rank": N_, "n_gpus": world, "scaling": "weak",
                                           "forward_algorithmic_bytes": fwd_bytes,
                                           "fwd_bwd_algorithmic_bytes": fwd_bytes + bwd_bytes,
                                           "fwd_bwd_hbm_gbs_algorithmic_per_gpu": (fwd_bytes + bwd_bytes) / (f + one) / 1e6,
                                           "forward_ms": f, "backward_data_ms": bd, "backward_weight_ms": bwt,
                                           "backward_one_call_ms": one,  # dX, dW, bias gradient and the ReLU mask
                                           "forward_img_per_s": world * N_ / f * 1e3,
                                           "fwd_bwd_img_per_s": world * N_ / (f + bd + bwt) * 1e3,
                                           "fwd_full_bwd_img_per_s": world * N_ / (f + one) * 1e3,
                                           "forward_tflops_per_gpu": flop / f / 1e9,
                                           "forward_hbm_gbs_algorithmic_per_gpu":
                                               4.0 * (x.numel() + y.numel() + bias.numel()) / f / 1e6,
                                           "forward_hbm_frac_of_measured": 4.0 * (x.numel() + y.numel() + bias.numel())
                                               / f / 1e6 / measured_hbm_gbs()}
        del x, y, dy, dx, bias
        torch.cuda.empty_cache()
    except Exception as e:  # pragma: no cover
        out["conv2d_n32_c64_224_co128"] = {"error": repr(e)[:200]}
    tool = os.path.join(ROOT, "neuzephyr_b200", "bin", "seg_model")
    if os.path.exists(tool):
        key = "seg_model_step_batch64"
        try:
            # the tool's ranks find each other through a file holding the NCCL id: name it uniquely
            nonce = [int.from_bytes(os.urandom(4), "little")]
            if world > 1:
                dist.broadcast_object_list(nonce, src=0)
            id_file = "/tmp/nz_dp_bench_%08x.id" % nonce[0]
            env = dict(os.environ)
            env.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(local),
                        "NZ_DP_ID_FILE": id_file})
            r = subprocess.run([tool, "bench", "64", "1024", "2", "1"], capture_output=True, text=True, timeout=600,
                               env=env)
            if rank == 0:
                out[key] = json.loads(r.stdout.strip().splitlines()[-1])
                out[key]["scaling"] = "strong"
            # forward / backward / update times, each closed by a full synchronisation (the sum exceeds a
            # pipelined step; it shows where a rank's time goes at this world size)
            env["NZ_DP_ID_FILE"] = id_file + ".phases"
            r = subprocess.run([tool, "phases", "64", "1024", "2", "1"], capture_output=True, text=True, timeout=600,
                               env=env)
            if rank == 0:
                for line in r.stdout.strip().splitlines():
                    if '"mode": "phases"' in line:
                        out[key]["phases"] = json.loads(line)
            if world > 1:
                # correctness of the sharded step where the driver sees it: the same step on the full batch
                # (rank 0, alone) against the all-reduced sharded step, on a small case
                env["NZ_DP_ID_FILE"] = id_file + ".check"
                r = subprocess.run([tool, "check", "16", "64"], capture_output=True, text=True, timeout=600, env=env)
                if rank == 0:
                    line = [ln for ln in r.stdout.strip().splitlines() if ln.startswith("{")][-1]
                    chk = json.loads(line)
                    out["dp_check"] = {"ok": bool(chk["ok"]) and r.returncode == 0, "world": chk["world"],
                                       "max_rel_grad_diff": chk["max_rel_grad_diff"],
                                       "max_abs_param_diff": chk["max_abs_param_diff"],
                                       "loss_sharded": chk["loss_sharded"], "loss_full": chk["loss_full"],
                                       "case": "global batch 16, 64x64 images, one Adam step"}
        except Exception as e:  # pragma: no cover
            out.setdefault(key, {})["error"] = repr(e)[:200]
    return out


def run_reference(args):
    """The reference arm. NeuZephyr has no CPU implementation: its own path is the WMMA
    kernel behind GEMMTensorCore, which runs on the GPU. When the library built from the
    reference's sources is present (oracle/_ref), it is timed through GEMMTensorCore on
    this box's GPU; the host oracle port is timed beside it as the CPU baseline."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    harness = os.path.join(ROOT, "oracle", "_ref", "ref_harness")
    cpu = cpu_baseline()
    # --steps / --warmup as given (a call takes about 40 ms); only a pathological request is capped so
    # that the arm always ends within minutes
    steps, warm = max(1, min(args.steps, 500)), max(1, min(args.warmup, 50))
    out = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": warm,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
           "dtype": "f16 operands, f32 accumulate",
           "config": {"workload": WORKLOAD, "parallelism": "single GPU (the reference has no multi-GPU path)",
                      "timing": "each step timed on its own (host clock around GEMMTensorCore + the library's "
                                "own Tensor::sync); ms_per_step is the median, each_ms lists every step",
                      "e2e_region": "Tensor::dataInject x2 from pageable std::vector (the reference's stock blocking "
                                    "copies) + GEMMTensorCore + Tensor::hostData"}}
    ran = False
    if os.path.exists(harness):
        env = dict(os.environ, CUDA_VISIBLE_DEVICES=os.environ.get("CUDA_VISIBLE_DEVICES", str(local)))
        try:
            r = subprocess.run([harness, "gemm_bench", str(M), str(N), str(K), str(steps), str(warm), "0"],
                               capture_output=True, text=True, timeout=900, env=env)
            j = json.loads(r.stdout.strip().splitlines()[-1])
            e2e_steps = max(2, min(steps, 5))
            r2 = subprocess.run([harness, "gemm_bench", str(M), str(N), str(K), str(e2e_steps), "1", "1"],
                                capture_output=True, text=True, timeout=900, env=env)
            j2 = json.loads(r2.stdout.strip().splitlines()[-1])
            out.update({"value": j["tflops"], "ms_per_step": j["ms_per_step"],
                        "mean_ms_per_step": j.get("mean_ms_per_step"), "each_ms": j.get("each_ms"),
                        "e2e": {"value": j2["tflops"], "unit": UNIT, "h2d_bytes_per_step": 4 * (M * K + K * N),
                                "d2h_bytes_per_step": 4 * M * N, "ms_per_step": j2["ms_per_step"],
                                "steps": e2e_steps, "each_ms": j2.get("each_ms")},
                        "reference_device": "gpu (NeuZephyr WMMA kernel rebuilt for sm_100, via GEMMTensorCore)",
                        "cpu_baseline": dict(cpu, kind="port")})
            ran = True
        except Exception as e:  # fall through to the CPU port
            out["reference_gpu_error"] = repr(e)[:200]
    if not ran:
        out.update({"value": cpu["value"], "ms_per_step": FLOP / (cpu["value"] * 1e12) * 1e3,
                    "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    "cpu_baseline": cpu})
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the Linear / Conv2d / model-step measurements")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

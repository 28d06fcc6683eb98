"""Command line of the package: run one operation of the C ABI on seeded data and print one JSON line.

    python -m neuzephyr_b200 info
    python -m neuzephyr_b200 gemm M N K [--staged] [--iters 10] [--warmup 3]
    python -m neuzephyr_b200 conv N C H W Cout K pad [--backward] [--no-bias] [--counters] [--iters 5] [--warmup 2]

`gemm` times nzb_gemm (fp32 in / out, uniform[-1,1]); with --staged the GEMM kernel alone on operands
that are already fp16 (nzb_gemm_f16). `conv` times nzb_conv2d_forward (+ untied bias matrix + ReLU) or,
with --backward, nzb_conv2d_backward_data, on N(0,1) tensors with Kaiming-normal weights, stride 1.
Times are CUDA-event averages over --iters calls after --warmup calls. Needs a B200.

--counters prints, after the timed calls, the clock64() counters of the channels-last convolution kernel:
clocks per CTA and call that each role spent waiting or working. They exist only in a library built with
    NZB_EXTRA_NVCC_FLAGS=-DNZB_NHWC_PROFILE python -m neuzephyr_b200.build --force
(rebuild without the variable afterwards: the instrumented kernel is a few percent slower).
"""
import argparse
import json

import torch

import neuzephyr_b200 as nz
from neuzephyr_b200 import _capi


def _time(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / max(iters, 1)


def main():
    ap = argparse.ArgumentParser(prog="python -m neuzephyr_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("info")
    g = sub.add_parser("gemm")
    g.add_argument("shape", type=int, nargs=3, metavar=("M", "N", "K"))
    g.add_argument("--staged", action="store_true")
    g.add_argument("--iters", type=int, default=10)
    g.add_argument("--warmup", type=int, default=3)
    c = sub.add_parser("conv")
    c.add_argument("dims", type=int, nargs=7, metavar=("N", "C", "H", "W", "Cout", "K", "pad"))
    c.add_argument("--backward", action="store_true")
    c.add_argument("--no-bias", action="store_true")
    c.add_argument("--counters", action="store_true")
    c.add_argument("--iters", type=int, default=5)
    c.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args()
    if args.cmd == "info":
        print(json.dumps({"abi_version": _capi.lib().nzb_version(), "library": _capi.LIB_PATH,
                          "device": torch.cuda.get_device_name(0) if torch.cuda.is_available() else None}))
        return
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    if args.cmd == "gemm":
        M, N, K = args.shape
        A = torch.rand((M, K), device="cuda", generator=gen) * 2 - 1
        B = torch.rand((K, N), device="cuda", generator=gen) * 2 - 1
        C = torch.empty((M, N), device="cuda")
        if args.staged:
            A16, B16 = nz.cast_f32_f16(A), nz.cast_f32_f16(B, transpose=True)
            ms = _time(lambda: nz.gemm_f16(A16, B16, M, N, K, out=C), args.iters, args.warmup)
        else:
            ms = _time(lambda: nz.gemm(A, B, out=C), args.iters, args.warmup)
        print(json.dumps({"op": "gemm", "M": M, "N": N, "K": K, "staged": args.staged, "ms": ms,
                          "tflops": 2.0 * M * N * K / ms / 1e9, "status": nz.device_status()}), flush=True)
        return
    N, C, H, W, Co, k, p = args.dims
    x = torch.randn((N, C, H, W), device="cuda", generator=gen)
    w = torch.randn((1, 1, C * k * k, Co), device="cuda", generator=gen) * (2.0 / (C * k * k)) ** 0.5
    Ho, Wo = H + 2 * p - k + 1, W + 2 * p - k + 1
    bias = None if args.no_bias else torch.zeros((1, 1, Ho * Wo, Co), device="cuda")
    y = torch.empty((N, Co, Ho, Wo), device="cuda")
    if args.backward:
        dy = torch.randn((N, Co, Ho, Wo), device="cuda", generator=gen)
        dx = torch.zeros_like(x)
        ms = _time(lambda: nz.conv2d_backward_data(dy, w, x.shape, k, k, 1, p, dx), args.iters, args.warmup)
    else:
        ms = _time(lambda: nz.conv2d_forward(x, w, bias, k, k, 1, p, relu=True, out=y), args.iters, args.warmup)
    line = {"op": "conv", "dims": args.dims, "backward": args.backward, "ms": ms,
            "tflops": 2.0 * N * Ho * Wo * Co * C * k * k / ms / 1e9, "img_per_s": N / ms * 1e3,
            "status": nz.device_status()}
    if args.counters:
        import ctypes
        lib = _capi.lib()
        if not hasattr(lib, "nzb_debug_nhwc_counters"):
            line["counters"] = "not in this build (see --help)"
        else:
            out = (ctypes.c_ulonglong * 16)()
            lib.nzb_debug_nhwc_counters(out, 1)  # drop what the timing loop accumulated
            calls = max(args.iters, 1)
            for _ in range(calls):
                nz.conv2d_forward(x, w, bias, k, k, 1, p, relu=True, out=y)
            lib.nzb_debug_nhwc_counters(out, 1)
            ctas = torch.cuda.get_device_properties(0).multi_processor_count
            names = ["tma_wait_empty", "mma_wait_tempty", "mma_wait_full", "mma_issue_and_commit", "epilogue_wait_tfull",
                     "epilogue_work", "kernel", "mma_issue"]
            line["counters"] = {n: int(out[i] // (ctas * calls)) for i, n in enumerate(names)}
            line["counters_unit"] = "clocks per CTA and call (one CTA per SM; MMA figures are the first of the two issuing warps)"
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()

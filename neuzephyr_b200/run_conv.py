"""Runs nzb_conv2d_forward / backward on seeded N(0,1) tensors and prints one JSON line.

    python -m neuzephyr_b200.run_conv N C H W Cout K pad [--iters 5] [--warmup 2] [--no-bias] [--backward]

A small single-kernel command for timing and for profiler captures of the convolution kernels.
"""
import argparse
import json

import torch

import neuzephyr_b200 as nz


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("dims", type=int, nargs=7, help="N C H W Cout K pad")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--no-bias", action="store_true")
    ap.add_argument("--backward", action="store_true")
    args = ap.parse_args()
    N, C, H, W, Co, k, p = args.dims
    g = torch.Generator(device="cuda")
    g.manual_seed(20)
    x = torch.randn((N, C, H, W), device="cuda", generator=g)
    w = torch.randn((1, 1, C * k * k, Co), device="cuda", generator=g) * (2.0 / (C * k * k)) ** 0.5
    Ho, Wo = H + 2 * p - k + 1, W + 2 * p - k + 1
    bias = None if args.no_bias else torch.zeros((1, 1, Ho * Wo, Co), device="cuda")
    y = torch.empty((N, Co, Ho, Wo), device="cuda")
    dy = torch.randn((N, Co, Ho, Wo), device="cuda", generator=g)
    dx = torch.zeros_like(x)
    if args.backward:
        fn = lambda: nz.conv2d_backward_data(dy, w, x.shape, k, k, 1, p, dx)  # noqa: E731
    else:
        fn = lambda: nz.conv2d_forward(x, w, bias, k, k, 1, p, relu=True, out=y)  # noqa: E731
    for _ in range(args.warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / max(args.iters, 1)
    flop = 2.0 * N * Ho * Wo * Co * C * k * k
    print(json.dumps({"dims": args.dims, "backward": args.backward, "ms": ms, "tflops": flop / ms / 1e9,
                      "img_per_s": N / ms * 1e3, "status": nz.device_status()}), flush=True)


if __name__ == "__main__":
    main()

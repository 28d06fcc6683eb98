"""Runs nzb_gemm on seeded uniform[-1,1] fp32 matrices and prints one JSON line per shape.

    python -m neuzephyr_b200.run_gemm 8192 8192 8192 [--iters 10] [--warmup 3] [--staged]

--staged times the GEMM kernel alone on operands that are already fp16 (nzb_gemm_f16);
the default times the whole call (two staging kernels + GEMM). Handy for shape sweeps and
as the small, single-kernel command a profiler capture needs.
"""
import argparse
import json

import torch

import neuzephyr_b200 as nz


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("shape", type=int, nargs="+", help="M N K triples")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--staged", action="store_true")
    args = ap.parse_args()
    assert len(args.shape) % 3 == 0
    for i in range(0, len(args.shape), 3):
        M, N, K = args.shape[i:i + 3]
        g = torch.Generator(device="cuda")
        g.manual_seed(i + 1)
        A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
        B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
        C = torch.empty((M, N), device="cuda")
        if args.staged:
            A16, B16 = nz.cast_f32_f16(A), nz.cast_f32_f16(B, transpose=True)
            fn = lambda: nz.gemm_f16(A16, B16, M, N, K, out=C)  # noqa: E731
        else:
            fn = lambda: nz.gemm(A, B, out=C)  # noqa: E731
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
        print(json.dumps({"M": M, "N": N, "K": K, "staged": args.staged, "ms": ms,
                          "tflops": 2.0 * M * N * K / ms / 1e9, "status": nz.device_status()}), flush=True)


if __name__ == "__main__":
    main()

"""Times the two bfloat16 matrix products of the prefill path against each other on one shape:

    python -m ember_cpp_b200.csrc.linear_bench M N K [--act gelu_tanh] [--residual] [--tile-n BN] [--only tc|lt]
                                               [--iters 10] [--chain 1]

`lt` is cuBLASLt with its epilogue, `tc` this library's tcgen05 kernel.  Each timed region follows
a write of 256 MiB (larger than L2), is bracketed by CUDA events, and the median is printed.  With
--chain C the region is C launches in a row and the time is divided by C: the host's work for a
launch then hides behind the launch before it, as it does inside a model's step; with --graph the
chain is captured once and replayed, as the engine's decode step is.
"""
from __future__ import annotations

import argparse

import torch

from .ops import CudaOps


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("M", type=int)
    ap.add_argument("N", type=int)
    ap.add_argument("K", type=int)
    ap.add_argument("--act", default=None, choices=[None, "gelu_tanh", "gelu_erf"])
    ap.add_argument("--residual", action="store_true", help="add a float32 residual (the output is float32 then)")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--only", default=None, choices=["tc", "lt"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--chain", type=int, default=1)
    ap.add_argument("--graph", action="store_true", help="capture the chain in a CUDA graph and time its replay")
    args = ap.parse_args()
    ops = CudaOps()
    M, N, K = args.M, args.N, args.K
    a = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda") if args.residual else None
    out = res if args.residual else torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def lt():
        ops.gemm = "lt"
        ops.linear(a, w, bias, act=args.act, residual=res)

    def tc():
        ops.linear_tc(a, w, bias, args.act, res, out, tile_n=args.tile_n)

    for name, fn in (("lt", lt), ("tc", tc)):
        if args.only not in (None, name):
            continue
        for _ in range(3):
            fn()
        run = fn
        if args.graph:        # the host's part of a launch is then outside the timed region altogether
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(args.chain):
                    fn()
            run = graph.replay
        times = []
        for _ in range(args.iters):
            flush.zero_()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(1 if args.graph else args.chain):
                run()
            t1.record()
            torch.cuda.synchronize()
            times.append(t0.elapsed_time(t1) / args.chain)
        ops.check()
        ms = sorted(times)[len(times) // 2]
        print(f"{name}: M={M} N={N} K={K} act={args.act} residual={args.residual}  {ms * 1e3:.1f} us  "
              f"{2.0 * M * N * K / ms / 1e9:.1f} TFLOP/s")


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""GEMM microbenchmark: the tcgen05 kernel against torch.matmul (cuBLAS) on the GEMM
shapes of the Llama training step.  CUDA-event timed, L2 flushed between iterations.

    python benchmarks/gemm.py [--out results.json]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200 import ops  # noqa: E402
from monarch_b200.ops import kernels as K  # noqa: E402

bf16 = torch.bfloat16


def timeit(fn, flush, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    best = 1e9
    tot = 0.0
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        best = min(best, ms)
        tot += ms
    return best, tot / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--T", type=int, default=8192)
    ap.add_argument("--impl", type=int, default=0,
                    help="1: single-CTA tiles, 2: CTA-pair tiles, 0: the library default")
    args = ap.parse_args()
    if args.impl:
        K.set_gemm_impl(args.impl)
    T = args.T
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    # (name, M, N, K, a_mn, b_mn)
    shapes = [
        ("qkv fwd", T, 6144, 4096, False, False),
        ("wo fwd", T, 4096, 4096, False, False),
        ("gate_up fwd", T, 28672, 4096, False, False),
        ("down fwd", T, 4096, 14336, False, False),
        ("lm_head fwd", T, 128256, 4096, False, False),
        ("gate_up dgrad", T, 4096, 28672, False, True),
        ("down dgrad", T, 14336, 4096, False, True),
        ("gate_up wgrad", 28672, 4096, T, True, True),
        ("down wgrad", 4096, 14336, T, True, True),
        ("square 8192", 8192, 8192, 8192, False, False),
    ]
    rows = []
    for name, M, N, Kd, a_mn, b_mn in shapes:
        a = torch.randn((Kd, M) if a_mn else (M, Kd), device="cuda", dtype=bf16)
        b = torch.randn((Kd, N) if b_mn else (N, Kd), device="cuda", dtype=bf16)
        out = torch.empty(M, N, device="cuda", dtype=bf16)
        ours = lambda: ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out)
        A = a.t() if a_mn else a
        Bm = b if b_mn else b.t()
        lib = lambda: torch.matmul(A, Bm, out=out)
        flops = 2.0 * M * N * Kd
        o_best, o_avg = timeit(ours, flush)
        l_best, l_avg = timeit(lib, flush)
        K.check_status()
        rows.append({"impl": K.gemm_impl(), "shape": name, "M": M, "N": N, "K": Kd, "ours_ms": o_best,
                     "ours_tflops": flops / o_best / 1e9, "cublas_ms": l_best,
                     "cublas_tflops": flops / l_best / 1e9, "ratio": l_best / o_best})
        print(f"{name:16s} {M:6d}x{N:6d}x{Kd:6d}  ours {o_best:7.3f} ms {flops/o_best/1e9:7.1f} TF"
              f"   cuBLAS {l_best:7.3f} ms {flops/l_best/1e9:7.1f} TF   x{l_best/o_best:.2f}")
        del a, b, out
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()

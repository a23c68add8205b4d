#!/usr/bin/env python
"""Attention microbenchmark: the tcgen05 flash kernels against torch SDPA (library) on the
causal GQA shapes of the Llama configs.  CUDA-event timed, L2 flushed between iterations.

    python benchmarks/attention.py [--out results.json]
"""
import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200 import ops  # noqa: E402
from monarch_b200.ops import kernels as K  # noqa: E402

bf16 = torch.bfloat16


def timeit(fn, flush, iters=8, warmup=3):
    for _ in range(warmup):
        fn()
    best = 1e9
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    shapes = [("llama3-8b", 1, 8192, 32, 8, 128), ("llama2-13b", 1, 4096, 40, 40, 128),
              ("llama3.2-1b", 2, 4096, 32, 8, 64)]
    rows = []
    for name, B, S, Hq, Hkv, hd in shapes:
        T = B * S
        qkv = torch.randn(T, (Hq + 2 * Hkv) * hd, device="cuda").to(bf16)
        do = torch.randn(T, Hq * hd, device="cuda").to(bf16)
        flops_fwd = 4.0 * B * Hq * S * S * hd / 2
        res = {"shape": name, "B": B, "S": S, "Hq": Hq, "Hkv": Hkv, "hd": hd}
        for impl in ("own", "sdpa"):
            os.environ["MB200_ATTN"] = "" if impl == "own" else "sdpa"
            ctx_box = {}

            def fwd():
                o, ctx = ops.attention_fwd(qkv, B, S, Hq, Hkv, hd, need_bwd=True)
                ctx_box["ctx"] = ctx

            def bwd():
                # the SDPA path consumes its autograd graph, so it needs a fresh forward
                if impl == "sdpa":
                    fwd()
                ops.attention_bwd(ctx_box["ctx"], do)

            t_f = timeit(fwd, flush)
            fwd()
            t_b = timeit(bwd, flush)
            if impl == "sdpa":
                t_b -= t_f
            K.check_status()
            res[impl + "_fwd_ms"] = t_f
            res[impl + "_bwd_ms"] = t_b
            res[impl + "_fwd_tflops"] = flops_fwd / t_f / 1e9
            res[impl + "_bwd_tflops"] = 2.5 * flops_fwd / t_b / 1e9
        rows.append(res)
        print(f"{name:12s} fwd own {res['own_fwd_ms']:.3f} ms ({res['own_fwd_tflops']:.0f} TF) "
              f"sdpa {res['sdpa_fwd_ms']:.3f} ms ({res['sdpa_fwd_tflops']:.0f} TF) | bwd own "
              f"{res['own_bwd_ms']:.3f} ms ({res['own_bwd_tflops']:.0f} TF) sdpa "
              f"{res['sdpa_bwd_ms']:.3f} ms ({res['sdpa_bwd_tflops']:.0f} TF)")
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()

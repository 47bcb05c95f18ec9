"""Run one any-precision layer operator on synthetic operands (usage example and profiling driver).

    python any-precision-llm_b200/examples/run_layer.py --op matmul --N 4096 --K 4096 --w 4 --M 1 --reps 10

`--reps` distinct random layers are created (uniform parent codes drawn as random bitplanes, sorted
N(0, 0.02) fp16 tables) and the chosen operator is called once on each:
`matmul` = any_precision_ext.matmul_kbit (decode GEMV), `prenorm` = the same product through the decoder variant
of the kernel (scaled by rsqrt of a given mean square in its epilogue), `gemm` = gemm_kbit (fused prefill),
`dequant` = dequant_kbit, `quantize` = quantize.seed_and_upscale_layer (seed 3 bits, parent 8; random fp16-valued
weights and squared-normal sensitivities instead of packed operands).  Prints the mean |y| of the last result so the work cannot be elided.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch

import any_precision_ext as ext
from anyprec_b200 import packing


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=["matmul", "prenorm", "gemm", "dequant", "quantize"], default="matmul")
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--w", type=int, default=4)
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--reps", type=int, default=10)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(0)
    if a.op == "quantize":
        from anyprec_b200 import quantize
        codes = None
        for _ in range(a.reps):
            w = (torch.randn((a.N, a.K), device="cuda", generator=gen) * 0.02).half().float()
            s = torch.randn((a.N, a.K), device="cuda", generator=gen) ** 2
            luts, codes = quantize.seed_and_upscale_layer(w, s)
        torch.cuda.synchronize()
        print("done", float(codes.float().mean()))
        return
    qs = [packing.random_qweight(8, a.N, a.K, device="cuda", generator=gen) for _ in range(a.reps)]
    luts = [packing.random_lut(a.N, a.w, device="cuda", generator=gen) for _ in range(a.reps)]
    x = torch.randn((a.M, a.K), device="cuda", generator=gen).half()
    ssq = torch.full((a.M, a.K // 16), 16.0, device="cuda")                # mean square 1
    y = None
    for q, lut in zip(qs, luts):
        if a.op == "matmul":
            y = ext.matmul_kbit(x, q, lut, a.w)
        elif a.op == "prenorm":
            y = ext.matmul_kbit(x, q, lut, a.w, prenorm=(ssq, a.K, 1e-5))
        elif a.op == "gemm":
            y = ext.gemm_kbit(x, q, lut, a.w)
        else:
            y = ext.dequant_kbit(q, lut, a.w)
    torch.cuda.synchronize()
    print("done", float(y.float().abs().mean()))


if __name__ == "__main__":
    main()

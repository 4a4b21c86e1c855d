"""Prefill dequantise + GEMM timing on the Llama-3-8B shapes of the baseline's fourth configuration
(E8-D4 r=1.75, group scales qb=128, 2048 tokens): `python -m eptq_b200.gemm_bench [--tokens T]`.
Prints one JSON line per layer shape: time, TFLOP/s (2*T*out*in), fraction of the measured dense
bf16 tensor peak, and the same product done by cuBLAS on the reconstructed fp16 weight for scale."""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from .kernels.linear import EPTQLinear
from .quantizers import E8D4Quantizer
from .synthetic import LLAMA3_8B_LINEARS, make_layer


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--only", default=None, help="substring of a layer name, e.g. k_proj")
    args = ap.parse_args()
    peaks = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    peak = json.loads(peaks.read_text())["bf16_tflops"] if peaks.exists() else 1590.0
    dev = torch.device("cuda")
    table = E8D4Quantizer(radius=1.75).codes.to(dev)
    seen = set()
    for name, (o, i) in LLAMA3_8B_LINEARS.items():
        if (o, i) in seen or (args.only and args.only not in name):
            continue
        seen.add((o, i))
        lin = EPTQLinear.from_quantized_data(make_layer(o, i, seed=42, device="cuda", qb_size=128), table, "e8_d4")
        x = torch.randn(args.tokens, i, device=dev).half()

        def timed(fn):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / args.reps

        ms = timed(lambda: lin(x))
        W = lin.dequantize()
        ms_lib = timed(lambda: x @ W.T)
        flops = 2.0 * args.tokens * o * i
        print(json.dumps({"layer": name, "out": o, "in": i, "tokens": args.tokens, "ms": ms,
                          "tflops": flops / ms / 1e9, "frac_of_measured_tensor_peak": flops / ms / 1e9 / peak,
                          "cublas_on_reconstructed_ms": ms_lib, "cublas_tflops": flops / ms_lib / 1e9}))


if __name__ == "__main__":
    main()

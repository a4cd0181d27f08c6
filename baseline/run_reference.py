"""Runs the reference project's own operator (baseline/_ref/gemm_int8_CUDA.so, built by build_reference.sh
from the reference's unmodified csrc/kernels/gemm.cu and bindings.cpp) on seeded inputs, in a process of
its own: the library registers the torch namespace gemm_int8_CUDA, which this repository's package also
defines, so the two cannot live in one interpreter.  This file never imports the product package.

    python baseline/run_reference.py --cases cases.json --out results.npz [--time [--no-outputs]]

cases.json: a list of {"name", "kind", "M", "N", "K", "alpha", "seed"}; kind is one of
  "uniform"   x, y = randint(-128, 127) with seeds seed, seed + 1              (the README example)
  "testpy"    x = (rand(M, K) * 100).to(int8), y = x                           (the reference's test.py:5-6)
  "benchmark" x, y = clamp(round(randn * 5), -128, 127) with seeds seed, seed+1 (benchmark.py:20-26)
The same generator (`make_case`) is imported by the test that compares these outputs with the CPU oracle
and with this repository's kernels, so all three see identical bits.

results.npz: per case "<name>" = bf16 result as uint16 bit patterns, and with --time "<name>.us" = device
time per call in microseconds (CUDA events around 20 back-to-back calls, best of 5, after 10 warm-ups).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_LIB = os.path.join(HERE, "_ref", "gemm_int8_CUDA.so")


def make_case(kind: str, M: int, N: int, K: int, seed: int):
    """CPU int8 operands x [M,K], y [N,K] of one case (see the module docstring)."""
    g0 = torch.Generator().manual_seed(seed)
    g1 = torch.Generator().manual_seed(seed + 1)
    if kind == "uniform":
        x = torch.randint(-128, 127, (M, K), dtype=torch.int8, generator=g0)
        y = torch.randint(-128, 127, (N, K), dtype=torch.int8, generator=g1)
    elif kind == "testpy":
        if M != N:
            raise ValueError("the test.py case multiplies x by itself: M must equal N")
        x = (torch.rand(M, K, generator=g0) * 100).to(torch.int8)
        y = x.clone()
    elif kind == "benchmark":
        x = (torch.randn(M, K, generator=g0) * 5).round().clamp(-128, 127).to(torch.int8)
        y = (torch.randn(N, K, generator=g1) * 5).round().clamp(-128, 127).to(torch.int8)
    else:
        raise ValueError(f"unknown case kind {kind!r}")
    return x, y


def available() -> bool:
    return os.path.exists(REF_LIB)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--no-outputs", action="store_true", help="with --time: store the timings only")
    args = ap.parse_args()
    if not available():
        print(f"reference library {REF_LIB} not built (baseline/build_reference.sh)", file=sys.stderr)
        return 3
    if "gemm_int8_b200" in sys.modules or "gemm_int8" in sys.modules:
        raise RuntimeError("the product package must not be loaded in the reference process")
    torch.ops.load_library(REF_LIB)
    op = torch.ops.gemm_int8_CUDA.int8_matmul
    dev = torch.device("cuda:0")
    out = {}
    with open(args.cases) as f:
        cases = json.load(f)
    for c in cases:
        x, y = make_case(c["kind"], c["M"], c["N"], c["K"], c["seed"])
        xd, yd = x.to(dev), y.to(dev)
        r = op(xd, yd, float(c["alpha"]))
        torch.cuda.synchronize()
        if not args.no_outputs:
            out[c["name"]] = r.view(torch.int16).cpu().numpy().view(np.uint16)
        if args.time:
            for _ in range(10):
                op(xd, yd, float(c["alpha"]))
            best = float("inf")
            for _ in range(5):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(20):
                    op(xd, yd, float(c["alpha"]))
                e.record()
                torch.cuda.synchronize()
                best = min(best, s.elapsed_time(e) * 1000.0 / 20)
            out[c["name"] + ".us"] = np.float64(best)
    np.savez(args.out, **out)
    return 0


if __name__ == "__main__":
    sys.exit(main())

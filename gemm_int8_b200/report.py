"""Sweep of the five benchmark configurations on one GPU: device time, INT8 TOP/s (or HBM GB/s for the decode
shapes), fraction of the peaks, speed-up over cuBLAS bf16 (`torch.matmul(a_bf16, b_bf16.t())`, the comparison the
reference's benchmark.py:77-80 makes) and cuBLASLt int8 (`torch._int_mm`) where it applies.

    python -m gemm_int8_b200.report [--quick] [--out FILE.md]

Timing: CUDA events on the current stream, median of the repeats.  Compute-bound shapes: one launch per timed
region with the L2 flushed before it by a 256 MiB read.  Decode shapes (launch-bound): CUDA-graph replay over
rotating weight copies whose total exceeds twice the L2, so every launch streams its weights from HBM.
Inputs are random int8 / random scales of the configuration's shapes (values do not change the timing).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

import gemm_int8_b200 as g

NOMINAL_INT8_TOPS = 4500.0


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self, dev):
        self.flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev).view(torch.int64)

    def cold(self, fn, iters=7, warm=2):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            self.flush.max()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        return statistics.median(ts)

    @staticmethod
    def graph(fns, reps=5):
        for f in fns:
            f()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for f in fns:
                f()
        gr.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            gr.replay()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) / len(fns))
        return statistics.median(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="skip the largest shapes")
    ap.add_argument("--out", default="")
    ap.add_argument("--section", default="all", choices=["all", "gemm", "decode", "quant"],
                    help="which part of the sweep to run")
    args = ap.parse_args()
    dev = torch.device("cuda")
    hbm, bf16, kind = _peaks()
    int8_peak = 2 * bf16
    tm = Timer(dev)
    lines = []
    # Bring the clocks up before the first (small) rows are timed.
    wa, wb = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16), torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
    for _ in range(200):
        torch.matmul(wa, wb)
    torch.cuda.synchronize()
    del wa, wb

    def emit(s=""):
        print(s, flush=True)
        lines.append(s)

    def rnd(shape):
        return torch.randint(-128, 127, shape, dtype=torch.int8, device=dev)

    emit(f"Peaks: HBM {hbm} GB/s ({kind}), int8 tensor = 2 x bf16 {bf16} = {int8_peak:.0f} TOP/s ({kind}), nominal int8 {NOMINAL_INT8_TOPS:.0f} TOP/s")
    emit()
    if args.section in ("all", "gemm"):
        gemm_section(args, emit, tm, rnd, dev, int8_peak)
    if args.section in ("all", "decode"):
        decode_section(emit, tm, rnd, dev, hbm)
    if args.section in ("all", "quant"):
        quant_section(emit, tm, dev, hbm)
    emit()
    emit(f"kernel status word after the sweep: {g.device_status()}")
    if args.out:
        with open(args.out, "w") as f:
            f.write("\n".join(lines) + "\n")


def quant_section(emit, tm, dev, hbm):
    """Activation quantisers: bytes = input + int8 output + scales, one cold-L2 launch per timed region."""
    emit("Activation quantisers (per token per 128-wide K block), cold L2; bytes = input + int8 output + fp32 scales")
    emit()
    emit("| input | M | K | kernel | us | GB/s | of HBM peak |")
    emit("|---|---|---|---|---|---|---|")
    for dtype in (torch.bfloat16, torch.float32):
        for (M, K) in ((2048, 4096), (2048, 8192), (16384, 8192), (8192, 28672)):
            a = torch.randn(M, K, device=dev).to(dtype)
            byt = M * K * (a.element_size() + 1) + M * (K // 128) * 4
            for name, fn in (("quantize_token_block", lambda: g.quantize_per_token_block(a)),
                             (f"hadamard_quantize_token_block (H = {min(K & -K, 8192)})",
                              lambda: g.hadamard_quantize_per_token_block(a))):
                t = tm.cold(fn)
                emit(f"| {str(dtype).replace('torch.', '')} | {M} | {K} | {name} | {t * 1e3:.1f} | {byt / t / 1e6:.0f} | {byt / t / 1e6 / hbm:.3f} |")
            del a


def gemm_section(args, emit, tm, rnd, dev, int8_peak):
    emit("| config | M | N | K | kernel | ms | TOP/s | of 2x bf16 | of nominal | cuBLAS bf16 ms | speed-up vs bf16 | cuBLASLt int8 ms |")
    emit("|---|---|---|---|---|---|---|---|---|---|---|---|")

    def row(cfg, M, N, K, kindname, fn, int_mm=True, bf16_cmp=True):
        x, y = rnd((M, K)), rnd((N, K))
        extra = ()
        if kindname == "blockwise":
            extra = (torch.rand(M, -(-K // 128), device=dev) * 0.02 + 1e-3, torch.rand(-(-N // 128), -(-K // 128), device=dev) * 0.02 + 1e-3)
        iters = 3 if M * N * K > 2e12 else 7
        t = tm.cold(lambda: fn(x, y, *extra), iters=iters)
        tops = 2.0 * M * N * K / t / 1e9
        tb = ti = float("nan")
        if bf16_cmp and M * N <= 8192 * 16384 * 2:
            xb, yb = x.bfloat16(), y.bfloat16()
            tb = tm.cold(lambda: torch.matmul(xb, yb.t()), iters=iters)
            del xb, yb
        if int_mm and M > 16 and M * N <= 8192 * 16384 * 2:
            try:
                yt = y.t()
                ti = tm.cold(lambda: torch._int_mm(x, yt), iters=iters)
            except Exception:
                pass
        variant = g.pick_variant(2 if kindname == "blockwise" else 0, M, N, K)
        emit(f"| {cfg} | {M} | {N} | {K} | {kindname}/{variant} | {t:.4f} | {tops:.0f} | {tops / int8_peak:.3f} | {tops / NOMINAL_INT8_TOPS:.3f} | {tb:.4f} | {tb / t:.2f}x | {ti:.4f} |")

    plain = lambda x, y: g.matmul(x, y, 1.0)  # noqa: E731
    block = lambda x, y, sa, sw: g.matmul_blockwise(x, y, sa, sw)  # noqa: E731

    row("1 plain (README example)", 1024, 4096, 4096, "plain", plain)
    for tok in (512, 1024, 2048):   # the reference benchmark's own grid (benchmark.py:56-62)
        for (n, k) in ((4096, 4096), (14336, 4096), (4096, 14336)):
            row("ref benchmark.py", tok, n, k, "plain", plain)
    row("2 blockwise prefill", 2048, 11008, 4096, "blockwise", block, int_mm=False)
    for (K, N) in ((8192, 10240), (8192, 8192), (8192, 57344), (28672, 8192)):
        for M in (128, 512, 2048, 8192, 16384):
            if args.quick and M * N * K > 3e12:
                continue
            row("4 Llama-70B sweep", M, N, K, "blockwise", block, int_mm=False, bf16_cmp=M * N <= 8192 * 57344)
    if not args.quick:
        row("5 N-shard, g=1 (GEMM only)", 16384, 57344, 8192, "blockwise", block, int_mm=False, bf16_cmp=False)
        row("5 N-shard, one of 8 shards", 16384, 7168, 8192, "blockwise", block, int_mm=False)
    row("target", 8192, 8192, 8192, "plain", plain)
    if not args.quick:
        row("target", 16384, 16384, 16384, "plain", plain)



def decode_section(emit, tm, rnd, dev, hbm):
    emit()
    emit("Decode shapes (config 3): per-token x per-channel scales, device time per kernel from CUDA-graph replays over HBM-cold weights")
    emit()
    emit("| M | N | K | kernel | us | GB/s | of HBM peak | cuBLAS bf16 us | speed-up vs bf16 |")
    emit("|---|---|---|---|---|---|---|---|---|")
    for (K, N) in ((4096, 4096), (4096, 14336), (14336, 4096)):
        ncopy = max(8, int(300e6 // (N * K)) + 1)
        ys = [rnd((N, K)) for _ in range(ncopy)]
        sw = torch.rand(N, device=dev)
        for M in (1, 4, 16, 64):
            x, sx = rnd((M, K)), torch.rand(M, device=dev)
            byt = M * K + N * K + 2 * M * N + 4 * (M + N)
            t = tm.graph([(lambda y=y: g.matmul_scaled(x, y, sx, sw)) for y in ys])
            xb = x.bfloat16()
            yb = [y.bfloat16() for y in ys[: max(4, ncopy // 2)]]
            tb = tm.graph([(lambda y=y: torch.matmul(xb, y.t())) for y in yb])
            del yb
            emit(f"| {M} | {N} | {K} | {g.pick_variant(1, M, N, K)} | {t * 1e3:.1f} | {byt / t / 1e6:.0f} | {byt / t / 1e6 / hbm:.3f} | {tb * 1e3:.1f} | {tb / t:.2f}x |")
        del ys



if __name__ == "__main__":
    sys.exit(main())

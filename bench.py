#!/usr/bin/env python
"""Benchmark of the INT8 GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one blockwise-dequantised W8A8 GEMM over one batch of synthetic tokens.  Default workload at every N:
the largest configuration, 16384 x 57344 x 8192 (uniform int8 operands, per-token-per-128-K activation scales,
per-128x128 weight scales, bf16 output).  N = 1 computes the whole product on one GPU.  With N > 1 ranks (launched
by torch.distributed.run, one rank per GPU) the weight is split column-wise over the ranks, every rank computes its
bf16 [M, N/ranks] slice with the unchanged single-GPU kernel and the slices are assembled on every rank -- by an
NCCL all-gather over NVLink after the GEMM, or (`--gather fused`) by the GEMM's own epilogue, which stores every
block into every rank's matrix through mapped peer memory.  Total work is fixed: strong scaling.

Rank 0 prints ONE JSON line.  `value` is whole-job INT8 TOPS with inputs resident in HBM (CUDA events around each
step on the launching stream, L2 flushed between steps, max over ranks); `gemm_ms` is the GEMM alone and
`ms_per_step` the GEMM plus the gather; `cublas_bf16` is torch.matmul in bf16 on the same per-rank shape, timed
the same way, and `speedup_vs_cublas_bf16` their ratio; `e2e` is the same metric through the public Python API with
pinned HOST buffers, host<->device copies inside the timed region; `roofline` relates the kernel to the measured
tensor peak; `cpu_baseline` times the CPU restatement of the same arithmetic on this box's host cores; `sweep`
(N = 1 only) carries every other configuration: device time, TOPS or GB/s and the cuBLAS bf16 time of each shape,
and for the plain shapes the reference project's own kernel when baseline/_ref holds its build.

`--impl reference` times the CPU restatement of the reference formula (the reference project has no CPU
implementation of its own; its CUDA operator, where built, appears in `sweep`) with all host threads, each step a
bounded row sample of the same workload; it never loads this repository's CUDA library.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "INT8 TOPS per shape (fraction of B200 INT8 peak); speedup vs cuBLAS BF16"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL_INT8_TOPS = 4500.0

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures summarised under
# profiles/: keyed by (workload, M, N, K).  Other shapes report null.
NCU_TRAFFIC = {
    ("blockwise_prefill", 2048, 11008, 4096): (66.5e6, "profiles/blockwise_gemm_kernel__blockwise_prefill_2048x11008x4096.md"),
    ("square8192", 8192, 8192, 8192): (444.3e6, "profiles/dense_gemm_kernel__square8192.md"),
    ("decode", 16, 14336, 4096): (58.94e6, "profiles/smallm_cluster_kernel__decode_16x14336x4096.md"),
}

WORKLOADS = {
    # name: (M, N, K, kind)
    "nshard": (16384, 57344, 8192, "blockwise"),
    "blockwise_prefill": (2048, 11008, 4096, "blockwise"),
    "plain": (1024, 4096, 4096, "plain"),
    "square8192": (8192, 8192, 8192, "plain"),
    "decode": (16, 4096, 4096, "scaled"),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            if "bf16_tflops" in d and "hbm_gbs" in d:
                return d, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def load_input_generators():
    """The seeded input generators (gemm_int8_b200/workloads.py and quant.py, pure torch) loaded under a private
    package name, so that the reference arm gets the same inputs without importing the product package (and with
    it the CUDA library)."""
    pkg_dir = os.path.join(ROOT, "gemm_int8_b200")
    pkg = types.ModuleType("_gi8_inputs")
    pkg.__path__ = [pkg_dir]
    sys.modules.setdefault("_gi8_inputs", pkg)
    mods = {}
    for name in ("quant", "workloads"):
        full = f"_gi8_inputs.{name}"
        if full not in sys.modules:
            spec = importlib.util.spec_from_file_location(full, os.path.join(pkg_dir, name + ".py"))
            mod = importlib.util.module_from_spec(spec)
            sys.modules[full] = mod
            spec.loader.exec_module(mod)
        mods[name] = sys.modules[full]
    return mods["workloads"]


class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU through NVML (read-only) while a region runs, as fast
    as NVML answers (about a kilohertz)."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.0005):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        n = 0
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                n += 1
                if n % 8 == 1:  # the reasons change slowly; the clock is what needs the rate
                    try:
                        mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                    except Exception:
                        mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                    for bit, name in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return False

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_min_mhz": min(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


def make_inputs(workloads, name: str, rows: int | None = None):
    """CPU tensors of the workload (seeded); `rows` restricts it to a token slice."""
    M, N, K, kind = WORKLOADS[name]
    M = rows if rows is not None else M
    if name == "blockwise_prefill":
        return workloads.blockwise_prefill(M, N, K), kind
    if name == "nshard":
        return workloads.nshard(M, N, K), kind
    if name == "decode":
        return workloads.decode(M, N, K), kind
    x, y, _ = workloads.plain(M, N, K, seed=1001 if name == "plain" else 6001)
    return (x, y), kind


def oracle_runner(O, kind, inp):
    if kind == "blockwise":
        return lambda: O.c_matmul_blockwise(inp[0], inp[1], inp[2], inp[3])
    if kind == "scaled":
        return lambda: O.c_matmul_scaled(inp[0], inp[1], inp[2], inp[3])
    return lambda: O.c_matmul(inp[0], inp[1], 1.0)


def cpu_baseline(name: str, sample_seconds: float = 12.0):
    """Times the CPU restatement (oracle C port, all host threads) on a bounded sample of the workload."""
    from oracle import oracle as O

    O.build()
    M, N, K, kind = WORKLOADS[name]
    rows = min(M, 128)
    inp, _ = make_inputs(load_input_generators(), name, rows)
    run_once = oracle_runner(O, kind, inp)
    run_once()
    t0 = time.perf_counter()
    reps = 0
    while True:
        run_once()
        reps += 1
        el = time.perf_counter() - t0
        if el > sample_seconds or reps >= 50:
            break
    tops = 2.0 * rows * N * K * reps / el / 1e12
    return {"value": tops, "unit": "TOPS", "cores": O.num_threads(), "kind": "port",
            "sample": f"{reps} passes over a {rows}-token slice of the {M}x{N}x{K} {kind} workload "
                      f"({el:.1f} s of CPU time, C restatement, {O.num_threads()} threads)"}


def run_reference(args, rank):
    """The reference arm: the CPU restatement of the reference formula on the host cores (rank 0 only).  Each step is
    a row sample of the workload, sized by a short calibration so that warm-up + steps take about two minutes."""
    if rank != 0:
        return
    name = args.workload
    M, N, K, kind = WORKLOADS[name]
    from oracle import oracle as O

    O.build()
    workloads = load_input_generators()
    probe_rows = min(M, 16)
    inp, _ = make_inputs(workloads, name, probe_rows)
    fn = oracle_runner(O, kind, inp)
    fn()
    t0 = time.perf_counter()
    fn()
    per_row = (time.perf_counter() - t0) / probe_rows
    rows = int(120.0 / max(1, args.steps + args.warmup) / max(per_row, 1e-9))
    rows = max(1, min(M, rows))
    if rows >= 16:
        rows -= rows % 16
    if rows != probe_rows:
        inp, _ = make_inputs(workloads, name, rows)
        fn = oracle_runner(O, kind, inp)
    for _ in range(args.warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    el = time.perf_counter() - t0
    tops = 2.0 * rows * N * K * args.steps / el / 1e12
    cb = {"value": tops, "unit": "TOPS", "cores": O.num_threads(), "kind": "port",
          "sample": f"each step = a {rows}-token slice of the {M}x{N}x{K} {kind} workload, C restatement of the "
                    f"reference formula on {O.num_threads()} host threads"}
    assert "gemm_int8_b200" not in sys.modules, "the reference arm must not load the product package"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong" if name == "nshard" else "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": name, "M": M, "N": N, "K": K, "kind": kind},
        "cpu_baseline": cb,
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------------------------
# sweep: every other configuration, device-timed on one GPU with inputs generated on the device
# ---------------------------------------------------------------------------------------------------------------
def _time_interleaved(torch, fns, flush, iters, warm=3):
    """Median device time (ms) of each function in `fns` over `iters` launches, every launch preceded by an L2 flush
    outside its timed pair.  The functions take turns (a, b, c, a, b, c, ...), so that all of them see the same clock
    and thermal state: timed one after the other, the ratio between two libraries moved by 20 % from run to run."""
    for fn in fns:
        for _ in range(warm):
            fn()
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)] for _ in fns]
    for i in range(iters):
        for j, fn in enumerate(fns):
            a, b = ev[j][i]
            flush.max()
            a.record()
            fn()
            b.record()
    torch.cuda.synchronize()
    return [statistics.median(a.elapsed_time(b) for a, b in e) for e in ev]


def _wall_per_call(torch, fn, iters=100, warm=10, repeats=10):
    """Microseconds per call as the reference's benchmark.py measures them: time.time around `iters` calls issued
    back to back and one synchronize, mean over `repeats`."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(repeats):
        t0 = time.time()
        for _ in range(iters):
            fn()
        torch.cuda.synchronize()
        ts.append((time.time() - t0) * 1e6 / iters)
    return statistics.mean(ts)


def _time_graph_rotating(torch, make_call, sets, replays=5):
    """Launch-bound kernels: one CUDA graph walks over `sets` operand copies (more than twice the L2 in total, so
    every launch streams its weights from HBM); returns the median device time per launch (ms)."""
    for s in sets:
        make_call(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for s in sets:
            make_call(s)
    graph.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) / len(sets))
    return statistics.median(ts)


def reference_kernel_times(shapes):
    """Device time of the reference project's own operator (its Sm80 mma.sync kernel compiled for sm_100, see
    baseline/build_reference.sh) on plain shapes, measured in a process of its own; {} when it has not been built."""
    runner = os.path.join(ROOT, "baseline", "run_reference.py")
    if not os.path.exists(os.path.join(ROOT, "baseline", "_ref", "gemm_int8_CUDA.so")):
        return {}
    cases = [{"name": f"{m}x{n}x{k}", "kind": "uniform", "M": m, "N": n, "K": k, "alpha": 1.0, "seed": 1} for (m, n, k) in shapes]
    try:
        with tempfile.TemporaryDirectory() as d:
            cf, of = os.path.join(d, "cases.json"), os.path.join(d, "out.npz")
            with open(cf, "w") as f:
                json.dump(cases, f)
            res = subprocess.run([sys.executable, runner, "--cases", cf, "--out", of, "--time", "--no-outputs"], capture_output=True,
                                 text=True, timeout=600, cwd=ROOT)
            if res.returncode != 0:
                return {}
            import numpy as np

            z = np.load(of)
            return {c["name"]: float(z[c["name"] + ".us"]) for c in cases}
    except Exception:
        return {}


def run_sweep(torch, g, dev, flush, peaks, sections=None):
    """sections: None for all, or a subset of {'plain', 'blockwise', 'decode', 'quant'}."""
    rows = []
    want = lambda name: sections is None or name in sections  # noqa: E731
    gen = torch.Generator(device=dev).manual_seed(99)

    def ri8(shape):
        return torch.randint(-128, 127, shape, dtype=torch.int8, device=dev, generator=gen)

    def rf(shape, lo=0.001, span=0.02):
        return torch.rand(shape, device=dev, generator=gen) * span + lo

    def entry(config, kind, M, N, K, t_ms, t_bf16_ms, extra=None):
        ops = 2.0 * M * N * K
        n_sc = {"plain": 0, "scaled": M + N, "blockwise": (M + -(-N // 128)) * -(-K // 128)}[kind]
        byts = M * K + N * K + 2 * M * N + 4 * n_sc
        e = {"config": config, "kind": kind, "M": M, "N": N, "K": K, "us": round(t_ms * 1e3, 2),
             "tops": round(ops / t_ms / 1e9, 1), "frac_nominal_int8": round(ops / t_ms / 1e9 / NOMINAL_INT8_TOPS, 4),
             "gbs": round(byts / t_ms / 1e6, 1), "frac_hbm": round(byts / t_ms / 1e6 / peaks["hbm_gbs"], 4),
             "cublas_bf16_us": round(t_bf16_ms * 1e3, 2), "speedup_vs_cublas_bf16": round(t_bf16_ms / t_ms, 3),
             "variant": g.pick_variant({"blockwise": 2, "scaled": 1}[kind] if kind != "plain" else 0, M, N, K)}
        if extra:
            e.update(extra)
        rows.append(e)

    # plain: config 1, the target squares and the reference benchmark's nine layer shapes (benchmark.py:56-62)
    plain = [("1", 1024, 4096, 4096), ("target", 8192, 8192, 8192), ("target", 16384, 16384, 16384)]
    plain += [("reference benchmark", m, n, k) for m in (512, 1024, 2048) for (n, k) in ((4096, 4096), (14336, 4096), (4096, 14336))]
    if not want("plain"):
        plain = []
    ref_us = reference_kernel_times([(m, n, k) for (_, m, n, k) in plain]) if plain else {}
    for (cfg, M, N, K) in plain:
        x, y = ri8((M, K)), ri8((N, K))
        xb, yb = x.bfloat16(), y.bfloat16()
        iters = 5 if M * N * K > 1e12 else 30
        fns = [lambda: g.matmul(x, y, 1.0), lambda: torch.matmul(xb, yb.t())]
        if M > 16:
            fns.append(lambda: torch._int_mm(x, y.t()))
        ts = _time_interleaved(torch, fns, flush, iters)
        t, tb, ti = ts[0], ts[1], (ts[2] if M > 16 else None)
        extra = {"cublaslt_int8_us": round(ti * 1e3, 2) if ti else None}
        if cfg == "reference benchmark":
            # the reference benchmark's own measurement (benchmark.py:39-53): wall clock around 100 back-to-back calls
            # through the Python entry point after 10 warm-ups, mean of 10 repeats, no flush (warm L2)
            extra["wall_us_per_call"] = round(_wall_per_call(torch, lambda: g.matmul(x, y, 1.0)), 2)
            extra["wall_us_per_call_cublas_bf16"] = round(_wall_per_call(torch, lambda: torch.matmul(xb, yb.t())), 2)
        if f"{M}x{N}x{K}" in ref_us:
            extra["reference_sm80_kernel_us"] = round(ref_us[f"{M}x{N}x{K}"], 2)
        entry(cfg, "plain", M, N, K, t, tb, extra)
        del x, y, xb, yb
    # blockwise: config 2 and the Llama-70B sweep (config 4)
    bw = [("2", 2048, 11008, 4096)]
    bw += [("4", m, n, k) for (k, n) in ((8192, 10240), (8192, 8192), (8192, 57344), (28672, 8192)) for m in (128, 512, 2048, 8192, 16384)]
    for (cfg, M, N, K) in (bw if want("blockwise") else []):
        x, y = ri8((M, K)), ri8((N, K))
        sa, sw = rf((M, K // 128)), rf((-(-N // 128), K // 128))
        xb, yb = x.bfloat16(), y.bfloat16()
        iters = 5 if M * N * K > 1e12 else 30
        t, tb = _time_interleaved(torch, [lambda: g.matmul_blockwise(x, y, sa, sw), lambda: torch.matmul(xb, yb.t())], flush, iters)
        entry(cfg, "blockwise", M, N, K, t, tb)
        del x, y, xb, yb, sa, sw
    # decode (config 3): HBM-bound, launch-bound; CUDA-graph replays over rotating weight copies
    for (K, N) in (((4096, 4096), (4096, 14336), (14336, 4096)) if want("decode") else ()):
        n_sets = max(4, int(2.2 * 126e6 // (N * K)) + 1)
        ws = [ri8((N, K)) for _ in range(n_sets)]
        wbs = [w.bfloat16() for w in ws[: max(2, n_sets // 2)]]
        swc = rf((N,))
        for M in (1, 4, 16, 64):
            x, sx = ri8((M, K)), rf((M,))
            xb = x.bfloat16()
            t = _time_graph_rotating(torch, lambda w: g.matmul_scaled(x, w, sx, swc), ws)
            tb = _time_graph_rotating(torch, lambda w: torch.matmul(xb, w.t()), wbs)
            entry("3", "scaled", M, N, K, t, tb)
            if M == 16:
                # The same with the library's static-weights option (the host promises that the weights are not written
                # by the preceding kernel, true of this loop as of any decode loop over a loaded model): the first weight
                # tiles are requested before the dependency wait.  Off by default; reported as a row of its own.
                os.environ["GEMM_INT8_STATIC_WEIGHTS"] = "1"
                g.reload_env()
                try:
                    t2 = _time_graph_rotating(torch, lambda w: g.matmul_scaled(x, w, sx, swc), ws)
                finally:
                    os.environ.pop("GEMM_INT8_STATIC_WEIGHTS", None)
                    g.reload_env()
                entry("3", "scaled", M, N, K, t2, tb, {"option": "GEMM_INT8_STATIC_WEIGHTS=1"})
        del ws, wbs
    # activation quantisers (the step before every W8A8 GEMM): HBM-bound; bytes = input + int8 output + fp32 scales
    if want("quant"):
        shapes = [(torch.bfloat16, 2048, 4096), (torch.bfloat16, 2048, 8192), (torch.bfloat16, 16384, 8192), (torch.bfloat16, 8192, 28672),
                  (torch.float32, 2048, 8192), (torch.float32, 16384, 8192), (torch.float32, 8192, 28672)]
        for (dt, M, K) in shapes:
            a = torch.randn((M, K), device=dev, generator=gen, dtype=torch.float32).to(dt)
            fns = [lambda: g.quantize_per_token_block(a), lambda: g.hadamard_quantize_per_token_block(a), lambda: g.quantize_per_token(a)]
            names = ["quantize_per_token_block", "hadamard_quantize_per_token_block", "quantize_per_token"]
            ts = _time_interleaved(torch, fns, flush, 20)
            for nm, t in zip(names, ts):
                n_sc = M if nm == "quantize_per_token" else M * -(-K // 128)
                byts = M * K * a.element_size() + M * K + 4 * n_sc
                rows.append({"config": "f1/f2", "kind": "quantize", "op": nm, "dtype": str(dt).replace("torch.", ""), "M": M, "K": K,
                             "us": round(t * 1e3, 2), "gbs": round(byts / t / 1e6, 1), "frac_hbm": round(byts / t / 1e6 / peaks["hbm_gbs"], 4)})
            del a
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="nshard", choices=sorted(WORKLOADS))
    ap.add_argument("--M", type=int, default=0, help="override the workload's M")
    ap.add_argument("--N", type=int, default=0, help="override the workload's N")
    ap.add_argument("--K", type=int, default=0, help="override the workload's K")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--only-sweep", default="", help="skip the main workload and print only the named sweep sections "
                    "(comma-separated: plain, blockwise, decode, quant) as one JSON line; used by the profiling commands")
    ap.add_argument("--gather", default="auto", choices=["auto", "fused", "nccl"],
                    help="N > 1: all-gather fused into the GEMM epilogue (peer stores; auto), or NCCL after it")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.M or args.N or args.K:
        m, n, k, kd = WORKLOADS[args.workload]
        WORKLOADS[args.workload] = (args.M or m, args.N or n, args.K or k, kd)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch

    import gemm_int8_b200 as g
    from gemm_int8_b200 import workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    if args.only_sweep:
        # Not a bench line: the named sweep sections alone, for the profiling commands under profiles/.
        if world > 1:
            raise SystemExit("--only-sweep runs on one GPU")
        flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev).view(torch.int64)
        peaks_, _ = load_peaks()
        rows = run_sweep(torch, g, dev, flush, peaks_, sections=set(args.only_sweep.split(",")))
        print(json.dumps({"sweep_only": sorted(set(args.only_sweep.split(","))), "kernel_status": g.device_status(), "sweep": rows}))
        return

    name = args.workload
    M, N, K, kind = WORKLOADS[name]
    inputs, _ = make_inputs(workloads, name)
    sharded = world > 1 and kind == "blockwise"
    if world > 1 and not sharded:
        raise SystemExit("only the blockwise workloads shard over several GPUs")
    if args.gather == "auto":
        args.gather = "fused"  # measured faster than GEMM + NCCL all-gather at 2, 4 and 8 GPUs
    if sharded:
        from gemm_int8_b200 import dist as gdist

        x, y, sa, sw = inputs
        y, sw = gdist.shard_weight(y, sw, rank, world)
        inputs = (x, y, sa, sw)
    n_local = inputs[1].shape[0]

    # Several rotating copies of the operands so that consecutive steps never reuse lines left in L2
    # (in addition to the explicit flush below); one copy when the operands alone exceed the L2 several times.
    bytes_one = sum(t.numel() * t.element_size() for t in inputs) + 2 * M * n_local
    copies = 1 if bytes_one > 300e6 else max(3, int(300e6 // bytes_one) + 1)
    copies = min(copies, 24)
    dev_sets = [[t.to(dev) for t in inputs] for _ in range(copies)]
    # L2 flush by READING a 256 MiB buffer: it leaves clean lines behind, so the timed kernel does not pay for
    # write-backs of somebody else's dirty data (a write-based flush would add that DRAM traffic to it).
    flush_buf = torch.zeros(256 << 20, dtype=torch.uint8, device=dev).view(torch.int64)

    if kind == "blockwise":
        gemm = lambda s: g.matmul_blockwise(s[0], s[1], s[2], s[3])  # noqa: E731
    elif kind == "scaled":
        gemm = lambda s: g.matmul_scaled(s[0], s[1], s[2], s[3])  # noqa: E731
    else:
        gemm = lambda s: g.matmul(s[0], s[1], 1.0)  # noqa: E731
    op = gemm

    fused = None
    if sharded:
        if args.gather == "fused":
            # every rank's kernel writes its column slice into every rank's full [M, N] matrix; the step ends with
            # the barrier after which that matrix is complete
            fused = gdist.FusedGatherGemm(M, N)
            op = lambda s: fused.run(s[0], s[1], s[2], s[3])  # noqa: E731
        else:
            gather_out = torch.empty((world, M, n_local), dtype=torch.bfloat16, device=dev)
            op = lambda s: gdist.all_gather_slices(gemm(s), gather_out)  # noqa: E731

    def timed_steps(fn, n):
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        for i in range(n):
            flush_buf.max()  # reads 256 MiB: evicts L2 (126 MB) without leaving dirty lines
            starts[i].record()
            fn(dev_sets[i % copies])
            ends[i].record()
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in zip(starts, ends)]

    def max_over_ranks(v):
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    use_graph = kind == "scaled" and M <= 64 and dist is None
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        if use_graph:
            # Launch-bound kernels (tens of microseconds): the steps are captured in a CUDA graph that walks over the
            # rotating operand copies (their total exceeds twice the L2, so every launch streams its weights from
            # HBM) and the replays are timed with events; no flush kernels sit between the steps.
            copies_needed = max(copies, int(300e6 // bytes_one) + 1)
            while len(dev_sets) < copies_needed:
                dev_sets.append([t.to(dev) for t in inputs])
            copies = len(dev_sets)
            for s_ in dev_sets:
                op(s_)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for s_ in dev_sets:
                    op(s_)
            replays_w = max(1, -(-args.warmup // copies))
            replays = max(1, -(-args.steps // copies))
            args.steps = replays * copies
            for _ in range(replays_w):
                graph.replay()
            torch.cuda.synchronize()
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(replays)]
            for a, b in evs:
                a.record()
                graph.replay()
                b.record()
            torch.cuda.synchronize()
            times = [a.elapsed_time(b) / copies for a, b in evs for _ in range(copies)]
            gemm_times = times
        else:
            timed_steps(op, args.warmup)
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            times = timed_steps(op, args.steps)
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
            gemm_times = times
            if sharded:  # the GEMM alone (the fused form has no GEMM-only step: it is run without its barrier)
                only = (lambda s: fused.run(s[0], s[1], s[2], s[3], barrier=False)) if fused is not None else gemm
                timed_steps(only, 3)
                torch.cuda.synchronize()
                dist.barrier()
                gemm_times = timed_steps(only, max(5, min(args.steps, 20)))
                torch.cuda.synchronize()
                dist.barrier()
    ms_per_step = max_over_ranks(sum(times)) / args.steps
    gemm_ms = max_over_ranks(statistics.mean(gemm_times))
    clock_summary = clocks.summary()

    # ---- cuBLAS bf16 on the same per-rank shape (torch.matmul(a_bf16, b_bf16.t()), as the reference's benchmark.py:77)
    cublas = None
    if kind != "scaled" or M > 64:
        xb, yb = dev_sets[0][0].bfloat16(), dev_sets[0][1].bfloat16()
        bf = lambda s: torch.matmul(xb, yb.t())  # noqa: E731
        timed_steps(bf, 3)
        tb = timed_steps(bf, max(5, min(args.steps, 20)))
        tb_ms = max_over_ranks(statistics.mean(tb))
        cublas = {"ms": tb_ms, "tflops": 2.0 * M * n_local * K / tb_ms / 1e9, "shape": [M, n_local, K],
                  "how": "torch.matmul(x.bfloat16(), y.bfloat16().t()), same flush and events, max over ranks"}
        del xb, yb
    status = g.device_status()

    # ---- end to end through the public API with HOST buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e:
        host_in = [t.pin_memory() for t in inputs]
        # Sharded: every rank copies its operands in.  Fused gather: every rank holds the assembled [M, N] matrix and reads
        # back its own block of M / world rows, so that the whole result reaches host memory exactly once, spread over
        # the ranks' PCIe links.  NCCL gather (block layout [world, M, n_local]): rank 0 reads everything back.
        rows_each = M // world if (sharded and fused is not None and M % world == 0) else 0
        reads_back = (not sharded) or rank == 0 or rows_each > 0
        if sharded:
            out_shape = ((rows_each, N) if rows_each else (M, N)) if fused is not None else (world, M, n_local)
        else:
            out_shape = (M, n_local)
        host_out = torch.empty(out_shape if reads_back else (1,), dtype=torch.bfloat16).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host_in)
        d2h = host_out.numel() * host_out.element_size() if reads_back else 0
        e2e_steps = max(3, min(args.steps, 10))

        pipe = None
        if not sharded:
            # The library's host-buffer front end: H2D, GEMM and D2H of consecutive steps overlap on three streams
            # (every step still copies all of its operands in and its whole result out).
            from gemm_int8_b200.host import HostPipeline

            pipe = HostPipeline({"blockwise": "blockwise", "scaled": "scaled"}.get(kind, "plain"), depth=2, device=dev)

        def e2e_step():
            if pipe is not None:
                pipe.submit(host_in, host_out)
                return
            s = [t.to(dev, non_blocking=True) for t in host_in]
            out = op(s)
            if reads_back:
                host_out.copy_(out[rank * rows_each:(rank + 1) * rows_each] if rows_each else out, non_blocking=True)

        for _ in range(2):
            e2e_step()
        if pipe is not None:
            pipe.drain()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        es, ee = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        es.record()
        if pipe is not None:
            pipe.start_after(es)
        for _ in range(e2e_steps):
            e2e_step()
        if pipe is not None:
            ee = pipe.finish_event()
        else:
            ee.record()
        torch.cuda.synchronize()
        e2e_ms = max_over_ranks(es.elapsed_time(ee))
        tot = torch.tensor([float(h2d), float(d2h)], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(tot)
        e2e = {"value": 2.0 * M * N * K * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS",
               "h2d_bytes_per_step": int(tot[0].item()), "d2h_bytes_per_step": int(tot[1].item()), "steps": e2e_steps,
               "api": ("gemm_int8_b200.host.HostPipeline (2 calls in flight)" if pipe is not None else
                       "gemm_int8_b200 ops + gather on one stream per rank; every rank copies its operands in and " +
                       ("its own M / world rows of the assembled matrix out (the whole result is read back once, spread "
                        "over the ranks)" if rows_each else "rank 0 copies the assembled matrix out"))}
        del host_in, host_out

    sweep = None
    if world == 1 and rank == 0 and not args.no_sweep:
        for s_ in dev_sets:
            s_.clear()
        torch.cuda.empty_cache()
        peaks_, _ = load_peaks()
        try:
            sweep = run_sweep(torch, g, dev, flush_buf, peaks_)
        except Exception as exc:  # the main line must not be lost to the extra rows
            sweep = [{"error": repr(exc)[:300]}]
        status = status or g.device_status()

    # N > 1: the K-sharded (row-parallel) form on the Llama-70B down-projection shape of config 4 (K = 28672 split over the
    # ranks): GEMM with the reduce-scatter fused into its epilogue against GEMM + NCCL all-to-all + ordered sum.
    kshard = None
    if sharded and not args.no_sweep:
        try:
            from gemm_int8_b200 import dist as gdist2

            for s_ in dev_sets:
                s_.clear()
            torch.cuda.empty_cache()
            Mk, Nk, Kk = 16384, 8192, 28672
            k0, k1 = gdist2.kshard_bounds(Kk, world, rank)
            genk = torch.Generator(device=dev).manual_seed(77)
            xk = torch.randint(-128, 127, (Mk, k1 - k0), dtype=torch.int8, device=dev, generator=genk)
            yk = torch.randint(-128, 127, (Nk, k1 - k0), dtype=torch.int8, device=dev, generator=genk)
            sak = torch.rand((Mk, (k1 - k0) // 128), device=dev, generator=genk) * 0.02 + 0.001
            swk = torch.rand((Nk // 128, (k1 - k0) // 128), device=dev, generator=genk) * 0.02 + 0.001
            frs = gdist2.FusedReduceScatterGemm(Mk, Nk)

            def timed_k(fn, n=6):
                ts = []
                for _ in range(n):
                    dist.barrier()
                    flush_buf.max()
                    torch.cuda.synchronize()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    fn()
                    b.record()
                    torch.cuda.synchronize()
                    ts.append(a.elapsed_time(b))
                return max_over_ranks(statistics.median(ts[1:]))

            t_f = timed_k(lambda: frs.run(xk, yk, sak, swk))
            t_n = timed_k(lambda: gdist2.matmul_blockwise_ksharded(xk, yk, sak, swk))
            same = bool(torch.equal(frs.run(xk, yk, sak, swk).view(torch.int16),
                                    gdist2.matmul_blockwise_ksharded(xk, yk, sak, swk).view(torch.int16)))
            frs.close()
            kshard = {"shape": [Mk, Nk, Kk], "ranks": world, "fused_reduce_scatter_ms": round(t_f, 4),
                      "gemm_nccl_all_to_all_sum_ms": round(t_n, 4), "tops_fused": round(2.0 * Mk * Nk * Kk / t_f / 1e9, 1),
                      "results_identical": same,
                      "how": "device time per call incl. the cross-rank barrier and the ordered sum, L2 flushed before, median of 5, max over ranks"}
            del xk, yk, sak, swk
        except Exception as exc:  # the main line must not be lost to this extra
            kshard = {"error": repr(exc)[:200]}
        status = status or g.device_status()

    if rank == 0:
        peaks, peak_kind = load_peaks()
        total_ops = 2.0 * M * N * K
        tops = total_ops / (ms_per_step * 1e-3) / 1e12
        per_gpu_ops = 2.0 * M * n_local * K
        achieved = per_gpu_ops / (gemm_ms * 1e-3) / 1e12
        # a step of several milliseconds runs at the sustained clock: compare with the sustained peak there
        long_step = gemm_ms > 2.0
        bf16_peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) if long_step else peaks["bf16_tflops"]
        int8_peak = 2.0 * bf16_peak
        cb = None if args.no_cpu_baseline else cpu_baseline(name)
        n_scales = sum(t.numel() for t in inputs[2:]) if len(inputs) > 2 else 0
        algo_bytes = M * K + n_local * K + 2 * M * n_local + 4 * n_scales
        if kind == "scaled" and M <= 64:
            gbs = algo_bytes / (gemm_ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                        "note": f"algorithmic bytes {algo_bytes} per launch; peak = {peak_kind} copy bandwidth "
                                f"({peaks['hbm_gbs']} GB/s) of {peak_kind}; min step {min(times):.4f} ms"}
        else:
            roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s",
                        "frac": achieved / int8_peak, "traffic": None,
                        "note": f"int8 TOP/s of the GEMM launch (per GPU); peak = 2 x {peak_kind} bf16 "
                                f"{'sustained' if long_step else 'burst'} ({bf16_peak} TFLOP/s) of {peak_kind}; "
                                f"against the nominal {NOMINAL_INT8_TOPS:.0f} TOP/s: {achieved / NOMINAL_INT8_TOPS:.3f}; "
                                f"min step {min(times):.4f} ms"}
        if (name, M, N, K) in NCU_TRAFFIC and world == 1:
            roofline["traffic"], roofline["traffic_source"] = NCU_TRAFFIC[(name, M, N, K)]
            roofline["algorithmic_bytes"] = algo_bytes
        mhz = clock_summary.get("sm_mhz")
        line = {
            "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "gemm_ms": gemm_ms,
            "ms_x_median_mhz": ms_per_step * mhz if mhz else None,
            "higher_is_better": True,
            "scaling": "strong" if sharded or name == "nshard" else "weak", "vs_baseline": None,
            "speedup_vs_cublas_bf16": (cublas["ms"] / gemm_ms) if cublas else None, "cublas_bf16": cublas,
            "dtype": "int8", "data": "synthetic",
            "config": {"workload": name, "M": M, "N": N, "K": K, "kind": kind, "per_gpu_N": n_local,
                       "variant": g.pick_variant({"blockwise": 2, "scaled": 1}.get(kind, 0), M, n_local, K),
                       "l2": (f"CUDA-graph replay over {copies} rotating operand copies (> 2 x L2 in total), no flush"
                              if use_graph else
                              f"flushed between steps (256 MiB read); operands {bytes_one / 1e6:.0f} MB per rank"
                              + (f", rotated over {copies} copies" if copies > 1 else "")),
                       "parallelism": (f"nshard{world}+allgather({args.gather})" if sharded else "single GPU"),
                       "frac_of_nominal_int8_peak_4500": tops / world / NOMINAL_INT8_TOPS},
            "roofline": roofline,
            "cpu_baseline": cb,
            "e2e": e2e,
            # one GEMM kernel of this library per step; two where the dispatch adds a second launch for a thin last wave
            # (dense: split-K kernel; blockwise: the remaining columns with narrower tiles)
            "gpu_launches": args.steps * (2 if any(t in g.pick_variant({"blockwise": 2, "scaled": 1}.get(kind, 0), M, n_local, K)
                                                   for t in ("+splitk", "+columns")) and not sharded else 1),
            "clocks": clock_summary,
            "kernel_status": status,
            "kshard": kshard,
            "sweep": sweep,
        }
        print(json.dumps(line))
    if fused is not None:
        fused.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

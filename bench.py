#!/usr/bin/env python
"""Benchmark of the INT8 GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one blockwise-dequantised W8A8 GEMM over one batch of synthetic tokens.  Default workload:
the prefill configuration M=2048, K=4096, N=11008 (per-token-per-128-K activation scales, per-128x128
weight scales, bf16 output).  With N > 1 ranks (launched by torch.distributed.run, one rank per GPU)
every rank processes its own token batch against its own copy of the weights -- data parallel, no
collective on the data path (weak scaling); `--workload nshard` instead runs the 16384 x 57344 x 8192
GEMM split column-wise over the ranks followed by an NCCL all-gather of the bf16 slices (strong scaling).

Rank 0 prints ONE JSON line.  `value` is whole-job INT8 TOPS with inputs resident in HBM (CUDA events
around each step on the launching stream, L2 flushed between steps, max over ranks); `e2e` is the same
metric through the public Python op with pinned HOST buffers, host<->device copies inside the timed
region; `roofline` relates the kernel to the measured tensor peak; `cpu_baseline` times the CPU
restatement of the same arithmetic on this box's host cores.

`--impl reference` times only that CPU restatement (the reference project has no CPU implementation of
its own and its CUDA build needs CUTLASS, which is not vendored), with all host threads, on the same
workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "INT8 TOPS per shape (fraction of B200 INT8 peak); speedup vs cuBLAS BF16"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures summarised under
# profiles/: keyed by (workload, M, N, K).  Other shapes report null.
NCU_TRAFFIC = {
    ("blockwise_prefill", 2048, 11008, 4096): (65.9e6, "profiles/blockwise_gemm_kernel__blockwise_prefill_2048x11008x4096.md"),
    ("square8192", 8192, 8192, 8192): (444.3e6, "profiles/dense_gemm_kernel__square8192.md"),
    ("decode", 16, 14336, 4096): (58.97e6, "profiles/smallm_cluster_kernel__decode_16x14336x4096.md"),
}

WORKLOADS = {
    # name: (M, N, K, kind)
    "blockwise_prefill": (2048, 11008, 4096, "blockwise"),
    "plain": (1024, 4096, 4096, "plain"),
    "nshard": (16384, 57344, 8192, "blockwise"),
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


class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU through NVML (read-only) while a region runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.005):
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
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
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
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


def make_inputs(name: str, world: int, rank: int):
    """CPU tensors of the workload (seeded; rank r uses its own token batch in the data-parallel mode)."""
    from gemm_int8_b200 import workloads

    M, N, K, kind = WORKLOADS[name]
    if name == "blockwise_prefill":
        return workloads.blockwise_prefill(M, N, K, seed=2001 + 10 * rank), kind
    if name == "nshard":
        return workloads.nshard(M, N, K), kind
    if name == "decode":
        return workloads.decode(M, N, K), kind
    x, y, _ = workloads.plain(M, N, K, seed=1001 if name == "plain" else 6001)
    return (x, y), kind


def cpu_baseline(name: str, budget_s: float = 12.0):
    """Times the CPU restatement (oracle C port, all host threads) on a bounded sample of the workload."""
    from oracle import oracle as O

    O.build()
    M, N, K, kind = WORKLOADS[name]
    (inputs, _) = make_inputs(name, 1, 0) if name != "nshard" else (None, None)
    if name == "nshard":
        from gemm_int8_b200 import workloads

        inputs = workloads.nshard(256, N, K)  # a 256-token slice of the full workload
    rows = min(M, 256)
    x = inputs[0][:rows].contiguous()

    def run_once():
        if kind == "blockwise":
            O.c_matmul_blockwise(x, inputs[1], inputs[2][:rows].contiguous(), inputs[3])
        elif kind == "scaled":
            O.c_matmul_scaled(x, inputs[1], inputs[2][:rows].contiguous(), inputs[3])
        else:
            O.c_matmul(x, inputs[1], 1.0)

    run_once()
    t0 = time.perf_counter()
    reps = 0
    while True:
        run_once()
        reps += 1
        el = time.perf_counter() - t0
        if el > budget_s or reps >= 50:
            break
    tops = 2.0 * rows * N * K * reps / el / 1e12
    return {"value": tops, "unit": "TOPS", "cores": O.num_threads(), "kind": "port",
            "sample": f"{reps} passes over a {rows}-token slice of the {M}x{N}x{K} {kind} workload "
                      f"({el:.1f} s of CPU time, C restatement, {O.num_threads()} threads)"}


def run_reference(args, rank):
    """The reference arm: the CPU restatement of the reference formula on the host cores (rank 0 only)."""
    if rank != 0:
        return
    name = args.workload
    M, N, K, kind = WORKLOADS[name]
    from oracle import oracle as O

    O.build()
    rows = min(M, 256)
    from gemm_int8_b200 import workloads

    if kind == "blockwise":
        inp = workloads.blockwise_prefill(rows, N, K) if name == "blockwise_prefill" else workloads.nshard(rows, N, K)
        fn = lambda: O.c_matmul_blockwise(inp[0], inp[1], inp[2], inp[3])  # noqa: E731
    elif kind == "scaled":
        inp = workloads.decode(rows, N, K)
        fn = lambda: O.c_matmul_scaled(inp[0], inp[1], inp[2], inp[3])  # noqa: E731
    else:
        inp = workloads.plain(rows, N, K)
        fn = lambda: O.c_matmul(inp[0], inp[1], 1.0)  # noqa: E731
    steps = max(1, min(args.steps, 20))
    warm = max(1, min(args.warmup, 3))
    for _ in range(warm):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    el = time.perf_counter() - t0
    tops = 2.0 * rows * N * K * steps / el / 1e12
    cb = {"value": tops, "unit": "TOPS", "cores": O.num_threads(), "kind": "port",
          "sample": f"each step = a {rows}-token slice of the {M}x{N}x{K} {kind} workload, C restatement of the "
                    f"reference formula on {O.num_threads()} host threads"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": el / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": name, "M": M, "N": N, "K": K, "sample_rows": rows},
        "cpu_baseline": cb,
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="blockwise_prefill", choices=sorted(WORKLOADS))
    ap.add_argument("--M", type=int, default=0, help="override the workload's M")
    ap.add_argument("--N", type=int, default=0, help="override the workload's N")
    ap.add_argument("--K", type=int, default=0, help="override the workload's K")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--gather", default="auto", choices=["auto", "fused", "nccl"],
                    help="nshard workload: all-gather fused into the GEMM epilogue (peer stores), or NCCL after it; "
                         "auto = fused on 2 GPUs (measured faster), NCCL on more (the fused form needs its opt-in "
                         "wide store boxes to win there)")
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

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    name = args.workload
    M, N, K, kind = WORKLOADS[name]
    inputs, _ = make_inputs(name, world, rank)
    nshard = name == "nshard"
    if args.gather == "auto":
        args.gather = "fused" if world == 2 else "nccl"
    if nshard:
        from gemm_int8_b200 import dist as gdist

        x, y, sa, sw = inputs
        y, sw = gdist.shard_weight(y, sw, rank, world)
        inputs = (x, y, sa, sw)
    n_local = inputs[1].shape[0]

    # Several rotating copies of the operands so that consecutive steps never reuse lines left in L2
    # (in addition to the explicit flush below).
    bytes_one = sum(t.numel() * t.element_size() for t in inputs) + 2 * M * n_local
    copies = 1 if bytes_one > 300e6 else max(3, int(300e6 // bytes_one) + 1)
    copies = min(copies, 24)
    dev_sets = [[t.to(dev) for t in inputs] for _ in range(copies)]
    # L2 flush by READING a 256 MiB buffer: it leaves clean lines behind, so the timed kernel does not pay for
    # write-backs of somebody else's dirty data (a write-based flush would add that DRAM traffic to it).
    flush_buf = torch.zeros(256 << 20, dtype=torch.uint8, device=dev).view(torch.int64)

    if kind == "blockwise":
        op = lambda s: g.matmul_blockwise(s[0], s[1], s[2], s[3])  # noqa: E731
    elif kind == "scaled":
        op = lambda s: g.matmul_scaled(s[0], s[1], s[2], s[3])  # noqa: E731
    else:
        op = lambda s: g.matmul(s[0], s[1], 1.0)  # noqa: E731

    gather_out = None
    if nshard and world > 1:
        from gemm_int8_b200 import dist as gdist

        if args.gather == "fused":
            # every rank's kernel writes its column slice into every rank's full [M, N] matrix; the step ends with
            # the barrier after which that matrix is complete
            fused = gdist.FusedGatherGemm(M, N)
            op = lambda s: fused.run(s[0], s[1], s[2], s[3])  # noqa: E731
        else:
            gather_out = torch.empty((world, M, n_local), dtype=torch.bfloat16, device=dev)
            inner = op
            op = lambda s: gdist.all_gather_slices(inner(s), gather_out)  # noqa: E731

    def timed_steps(n):
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        for i in range(n):
            flush_buf.max()  # reads 256 MiB: evicts L2 (126 MB) without leaving dirty lines
            starts[i].record()
            op(dev_sets[i % copies])
            ends[i].record()
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in zip(starts, ends)]

    use_graph = kind == "scaled" and M <= 64 and dist is None
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
        with ClockSampler(physical_gpu_index(local_rank)) as clocks:
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(replays)]
            for a, b in evs:
                a.record()
                graph.replay()
                b.record()
            torch.cuda.synchronize()
        times = [a.elapsed_time(b) / copies for a, b in evs for _ in range(copies)]
    else:
        timed_steps(args.warmup)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        with ClockSampler(physical_gpu_index(local_rank)) as clocks:
            times = timed_steps(args.steps)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
    total_ms = sum(times)
    if dist is not None:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    status = g.device_status()

    # ---- end to end through the public op with HOST buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e:
        host_in = [t.pin_memory() for t in inputs]
        # N-shard: every rank reads back the gathered result ([world, M, N/world], the collective's block layout)
        out_shape = ((M, N) if args.gather == "fused" else (world, M, n_local)) if (nshard and world > 1) else (M, n_local)
        host_out = torch.empty(out_shape, dtype=torch.bfloat16).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host_in)
        d2h = host_out.numel() * host_out.element_size()
        e2e_steps = max(3, min(args.steps, 20))

        pipe = None
        if not nshard:
            # The library's host-buffer front end: H2D, GEMM and D2H of consecutive steps overlap on three streams
            # (every step still copies all of its operands in and its whole result out).
            from gemm_int8_b200.host import HostPipeline

            pipe = HostPipeline({"blockwise": "blockwise", "scaled": "scaled"}.get(kind, "plain"), depth=3, device=dev)

        def e2e_step():
            if pipe is not None:
                pipe.submit(host_in, host_out)
                return
            s = [t.to(dev, non_blocking=True) for t in host_in]
            out = op(s)
            host_out.copy_(out, non_blocking=True)

        for _ in range(3):
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
        e2e_ms = es.elapsed_time(ee)
        if dist is not None:
            t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        units = world if not nshard else 1
        e2e = {"value": 2.0 * M * (N if nshard else n_local) * K * units * e2e_steps / (e2e_ms * 1e-3) / 1e12,
               "unit": "TOPS", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "api": "gemm_int8_b200.host.HostPipeline (3 calls in flight)" if pipe is not None else "gemm_int8_b200 ops, one stream"}

    if rank == 0:
        peaks, peak_kind = load_peaks()
        total_ops = 2.0 * M * N * K * (1 if nshard else world)
        tops = total_ops / (ms_per_step * 1e-3) / 1e12
        per_gpu_ops = 2.0 * M * n_local * K
        kernel_ms = statistics.mean(times)  # rank 0's own kernel time (the GEMM launch dominates a step)
        achieved = per_gpu_ops / (kernel_ms * 1e-3) / 1e12
        int8_peak = 2.0 * peaks["bf16_tflops"]
        cb = None if args.no_cpu_baseline else cpu_baseline(name)
        n_scales = sum(t.numel() for t in inputs[2:]) if len(inputs) > 2 else 0
        algo_bytes = M * K + n_local * K + 2 * M * n_local + 4 * n_scales
        if kind == "scaled" and M <= 64:
            gbs = algo_bytes / (kernel_ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                        "note": f"algorithmic bytes {algo_bytes} per launch; peak = {peak_kind} copy bandwidth "
                                f"({peaks['hbm_gbs']} GB/s) of {peak_kind}; min step {min(times):.4f} ms"}
        else:
            roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s",
                        "frac": achieved / int8_peak, "traffic": None,
                        "note": f"int8 TOP/s of the GEMM launch; peak = 2 x {peak_kind} bf16 burst "
                                f"({peaks['bf16_tflops']} TFLOP/s) of {peak_kind}; min step {min(times):.4f} ms"}
        if (name, M, N, K) in NCU_TRAFFIC and world == 1:
            roofline["traffic"], roofline["traffic_source"] = NCU_TRAFFIC[(name, M, N, K)]
            roofline["algorithmic_bytes"] = algo_bytes
        line = {
            "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if nshard else "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": name, "M": M, "N": N, "K": K, "kind": kind, "per_gpu_N": n_local,
                       "variant": g.pick_variant({"blockwise": 2, "scaled": 1}.get(kind, 0), M, n_local, K),
                       "l2": (f"CUDA-graph replay over {copies} rotating operand copies (> 2 x L2 in total), no flush"
                              if use_graph else
                              f"flushed between steps (256 MiB read) and operands rotated over {copies} copies"), "parallelism": f"dp{world}" if not nshard else f"nshard{world}+allgather({args.gather if world > 1 else 'none'})",
                       "frac_of_nominal_int8_peak_4500": tops / world / 4500.0 if not nshard else None},
            "roofline": roofline,
            "cpu_baseline": cb,
            "e2e": e2e,
            "gpu_launches": args.steps,
            "clocks": clocks.summary(),
            "kernel_status": status,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Host-buffer front end: operands in pinned host memory, result written to pinned host memory.

The C ABI and the torch ops take device pointers, like the reference's `gemm_int8.matmul` (which asserts CUDA
tensors, gemm_int8/__init__.py:16-35).  A caller whose operands live on the host pays two PCIe transfers per call;
`HostPipeline` overlaps them across consecutive calls: three streams (host-to-device, compute, device-to-host)
and `depth` slots of device buffers, so that while call i computes, call i+1's operands are on their way in and
call i-1's result is on its way out (PCIe is full duplex).  Every call still copies all of its operands in and its
whole result out; results are bit-identical to the device-tensor ops.

    pipe = HostPipeline("blockwise", depth=3)
    for x, w, sa, sw, out in batches:          # pinned CPU tensors
        pipe.submit((x, w, sa, sw), out)
    pipe.drain()                               # all `out` tensors are complete after this
"""
from __future__ import annotations

import torch

import gemm_int8_b200 as g

_OPS = {
    "plain": lambda s: g.matmul(s[0], s[1], 1.0),
    "scaled": lambda s: g.matmul_scaled(s[0], s[1], s[2], s[3]),
    "blockwise": lambda s: g.matmul_blockwise(s[0], s[1], s[2], s[3]),
}


class _Slot:
    def __init__(self):
        self.dev_in = None          # device copies of the operands (reused while shapes stay the same)
        self.dev_out = None
        self.loaded = torch.cuda.Event()
        self.computed = torch.cuda.Event()
        self.stored = torch.cuda.Event()
        self.busy = False


class HostPipeline:
    """Runs one of the GEMM ops ("plain", "scaled", "blockwise") on pinned host operands, `depth` calls in flight."""

    def __init__(self, kind: str = "blockwise", depth: int = 3, device: torch.device | int | None = None):
        if kind not in _OPS:
            raise ValueError(f"kind must be one of {sorted(_OPS)}")
        if depth < 1:
            raise ValueError("depth must be at least 1")
        if not torch.cuda.is_available():
            raise RuntimeError("HostPipeline needs a CUDA device (there is no CPU path)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.op = _OPS[kind]
        self.slots = [_Slot() for _ in range(depth)]
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.calls = 0

    def start_after(self, event: torch.cuda.Event) -> None:
        """Orders everything submitted from now on after `event` (used to bracket a timed region)."""
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(event)

    def submit(self, host_in, host_out: torch.Tensor) -> None:
        """Queues one call.  `host_in` and `host_out` must be pinned and must stay untouched until drain()
        (or until `depth` further calls have been submitted)."""
        for t in (*host_in, host_out):
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError("HostPipeline operands and result must be pinned CPU tensors")
        slot = self.slots[self.calls % len(self.slots)]
        self.calls += 1
        if slot.busy:
            slot.stored.synchronize()  # the slot's previous result has left the device; its buffers are free
        if slot.dev_in is None or any(d.shape != h.shape or d.dtype != h.dtype for d, h in zip(slot.dev_in, host_in)) \
                or len(slot.dev_in) != len(host_in):
            slot.dev_in = [torch.empty(h.shape, dtype=h.dtype, device=self.device) for h in host_in]
        with torch.cuda.stream(self.s_in):
            for d, h in zip(slot.dev_in, host_in):
                d.copy_(h, non_blocking=True)
            slot.loaded.record()
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(slot.loaded)
            slot.dev_out = self.op(slot.dev_in)
            slot.computed.record()
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(slot.computed)
            host_out.copy_(slot.dev_out, non_blocking=True)
            slot.stored.record()
        # The caching allocator must not hand the result buffer to another stream's allocation before the copy-out.
        slot.dev_out.record_stream(self.s_out)
        slot.busy = True

    def finish_event(self) -> torch.cuda.Event:
        """An event on the current stream that completes after everything submitted so far."""
        cur = torch.cuda.current_stream(self.device)
        for slot in self.slots:
            if slot.busy:
                cur.wait_event(slot.stored)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(cur)
        return ev

    def drain(self) -> None:
        for slot in self.slots:
            if slot.busy:
                slot.stored.synchronize()
                slot.busy = False

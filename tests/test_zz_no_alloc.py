"""GPU test of gi8_matmul_scaled_static, the entry point for callers that must not allocate device memory
(a runtime whose pool already owns all of HBM, a decode loop that cannot take cudaMalloc's device-wide
synchronisation, a C host without a device allocator).  Its split-K scratch is a fixed array inside the
library, so the caller passes inputs and outputs only.

The file name sorts last on purpose: under `pytest -x` every other test has run before this one can fail.
It is self-contained (own inputs, own library handle) and passes alone in a fresh process as well as after
the rest of the suite.  The result must equal gi8_matmul_scaled (caller-owned workspace) AND the CPU oracle bit
for bit -- the same bar the other parity tests use -- on two calls in a row that share the static array."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _call_static(C, x, y, sx, sw, stream):
    M, N, K = x.shape[0], y.shape[0], x.shape[1]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    rc = C.gi8_matmul_scaled_static(_p(x), _p(y), _p(sx), _p(sw), _p(out), M, N, K, stream)
    assert rc == 0, C.gi8_last_error()
    return out


def _call_workspace(C, x, y, sx, sw, stream):
    M, N, K = x.shape[0], y.shape[0], x.shape[1]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    nbytes = int(C.gi8_matmul_scaled_workspace_bytes(M, N, K))
    ws = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    rc = C.gi8_matmul_scaled(_p(x), _p(y), _p(sx), _p(sw), _p(out), M, N, K, _p(ws), nbytes, stream)
    assert rc == 0, C.gi8_last_error()
    return out


def test_static_scratch_entry_matches_workspace_entry_twice(oracle):
    import gemm_int8_b200 as g

    C = g._C
    g.force_variant("smallm")    # the comparison entry point then runs the same split-K kernel with caller scratch
    try:
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        gen = torch.Generator().manual_seed(2718)
        # two calls in a row with different shapes and data: the second must not see the first one's leftovers
        for (M, N, K) in [(16, 4096, 4096), (48, 1000, 2048)]:
            xc = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=gen)
            yc = torch.randint(-128, 128, (N, K), dtype=torch.int8, generator=gen)
            sxc = torch.rand(M, generator=gen) * 0.05 + 1e-3
            swc = torch.rand(N, generator=gen) * 0.05 + 1e-3
            x, y, sx, sw = xc.to(dev), yc.to(dev), sxc.to(dev), swc.to(dev)
            assert int(C.gi8_matmul_scaled_workspace_bytes(M, N, K)) > 0, "shape must exercise the split-K scratch"
            expect = _call_workspace(C, x, y, sx, sw, stream)
            got = _call_static(C, x, y, sx, sw, stream)
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int16), expect.view(torch.int16))
            again = _call_static(C, x, y, sx, sw, stream)       # same inputs, straight after
            torch.cuda.synchronize()
            assert torch.equal(again.view(torch.int16), expect.view(torch.int16))
            ref_bits = oracle.c_matmul_scaled(xc, yc, sxc, swc)  # the CPU restatement, independent of both entry points
            assert (oracle.bf16_bits(got) == ref_bits).all() and (oracle.bf16_bits(again) == ref_bits).all()
    finally:
        g.force_variant(None)
    assert g.device_status() == 0


def test_static_scratch_entry_rejects_what_does_not_fit():
    import gemm_int8_b200 as g

    C = g._C
    dev = torch.device("cuda", 0)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    # M = 100 -> token tile 128; N = 12544 -> 98 weight tiles, split in two over K:
    # 98 * 128 * 512 bytes = 6.4 MB of scratch > 4 MiB
    M, big_n, K = 100, 12544, 512
    x = torch.zeros((M, K), dtype=torch.int8, device=dev)
    y = torch.zeros((big_n, K), dtype=torch.int8, device=dev)
    sx = torch.ones(M, device=dev)
    sw = torch.ones(big_n, device=dev)
    out = torch.empty((M, big_n), dtype=torch.bfloat16, device=dev)
    rc = C.gi8_matmul_scaled_static(_p(x), _p(y), _p(sx), _p(sw), _p(out), M, big_n, K, stream)
    assert rc == 2 and b"GI8_STATIC_SCRATCH_BYTES" in C.gi8_last_error()
    x2 = torch.zeros((129, K), dtype=torch.int8, device=dev)
    rc = C.gi8_matmul_scaled_static(_p(x2), _p(y), _p(sx), _p(sw), _p(out), 129, 128, K, stream)
    assert rc == 2 and b"M <= 128" in C.gi8_last_error()

"""The gathering form of the blockwise GEMM (gi8_matmul_blockwise_allgather) driven on ONE GPU through the C ABI:
the output matrices are all local, so the epilogue that multi-GPU runs use for their peer stores is compared with
the CPU oracle without a second device.  Covers the kernel that entry point dispatches to on edge shapes, on the
prefill configuration at full size and on the 128-token Llama-70B shapes, and the column-slice rules: a slice must
never write outside its own columns, whatever its width."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SENTINEL = 0x7FC1  # a bf16 NaN pattern no GEMM result takes


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _gather_call(g, x, y, sa, sw, outs, n_total, col0):
    M, K = x.shape
    N = y.shape[0]
    arr = (ctypes.c_void_p * len(outs))(*[o.data_ptr() for o in outs])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return g._C.gi8_matmul_blockwise_allgather(_p(x), _p(y), _p(sa), sa.stride(0), _p(sw), sw.stride(0), arr, len(outs),
                                               M, N, K, n_total, col0, stream)


def _inputs(M, N, K, seed):
    gen = torch.Generator().manual_seed(seed)
    KB, NB = -(-K // 128), -(-N // 128)
    x = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=gen)
    y = torch.randint(-128, 128, (N, K), dtype=torch.int8, generator=gen)
    sa = torch.rand(M, KB, generator=gen) * 0.02 + 1e-3
    sw = torch.rand(NB, KB, generator=gen) * 0.02 + 1e-3
    return x, y, sa, sw


@pytest.fixture(scope="module")
def g():
    import gemm_int8_b200 as g

    yield g
    g.force_variant(None)
    assert g.device_status() == 0, "a kernel recorded an expired wait"


@pytest.mark.parametrize("variant", [None, "dense_bn256", "dense_bn128", "dense_bn64", "pair"])
def test_gather_entry_one_matrix_matches_oracle(g, oracle, variant):
    g.force_variant(variant)
    for i, (M, N, K) in enumerate([(1, 32, 16), (33, 160, 144), (129, 256, 400), (257, 992, 1040), (130, 512, 4096),
                                   (140, 544, 8192)]):
        x, y, sa, sw = _inputs(M, N, K, 700 + i)
        out = torch.full((M, N), SENTINEL, dtype=torch.int16, device="cuda").view(torch.bfloat16)
        rc = _gather_call(g, x.cuda(), y.cuda(), sa.cuda(), sw.cuda(), [out], N, 0)
        assert rc == 0, g._C.gi8_last_error()
        torch.cuda.synchronize()
        ref = oracle.c_matmul_blockwise(x, y, sa, sw)
        assert np.array_equal(oracle.bf16_bits(out), ref), (variant, M, N, K)
    g.force_variant(None)


def test_gather_entry_config2_and_llama_m128(g, oracle):
    from gemm_int8_b200 import workloads

    cases = [("config 2", workloads.blockwise_prefill())]
    cases += [(f"config 4 M=128 K={K} N={N}", workloads.llama70b(128, N, K)) for (K, N) in [(8192, 10240), (8192, 8192), (28672, 8192)]]
    for name, (xq, wq, sa, sw) in cases:
        M, N = xq.shape[0], wq.shape[0]
        out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        rc = _gather_call(g, xq.cuda(), wq.cuda(), sa.cuda(), sw.cuda(), [out], N, 0)
        assert rc == 0, g._C.gi8_last_error()
        torch.cuda.synchronize()
        assert np.array_equal(oracle.bf16_bits(out), oracle.c_matmul_blockwise(xq, wq, sa, sw)), name


@pytest.mark.parametrize("n_first", [96, 128, 160, 320])
def test_gather_slices_stay_inside_their_columns(g, oracle, n_first):
    """Two column slices written one after the other into TWO local matrices filled with sentinels.  After the first
    slice (whose width is not always a multiple of the 64-column store box) the neighbour's columns must still hold
    the sentinel in both matrices; after the second, both matrices equal the oracle's full product."""
    M, K, n_total = 200, 1024, 448
    x, y, sa, sw_full = _inputs(M, n_total, K, 900 + n_first)
    # weight scales per slice: scale block b of a slice covers the slice's rows [128 b, 128 b + 128)
    gen = torch.Generator().manual_seed(17)
    n_second = n_total - n_first
    sw1 = torch.rand(-(-n_first // 128), K // 128, generator=gen) * 0.02 + 1e-3
    sw2 = torch.rand(-(-n_second // 128), K // 128, generator=gen) * 0.02 + 1e-3
    y1, y2 = y[:n_first].contiguous(), y[n_first:].contiguous()
    ref1 = oracle.c_matmul_blockwise(x, y1, sa, sw1)
    ref2 = oracle.c_matmul_blockwise(x, y2, sa, sw2)
    outs = [torch.full((M, n_total), SENTINEL, dtype=torch.int16, device="cuda").view(torch.bfloat16) for _ in range(2)]
    xd, sad = x.cuda(), sa.cuda()
    rc = _gather_call(g, xd, y1.cuda(), sad, sw1.cuda(), outs, n_total, 0)
    assert rc == 0, g._C.gi8_last_error()
    torch.cuda.synchronize()
    for o in outs:
        bits = oracle.bf16_bits(o)
        assert np.array_equal(bits[:, :n_first], ref1)
        assert (bits[:, n_first:] == SENTINEL).all(), "the first slice wrote into its neighbour's columns"
    rc = _gather_call(g, xd, y2.cuda(), sad, sw2.cuda(), outs, n_total, n_first)
    assert rc == 0, g._C.gi8_last_error()
    torch.cuda.synchronize()
    for o in outs:
        bits = oracle.bf16_bits(o)
        assert np.array_equal(bits[:, :n_first], ref1) and np.array_equal(bits[:, n_first:], ref2)


def test_gather_entry_rejects_bad_slices(g):
    x, y, sa, sw = (t.cuda() for t in _inputs(64, 64, 256, 5))
    out = torch.empty((64, 128), dtype=torch.bfloat16, device="cuda")
    assert _gather_call(g, x, y, sa, sw, [out], 128, 16) == 2       # start not a multiple of 32
    assert _gather_call(g, x, y[:48].contiguous(), sa, sw, [out], 128, 0) == 2   # ragged end inside the matrix
    assert _gather_call(g, x, y, sa, sw, [out], 96, 64) == 2        # slice runs past n_total

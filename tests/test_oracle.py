"""CPU tests of the oracle itself: pinned to the golden fixtures made from the reference test's own
formula (reference test.py:8), and its C and numpy restatements checked against each other."""
import glob
import os

import numpy as np
import pytest
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "*.npz"))), ids=os.path.basename)
def test_oracle_matches_golden(oracle, path):
    d = np.load(path)
    exp = d["expected_bf16_bits"]
    assert np.array_equal(oracle.c_matmul(d["x"], d["y"], float(d["alpha"])), exp)
    assert np.array_equal(oracle.np_matmul(d["x"], d["y"], float(d["alpha"])), exp)


def test_golden_files_present():
    names = {os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "*.npz"))}
    assert {"ref_test_py.npz", "ref_benchmark_py.npz", "readme_uniform.npz"} <= names


def test_reference_test_case_formula(oracle):
    """The reference's own test: values 0..99, 32x32, same tensor as both operands, alpha = 1
    (test.py:5-9,15): the oracle must equal x.bfloat16() @ x.bfloat16().t() exactly."""
    g = torch.Generator().manual_seed(7)
    x = (torch.rand(32, 32, generator=g) * 100).to(torch.int8)
    expect = x.bfloat16() @ x.bfloat16().t()
    got = oracle.to_torch_bf16(oracle.c_matmul(x, x, 1.0))
    assert torch.equal(got, expect)
    torch.testing.assert_close(got, expect)  # the reference's own criterion


@pytest.mark.parametrize("M,N,K", [(1, 8, 16), (37, 200, 400), (130, 136, 144), (5, 120, 4096)])
def test_c_vs_numpy_i32_and_alpha(oracle, M, N, K):
    rng = np.random.default_rng(M * 1000 + N)
    x = rng.integers(-128, 128, (M, K), dtype=np.int8)
    y = rng.integers(-128, 128, (N, K), dtype=np.int8)
    assert np.array_equal(oracle.c_matmul_i32(x, y), oracle.np_matmul_i32(x, y))
    for alpha in (1.0, 0.5, 1.0 / 127 ** 2, -3.7, 0.0):
        assert np.array_equal(oracle.c_matmul(x, y, alpha), oracle.np_matmul(x, y, alpha)), alpha


def test_extreme_values_do_not_overflow(oracle):
    K = 28672
    x = np.full((2, K), -128, np.int8)
    y = np.full((3, K), -128, np.int8)
    acc = oracle.c_matmul_i32(x, y)
    assert (acc == 128 * 128 * K).all() and acc.dtype == np.int32
    y[1] = 127
    assert oracle.c_matmul_i32(x, y)[0, 1] == -128 * 127 * K


def test_k_limit_rejected(oracle):
    x = np.zeros((1, 131072), np.int8)
    with pytest.raises(ValueError):
        oracle.c_matmul_i32(x, x)


@pytest.mark.parametrize("M,N,K", [(3, 8, 16), (37, 200, 400), (64, 136, 1024)])
def test_c_vs_numpy_scaled(oracle, M, N, K):
    rng = np.random.default_rng(5)
    x = rng.integers(-128, 128, (M, K), dtype=np.int8)
    y = rng.integers(-128, 128, (N, K), dtype=np.int8)
    sx = rng.random(M, dtype=np.float32) * 0.1
    sw = rng.random(N, dtype=np.float32) * 0.1
    sx[0] = 0.0
    assert np.array_equal(oracle.c_matmul_scaled(x, y, sx, sw), oracle.np_matmul_scaled(x, y, sx, sw))


@pytest.mark.parametrize("M,N,K", [(3, 8, 16), (37, 200, 400), (20, 300, 1296)])
def test_c_vs_numpy_blockwise(oracle, M, N, K):
    rng = np.random.default_rng(6)
    x = rng.integers(-128, 128, (M, K), dtype=np.int8)
    y = rng.integers(-128, 128, (N, K), dtype=np.int8)
    KB, NB = -(-K // 128), -(-N // 128)
    sa = rng.random((M, KB), dtype=np.float32) * 0.02 + 0.001
    sw = rng.random((NB, KB), dtype=np.float32) * 0.02 + 0.001
    sw[0, 0] = 0.0
    o1, a1 = oracle.c_matmul_blockwise(x, y, sa, sw, return_acc=True)
    o2, a2 = oracle.np_matmul_blockwise(x, y, sa, sw, return_acc=True)
    assert np.array_equal(a1.view(np.uint32), a2.view(np.uint32))
    assert np.array_equal(o1, o2)


def test_blockwise_unit_scales_equal_plain(oracle):
    """With every scale 1 and sums below 2^24 the blockwise result is bf16 of the exact int32 product."""
    rng = np.random.default_rng(8)
    x = rng.integers(-20, 21, (16, 512), dtype=np.int8)
    y = rng.integers(-20, 21, (136, 512), dtype=np.int8)
    sa = np.ones((16, 4), np.float32)
    sw = np.ones((2, 4), np.float32)
    assert np.array_equal(oracle.c_matmul_blockwise(x, y, sa, sw), oracle.c_matmul(x, y, 1.0))


def test_blockwise_within_fp64_bound(oracle):
    """Sanity: the fp32 block accumulation stays within a cancellation-aware bound of a float64 evaluation."""
    rng = np.random.default_rng(9)
    M, N, K = 32, 256, 1024
    x = rng.integers(-128, 128, (M, K), dtype=np.int8)
    y = rng.integers(-128, 128, (N, K), dtype=np.int8)
    sa = rng.random((M, 8), dtype=np.float32) * 0.02 + 0.001
    sw = rng.random((2, 8), dtype=np.float32) * 0.02 + 0.001
    _, acc = oracle.c_matmul_blockwise(x, y, sa, sw, return_acc=True)
    ref = np.zeros((M, N)); mag = np.zeros((M, N))
    for kb in range(8):
        P = x[:, kb * 128:(kb + 1) * 128].astype(np.int64) @ y[:, kb * 128:(kb + 1) * 128].astype(np.int64).T
        t = sa[:, kb:kb + 1].astype(np.float64) * sw[np.arange(N) // 128, kb][None, :].astype(np.float64)
        ref += P * t
        mag += np.abs(P * t)
    assert (np.abs(acc - ref) <= 2.0 ** -21 * mag + 1e-30).all()


def test_bf16_rounding_ties_and_nan(oracle):
    f = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, np.inf, np.nan, 3.0e38], np.float32)
    got = oracle.np_bf16_rne(f)
    exp = torch.from_numpy(f).bfloat16().view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got[:5], exp[:5]) and got[6] == exp[6]
    assert (got[5] & 0x7F80) == 0x7F80 and (got[5] & 0x7F) != 0


def test_quantisers_match_package(oracle):
    from gemm_int8_b200 import quant

    g = torch.Generator().manual_seed(0)
    a = torch.randn(33, 300, generator=g)
    a[5] = 0.0
    q, s = quant.quantize_per_token_block(a)
    q2, s2 = oracle.c_quantize_blocks(a, 1, 128)
    assert np.array_equal(q.numpy(), q2) and np.array_equal(s.numpy(), s2)
    w = torch.randn(200, 300, generator=g) * 0.02
    q, s = quant.quantize_weight_block(w)
    q2, s2 = oracle.np_quantize_blocks(w, 128, 128)
    assert np.array_equal(q.numpy(), q2) and np.array_equal(s.numpy(), s2)
    q, s = quant.quantize_per_row(a)
    q2, s2 = oracle.c_quantize_blocks(a, 1, 300)
    assert np.array_equal(q.numpy(), q2) and np.array_equal(s.numpy(), s2.reshape(-1))


def test_ulp_distance_helper(oracle):
    a = torch.tensor([1.0, -1.0, 0.0, 256.0]).bfloat16()
    b = torch.tensor([1.0078125, -1.0078125, 0.0, 258.0]).bfloat16()
    d = oracle.bf16_ulp_distance(oracle.bf16_bits(a), oracle.bf16_bits(b))
    assert d.tolist() == [1, 1, 0, 1]


def test_hadamard_rotation_oracle(oracle):
    """The C rotation equals the package's torch restatement bit for bit, equals the Sylvester matrix product to
    fp32 accuracy, is an involution up to rounding, and preserves the Euclidean norm."""
    from scipy.linalg import hadamard

    from gemm_int8_b200 import quant

    gen = torch.Generator().manual_seed(5)
    for (R, C, H) in [(3, 256, 128), (2, 1024, 1024), (2, 12288, 4096), (1, 8192, 8192)]:
        a = torch.randn(R, C, generator=gen)
        got = oracle.c_hadamard_rotate(a, H)
        ref = quant.hadamard_rotate(a, H).numpy()
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), (R, C, H)
        back = oracle.c_hadamard_rotate(got, H)
        assert np.abs(back - a.numpy()).max() < 1e-5
        assert np.allclose(np.linalg.norm(got, axis=1), np.linalg.norm(a.numpy(), axis=1), rtol=1e-5)
        if H <= 1024:
            mat = hadamard(H).astype(np.float64) / np.sqrt(H)
            exact = a.numpy().astype(np.float64).reshape(R, C // H, H) @ mat.T
            assert np.abs(exact.reshape(R, C) - got).max() < 1e-5
    one = np.zeros((1, 128), np.float32)
    one[0, 0] = 1.0
    assert np.array_equal(oracle.c_hadamard_rotate(one, 128), np.full((1, 128), np.float32(128 ** -0.5)))
    with pytest.raises(Exception):
        oracle.c_hadamard_rotate(np.zeros((1, 96), np.float32), 96)

"""GPU parity tests: the CUDA path, called through the torch ops (which call the C ABI) and through the
C ABI directly, against the CPU oracle on identical seeded inputs.

Bars: the int32 accumulators and every bf16 result are compared BIT FOR BIT with the oracle (the stated
tolerance for the scaled outputs is 1 bf16 ulp; the kernels reproduce the oracle's operation order, so
the tests demand 0 and would report the ulp distance on failure)."""
import ctypes
import glob
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DENSE_VARIANTS = ["dense_bn64", "dense_bn128", "dense_bn256", "pair"]


@pytest.fixture(scope="module")
def g():
    import gemm_int8_b200 as g

    assert os.path.exists(g._lib.LIB_PATH)
    yield g
    g.force_variant(None)
    assert g.device_status() == 0, "a kernel recorded an expired wait"


def rand_i8(shape, seed, lo=-128, hi=128):
    return torch.randint(lo, hi, shape, dtype=torch.int8, generator=torch.Generator().manual_seed(seed))


def assert_bits_equal(oracle, got_bf16, ref_bits, what=""):
    got = oracle.bf16_bits(got_bf16)
    if not np.array_equal(got, ref_bits):
        d = oracle.bf16_ulp_distance(got, ref_bits)
        bad = np.argwhere(got != ref_bits)
        raise AssertionError(f"{what}: {len(bad)} of {got.size} differ, max ulp distance {d.max()}, first at {bad[0].tolist()}")


# ---------------------------------------------------------------------------------------- golden / reference test
@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "*.npz"))), ids=os.path.basename)
def test_golden_vectors(g, oracle, path):
    d = np.load(path)
    x, y = torch.from_numpy(d["x"]).cuda(), torch.from_numpy(d["y"]).cuda()
    for v in DENSE_VARIANTS + [None]:
        g.force_variant(v)
        out = g.matmul(x, y, float(d["alpha"]))
        assert_bits_equal(oracle, out, d["expected_bf16_bits"], f"{os.path.basename(path)} {v}")
    g.force_variant(None)


def test_reference_test_script_flow(g):
    """The reference's test.py, step for step: opcheck, assert_close against the bf16 matmul, torch.compile."""
    import gemm_int8

    x = (torch.rand(32, 32).cuda() * 100).to(torch.int8)
    y_torch = x.bfloat16() @ x.bfloat16().t()
    y_int8 = gemm_int8.matmul(x, x, 1.0)
    torch.library.opcheck(torch.ops.gemm_int8_CUDA.int8_matmul.default, (x, x, 1.0))
    torch.testing.assert_close(y_torch, y_int8)

    @torch.compile(dynamic=True)
    def compiled(x, y, alpha):
        return gemm_int8.matmul(x, y, alpha)

    torch.testing.assert_close(y_torch, compiled(x, x, 1.0))
    x2 = (torch.rand(48, 64).cuda() * 100).to(torch.int8)
    torch.testing.assert_close((x2.float() @ x2.float().t()).bfloat16(), compiled(x2, x2, 1.0))


def test_opcheck_new_ops(g):
    x, y = rand_i8((40, 256), 1).cuda(), rand_i8((136, 256), 2).cuda()
    sa, sw = torch.rand(40, 2).cuda(), torch.rand(2, 2).cuda()
    torch.library.opcheck(torch.ops.gemm_int8_CUDA.int8_matmul_blockwise.default, (x, y, sa, sw))
    torch.library.opcheck(torch.ops.gemm_int8_CUDA.int8_matmul_scaled.default, (x, y, torch.rand(40).cuda(), torch.rand(136).cuda()))


# ---------------------------------------------------------------------------------------- integer main loop, bit exact
@pytest.mark.parametrize("variant", DENSE_VARIANTS)
def test_i32_edge_shapes(g, oracle, variant):
    g.force_variant(variant)
    Ms = [1, 2, 7, 31, 32, 33, 64, 65, 127, 128, 129, 130, 255, 257]
    Ns = [8, 16, 120, 128, 136, 264]
    Ks = [16, 32, 128, 144, 400]
    seed = 0
    for K in Ks:
        y_all = rand_i8((max(Ns), K), 100 + K)
        for M in Ms:
            x = rand_i8((M, K), 200 + M)
            xd = x.cuda()
            for N in Ns:
                seed += 1
                y = y_all[:N].contiguous()
                out = g.matmul_i32(xd, y.cuda()).cpu().numpy()
                ref = oracle.c_matmul_i32(x, y)
                assert np.array_equal(out, ref), (variant, M, N, K)
    g.force_variant(None)


def test_i32_all_m_1_to_130(g, oracle):
    K, N = 144, 136
    y = rand_i8((N, K), 5)
    x = rand_i8((130, K), 6)
    ref = oracle.c_matmul_i32(x, y)
    yd = y.cuda()
    for M in range(1, 131):
        out = g.matmul_i32(x[:M].contiguous().cuda(), yd).cpu().numpy()
        assert np.array_equal(out, ref[:M]), M


def test_i32_extreme_values_largest_k(g, oracle):
    K = 28672
    x = torch.full((130, K), -128, dtype=torch.int8)
    y = torch.full((136, K), -128, dtype=torch.int8)
    y[1::2] = 127
    out = g.matmul_i32(x.cuda(), y.cuda()).cpu().numpy()
    assert out[0, 0] == 128 * 128 * K and out[0, 1] == -128 * 127 * K
    assert np.array_equal(out, oracle.c_matmul_i32(x, y))


def test_i32_odd_n_scalar_store_path(g, oracle):
    x, y = rand_i8((70, 160), 11), rand_i8((37, 160), 12)
    assert np.array_equal(g.matmul_i32(x.cuda(), y.cuda()).cpu().numpy(), oracle.c_matmul_i32(x, y))
    out = g.matmul(x.cuda(), y.cuda(), 0.25)
    assert_bits_equal(oracle, out, oracle.c_matmul(x, y, 0.25), "odd N bf16")


# ---------------------------------------------------------------------------------------- plain matmul (alpha epilogue)
@pytest.mark.parametrize("alpha", [1.0, 0.5, 1.0 / 127 ** 2, -3.7, 0.0])
def test_matmul_alpha_values(g, oracle, alpha):
    x, y = rand_i8((257, 1040), 21), rand_i8((520, 1040), 22)
    out = g.matmul(x.cuda(), y.cuda(), alpha)
    assert out.dtype == torch.bfloat16 and out.shape == (257, 520)
    assert_bits_equal(oracle, out, oracle.c_matmul(x, y, alpha), f"alpha={alpha}")


def test_config1_plain_full_size(g, oracle):
    from gemm_int8_b200 import workloads

    x, y, alpha = workloads.plain()
    out = g.matmul(x.cuda(), y.cuda(), alpha)
    assert_bits_equal(oracle, out, oracle.c_matmul(x, y, alpha), "config 1")
    acc = g.matmul_i32(x.cuda(), y.cuda()).cpu().numpy()
    assert np.array_equal(acc, oracle.c_matmul_i32(x, y))


def test_reference_benchmark_shapes(g, oracle):
    """Input recipe and layer shapes of the reference benchmark (benchmark.py:17-26,56-62), smallest token count."""
    gen = torch.Generator().manual_seed(31)
    for (n, k) in [(4096, 4096), (14336, 4096), (4096, 14336)]:
        a = torch.round((torch.randn(512, k, generator=gen) * 5).clamp(-128, 127)).to(torch.int8)
        b = torch.round((torch.randn(n, k, generator=gen) * 5).clamp(-128, 127)).to(torch.int8)
        out = g.matmul(a.cuda(), b.cuda(), 1.0)
        assert_bits_equal(oracle, out, oracle.c_matmul(a, b, 1.0), f"benchmark shape {n}x{k}")


# ---------------------------------------------------------------------------------------- split-K tail of the dense kernels
@pytest.mark.parametrize("variant", ["dense_bn256", "pair", None])
def test_dense_split_k_tail(g, oracle, variant, monkeypatch):
    """GEMM_INT8_TAIL_SPLIT=2 sends the last wave of the 256-wide forms (or the whole grid, when it is thin) to the
    split-K cluster kernel whenever that is possible: results must stay the oracle's bits for the plain and the
    per-token x per-channel entry points -- ragged M and N, a 256-row tile whose lower half lies below M, extreme
    values, and grids of more than one wave (main launch + split-K launch)."""
    monkeypatch.setenv("GEMM_INT8_TAIL_SPLIT", "2")
    g.reload_env()
    try:
        g.force_variant(variant)
        gen = torch.Generator().manual_seed(91)
        shapes = [(130, 264, 400), (300, 1000, 2048), (257, 520, 4096), (256, 20480, 512), (512, 10240, 640),
                  (100, 38400, 256), (1, 8, 256)]
        for (M, N, K) in shapes:
            x, y = rand_i8((M, K), M + 11), rand_i8((N, K), N + 11)
            if K >= 2048:
                x[0], y[0] = -128, -128   # the largest possible sums
            xd, yd = x.cuda(), y.cuda()
            for alpha in (1.0, -3.7):
                ref = oracle.c_matmul(x, y, alpha)
                for pdl in ("1", "0"):   # split-K launch released as the main launch's CTAs leave / an ordinary second launch
                    monkeypatch.setenv("GEMM_INT8_PDL", pdl)
                    g.reload_env()
                    outs = [g.matmul(xd, yd, alpha).clone() for _ in range(2)]   # back to back, a reader right behind each
                    for out in outs:
                        assert_bits_equal(oracle, out, ref, f"split-K plain {variant} {(M, N, K)} alpha {alpha} pdl {pdl}")
                monkeypatch.delenv("GEMM_INT8_PDL", raising=False)
                g.reload_env()
            if M > 64:   # (smaller M goes to the small-M kernel)
                sx = torch.rand(M, generator=gen) * 0.05 + 1e-3
                sw = torch.rand(N, generator=gen) * 0.05 + 1e-3
                out = g.matmul_scaled(xd, yd, sx.cuda(), sw.cuda())
                assert_bits_equal(oracle, out, oracle.c_matmul_scaled(x, y, sx, sw), f"split-K scaled {variant} {(M, N, K)}")
        assert g.device_status() == 0
    finally:
        g.force_variant(None)
        monkeypatch.delenv("GEMM_INT8_TAIL_SPLIT", raising=False)
        g.reload_env()


def test_dense_split_k_is_chosen_for_thin_last_waves(g):
    """The dispatch hands a thin last wave, or a thin grid with a long K, to the split-K kernel (names as
    gi8_pick_variant reports them) and leaves well-filled grids alone."""
    assert g.pick_variant(0, 1024, 14336, 16384).endswith("+splitk8")
    assert g.pick_variant(0, 256, 4096, 28672).startswith("splitk")
    assert g.pick_variant(0, 8192, 8192, 8192) == "pair"
    assert g.pick_variant(0, 1024, 4096, 4096) == "pair"


# ---------------------------------------------------------------------------------------- scaled (per token x per channel)
@pytest.mark.parametrize("variant", DENSE_VARIANTS + ["smallm", "smallm_cluster", None])
def test_scaled_edge_shapes(g, oracle, variant):
    g.force_variant(variant)
    gen = torch.Generator().manual_seed(41)
    for (M, N, K) in [(1, 8, 16), (4, 136, 144), (16, 520, 1024), (64, 128, 4096), (130, 264, 400), (300, 1000, 512)]:
        x, y = rand_i8((M, K), M), rand_i8((N, K), N)
        sx = torch.rand(M, generator=gen) * 0.05 + 1e-3
        sw = torch.rand(N, generator=gen) * 0.05 + 1e-3
        sx[0] = 0.0
        out = g.matmul_scaled(x.cuda(), y.cuda(), sx.cuda(), sw.cuda())
        assert_bits_equal(oracle, out, oracle.c_matmul_scaled(x, y, sx, sw), f"scaled {variant} {(M, N, K)}")
    g.force_variant(None)


@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 14336), (14336, 4096)])
def test_config3_decode_shapes(g, oracle, K, N):
    from gemm_int8_b200 import workloads

    for M in (1, 4, 16, 64):
        xq, wq, sx, sw = workloads.decode(M, N, K)
        assert g.pick_variant(1, M, N, K) == "smallm_cluster"
        ref = oracle.c_matmul_scaled(xq, wq, sx, sw)
        # the automatic choice, the cluster reduction and the global-scratch reduction
        for variant in (None, "smallm_cluster", "smallm"):
            g.force_variant(variant)
            out = g.matmul_scaled(xq.cuda(), wq.cuda(), sx.cuda(), sw.cuda())
            assert_bits_equal(oracle, out, ref, f"decode {variant} M={M} N={N} K={K}")
        g.force_variant(None)


def test_smallm_static_weights_option(g, oracle, monkeypatch):
    """GEMM_INT8_STATIC_WEIGHTS=1 lets the small-M kernel request its first weight tiles before the preceding
    kernel has ended; activations and scales are still read after it.  Here the activations of every call are
    written by a kernel directly before it (a device copy), back to back, and the bits must stay the oracle's."""
    from gemm_int8_b200 import workloads

    monkeypatch.setenv("GEMM_INT8_STATIC_WEIGHTS", "1")
    g.reload_env()
    try:
        for (M, N, K) in [(16, 4096, 4096), (3, 1000, 1040), (64, 14336, 4096)]:
            xq, wq, sx, sw = workloads.decode(M, N, K)
            cases = [(xq, wq, sx, sw)]
            for i in range(3):   # further activations for the same weights
                cases.append((rand_i8((M, K), 70 + i), wq, torch.rand(M, generator=torch.Generator().manual_seed(80 + i)) * 0.05, sw))
            wd, swd = wq.cuda(), sw.cuda()
            srcs = [(c[0].cuda(), c[2].cuda()) for c in cases]
            xd, sxd = torch.empty_like(srcs[0][0]), torch.empty_like(srcs[0][1])
            outs = []
            for (xs, ss) in srcs:
                xd.copy_(xs)
                sxd.copy_(ss)
                outs.append(g.matmul_scaled(xd, wd, sxd, swd))
            for (c, out) in zip(cases, outs):
                assert_bits_equal(oracle, out, oracle.c_matmul_scaled(c[0], wq, c[2], sw), f"static weights {(M, N, K)}")
    finally:
        monkeypatch.delenv("GEMM_INT8_STATIC_WEIGHTS", raising=False)
        g.reload_env()


def test_smallm_split_k_scratch_is_left_zeroed(g, oracle):
    """The split-K kernel adds int32 partials into caller-provided scratch and must leave it zero-filled, so
    back-to-back calls sharing one buffer stay exact; also checks extreme values and ragged N."""
    M, N, K = 33, 1000, 4096
    x = torch.full((M, K), -128, dtype=torch.int8)
    y = torch.full((N, K), -128, dtype=torch.int8)
    y[1::2] = 127
    sx, sw = torch.rand(M) + 0.5, torch.rand(N) + 0.5
    xd, yd, sxd, swd = x.cuda(), y.cuda(), sx.cuda(), sw.cuda()
    g.force_variant("smallm")
    nbytes = int(g._C.gi8_matmul_scaled_workspace_bytes(M, N, K))
    assert nbytes > 0
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    ref = oracle.c_matmul_scaled(x, y, sx, sw)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(3):
        out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        rc = g._C.gi8_matmul_scaled(ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(yd.data_ptr()),
                                    ctypes.c_void_p(sxd.data_ptr()), ctypes.c_void_p(swd.data_ptr()),
                                    ctypes.c_void_p(out.data_ptr()), M, N, K, ctypes.c_void_p(ws.data_ptr()), nbytes, stream)
        assert rc == 0, g._C.gi8_last_error()
        assert_bits_equal(oracle, out, ref, "split-K")
        assert int(ws.count_nonzero()) == 0, "scratch not restored to zero"
    # too small / missing workspace is refused, not overrun
    rc = g._C.gi8_matmul_scaled(ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(yd.data_ptr()),
                                ctypes.c_void_p(sxd.data_ptr()), ctypes.c_void_p(swd.data_ptr()),
                                ctypes.c_void_p(out.data_ptr()), M, N, K, ctypes.c_void_p(ws.data_ptr()), 16, stream)
    assert rc == 6
    g.force_variant(None)
    assert int(g._C.gi8_matmul_scaled_workspace_bytes(M, N, K)) == 0   # the default (cluster) path needs none
    out = g.matmul_scaled(xd, yd, sxd, swd)
    assert_bits_equal(oracle, out, ref, "cluster split-K, extreme values")


# ---------------------------------------------------------------------------------------- blockwise
@pytest.fixture
def bw_knobs(g, monkeypatch):
    """Sets the blockwise kernel's tuning variables for one test and restores the defaults afterwards."""
    def set_knobs(halves, issuers):
        monkeypatch.setenv("GEMM_INT8_BW_HALVES", str(halves))
        monkeypatch.setenv("GEMM_INT8_BW_ISSUERS", str(issuers))
        g.reload_env()
    yield set_knobs
    monkeypatch.delenv("GEMM_INT8_BW_HALVES", raising=False)
    monkeypatch.delenv("GEMM_INT8_BW_ISSUERS", raising=False)
    g.reload_env()


@pytest.mark.parametrize("issuers", [1, 2])
@pytest.mark.parametrize("variant", ["dense_bn64", "dense_bn128", "dense_bn256", "pair", None])
def test_blockwise_edge_shapes(g, oracle, variant, issuers, bw_knobs):
    bw_knobs(issuers, issuers)   # (1, 1): N = 256 MMAs, one issuer; (2, 2): column halves, one issuer per half
    g.force_variant(variant)
    gen = torch.Generator().manual_seed(51)
    shapes = [(1, 8, 16), (7, 120, 128), (33, 136, 144), (128, 128, 128), (129, 264, 400), (257, 1000, 1040),
              (130, 520, 4096)]
    for (M, N, K) in shapes:
        KB, NB = -(-K // 128), -(-N // 128)
        x, y = rand_i8((M, K), M + 1), rand_i8((N, K), N + 1)
        sa = torch.rand(M, KB, generator=gen) * 0.02 + 1e-3
        sw = torch.rand(NB, KB, generator=gen) * 0.02 + 1e-3
        sa[0, 0] = 0.0
        sw[-1, -1] = 0.0
        out = g.matmul_blockwise(x.cuda(), y.cuda(), sa.cuda(), sw.cuda())
        assert_bits_equal(oracle, out, oracle.c_matmul_blockwise(x, y, sa, sw), f"blockwise {variant} {(M, N, K)}")
    g.force_variant(None)


@pytest.mark.parametrize("halves", [1, 2])
@pytest.mark.parametrize("issuers", [1, 2])
def test_blockwise_mma_forms_agree(g, oracle, halves, issuers, bw_knobs):
    """The MMA shapes of the 256-wide tile (N = 256, or two column halves with N = 128) and one or two issuing
    threads give the oracle's bits, including the largest possible block partial and many K blocks per tile
    (the barrier rings wrap many times)."""
    bw_knobs(halves, issuers)
    gen = torch.Generator().manual_seed(52)
    for variant in ("dense_bn64", "dense_bn128", "dense_bn256", "pair"):
        g.force_variant(variant)
        for (M, N, K) in [(130, 264, 400), (300, 1000, 2048), (140, 520, 8192)]:
            KB, NB = -(-K // 128), -(-N // 128)
            x, y = rand_i8((M, K), M + 3), rand_i8((N, K), N + 3)
            x[0], y[0] = -128, -128          # largest possible block partial, 2^21
            sa = torch.rand(M, KB, generator=gen) * 0.02 + 1e-3
            sw = torch.rand(NB, KB, generator=gen) * 0.02 + 1e-3
            out = g.matmul_blockwise(x.cuda(), y.cuda(), sa.cuda(), sw.cuda())
            assert_bits_equal(oracle, out, oracle.c_matmul_blockwise(x, y, sa, sw), f"halves {halves} issuers {issuers} {variant}")
    g.force_variant(None)


def test_blockwise_column_split_second_launch(g, oracle, monkeypatch):
    """A blockwise grid of W full waves plus a few tiles is run as two launches over disjoint column ranges (the second with
    narrower tiles, released as the first one's CTAs leave).  Forced wherever possible: the bits must stay the oracle's,
    also for a ragged last tile, for back-to-back calls, and for a kernel that reads the result right behind the pair
    (it must see both launches' columns)."""
    monkeypatch.setenv("GEMM_INT8_TAIL_SPLIT", "2")
    g.reload_env()
    try:
        gen = torch.Generator().manual_seed(77)
        for (M, N, K) in [(512, 10240, 512), (512, 10232, 640), (256, 38400, 384)]:
            assert "+columns_bn" in g.pick_variant(2, M, N, K), (M, N, K)
            KB, NB = -(-K // 128), -(-N // 128)
            x, y = rand_i8((M, K), M + 5), rand_i8((N, K), N + 5)
            sa = torch.rand(M, KB, generator=gen) * 0.02 + 1e-3
            sw = torch.rand(NB, KB, generator=gen) * 0.02 + 1e-3
            ref = oracle.c_matmul_blockwise(x, y, sa, sw)
            xd, yd, sad, swd = x.cuda(), y.cuda(), sa.cuda(), sw.cuda()
            for pdl in ("1", "0"):   # second launch released as the first one's CTAs leave / an ordinary second launch
                monkeypatch.setenv("GEMM_INT8_PDL", pdl)
                g.reload_env()
                copies = []
                for _ in range(3):
                    out = g.matmul_blockwise(xd, yd, sad, swd)
                    copies.append(out.clone())          # a kernel right behind the pair, on the same stream
                for c in copies:
                    assert_bits_equal(oracle, c, ref, f"column split {(M, N, K)} pdl {pdl}")
            monkeypatch.delenv("GEMM_INT8_PDL", raising=False)
        assert g.device_status() == 0
    finally:
        monkeypatch.delenv("GEMM_INT8_TAIL_SPLIT", raising=False)
        g.reload_env()
    assert g.pick_variant(2, 512, 10240, 8192) == "blockwise_bn256+columns_bn64"
    assert g.pick_variant(2, 8192, 8192, 8192) == "blockwise_bn256"


def test_blockwise_unit_scales_are_exact_integers(g, oracle):
    """All scales 1 and |sums| < 2^24: the blockwise kernel must return bf16 of the exact int32 product, and
    single-K-block slices expose each int32 partial exactly."""
    x, y = rand_i8((200, 512), 61, -20, 21), rand_i8((264, 512), 62, -20, 21)
    ones_a, ones_w = torch.ones(200, 4), torch.ones(3, 4)
    out = g.matmul_blockwise(x.cuda(), y.cuda(), ones_a.cuda(), ones_w.cuda())
    assert_bits_equal(oracle, out, oracle.c_matmul(x, y, 1.0), "unit scales")
    xs, ys = rand_i8((200, 128), 63), rand_i8((264, 128), 64)
    out = g.matmul_blockwise(xs.cuda(), ys.cuda(), torch.ones(200, 1).cuda(), torch.ones(3, 1).cuda())
    assert torch.equal(out.cpu(), torch.from_numpy(oracle.c_matmul_i32(xs, ys)).float().bfloat16())


def test_blockwise_strided_scales(g, oracle):
    M, N, K = 70, 264, 512
    x, y = rand_i8((M, K), 65), rand_i8((N, K), 66)
    sa_big = torch.rand(M, 9, generator=torch.Generator().manual_seed(67)) * 0.02 + 1e-3
    sw_big = torch.rand(3, 7, generator=torch.Generator().manual_seed(68)) * 0.02 + 1e-3
    sa, sw = sa_big[:, :4], sw_big[:, :4]  # row strides 9 and 7
    out = g.matmul_blockwise(x.cuda(), y.cuda(), sa_big.cuda()[:, :4], sw_big.cuda()[:, :4])
    assert_bits_equal(oracle, out, oracle.c_matmul_blockwise(x, y, sa.contiguous(), sw.contiguous()), "strided scales")


def test_blockwise_f32_accumulators_and_ksharded_sum(g, oracle):
    """The fp32-result entry point returns the oracle's accumulators bit for bit (every tile width, ragged shapes),
    and the K-sharded form -- per-slice accumulators added in slice order, then cast -- equals the oracle's
    restatement of it, emulated on one GPU for 2, 3 and 4 slices."""
    gen = torch.Generator().manual_seed(53)
    for variant in (None, "dense_bn256", "dense_bn128", "dense_bn64", "pair"):
        g.force_variant(variant)
        for (M, N, K) in [(7, 120, 128), (129, 264, 400), (300, 1000, 2048)]:
            KB, NB = -(-K // 128), -(-N // 128)
            x, y = rand_i8((M, K), M + 5), rand_i8((N, K), N + 5)
            sa = torch.rand(M, KB, generator=gen) * 0.02 + 1e-3
            sw = torch.rand(NB, KB, generator=gen) * 0.02 + 1e-3
            acc = g.matmul_blockwise_f32(x.cuda(), y.cuda(), sa.cuda(), sw.cuda())
            assert acc.dtype == torch.float32
            _, ref_acc = oracle.c_matmul_blockwise(x, y, sa, sw, return_acc=True)
            assert np.array_equal(acc.cpu().numpy().view(np.uint32), ref_acc.view(np.uint32)), (variant, M, N, K)
    g.force_variant(None)
    M, N, K = 96, 520, 2048 + 128
    KB, NB = K // 128, -(-N // 128)
    x, y = rand_i8((M, K), 71), rand_i8((N, K), 72)
    sa = torch.rand(M, KB, generator=gen) * 0.02 + 1e-3
    sw = torch.rand(NB, KB, generator=gen) * 0.02 + 1e-3
    from gemm_int8_b200 import dist as gdist

    for world in (2, 3, 4):
        parts = []
        for r in range(world):
            k0, k1 = gdist.kshard_bounds(K, world, r)
            parts.append(g.matmul_blockwise_f32(x[:, k0:k1].contiguous().cuda(), y[:, k0:k1].contiguous().cuda(),
                                                sa[:, k0 // 128:k1 // 128].contiguous().cuda(),
                                                sw[:, k0 // 128:k1 // 128].contiguous().cuda()))
        out = g.sum_parts_bf16(torch.stack(parts))
        assert_bits_equal(oracle, out, oracle.c_matmul_blockwise_ksharded(x, y, sa, sw, world), f"k-sharded world {world}")
    # the unaligned (scalar) form of the sum kernel
    odd = torch.stack([p[:, :519].contiguous() for p in parts])
    ref = oracle.c_matmul_blockwise_ksharded(x, y, sa, sw, 4)[:, :519]
    assert_bits_equal(oracle, g.sum_parts_bf16(odd), ref, "k-sharded, odd width")


def test_blockwise_f32_scatter_entry_on_one_gpu(g, oracle):
    """The reduce-scatter form through the C ABI with every rank's receive area on this GPU: rank r's launch must put
    rows [j R, (j + 1) R) of its fp32 accumulators into area j at part r (and nothing anywhere else: the areas start
    as NaN patterns and must be completely overwritten by the `world` launches), and the ordered sum of each area
    must equal the oracle's K-sharded restatement.  All tile forms, ragged N, 2 and 4 ranks."""
    from gemm_int8_b200 import dist as gdist

    gen = torch.Generator().manual_seed(54)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for variant in (None, "dense_bn256", "dense_bn128", "dense_bn64", "pair"):
        g.force_variant(variant)
        for (world, M, N, K) in [(2, 128, 520, 1024), (4, 384, 1000, 2048 + 128)]:
            KB, NB = K // 128, -(-N // 128)
            x, y = rand_i8((M, K), M + 9), rand_i8((N, K), N + 9)
            sa = torch.rand(M, KB, generator=gen) * 0.02 + 1e-3
            sw = torch.rand(NB, KB, generator=gen) * 0.02 + 1e-3
            R = M // world
            areas = [torch.full((world, R, N), float("nan"), dtype=torch.float32, device="cuda") for _ in range(world)]
            recv = (ctypes.c_void_p * world)(*[a.data_ptr() for a in areas])
            keep = []
            for r in range(world):
                k0, k1 = gdist.kshard_bounds(K, world, r)
                ops = (x[:, k0:k1].contiguous().cuda(), y[:, k0:k1].contiguous().cuda(),
                       sa[:, k0 // 128:k1 // 128].contiguous().cuda(), sw[:, k0 // 128:k1 // 128].contiguous().cuda())
                keep.append(ops)
                rc = g._C.gi8_matmul_blockwise_f32_scatter(
                    ctypes.c_void_p(ops[0].data_ptr()), ctypes.c_void_p(ops[1].data_ptr()), ctypes.c_void_p(ops[2].data_ptr()),
                    ops[2].stride(0), ctypes.c_void_p(ops[3].data_ptr()), ops[3].stride(0), recv, world, r, M, N, k1 - k0, stream)
                assert rc == 0, g._C.gi8_last_error()
            ref = oracle.c_matmul_blockwise_ksharded(x, y, sa, sw, world)
            for j in range(world):
                assert not torch.isnan(areas[j]).any(), f"area {j} not fully written ({variant}, world {world})"
                out = g.sum_parts_bf16(areas[j])
                assert_bits_equal(oracle, out, ref[j * R:(j + 1) * R], f"scatter {variant} world {world} rows of rank {j}")
    g.force_variant(None)
    # argument checks
    a = torch.zeros((2, 32, 64), dtype=torch.float32, device="cuda")
    recv = (ctypes.c_void_p * 2)(a.data_ptr(), a.data_ptr())
    xq = torch.zeros((64, 128), dtype=torch.int8, device="cuda")
    sc = torch.ones((64, 1), dtype=torch.float32, device="cuda")
    args = (ctypes.c_void_p(xq.data_ptr()), ctypes.c_void_p(xq.data_ptr()), ctypes.c_void_p(sc.data_ptr()), 1,
            ctypes.c_void_p(sc.data_ptr()), 1)
    assert g._C.gi8_matmul_blockwise_f32_scatter(*args, recv, 2, 2, 64, 64, 128, stream) == 1    # my_rank out of range
    assert g._C.gi8_matmul_blockwise_f32_scatter(*args, recv, 2, 0, 48, 64, 128, stream) == 2    # M not a multiple of 32 x ranks
    assert g._C.gi8_matmul_blockwise_f32_scatter(*args, recv, 9, 0, 288, 64, 128, stream) == 1   # more than 8 ranks


def test_config2_blockwise_prefill_full_size(g, oracle):
    from gemm_int8_b200 import workloads

    xq, wq, sa, sw = workloads.blockwise_prefill()
    out = g.matmul_blockwise(xq.cuda(), wq.cuda(), sa.cuda(), sw.cuda())
    assert out.shape == (2048, 11008)
    assert_bits_equal(oracle, out, oracle.c_matmul_blockwise(xq, wq, sa, sw), "config 2")


@pytest.mark.parametrize("K,N", [(8192, 10240), (8192, 8192), (8192, 57344), (28672, 8192)])
def test_config4_llama70b_sweep_all_m(g, oracle, K, N):
    """Config 4 inputs (outlier channels, Hadamard rotation, blockwise quantisation) for every M of the sweep.
    The oracle computes 128 distinct token rows once per (K, N); M = 128 is compared whole, and for
    M in {512, 2048, 8192, 16384} the 128 rows are tiled to M rows: the first, a middle and the last 128-row block
    of the result must each equal the oracle bit for bit (so every row block a CTA can be handed at that size meets
    the oracle's values at full K depth), and the run must leave the kernel status word clear."""
    from gemm_int8_b200 import workloads

    xq, wq, sa, sw = workloads.llama70b(128, N, K)
    ref = oracle.c_matmul_blockwise(xq, wq, sa, sw)
    xd, wd, sad, swd = xq.cuda(), wq.cuda(), sa.cuda(), sw.cuda()
    out = g.matmul_blockwise(xd, wd, sad, swd)
    assert_bits_equal(oracle, out, ref, f"config 4 M=128 K={K} N={N}")
    del out
    for M in (512, 2048, 8192, 16384):
        reps = M // 128
        x_big, sa_big = xd.repeat(reps, 1), sad.repeat(reps, 1)
        out = g.matmul_blockwise(x_big, wd, sad.repeat(reps, 1), swd)
        assert out.shape == (M, N)
        for blk in sorted({0, reps // 2, reps - 1}):
            assert_bits_equal(oracle, out[blk * 128:(blk + 1) * 128], ref, f"config 4 M={M} K={K} N={N} row block {blk}")
        del out, x_big, sa_big
    assert g.device_status() == 0


def test_config5_full_size_sampled_rows_and_properties(g, oracle):
    """Config 5 at full size (16384 x 57344 x 8192).  The oracle is too slow for the whole product, so:
    (1) 48 sampled rows are compared bit for bit with the oracle, (2) the run is repeated and must be
    bitwise identical, (3) duplicated input rows must give identical output rows."""
    from gemm_int8_b200 import workloads

    x, y, sa, sw = workloads.nshard()
    x[1001] = x[77]
    sa[1001] = sa[77]
    xd, yd, sad, swd = x.cuda(), y.cuda(), sa.cuda(), sw.cuda()
    out = g.matmul_blockwise(xd, yd, sad, swd)
    rows = torch.randperm(16384, generator=torch.Generator().manual_seed(5))[:48]
    ref = oracle.c_matmul_blockwise(x[rows].contiguous(), y, sa[rows].contiguous(), sw)
    assert_bits_equal(oracle, out[rows.cuda()], ref, "config 5 sampled rows")
    assert torch.equal(out[1001], out[77])
    out2 = g.matmul_blockwise(xd, yd, sad, swd)
    assert torch.equal(out, out2)
    del out2
    # N-shard consistency: each column shard computed separately equals the matching slice
    for gsz in (8,):
        n = 57344 // gsz
        r = 3
        shard = g.matmul_blockwise(xd, yd[r * n:(r + 1) * n], sad, swd[r * n // 128:(r + 1) * n // 128])
        assert torch.equal(shard, out[:, r * n:(r + 1) * n])


def test_large_square_sampled(g, oracle):
    """8192^3 plain GEMM: sampled rows bit-exact, plus linearity in alpha (alpha = 2 doubles every value exactly)."""
    x, y = rand_i8((8192, 8192), 71, -128, 127), rand_i8((8192, 8192), 72, -128, 127)
    xd, yd = x.cuda(), y.cuda()
    out = g.matmul(xd, yd, 1.0)
    rows = torch.randperm(8192, generator=torch.Generator().manual_seed(7))[:64]
    assert_bits_equal(oracle, out[rows.cuda()], oracle.c_matmul(x[rows].contiguous(), y, 1.0), "8192^3 rows")
    out2 = g.matmul(xd, yd, 2.0)
    assert torch.equal(out2.float(), out.float() * 2)


# ---------------------------------------------------------------------------------------- robustness
def test_determinism_repeated_runs(g):
    x, y = rand_i8((1024, 4096), 81).cuda(), rand_i8((4096, 4096), 82).cuda()
    first = g.matmul(x, y, 0.01)
    for _ in range(30):
        assert torch.equal(g.matmul(x, y, 0.01), first)
    sa, sw = torch.rand(1024, 32).cuda(), torch.rand(32, 32).cuda()
    firstb = g.matmul_blockwise(x, y, sa, sw)
    for _ in range(20):
        assert torch.equal(g.matmul_blockwise(x, y, sa, sw), firstb)


def test_c_abi_direct_call_with_guard_bands(g, oracle):
    """Calls the C ABI with raw pointers; the output sits inside a larger buffer of sentinels that must survive."""
    M, N, K = 130, 136, 400
    x, y = rand_i8((M, K), 91), rand_i8((N, K), 92)
    xd, yd = x.cuda(), y.cuda()
    guard = 4096
    buf = torch.full((M * N + 2 * guard,), 0x7FC1, dtype=torch.int16, device="cuda")
    out_ptr = buf.data_ptr() + guard * 2
    stream = torch.cuda.current_stream().cuda_stream
    rc = g._C.gi8_matmul(ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(yd.data_ptr()), ctypes.c_void_p(out_ptr),
                         M, N, K, 0.125, ctypes.c_void_p(stream))
    assert rc == 0, g._C.gi8_last_error()
    torch.cuda.synchronize()
    host = buf.cpu().numpy().view(np.uint16)
    assert (host[:guard] == 0x7FC1).all() and (host[-guard:] == 0x7FC1).all()
    assert np.array_equal(host[guard:-guard].reshape(M, N), oracle.c_matmul(x, y, 0.125))
    # int32 entry point the same way
    ibuf = torch.full((M * N + 2 * guard,), -7, dtype=torch.int32, device="cuda")
    rc = g._C.gi8_matmul_i32(ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(yd.data_ptr()),
                             ctypes.c_void_p(ibuf.data_ptr() + guard * 4), M, N, K, ctypes.c_void_p(stream))
    assert rc == 0
    torch.cuda.synchronize()
    ih = ibuf.cpu().numpy()
    assert (ih[:guard] == -7).all() and (ih[-guard:] == -7).all()
    assert np.array_equal(ih[guard:-guard].reshape(M, N), oracle.c_matmul_i32(x, y))


def test_side_stream_and_empty_problems(g, oracle):
    x, y = rand_i8((64, 256), 93), rand_i8((72, 256), 94)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        out = g.matmul(x.cuda(), y.cuda(), 1.0)
    s.synchronize()
    assert_bits_equal(oracle, out, oracle.c_matmul(x, y, 1.0), "side stream")
    e = torch.empty(0, 256, dtype=torch.int8, device="cuda")
    assert g.matmul(e, y.cuda(), 1.0).shape == (0, 72)
    assert g.matmul(x.cuda(), e, 1.0).shape == (64, 0)
    z = torch.empty(5, 0, dtype=torch.int8, device="cuda")
    out0 = g.matmul(z, torch.empty(9, 0, dtype=torch.int8, device="cuda"), 1.0)
    assert out0.shape == (5, 9) and (out0 == 0).all()


def test_error_paths(g):
    x, y = rand_i8((64, 256), 95).cuda(), rand_i8((72, 256), 96).cuda()
    with pytest.raises(RuntimeError):
        g.matmul(x.t(), y, 1.0)                      # not contiguous (reference: checkAllContiguous)
    with pytest.raises(RuntimeError):
        g.matmul(x, y[:, :128], 1.0)
    with pytest.raises(RuntimeError):
        g.matmul(x.to(torch.int32), y, 1.0)          # dtype
    with pytest.raises(RuntimeError):
        g.matmul(x[:, :24].contiguous(), y[:, :24].contiguous(), 1.0)   # K % 16 != 0
    with pytest.raises(RuntimeError):
        g.matmul(x, rand_i8((72, 128), 97).cuda(), 1.0)   # K mismatch
    with pytest.raises(RuntimeError):
        g.matmul(x, y.cpu(), 1.0)
    with pytest.raises(RuntimeError):
        g.matmul_blockwise(x, y, torch.rand(64, 3).cuda(), torch.rand(1, 2).cuda())   # bad scale shape
    with pytest.raises(RuntimeError):
        g.matmul_scaled(x, y, torch.rand(64).cuda().double(), torch.rand(72).cuda())
    assert g.device_status() == 0


# ---------------------------------------------------------------------------------------- callers of the GEMM
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_quantiser_kernels_match_oracle(g, oracle, dtype):
    gen = torch.Generator().manual_seed(101)
    for (M, K) in [(1, 128), (7, 136), (33, 4096), (300, 1000 if dtype == torch.float32 else 1008), (64, 14336)]:
        a = (torch.randn(M, K, generator=gen) * 3).to(dtype)
        a[0, : min(K, 128)] = 0  # an all-zero block: scale 1, zeros
        af = a.float()
        q, s = g.quantize_per_token_block(a.cuda())
        qr, sr = oracle.c_quantize_blocks(af, 1, 128)
        assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy(), sr), (dtype, M, K)
        q, s = g.quantize_per_token(a.cuda())
        qr, sr = oracle.c_quantize_blocks(af, 1, K)
        assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy(), sr.reshape(-1)), (dtype, M, K)
    # Rounding boundaries and extreme scales: the kernels multiply by 1/s and fall back to the exact division near
    # half-integers and for scales whose reciprocal is not accurate.
    if dtype == torch.float32:
        a = torch.zeros(6, 256)
        a[0, 0] = 127.0                                   # scale exactly 1
        a[0, 1:127] = torch.arange(1, 127) - 0.5          # exact ties: round half to even
        a[1, 0] = 127.0
        a[1, 1:127] = torch.nextafter(torch.arange(1, 127) - 0.5, torch.tensor(200.0))
        a[2, 0] = 127.0
        a[2, 1:127] = torch.nextafter(torch.arange(1, 127) - 0.5, torch.tensor(-200.0))
        a[3, :128] = torch.randn(128, generator=gen) * 1e-38   # subnormal scale
        a[4, :128] = torch.randn(128, generator=gen) * 1e35    # huge scale
        a[5, :256] = torch.randn(256, generator=gen) * 3.3
        a[:, 128:] = -a[:, :128] * 0.37
        q, s = g.quantize_per_token_block(a.cuda())
        qr, sr = oracle.c_quantize_blocks(a, 1, 128)
        assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy(), sr)
        q, s = g.quantize_per_token(a.cuda())
        qr, sr = oracle.c_quantize_blocks(a, 1, 256)
        assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy(), sr.reshape(-1))
    with pytest.raises(RuntimeError):
        g.quantize_per_token_block(torch.zeros(4, 130).cuda())       # K % 4 != 0
    with pytest.raises(RuntimeError):
        g.quantize_per_token_block(torch.zeros(4, 128))              # CPU tensor


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_hadamard_quantiser_matches_oracle(g, oracle, dtype):
    """Fused Walsh-Hadamard rotation + per-token-per-128 quantiser: int8 values and scales equal the oracle's
    rotate-then-quantise bit for bit, for every rotation block size the kernel has a code path for."""
    gen = torch.Generator().manual_seed(111)
    for (M, K, H) in [(3, 128, 128), (5, 768, 256), (2, 1536, 512), (4, 3072, 1024), (3, 2048, 2048), (2, 28672, 4096),
                      (3, 8192, 8192), (2, 16384, 8192), (130, 8192, None)]:
        a = (torch.randn(M, K, generator=gen) * 3).to(dtype)
        a[:, 5] *= 20.0   # an outlier channel, which the rotation spreads over its block
        a[0] = 0          # an all-zero row: scales 1, zeros
        q, s = g.hadamard_quantize_per_token_block(a.cuda(), H)
        block = H if H is not None else min(K & -K, 8192)
        qr, sr = oracle.c_quantize_blocks(oracle.c_hadamard_rotate(a.float(), block), 1, 128)
        assert np.array_equal(s.cpu().numpy(), sr), (dtype, M, K, H)
        assert np.array_equal(q.cpu().numpy(), qr), (dtype, M, K, H)
    with pytest.raises(RuntimeError):
        g.hadamard_quantize_per_token_block(torch.zeros(4, 384).cuda(), 256)    # block does not divide K
    with pytest.raises(RuntimeError):
        g.hadamard_quantize_per_token_block(torch.zeros(4, 192).cuda(), 64)     # block below 128
    with pytest.raises(RuntimeError):
        g.hadamard_quantize_per_token_block(torch.zeros(4, 384).cuda(), 384)    # not a power of two


def test_int8_linear_matches_oracle_pipeline(g, oracle):
    """Int8Linear = offline weight quantiser + fused activation quantiser + GEMM; every stage has an oracle, so
    the layer output must equal the oracle pipeline bit for bit, and stay close to the fp32 linear layer."""
    from gemm_int8_b200 import quant

    gen = torch.Generator().manual_seed(202)
    x = torch.randn(3, 50, 1024, generator=gen)
    w = torch.randn(520, 1024, generator=gen) * 0.02
    layer = g.Int8Linear.from_float(w, mode="blockwise").cuda()
    y = layer(x.cuda())
    assert y.shape == (3, 50, 520) and y.dtype == torch.bfloat16
    xq, xs = oracle.c_quantize_blocks(x.reshape(-1, 1024), 1, 128)
    wq, ws = oracle.c_quantize_blocks(w, 128, 128)
    ref = oracle.c_matmul_blockwise(xq, wq, xs, ws)
    assert np.array_equal(oracle.bf16_bits(y.reshape(-1, 520)), ref)
    dense = (x.reshape(-1, 1024) @ w.t())
    rel = (y.reshape(-1, 520).float().cpu() - dense).norm() / dense.norm()
    assert rel < 0.02, rel

    layer_c = g.Int8Linear.from_float(w, bias=torch.ones(520), mode="channel", out_dtype=torch.float32).cuda()
    y2 = layer_c(x[0, :4].cuda())
    xq, xs = oracle.c_quantize_blocks(x[0, :4], 1, 1024)
    wq, ws = quant.quantize_per_row(w)
    ref2 = oracle.to_torch_bf16(oracle.c_matmul_scaled(xq, wq, xs.reshape(-1), ws)) + torch.ones(520).bfloat16()
    assert y2.dtype == torch.float32 and torch.equal(y2.cpu(), ref2.float())

    compiled = torch.compile(layer, dynamic=True)
    assert torch.equal(compiled(x.cuda()), y)

    # Rotated layer: activations with outlier channels; bit-equal to the oracle pipeline, and closer to the fp32
    # layer than the unrotated one.
    xo = x.clone()
    xo[..., 7] *= 40.0
    xo[..., 300] *= 25.0
    rot = g.Int8Linear.from_float(w, mode="blockwise", hadamard_block=1024).cuda()
    yr = rot(xo.cuda())
    xq, xs = oracle.c_quantize_blocks(oracle.c_hadamard_rotate(xo.reshape(-1, 1024), 1024), 1, 128)
    wq, ws = oracle.c_quantize_blocks(oracle.c_hadamard_rotate(w, 1024), 128, 128)
    assert np.array_equal(oracle.bf16_bits(yr.reshape(-1, 520)), oracle.c_matmul_blockwise(xq, wq, xs, ws))
    dense_o = xo.reshape(-1, 1024) @ w.t()
    err_rot = (yr.reshape(-1, 520).float().cpu() - dense_o).norm() / dense_o.norm()
    err_plain = (layer(xo.cuda()).reshape(-1, 520).float().cpu() - dense_o).norm() / dense_o.norm()
    assert err_rot < err_plain and err_rot < 0.02, (err_rot, err_plain)


def test_host_pipeline_matches_oracle(g, oracle):
    """Host-buffer front end: pinned operands in, pinned result out, several calls in flight; every result is
    bit-identical to the oracle (and so to the device-tensor op)."""
    from gemm_int8_b200.host import HostPipeline

    gen = torch.Generator().manual_seed(77)
    pipe = HostPipeline("blockwise", depth=2)
    cases = []
    for i, (M, N, K) in enumerate([(130, 264, 400), (64, 512, 1024), (130, 264, 400), (257, 1000, 1040), (1, 8, 16)]):
        KB, NB = -(-K // 128), -(-N // 128)
        x, y = rand_i8((M, K), 100 + i), rand_i8((N, K), 200 + i)
        sa = torch.rand(M, KB, generator=gen) * 0.02 + 1e-3
        sw = torch.rand(NB, KB, generator=gen) * 0.02 + 1e-3
        host_in = [t.pin_memory() for t in (x, y, sa, sw)]
        host_out = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
        pipe.submit(host_in, host_out)
        cases.append((x, y, sa, sw, host_out))
    pipe.drain()
    for (x, y, sa, sw, host_out) in cases:
        assert_bits_equal(oracle, host_out, oracle.c_matmul_blockwise(x, y, sa, sw), "host pipeline")
    plain = HostPipeline("plain", depth=1)
    x, y = rand_i8((70, 256), 301), rand_i8((136, 256), 302)
    out = torch.empty((70, 136), dtype=torch.bfloat16).pin_memory()
    plain.submit([x.pin_memory(), y.pin_memory()], out)
    plain.drain()
    assert_bits_equal(oracle, out, oracle.c_matmul(x, y, 1.0), "host pipeline plain")
    with pytest.raises(ValueError):
        plain.submit([x, y.pin_memory()], out)  # not pinned

"""CPU tests of the drop-in boundary: the C-ABI library loads and exports every declared symbol, the
torch ops exist under the reference's names with working fake kernels, and argument validation that
needs no GPU behaves as documented."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "gemm_int8_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gi8_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from gemm_int8_b200 import _lib

    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert "gi8_matmul" in names and "gi8_matmul_blockwise" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_lib.SYMBOLS), "ctypes table and header disagree"


def test_version_and_error_string():
    import gemm_int8_b200 as g

    assert g._C.gi8_version() >= 100
    assert isinstance(g._C.gi8_last_error(), bytes)


def test_dispatch_table_choices_without_gpu():
    """The per-shape dispatch is host arithmetic over a table (148 SMs assumed without a device): tile form by waves x
    cycles, the two-CTA blockwise form only for long runs, the split-K kernel for thin grids with a long K and for thin
    last waves of long-K shapes, and nothing split where the grid fills the machine."""
    import gemm_int8_b200 as g

    pv = g.pick_variant
    assert pv(0, 8192, 8192, 8192) == "pair"                      # 13.8 waves of two-CTA tiles: no tail worth splitting
    assert pv(0, 1024, 4096, 4096) == "pair"                      # config 1: under one wave
    assert pv(0, 512, 4096, 4096) == "dense_bn128"                # few tiles, short K: narrow tiles, no split
    assert pv(0, 256, 4096, 28672).startswith("splitk")           # few tiles, long K: whole grid split
    assert pv(0, 1024, 14336, 16384) == "pair+splitk8"            # 3.03 waves of long tiles: the last two go to split-K
    assert pv(0, 1024, 14336, 4096) == "pair"                     # the same grid with short tiles: a second launch costs more
    assert pv(2, 2048, 11008, 4096) == "blockwise_bn256"
    assert pv(2, 16384, 57344, 8192) == "blockwise_pair"          # config 5: 193 waves
    assert pv(2, 128, 8192, 8192) == "blockwise_bn64"
    assert pv(2, 512, 10240, 8192) == "blockwise_bn256+columns_bn64"   # 160 tiles: one full wave + the last 768 columns narrow
    assert pv(2, 8192, 8192, 8192) == "blockwise_bn256"
    assert pv(1, 16, 4096, 4096) == "smallm_cluster" and pv(1, 64, 14336, 4096) == "smallm_cluster"
    assert pv(1, 2048, 4096, 4096) == "pair"                      # the scaled entry point above M = 64 is the dense kernel


def test_host_side_validation_without_gpu():
    """Shape/pointer checks run before any CUDA call, so they are testable on a CPU-only box."""
    import gemm_int8_b200 as g

    C = g._C
    buf = ctypes.create_string_buffer(4096 + 64)
    base = (ctypes.addressof(buf) + 63) & ~63
    p = ctypes.c_void_p
    assert C.gi8_matmul(p(base), p(base), p(base), -1, 8, 16, 1.0, None) == 1
    assert C.gi8_matmul(p(base), p(base), p(base), 8, 8, 24, 1.0, None) == 2      # K % 16
    assert b"multiple of 16" in C.gi8_last_error()
    assert C.gi8_matmul(p(base), p(base), p(base), 8, 8, 131072, 1.0, None) == 2  # K limit
    assert C.gi8_matmul(p(base + 1), p(base), p(base), 8, 8, 16, 1.0, None) == 3  # misaligned x
    assert C.gi8_matmul(None, p(base), p(base), 8, 8, 16, 1.0, None) == 1
    assert C.gi8_matmul(p(base), p(base), p(base + 1), 8, 8, 16, 1.0, None) == 3  # misaligned out
    assert C.gi8_matmul(p(base), p(base), None, 0, 8, 16, 1.0, None) == 0         # empty problem is a no-op
    assert C.gi8_matmul_i32(p(base), p(base), p(base + 2), 8, 8, 16, None) == 3
    assert C.gi8_force_variant(b"nonsense") == 1
    assert C.gi8_force_variant(b"dense_bn128") == 0 and C.gi8_force_variant(None) == 0
    # gathering form: argument checks come before any device work
    outs = (ctypes.c_void_p * 2)(base, base)
    args = (p(base), p(base), p(base), 1, p(base), 1)
    assert C.gi8_matmul_blockwise_allgather(*args, outs, 0, 8, 32, 128, 64, 0, None) == 1    # no outputs
    assert C.gi8_matmul_blockwise_allgather(*args, outs, 9, 8, 32, 128, 64, 0, None) == 1    # more than 8 ranks
    assert C.gi8_matmul_blockwise_allgather(*args, outs, 2, 8, 32, 128, 64, 16, None) == 2   # slice start % 32
    assert C.gi8_matmul_blockwise_allgather(*args, outs, 2, 8, 32, 128, 48, 32, None) == 2   # slice past n_total
    assert b"column slice" in C.gi8_last_error()
    bad = (ctypes.c_void_p * 2)(base, base + 2)
    assert C.gi8_matmul_blockwise_allgather(*args, bad, 2, 8, 32, 128, 64, 0, None) == 3     # misaligned peer matrix
    assert C.gi8_peer_alloc(None, 16) == 1 and C.gi8_peer_export(None, None) == 1 and C.gi8_peer_import(None, None) == 1


def test_ops_registered_under_reference_names():
    import gemm_int8  # noqa: F401  (the drop-in package name)

    op = torch.ops.gemm_int8_CUDA.int8_matmul.default
    assert str(op._schema) == "gemm_int8_CUDA::int8_matmul(Tensor A, Tensor B, float alpha) -> Tensor"
    assert gemm_int8.__all__ == ["matmul"]
    for name in ("int8_matmul_scaled", "int8_matmul_blockwise", "int8_matmul_i32"):
        assert hasattr(torch.ops.gemm_int8_CUDA, name)


def test_fake_kernels_propagate_shapes():
    import gemm_int8
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        x = torch.empty(33, 256, dtype=torch.int8, device="cuda")
        y = torch.empty(72, 256, dtype=torch.int8, device="cuda")
        out = gemm_int8.matmul(x, y, 0.5)
        assert out.shape == (33, 72) and out.dtype == torch.bfloat16 and out.device.type == "cuda"
        sa = torch.empty(33, 2, dtype=torch.float32, device="cuda")
        sw = torch.empty(1, 2, dtype=torch.float32, device="cuda")
        assert gemm_int8.matmul_blockwise(x, y, sa, sw).shape == (33, 72)
        sx = torch.empty(33, dtype=torch.float32, device="cuda")
        sc = torch.empty(72, dtype=torch.float32, device="cuda")
        assert gemm_int8.matmul_scaled(x, y, sx, sc).dtype == torch.bfloat16
        with pytest.raises(Exception):
            gemm_int8.matmul(x, torch.empty(72, 128, dtype=torch.int8, device="cuda"), 1.0)
        with pytest.raises(Exception):
            gemm_int8.matmul(x.to(torch.int32), y, 1.0)


def test_cpu_tensors_are_rejected_not_computed():
    """There is no CPU path: calling the op on CPU tensors must fail (the reference raises
    NotImplementedError for the missing CPU kernel as well)."""
    import gemm_int8

    x = torch.zeros(8, 16, dtype=torch.int8)
    with pytest.raises((NotImplementedError, RuntimeError)):
        gemm_int8.matmul(x, x, 1.0)


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "gemm_int8_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("CPU oracle's blockwise restatement", ""), f


def test_host_pipeline_rejects_bad_arguments_without_gpu():
    import torch

    from gemm_int8_b200.host import HostPipeline

    with pytest.raises(ValueError):
        HostPipeline("nonsense")
    with pytest.raises(ValueError):
        HostPipeline("plain", depth=0)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            HostPipeline("plain")  # no CPU path

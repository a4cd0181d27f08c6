"""CPU oracle for the INT8 GEMM path -- TEST INFRASTRUCTURE, not part of the shipped library.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this module;
the product package never does (it fails loudly when its CUDA library is missing instead).

Two independent restatements of the same arithmetic live here:

* ``c_*``  -- thin ctypes bindings to ``gi8_oracle.c`` (threaded C; fast enough for the full-size
  configurations), built by ``oracle/Makefile`` into ``oracle/_build/libgi8_oracle.so``.
* ``np_*`` -- a numpy restatement written separately, used to cross-check the C code on small cases.

Arithmetic contract (reference file:line, paths inside the reference project):

* ``gemm_int8/__init__.py:28-37``  matmul(x, y, alpha) = bf16((x @ y.T) * alpha); x [M,K], y [N,K] int8
* ``csrc/kernels/gemm.cu:33-37,46-58``  int8 products accumulated in int32
* ``csrc/kernels/gemm.cu:59-63,96``  epilogue: bf16_rne(fp32_rn(acc) * alpha), beta = 0
* ``test.py:8,15``  expected value x.bfloat16() @ x.bfloat16().t()

The scaled and blockwise variants have no reference counterpart; their definition is the one in
``gi8_oracle.c`` ("parity unpinned" by the reference, pinned by this restatement only).
All bf16 results are returned as uint16 bit patterns (numpy has no bf16); ``to_torch_bf16`` views
them as a torch.bfloat16 tensor.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libgi8_oracle.so")
_lib = None

KBLOCK = 128


def build(force: bool = False) -> str:
    """Compile gi8_oracle.c with the committed Makefile (gcc only); returns the .so path."""
    src = os.path.join(_HERE, "gi8_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        build()
    lib = ctypes.CDLL(_LIB_PATH)
    i64, p = ctypes.c_int64, ctypes.c_void_p
    lib.gi8o_matmul_i32.argtypes = [p, p, p, i64, i64, i64]
    lib.gi8o_matmul.argtypes = [p, p, p, i64, i64, i64, ctypes.c_float]
    lib.gi8o_matmul_scaled.argtypes = [p, p, p, p, p, i64, i64, i64]
    lib.gi8o_matmul_blockwise.argtypes = [p, p, p, i64, p, i64, p, p, i64, i64, i64]
    lib.gi8o_quantize_blocks.argtypes = [p, p, p, i64, i64, i64, i64]
    lib.gi8o_hadamard_rotate.argtypes = [p, p, i64, i64, i64]
    lib.gi8o_set_num_threads.argtypes = [ctypes.c_int]
    lib.gi8o_num_threads.restype = ctypes.c_int
    for f in ("gi8o_matmul_i32", "gi8o_matmul", "gi8o_matmul_scaled", "gi8o_matmul_blockwise",
              "gi8o_quantize_blocks", "gi8o_hadamard_rotate"):
        getattr(lib, f).restype = ctypes.c_int
    _lib = lib
    return lib


def set_num_threads(n: int) -> None:
    _load().gi8o_set_num_threads(int(n))


def num_threads() -> int:
    return int(_load().gi8o_num_threads())


def _np(a, dtype):
    """Accept numpy arrays or CPU torch tensors; return a C-contiguous numpy array of dtype."""
    if hasattr(a, "detach"):
        a = a.detach().cpu().contiguous().numpy()
    a = np.ascontiguousarray(a)
    if a.dtype != dtype:
        raise TypeError(f"expected {dtype}, got {a.dtype}")
    return a


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


def _check(st, what):
    if st != 0:
        raise ValueError(f"oracle {what}: bad arguments (status {st})")


def _mnk(x, y):
    if x.ndim != 2 or y.ndim != 2 or x.shape[1] != y.shape[1]:
        raise ValueError("x must be [M,K] and y [N,K] with the same K")
    return x.shape[0], y.shape[0], x.shape[1]


# ------------------------------------------------------------------ C oracle
def c_matmul_i32(x, y):
    x, y = _np(x, np.int8), _np(y, np.int8)
    M, N, K = _mnk(x, y)
    out = np.empty((M, N), np.int32)
    _check(_load().gi8o_matmul_i32(_ptr(x), _ptr(y), _ptr(out), M, N, K), "matmul_i32")
    return out


def c_matmul(x, y, alpha=1.0):
    x, y = _np(x, np.int8), _np(y, np.int8)
    M, N, K = _mnk(x, y)
    out = np.empty((M, N), np.uint16)
    _check(_load().gi8o_matmul(_ptr(x), _ptr(y), _ptr(out), M, N, K, ctypes.c_float(alpha)), "matmul")
    return out


def c_matmul_scaled(x, y, sx, sw):
    x, y = _np(x, np.int8), _np(y, np.int8)
    sx, sw = _np(sx, np.float32).reshape(-1), _np(sw, np.float32).reshape(-1)
    M, N, K = _mnk(x, y)
    if sx.shape[0] != M or sw.shape[0] != N:
        raise ValueError("scale shapes must be [M] and [N]")
    out = np.empty((M, N), np.uint16)
    _check(_load().gi8o_matmul_scaled(_ptr(x), _ptr(y), _ptr(sx), _ptr(sw), _ptr(out), M, N, K), "matmul_scaled")
    return out


def c_matmul_blockwise(x, y, sa, sw, return_acc=False):
    x, y = _np(x, np.int8), _np(y, np.int8)
    sa, sw = _np(sa, np.float32), _np(sw, np.float32)
    M, N, K = _mnk(x, y)
    KB, NB = -(-K // KBLOCK), -(-N // KBLOCK)
    if sa.shape != (M, KB) or sw.shape != (NB, KB):
        raise ValueError(f"scale shapes must be {(M, KB)} and {(NB, KB)}, got {sa.shape} and {sw.shape}")
    out = np.empty((M, N), np.uint16)
    acc = np.empty((M, N), np.float32) if return_acc else None
    st = _load().gi8o_matmul_blockwise(_ptr(x), _ptr(y), _ptr(sa), KB, _ptr(sw), KB, _ptr(out),
                                       _ptr(acc) if return_acc else None, M, N, K)
    _check(st, "matmul_blockwise")
    return (out, acc) if return_acc else out


def c_matmul_blockwise_ksharded(x, y, sa, sw, world, block=KBLOCK):
    """Restatement of the K-sharded (row-parallel) blockwise GEMM: the K blocks are dealt to `world` ranks in whole
    blocks (as evenly as possible, leading ranks one more), each rank's fp32 accumulator is the ascending
    fused-multiply-add chain over ITS blocks, the rank accumulators are added in rank order in fp32
    (round to nearest each step) and the sum is rounded to bf16.  Returns uint16 bit patterns [M, N]."""
    x, y = _np(x, np.int8), _np(y, np.int8)
    sa, sw = _np(sa, np.float32), _np(sw, np.float32)
    K = x.shape[1]
    nb = -(-K // block)
    base, extra = divmod(nb, world)
    total = None
    for r in range(world):
        b0 = r * base + min(r, extra)
        b1 = b0 + base + (1 if r < extra else 0)
        k0, k1 = min(b0 * block, K), min(b1 * block, K)
        if k1 == k0:
            acc = np.zeros((x.shape[0], y.shape[0]), np.float32)
        else:
            _, acc = c_matmul_blockwise(np.ascontiguousarray(x[:, k0:k1]), np.ascontiguousarray(y[:, k0:k1]),
                                        np.ascontiguousarray(sa[:, b0:b1]), np.ascontiguousarray(sw[:, b0:b1]),
                                        return_acc=True)
        total = acc if total is None else (total + acc).astype(np.float32)
    return np_bf16_rne(total)


def c_quantize_blocks(v, rb, cb):
    v = _np(v, np.float32)
    R, C = v.shape
    q = np.empty((R, C), np.int8)
    s = np.empty((-(-R // rb), -(-C // cb)), np.float32)
    _check(_load().gi8o_quantize_blocks(_ptr(v), _ptr(q), _ptr(s), R, C, rb, cb), "quantize_blocks")
    return q, s


def c_hadamard_rotate(v, block):
    """Normalised Walsh-Hadamard rotation along the last axis in blocks of `block` (fp32, butterfly order)."""
    v = _np(v, np.float32)
    R, C = v.shape
    out = np.empty((R, C), np.float32)
    _check(_load().gi8o_hadamard_rotate(_ptr(v), _ptr(out), R, C, block), "hadamard_rotate")
    return out


# ------------------------------------------------------------------ numpy restatement
def np_bf16_rne(f):
    """float32 array -> bf16 bit patterns (uint16), round to nearest even, NaN kept quiet."""
    f = np.ascontiguousarray(f, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    r = np.where(nan, (u >> 16) | 0x40, r)
    return r.astype(np.uint16)


def np_matmul_i32(x, y):
    x, y = _np(x, np.int8), _np(y, np.int8)
    return (x.astype(np.int64) @ y.astype(np.int64).T).astype(np.int32)


def np_matmul(x, y, alpha=1.0):
    acc = np_matmul_i32(x, y).astype(np.float32)  # int32 -> fp32, round to nearest even
    return np_bf16_rne(acc * np.float32(alpha))


def np_matmul_scaled(x, y, sx, sw):
    acc = np_matmul_i32(x, y).astype(np.float32)
    t = _np(sx, np.float32).reshape(-1, 1) * _np(sw, np.float32).reshape(1, -1)  # fp32 product first
    return np_bf16_rne(acc * t)


def np_matmul_blockwise(x, y, sa, sw, return_acc=False):
    """fp32 fused-multiply-add per K block in ascending order.

    numpy has no fmaf; the fused step is emulated exactly in float64: P (|P| < 2^22) times t (24-bit
    mantissa) is exact in float64 (<= 46 bits), and adding the fp32 accumulator then rounding once to
    fp32 equals fmaf unless the float64 sum itself had to round -- which is checked and, in that
    rare case, resolved with exact rational arithmetic.
    """
    from fractions import Fraction

    x, y = _np(x, np.int8), _np(y, np.int8)
    sa, sw = _np(sa, np.float32), _np(sw, np.float32)
    M, N, K = _mnk(x, y)
    KB = -(-K // KBLOCK)
    acc = np.zeros((M, N), np.float32)
    nb = np.arange(N) // KBLOCK
    for kb in range(KB):
        k0, k1 = kb * KBLOCK, min(K, (kb + 1) * KBLOCK)
        P = x[:, k0:k1].astype(np.int64) @ y[:, k0:k1].astype(np.int64).T
        t = (sa[:, kb].reshape(-1, 1) * sw[nb, kb].reshape(1, -1)).astype(np.float32)
        prod = P.astype(np.float64) * t.astype(np.float64)          # exact (<= 46 significant bits)
        a64 = acc.astype(np.float64)
        s64 = prod + a64                                             # may round to 53 bits
        bb = s64 - prod
        err = (prod - (s64 - bb)) + (a64 - bb)                       # TwoSum: exact rounding error of s64
        new = s64.astype(np.float32)
        # Rounding twice (to 53 bits, then to 24) differs from a single rounding only when the float64
        # sum is inexact AND sits exactly on a fp32 tie (or in the fp32 subnormal range): redo those
        # entries with exact rational arithmetic.
        dropped = s64.view(np.uint64) & np.uint64((1 << 29) - 1)
        risky = (err != 0) & ((dropped == np.uint64(1 << 28)) | (np.abs(s64) < 2.0 ** -126))
        for m, n in zip(*np.nonzero(risky)):
            exact = Fraction(int(P[m, n])) * Fraction(float(t[m, n])) + Fraction(float(acc[m, n]))
            new[m, n] = _round_fraction_to_f32(exact)
        acc = new
    out = np_bf16_rne(acc)
    return (out, acc) if return_acc else out


def _round_fraction_to_f32(fr):
    """Round an exact rational to the nearest float32 (ties to even)."""
    from fractions import Fraction

    if fr == 0:
        return np.float32(0.0)
    lo = np.float32(float(fr))  # float(fr) is correctly rounded to float64; then to fp32 -> candidate
    cands = [lo, np.nextafter(lo, np.float32(np.inf), dtype=np.float32),
             np.nextafter(lo, np.float32(-np.inf), dtype=np.float32)]
    best = None
    for c in cands:
        d = abs(Fraction(float(c)) - fr)
        key = (d, int(np.float32(c).view(np.uint32)) & 1)
        if best is None or key < best[0]:
            best = (key, c)
    return best[1]


def np_quantize_blocks(v, rb, cb):
    v = _np(v, np.float32)
    R, C = v.shape
    q = np.empty((R, C), np.int8)
    s = np.empty((-(-R // rb), -(-C // cb)), np.float32)
    for br in range(s.shape[0]):
        for bc in range(s.shape[1]):
            blk = v[br * rb:(br + 1) * rb, bc * cb:(bc + 1) * cb]
            amax = np.float32(np.abs(blk).max()) if blk.size else np.float32(0)
            sc = np.float32(amax / np.float32(127.0)) if amax > 0 else np.float32(1.0)
            s[br, bc] = sc
            q[br * rb:(br + 1) * rb, bc * cb:(bc + 1) * cb] = np.clip(np.rint(blk / sc), -127, 127).astype(np.int8)
    return q, s


# ------------------------------------------------------------------ helpers for tests
def to_torch_bf16(bits):
    import torch

    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)


def bf16_bits(t):
    """torch.bfloat16 tensor (any device) -> numpy uint16 bit patterns."""
    import torch

    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bf16_ulp_distance(a_bits, b_bits):
    """Distance in units of bf16 representable steps between two bit-pattern arrays (finite values)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(np.asarray(a_bits)) - key(np.asarray(b_bits)))

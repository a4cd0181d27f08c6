"""B200-native INT8 GEMM behind the reference's Python/PyTorch operator surface.

Mirrors gemm_int8/__init__.py of the reference:

* ``matmul(x, y, alpha=1.0)`` -> bf16 ``(x @ y.T) * alpha``            (gemm_int8/__init__.py:28-37)
* torch op ``gemm_int8_CUDA::int8_matmul(Tensor A, Tensor B, float alpha) -> Tensor`` with a CUDA
  implementation and a fake (meta) kernel                          (csrc/kernels/bindings.cpp:30-38,
                                                                     gemm_int8/__init__.py:16-25)

and adds the W8A8 entry points the reference lacks: ``matmul_scaled`` (per-token x per-channel scales)
and ``matmul_blockwise`` (per-token-per-128-K activation scales, per-128x128 weight scales).

The torch ops are registered from Python and call the C ABI of ``libgemm_int8_b200.so`` through ctypes
with raw device pointers and the current CUDA stream.  Importing this package without the compiled
library raises ImportError, as the reference does (gemm_int8/__init__.py:9-10); there is no CPU path.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_C = _lib.load()

KBLOCK = 128

# --------------------------------------------------------------------------------------------------
# op schemas.  Namespace, name and schema of int8_matmul are the reference's (bindings.cpp:30-33).
# --------------------------------------------------------------------------------------------------
_NS = "gemm_int8_CUDA"
_libdef = torch.library.Library(_NS, "DEF")
_libdef.define("int8_matmul(Tensor A, Tensor B, float alpha) -> Tensor")
_libdef.define("int8_matmul_i32(Tensor A, Tensor B) -> Tensor")
_libdef.define("int8_matmul_scaled(Tensor A, Tensor B, Tensor a_scale, Tensor b_scale) -> Tensor")
_libdef.define("int8_matmul_blockwise(Tensor A, Tensor B, Tensor A_scale, Tensor B_scale) -> Tensor")
_libdef.define("int8_matmul_blockwise_f32(Tensor A, Tensor B, Tensor A_scale, Tensor B_scale) -> Tensor")
_libdef.define("quantize_token_block(Tensor a) -> (Tensor, Tensor)")
_libdef.define("quantize_token(Tensor a) -> (Tensor, Tensor)")
_libdef.define("hadamard_quantize_token_block(Tensor a, int block) -> (Tensor, Tensor)")


def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class _on_device:
    """Makes `device` current for the duration of a launch (no-op when it already is)."""

    __slots__ = ("idx", "prev")

    def __init__(self, device: torch.device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def _check_operands(name: str, A: torch.Tensor, B: torch.Tensor) -> tuple[int, int, int]:
    # The reference checks contiguity, device type and same-GPU (bindings.cpp:15-20) and leaves dtype,
    # rank and the K match to its fake kernel (__init__.py:18-24); here the real kernel checks them all.
    if not (A.is_cuda and B.is_cuda):
        raise RuntimeError(f"{name}: A and B must be CUDA tensors")
    if A.device != B.device:
        raise RuntimeError(f"{name}: A and B must be on the same GPU, got {A.device} and {B.device}")
    if A.dtype != torch.int8 or B.dtype != torch.int8:
        raise RuntimeError(f"{name}: A and B must be int8, got {A.dtype} and {B.dtype}")
    if A.dim() != 2 or B.dim() != 2:
        raise RuntimeError(f"{name}: A and B must be 2-D")
    if A.shape[1] != B.shape[1]:
        raise RuntimeError(f"{name}: A.shape[1] ({A.shape[1]}) must equal B.shape[1] ({B.shape[1]})")
    if not A.is_contiguous() or not B.is_contiguous():
        raise RuntimeError(f"{name}: A and B must be contiguous")
    return A.shape[0], B.shape[0], A.shape[1]


def _check_scale(name: str, what: str, t: torch.Tensor, shape: tuple, device: torch.device) -> None:
    if t.device != device:
        raise RuntimeError(f"{name}: {what} must be on {device}, got {t.device}")
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name}: {what} must be float32, got {t.dtype}")
    if tuple(t.shape) != tuple(shape):
        raise RuntimeError(f"{name}: {what} must have shape {tuple(shape)}, got {tuple(t.shape)}")


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


# --------------------------------------------------------------------------------------------------
# CUDA implementations
# --------------------------------------------------------------------------------------------------
def _int8_matmul_cuda(A: torch.Tensor, B: torch.Tensor, alpha: float) -> torch.Tensor:
    M, N, K = _check_operands("int8_matmul", A, B)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    with _on_device(A.device):
        rc = _C.gi8_matmul(_ptr(A), _ptr(B), _ptr(out), M, N, K, float(alpha), _stream_ptr(A.device))
    _lib.check(_C, rc)
    return out


def _int8_matmul_i32_cuda(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    M, N, K = _check_operands("int8_matmul_i32", A, B)
    out = torch.empty((M, N), dtype=torch.int32, device=A.device)
    with _on_device(A.device):
        rc = _C.gi8_matmul_i32(_ptr(A), _ptr(B), _ptr(out), M, N, K, _stream_ptr(A.device))
    _lib.check(_C, rc)
    return out


_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int, stream: int) -> torch.Tensor | None:
    """Zero-filled scratch buffer, one per (device, stream); kernels leave it zero-filled."""
    if nbytes <= 0:
        return None
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _int8_matmul_scaled_cuda(A: torch.Tensor, B: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor) -> torch.Tensor:
    name = "int8_matmul_scaled"
    M, N, K = _check_operands(name, A, B)
    a_scale = a_scale.reshape(-1) if a_scale.dim() == 2 and a_scale.shape[-1] == 1 else a_scale
    b_scale = b_scale.reshape(-1) if b_scale.dim() == 2 and b_scale.shape[-1] == 1 else b_scale
    _check_scale(name, "a_scale", a_scale, (M,), A.device)
    _check_scale(name, "b_scale", b_scale, (N,), A.device)
    a_scale, b_scale = a_scale.contiguous(), b_scale.contiguous()
    out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    with _on_device(A.device):
        stream = _stream_ptr(A.device)
        nbytes = int(_C.gi8_matmul_scaled_workspace_bytes(M, N, K))
        ws = _workspace(A.device, nbytes, stream.value or 0)
        rc = _C.gi8_matmul_scaled(_ptr(A), _ptr(B), _ptr(a_scale), _ptr(b_scale), _ptr(out), M, N, K,
                                  _ptr(ws) if ws is not None else None, ws.numel() if ws is not None else 0, stream)
    _lib.check(_C, rc)
    return out


def _int8_matmul_blockwise_cuda(A: torch.Tensor, B: torch.Tensor, A_scale: torch.Tensor, B_scale: torch.Tensor,
                                f32: bool = False) -> torch.Tensor:
    name = "int8_matmul_blockwise_f32" if f32 else "int8_matmul_blockwise"
    M, N, K = _check_operands(name, A, B)
    KB, NB = -(-K // KBLOCK), -(-N // KBLOCK)
    _check_scale(name, "A_scale", A_scale, (M, KB), A.device)
    _check_scale(name, "B_scale", B_scale, (NB, KB), A.device)
    if A_scale.dim() == 2 and A_scale.stride(1) != 1 and KB > 1:
        A_scale = A_scale.contiguous()
    if B_scale.dim() == 2 and B_scale.stride(1) != 1 and KB > 1:
        B_scale = B_scale.contiguous()
    ld_sa = A_scale.stride(0) if M > 1 else KB
    ld_sw = B_scale.stride(0) if NB > 1 else KB
    if ld_sa < KB:
        A_scale, ld_sa = A_scale.contiguous(), KB
    if ld_sw < KB:
        B_scale, ld_sw = B_scale.contiguous(), KB
    out = torch.empty((M, N), dtype=torch.float32 if f32 else torch.bfloat16, device=A.device)
    fn = _C.gi8_matmul_blockwise_f32 if f32 else _C.gi8_matmul_blockwise
    with _on_device(A.device):
        rc = fn(_ptr(A), _ptr(B), _ptr(A_scale), ld_sa, _ptr(B_scale), ld_sw, _ptr(out), M, N, K, _stream_ptr(A.device))
    _lib.check(_C, rc)
    return out


_libdef.impl("int8_matmul", _int8_matmul_cuda, "CUDA")
_libdef.impl("int8_matmul_i32", _int8_matmul_i32_cuda, "CUDA")
_libdef.impl("int8_matmul_scaled", _int8_matmul_scaled_cuda, "CUDA")
_libdef.impl("int8_matmul_blockwise", _int8_matmul_blockwise_cuda, "CUDA")
_libdef.impl("int8_matmul_blockwise_f32", lambda A, B, sa, sw: _int8_matmul_blockwise_cuda(A, B, sa, sw, True), "CUDA")


# --------------------------------------------------------------------------------------------------
# fake (meta) kernels: shape/dtype propagation for torch.compile, as gemm_int8/__init__.py:16-25
# --------------------------------------------------------------------------------------------------
def _fake_common(x: torch.Tensor, y: torch.Tensor) -> None:
    torch._check(x.device.type == "cuda", lambda: "x must be a CUDA tensor")
    torch._check(y.device.type == "cuda", lambda: "y must be a CUDA tensor")
    torch._check(x.dtype == torch.int8, lambda: "x must be an int8 tensor")
    torch._check(y.dtype == torch.int8, lambda: "y must be an int8 tensor")
    torch._check(len(x.shape) == 2, lambda: "x must be a 2D tensor")
    torch._check(len(y.shape) == 2, lambda: "y must be a 2D tensor")
    torch._check(x.shape[1] == y.shape[1], lambda: "x.shape[1] must be equal to y.shape[1]")


@torch.library.register_fake(f"{_NS}::int8_matmul")
def _(x: torch.Tensor, y: torch.Tensor, alpha: float = 1.0):
    _fake_common(x, y)
    return torch.empty(x.shape[0], y.shape[0], device=x.device, dtype=torch.bfloat16)


@torch.library.register_fake(f"{_NS}::int8_matmul_i32")
def _(x: torch.Tensor, y: torch.Tensor):
    _fake_common(x, y)
    return torch.empty(x.shape[0], y.shape[0], device=x.device, dtype=torch.int32)


@torch.library.register_fake(f"{_NS}::int8_matmul_scaled")
def _(x: torch.Tensor, y: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor):
    _fake_common(x, y)
    torch._check(a_scale.dtype == torch.float32 and b_scale.dtype == torch.float32, lambda: "scales must be float32")
    return torch.empty(x.shape[0], y.shape[0], device=x.device, dtype=torch.bfloat16)


@torch.library.register_fake(f"{_NS}::int8_matmul_blockwise")
def _(x: torch.Tensor, y: torch.Tensor, A_scale: torch.Tensor, B_scale: torch.Tensor):
    _fake_common(x, y)
    torch._check(A_scale.dtype == torch.float32 and B_scale.dtype == torch.float32, lambda: "scales must be float32")
    torch._check(len(A_scale.shape) == 2 and len(B_scale.shape) == 2, lambda: "scales must be 2D tensors")
    return torch.empty(x.shape[0], y.shape[0], device=x.device, dtype=torch.bfloat16)


@torch.library.register_fake(f"{_NS}::int8_matmul_blockwise_f32")
def _(x: torch.Tensor, y: torch.Tensor, A_scale: torch.Tensor, B_scale: torch.Tensor):
    _fake_common(x, y)
    torch._check(A_scale.dtype == torch.float32 and B_scale.dtype == torch.float32, lambda: "scales must be float32")
    torch._check(len(A_scale.shape) == 2 and len(B_scale.shape) == 2, lambda: "scales must be 2D tensors")
    return torch.empty(x.shape[0], y.shape[0], device=x.device, dtype=torch.float32)


# --------------------------------------------------------------------------------------------------
# public functions
# --------------------------------------------------------------------------------------------------
def matmul(x: torch.Tensor, y: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
    """INT8 matrix product ``(x @ y.t()) * alpha`` returned as bf16.

    Same call as the reference's ``gemm_int8.matmul`` (gemm_int8/__init__.py:28-37).

    Arguments:
        x: int8 CUDA tensor of shape (M, K), contiguous
        y: int8 CUDA tensor of shape (N, K), contiguous
        alpha: scalar multiplied into the fp32-converted int32 accumulator before the bf16 cast
    """
    return torch.ops.gemm_int8_CUDA.int8_matmul(x, y, alpha)


def matmul_i32(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """Raw int32 accumulators ``x @ y.t()`` (bit-exact verification of the integer main loop)."""
    return torch.ops.gemm_int8_CUDA.int8_matmul_i32(x, y)


def matmul_scaled(x_q: torch.Tensor, w_q: torch.Tensor, x_scale: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """W8A8 GEMM with per-token and per-output-channel scales.

    ``out[m, n] = bf16( fp32(acc[m, n]) * (x_scale[m] * w_scale[n]) )`` with ``acc = x_q @ w_q.t()`` in int32.
    x_q (M, K) int8, w_q (N, K) int8, x_scale (M,) fp32, w_scale (N,) fp32.
    """
    return torch.ops.gemm_int8_CUDA.int8_matmul_scaled(x_q, w_q, x_scale, w_scale)


def matmul_blockwise(x_q: torch.Tensor, w_q: torch.Tensor, x_scale: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """Blockwise-dequantised W8A8 GEMM.

    ``out[m, n] = bf16( sum_kb fp32(P[m, n, kb]) * (x_scale[m, kb] * w_scale[n // 128, kb]) )`` where ``P`` is
    the exact int32 dot product over the kb-th 128-wide K block, accumulated in fp32 with one fused
    multiply-add per block in ascending kb order.
    x_q (M, K) int8, w_q (N, K) int8, x_scale (M, ceil(K/128)) fp32, w_scale (ceil(N/128), ceil(K/128)) fp32.
    """
    return torch.ops.gemm_int8_CUDA.int8_matmul_blockwise(x_q, w_q, x_scale, w_scale)


def matmul_blockwise_f32(x_q: torch.Tensor, w_q: torch.Tensor, x_scale: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """`matmul_blockwise` before its bf16 cast: the fp32 accumulators (one fused multiply-add per 128-wide K block,
    ascending).  The partial result of a K-sharded GEMM (see `dist.matmul_blockwise_ksharded`)."""
    return torch.ops.gemm_int8_CUDA.int8_matmul_blockwise_f32(x_q, w_q, x_scale, w_scale)


def sum_parts_bf16(parts: torch.Tensor) -> torch.Tensor:
    """parts fp32 [P, ...] (contiguous) -> bf16 [...]: ((parts[0] + parts[1]) + parts[2]) + ... in fp32, cast once."""
    if not parts.is_cuda or parts.dtype != torch.float32 or parts.dim() < 2:
        raise RuntimeError("sum_parts_bf16: a CUDA float32 tensor [P, ...] is expected")
    parts = parts.contiguous()
    P = parts.shape[0]
    count = parts[0].numel()
    out = torch.empty(parts.shape[1:], dtype=torch.bfloat16, device=parts.device)
    with _on_device(parts.device):
        rc = _C.gi8_sum_parts_bf16(_ptr(parts), P, count, _ptr(out), count, _stream_ptr(parts.device))
    _lib.check(_C, rc)
    return out


def _quantize(a: torch.Tensor, per_block: bool):
    if not a.is_cuda:
        raise RuntimeError("quantize: input must be a CUDA tensor (the torch reference lives in gemm_int8_b200.quant)")
    if a.dim() != 2:
        raise RuntimeError("quantize: input must be 2-D [tokens, features]")
    if a.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError(f"quantize: input must be float32 or bfloat16, got {a.dtype}")
    a = a.contiguous()
    M, K = a.shape
    q = torch.empty((M, K), dtype=torch.int8, device=a.device)
    s = torch.empty((M, -(-K // KBLOCK)) if per_block else (M,), dtype=torch.float32, device=a.device)
    fn = _C.gi8_quantize_token_block if per_block else _C.gi8_quantize_token
    with _on_device(a.device):
        rc = fn(_ptr(a), 0 if a.dtype == torch.float32 else 1, _ptr(q), _ptr(s), M, K, _stream_ptr(a.device))
    _lib.check(_C, rc)
    return q, s


def _hadamard_quantize(a: torch.Tensor, block: int):
    if not a.is_cuda:
        raise RuntimeError("hadamard_quantize: input must be a CUDA tensor (the torch reference lives in gemm_int8_b200.quant)")
    if a.dim() != 2:
        raise RuntimeError("hadamard_quantize: input must be 2-D [tokens, features]")
    if a.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError(f"hadamard_quantize: input must be float32 or bfloat16, got {a.dtype}")
    a = a.contiguous()
    M, K = a.shape
    q = torch.empty((M, K), dtype=torch.int8, device=a.device)
    s = torch.empty((M, -(-K // KBLOCK)), dtype=torch.float32, device=a.device)
    with _on_device(a.device):
        rc = _C.gi8_hadamard_quantize_token_block(_ptr(a), 0 if a.dtype == torch.float32 else 1, _ptr(q), _ptr(s), M, K,
                                                  block, _stream_ptr(a.device))
    _lib.check(_C, rc)
    return q, s


_libdef.impl("hadamard_quantize_token_block", _hadamard_quantize, "CUDA")
_libdef.impl("quantize_token_block", lambda a: _quantize(a, True), "CUDA")
_libdef.impl("quantize_token", lambda a: _quantize(a, False), "CUDA")


@torch.library.register_fake(f"{_NS}::quantize_token_block")
def _(a: torch.Tensor):
    torch._check(len(a.shape) == 2, lambda: "a must be a 2D tensor")
    kb = (a.shape[1] + KBLOCK - 1) // KBLOCK
    return (torch.empty(a.shape[0], a.shape[1], device=a.device, dtype=torch.int8),
            torch.empty(a.shape[0], kb, device=a.device, dtype=torch.float32))


@torch.library.register_fake(f"{_NS}::hadamard_quantize_token_block")
def _(a: torch.Tensor, block: int):
    torch._check(len(a.shape) == 2, lambda: "a must be a 2D tensor")
    kb = (a.shape[1] + KBLOCK - 1) // KBLOCK
    return (torch.empty(a.shape[0], a.shape[1], device=a.device, dtype=torch.int8),
            torch.empty(a.shape[0], kb, device=a.device, dtype=torch.float32))


@torch.library.register_fake(f"{_NS}::quantize_token")
def _(a: torch.Tensor):
    torch._check(len(a.shape) == 2, lambda: "a must be a 2D tensor")
    return (torch.empty(a.shape[0], a.shape[1], device=a.device, dtype=torch.int8),
            torch.empty(a.shape[0], device=a.device, dtype=torch.float32))


def quantize_per_token_block(a: torch.Tensor):
    """Fused activation quantiser for `matmul_blockwise`: a [M, K] fp32/bf16 (CUDA) -> (q int8 [M, K],
    scales fp32 [M, ceil(K/128)]), one symmetric scale per token per 128-wide K block (amax / 127, round half
    even, clamp to +-127) -- bit-identical to `quant.quantize_per_token_block`."""
    return torch.ops.gemm_int8_CUDA.quantize_token_block(a)


def hadamard_quantize_per_token_block(a: torch.Tensor, block: int | None = None):
    """Walsh-Hadamard rotation along K in blocks of `block` (default: the largest power of two dividing K, at most
    8192) fused with `quantize_per_token_block` in one pass over the activations -- bit-identical to
    `quant.quantize_per_token_block(quant.hadamard_rotate(a.float(), block))`.  The weights must have been rotated
    the same way before they were quantised (offline)."""
    K = a.shape[-1]
    if block is None:
        block = min(K & -K, 8192)
    return torch.ops.gemm_int8_CUDA.hadamard_quantize_token_block(a, block)


def quantize_per_token(a: torch.Tensor):
    """Fused per-token quantiser for `matmul_scaled`: a [M, K] -> (q int8 [M, K], scales fp32 [M])."""
    return torch.ops.gemm_int8_CUDA.quantize_token(a)


def force_variant(name: str | None) -> None:
    """Force a kernel variant ("dense_bn256", "dense_bn128", "dense_bn64", "pair", "smallm", "smallm_cluster");
    None = fitted dispatch."""
    _lib.check(_C, _C.gi8_force_variant(name.encode() if name else None))


def pick_variant(kind: int, M: int, N: int, K: int) -> str:
    """Variant the dispatch selects for a shape; kind 0 plain, 1 scaled, 2 blockwise."""
    return _C.gi8_pick_variant(kind, M, N, K).decode()


def device_status() -> int:
    """Synchronises the current device and returns (then clears) its kernel status word; 0 = healthy.

    A non-zero word means a kernel gave up a bounded wait and may have left the split-K scratch of the
    "smallm" variant half-summed, so the cached scratch buffers are dropped (the next call allocates zeroed ones)."""
    code = ctypes.c_uint32(0)
    _lib.check(_C, _C.gi8_device_status(ctypes.byref(code)))
    if code.value:
        _workspaces.clear()
    return int(code.value)


def check_device() -> None:
    """Synchronises the current device and raises GemmInt8Error (GI8_ERR_DEVICE_TIMEOUT) if a kernel since the
    last check gave up a bounded wait -- the counterpart of the reference's exception on a failed launch
    (csrc/kernels/gemm.cu:108-121)."""
    rc = _C.gi8_device_check()
    if rc:
        _workspaces.clear()
    _lib.check(_C, rc)


def reload_env() -> None:
    """Re-reads the GEMM_INT8_* tuning variables (they are otherwise read once, at first use)."""
    _lib.check(_C, _C.gi8_reload_env())


# GEMM_INT8_KERNEL=<variant> forces a kernel variant for the whole process (tuning and profiling).
import os as _os

if _os.environ.get("GEMM_INT8_KERNEL"):
    force_variant(_os.environ["GEMM_INT8_KERNEL"])


from .linear import Int8Linear  # noqa: E402

__all__ = ["matmul", "matmul_i32", "matmul_scaled", "matmul_blockwise", "matmul_blockwise_f32", "sum_parts_bf16",
           "quantize_per_token_block",
           "quantize_per_token", "Int8Linear", "force_variant", "pick_variant", "device_status", "check_device", "reload_env"]

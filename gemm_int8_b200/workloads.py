"""Seeded synthetic inputs for the five benchmark configurations (CPU tensors).

No public dataset is involved: the shapes are Llama-class layer shapes and the value distributions are
the ones the configurations state (uniform int8, or symmetric quantisation of Gaussians).  Inputs are
generated on the CPU with fixed seeds so that a CPU checker and the GPU kernels see identical bits.
"""
from __future__ import annotations

import torch

from . import quant


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def plain(M: int = 1024, N: int = 4096, K: int = 4096, seed: int = 1001):
    """Config 1: uniform int8 in [-128, 127) (upper bound exclusive), alpha = 1."""
    x = torch.randint(-128, 127, (M, K), dtype=torch.int8, generator=_gen(seed))
    y = torch.randint(-128, 127, (N, K), dtype=torch.int8, generator=_gen(seed + 1))
    return x, y, 1.0


def blockwise_prefill(M: int = 2048, N: int = 11008, K: int = 4096, seed: int = 2001):
    """Config 2: activations N(0,1) quantised per token per 128-K block; weights N(0, 0.02) per 128x128 block."""
    a = torch.randn(M, K, generator=_gen(seed))
    w = torch.randn(N, K, generator=_gen(seed + 1)) * 0.02
    xq, sa = quant.quantize_per_token_block(a)
    wq, sw = quant.quantize_weight_block(w)
    return xq, wq, sa, sw


def decode(M: int, N: int, K: int, seed: int = 3001):
    """Config 3: per-token activation scales [M], per-output-channel weight scales [N]."""
    a = torch.randn(M, K, generator=_gen(seed))
    w = torch.randn(N, K, generator=_gen(seed + 1)) * 0.02
    xq, sx = quant.quantize_per_row(a)
    wq, sw = quant.quantize_per_row(w)
    return xq, wq, sx, sw


def llama70b(M: int, N: int, K: int, seed: int = 4001, outliers_first: bool = True):
    """Config 4: Gaussian activations with 0.1 % outlier channels (x20), Hadamard-rotated along K in blocks of
    the largest power of two dividing K, quantised per token per 128-K block; weights per 128x128 block."""
    a = torch.randn(M, K, generator=_gen(seed))
    idx = torch.randperm(K, generator=_gen(seed + 1))[: max(1, round(0.001 * K))]
    if outliers_first:
        a[:, idx] *= 20.0
        a = quant.hadamard_rotate(a)
    else:
        a = quant.hadamard_rotate(a)
        a[:, idx] *= 20.0
    w = torch.randn(N, K, generator=_gen(seed + 2)) * 0.02
    xq, sa = quant.quantize_per_token_block(a)
    wq, sw = quant.quantize_weight_block(w)
    return xq, wq, sa, sw


def nshard(M: int = 16384, N: int = 57344, K: int = 8192, seed: int = 5001):
    """Config 5: uniform int8 operands with synthetic blockwise scales (rand * 0.02 + 0.001)."""
    x = torch.randint(-128, 127, (M, K), dtype=torch.int8, generator=_gen(seed))
    y = torch.randint(-128, 127, (N, K), dtype=torch.int8, generator=_gen(seed + 1))
    g = _gen(seed + 2)
    KB, NB = -(-K // 128), -(-N // 128)
    sa = torch.rand(M, KB, generator=g) * 0.02 + 0.001
    sw = torch.rand(NB, KB, generator=g) * 0.02 + 0.001
    return x, y, sa, sw


def ops(M: int, N: int, K: int) -> int:
    """Algorithmic integer operations of one GEMM (multiply and add counted separately)."""
    return 2 * M * N * K


def bytes_moved(M: int, N: int, K: int, n_scales: int = 0) -> int:
    """Algorithmic bytes: both int8 operands read once, bf16 result written once, fp32 scales read once."""
    return M * K + N * K + 2 * M * N + 4 * n_scales

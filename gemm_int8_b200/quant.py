"""Symmetric int8 quantisers and the Hadamard rotation that produce the W8A8 operands.

These are the callers' side of the GEMM (the reference ships none; its benchmark only rounds and clamps,
benchmark.py:17-18).  Plain torch ops, device-agnostic, used to build the synthetic workloads and by
users who do not have a fused quantiser of their own.  Rule everywhere:
    s = amax / 127   (s = 1 where the block is all zero),   q = clamp(round_half_even(v / s), -127, 127)
"""
from __future__ import annotations

import torch

KBLOCK = 128


def _quant(v: torch.Tensor, amax: torch.Tensor):
    s = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    return s


def quantize_per_token_block(a: torch.Tensor, block: int = KBLOCK):
    """a fp32 [M, K] -> (q int8 [M, K], s fp32 [M, ceil(K/block)]), one scale per row per K block."""
    M, K = a.shape
    KB = -(-K // block)
    pad = KB * block - K
    ap = torch.nn.functional.pad(a, (0, pad)) if pad else a
    blk = ap.reshape(M, KB, block)
    s = _quant(blk, blk.abs().amax(dim=2))
    q = torch.round(blk / s.unsqueeze(2)).clamp_(-127, 127).to(torch.int8).reshape(M, KB * block)
    return q[:, :K].contiguous(), s.contiguous()


def quantize_weight_block(w: torch.Tensor, block: int = KBLOCK):
    """w fp32 [N, K] -> (q int8 [N, K], s fp32 [ceil(N/block), ceil(K/block)]), one scale per block x block tile."""
    N, K = w.shape
    NB, KB = -(-N // block), -(-K // block)
    wp = torch.nn.functional.pad(w, (0, KB * block - K, 0, NB * block - N))
    blk = wp.reshape(NB, block, KB, block)
    s = _quant(blk, blk.abs().amax(dim=(1, 3)))
    q = torch.round(blk / s[:, None, :, None]).clamp_(-127, 127).to(torch.int8).reshape(NB * block, KB * block)
    return q[:N, :K].contiguous(), s.contiguous()


def quantize_per_row(a: torch.Tensor):
    """a fp32 [R, C] -> (q int8 [R, C], s fp32 [R]): per-token activations or per-output-channel weights."""
    s = _quant(a, a.abs().amax(dim=1))
    q = torch.round(a / s.unsqueeze(1)).clamp_(-127, 127).to(torch.int8)
    return q.contiguous(), s.contiguous()


def hadamard_rotate(a: torch.Tensor, block: int | None = None) -> torch.Tensor:
    """Normalised Walsh-Hadamard transform along the last dimension in blocks of `block` (a power of two;
    default: the largest power of two dividing the dimension)."""
    K = a.shape[-1]
    if block is None:
        block = K & -K
    if block & (block - 1) or K % block:
        raise ValueError("block must be a power of two dividing the last dimension")
    y = a.reshape(*a.shape[:-1], K // block, block).clone()
    h = 1
    while h < block:
        y = y.reshape(*y.shape[:-1], block // (2 * h), 2, h)
        y = torch.stack((y[..., 0, :] + y[..., 1, :], y[..., 0, :] - y[..., 1, :]), dim=-2)
        y = y.reshape(*y.shape[:-3], block)
        h *= 2
    return (y * (block ** -0.5)).reshape(a.shape)


def dequantize_blockwise(q: torch.Tensor, s: torch.Tensor, row_block: int, col_block: int = KBLOCK) -> torch.Tensor:
    """Inverse of the block quantisers (for accuracy checks): q * s broadcast over (row_block x col_block) tiles."""
    R, C = q.shape
    se = s.repeat_interleave(row_block, dim=0)[:R].repeat_interleave(col_block, dim=1)[:, :C]
    return q.to(torch.float32) * se

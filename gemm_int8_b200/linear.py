"""W8A8 linear layer built on the INT8 GEMM entry points.

The reference exposes only the raw matmul and leaves "arbitrary output dtype" and the layer around it to the
caller (gemm_int8/__init__.py:31, README usage section).  `Int8Linear` is that caller: weights are quantised once
(offline), activations are quantised on the fly by the fused CUDA quantiser, and the product runs on the blockwise
or the per-token x per-channel GEMM.  Inference only (the reference has no autograd either).
"""
from __future__ import annotations

import torch

from . import quant


class Int8Linear(torch.nn.Module):
    """y = x @ W.T (+ bias) with W and x in int8.

    mode="blockwise": per-128x128 weight scales, per-token-per-128-K activation scales (prefill-style shapes).
    mode="channel":   per-output-channel weight scales, per-token activation scales (decode-style shapes).

    hadamard_block (blockwise mode only): rotate activations and weights along the input features with a normalised
    Walsh-Hadamard transform in blocks of that size before quantising them (the rotation is orthogonal, so the
    product is unchanged; outlier channels are spread over their block, which is what the rotation is for).  The
    weights are rotated once in `from_float`; the activations by the fused rotate-and-quantise kernel.
    """

    def __init__(self, weight_q: torch.Tensor, weight_scale: torch.Tensor, bias: torch.Tensor | None = None,
                 mode: str = "blockwise", out_dtype: torch.dtype = torch.bfloat16, hadamard_block: int | None = None):
        super().__init__()
        if mode not in ("blockwise", "channel"):
            raise ValueError("mode must be 'blockwise' or 'channel'")
        if hadamard_block is not None and mode != "blockwise":
            raise ValueError("hadamard_block needs mode='blockwise'")
        self.mode = mode
        self.out_dtype = out_dtype
        self.hadamard_block = hadamard_block
        self.register_buffer("weight_q", weight_q.contiguous())
        self.register_buffer("weight_scale", weight_scale.contiguous())
        self.register_buffer("bias", bias)

    @classmethod
    def from_float(cls, weight: torch.Tensor, bias: torch.Tensor | None = None, mode: str = "blockwise",
                   out_dtype: torch.dtype = torch.bfloat16, hadamard_block: int | None = None) -> "Int8Linear":
        """Quantises an fp32/bf16 weight [out_features, in_features] once, on whatever device it lives."""
        w = weight.detach().to(torch.float32)
        if hadamard_block is not None:
            w = quant.hadamard_rotate(w, hadamard_block)
        if mode == "blockwise":
            wq, ws = quant.quantize_weight_block(w)
        else:
            wq, ws = quant.quantize_per_row(w)
        return cls(wq, ws, bias, mode, out_dtype, hadamard_block)

    @property
    def in_features(self) -> int:
        return self.weight_q.shape[1]

    @property
    def out_features(self) -> int:
        return self.weight_q.shape[0]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import gemm_int8_b200 as g

        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype not in (torch.float32, torch.bfloat16):
            x2 = x2.to(torch.bfloat16)
        if self.mode == "blockwise":
            if self.hadamard_block is not None:
                xq, xs = g.hadamard_quantize_per_token_block(x2, self.hadamard_block)
            else:
                xq, xs = g.quantize_per_token_block(x2)
            out = g.matmul_blockwise(xq, self.weight_q, xs, self.weight_scale)
        else:
            xq, xs = g.quantize_per_token(x2)
            out = g.matmul_scaled(xq, self.weight_q, xs, self.weight_scale)
        if self.bias is not None:
            out = out + self.bias.to(out.dtype)
        return out.to(self.out_dtype).reshape(*lead, self.out_features)

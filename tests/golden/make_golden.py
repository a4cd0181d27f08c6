"""Generates tests/golden/*.npz -- run in the build container, where torch (CPU) is available.

The reference has no golden vectors; the only values its own test pins are the torch formula
``x.bfloat16() @ x.bfloat16().t()`` compared with assert_close (reference test.py:5-8,15).  The
reference operator itself is CUDA-only and cannot run where these files are made, so the fixtures are
that FORMULA evaluated with torch on CPU on seeded inputs:

* ``ref_test_py``      the reference test's own case: x = (rand(32,32)*100).to(int8), both operands = x
* ``ref_benchmark_py`` the reference benchmark's input recipe (benchmark.py:17-26): randn*5 rounded and
                       clamped to int8, at a small shape
* ``readme_uniform``   uniform int8 in [-128, 127) as in the README example, small shape, alpha = 1

Each file holds x, y (int8), alpha and `expected_bf16_bits` (uint16 view of the bf16 result).  The
script asserts that the bf16 matmul is exact for these sizes (every partial sum fits 24 bits), so the
stored value equals bf16(exact int32 dot) and is independent of the BLAS used to make it.

Usage:  python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def formula(x, y):
    """Reference test.py:8 -- bf16 matmul of the int8 operands."""
    out = x.bfloat16() @ y.bfloat16().t()
    exact = (x.to(torch.int64) @ y.to(torch.int64).t())
    assert exact.abs().max() < 2 ** 24, "partial sums must stay exact in fp32 for this fixture"
    assert torch.equal(out, exact.to(torch.float32).bfloat16()), "bf16 matmul was not exact"
    return out


def save(name, x, y, alpha, out):
    np.savez_compressed(os.path.join(HERE, name + ".npz"), x=x.numpy(), y=y.numpy(),
                        alpha=np.float32(alpha), expected_bf16_bits=bits(out))
    print(name, tuple(x.shape), tuple(y.shape), "->", tuple(out.shape))


def main():
    g = torch.Generator().manual_seed(20240501)
    x = (torch.rand(32, 32, generator=g) * 100).to(torch.int8)          # test.py:5-6
    save("ref_test_py", x, x, 1.0, formula(x, x))

    def to_int8(t):                                                      # benchmark.py:17-18
        return torch.round(t.clamp(min=-128, max=127)).to(torch.int8)

    a = to_int8(torch.randn(96, 512, generator=g) * 5)                   # benchmark.py:22-26
    b = to_int8(torch.randn(160, 512, generator=g) * 5)
    save("ref_benchmark_py", a, b, 1.0, formula(a, b))

    x = torch.randint(-128, 127, (64, 256), dtype=torch.int8, generator=g)   # README example distribution
    y = torch.randint(-128, 127, (136, 256), dtype=torch.int8, generator=g)
    save("readme_uniform", x, y, 1.0, formula(x, y))


if __name__ == "__main__":
    main()

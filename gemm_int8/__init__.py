"""Drop-in name for the reference package: ``import gemm_int8; gemm_int8.matmul(x, y, alpha)``.

The reference's package (gemm_int8/__init__.py:28-40) exports ``matmul``; this shim forwards it, and the
W8A8 additions, to the B200 implementation in ``gemm_int8_b200``.
"""
from gemm_int8_b200 import (  # noqa: F401
    device_status,
    force_variant,
    matmul,
    matmul_blockwise,
    matmul_i32,
    matmul_scaled,
    pick_variant,
)

__all__ = ["matmul"]

"""Python face of the tcgen05 matrix product (gemm_tcgen05.cu)."""
from __future__ import annotations


def supports(weight) -> bool:
    return False

"""Python face of the tensor-core attention kernels (attention_flash.cu)."""
from __future__ import annotations


def supports(head_dim: int, group_size: int) -> bool:
    return False

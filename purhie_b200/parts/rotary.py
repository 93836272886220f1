"""Rotary position encoding, rotate-half pairing.

For pair i < n_rot/2 the angle at position p is p * theta^(-2i/n_rot); (x_i, x_{i+n_rot/2}) turns by it;
dimensions >= n_rot are left alone.  Angles are computed in double precision on the host and stored as
float32 cosines and sines.  Reference: src/qwen_ops.cpp:15-24 (double theta), src/attention.hip:225-240
(the device version); base and width: src/inference.cpp:1358-1359.
"""
from __future__ import annotations

import torch

from .base import BuildContext, PositionEncoding, register_part


class RotaryHalf(PositionEncoding):
    """params: theta, n_rot, max_position."""

    interleaved = False

    def __init__(self, params: dict, build: BuildContext):
        super().__init__(params, build)
        self.theta = float(params["theta"])
        self.n_rot = int(params["n_rot"])
        self.max_position = int(params["max_position"])
        if self.n_rot % 2 or self.n_rot < 2:
            raise ValueError(f"rotary width {self.n_rot} must be even and at least 2")
        self._table = None

    def angles(self) -> torch.Tensor:
        """float64 [max_position, n_rot/2]."""
        half = self.n_rot // 2
        i = torch.arange(half, dtype=torch.float64)
        inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.n_rot)
        pos = torch.arange(self.max_position, dtype=torch.float64)
        return pos[:, None] * inv_freq[None, :]

    def rotation_table(self, device) -> torch.Tensor:
        if self._table is None or self._table.device != torch.device(device):
            a = self.angles()
            self._table = torch.cat([torch.cos(a), torch.sin(a)], dim=1).to(torch.float32).contiguous().to(device)
        return self._table


register_part("position", "rope_neox", RotaryHalf)

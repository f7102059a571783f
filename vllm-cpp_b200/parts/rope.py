"""Rotary position encoding: the table of cosines and sines.

inv_freq_i = theta^(-2i/head_dim), angle = position * inv_freq_i
(src/model.cpp:582-589, 979-982); ``theta`` is a parameter (the reference's CPU
path uses the constant ROPE_BASE instead of config.json's rope_theta,
src/config.h:43).  The table [max_positions, head_dim] holds head_dim/2 cosines
then head_dim/2 sines per position, computed in 64-bit on the host and rounded
once to 32-bit, so large positions lose nothing to a fast sincos on the device.
The rotation itself pairs lanes (i, i + head_dim/2) (src/mlx_backend.cpp:411-412,
cuda/attention_kernels.cuh:275-287) and is applied inside the fused
norm-rotate-store kernel.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding


class RotaryEmbedding(PositionEncoding):
    """params: ``head_dim``, ``theta``, ``max_positions``; optional ``rotary_dim`` (how many lanes of a head turn,
    default all; angles theta^(-2i/rotary_dim)) and ``pairing`` ("half": lanes (i, i + rotary_dim/2), the default;
    "interleaved": lanes (2i, 2i+1)).

    What an attention part reads of its position part: ``table`` [max_positions, rotary_dim] (cosines, then
    sines), ``rotary_dim`` and ``pairing`` (absent: all lanes, "half")."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.head_dim = int(params["head_dim"])
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        self.rotary_dim = int(params.get("rotary_dim") or self.head_dim)
        self.pairing = str(params.get("pairing") or "half")
        if self.pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing '{self.pairing}' is not one of 'half', 'interleaved'")
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"{self.rotary_dim} rotated lanes of a head of {self.head_dim}: an even number up to head_dim")
        key = ("rope_table", self.rotary_dim, self.theta, self.max_positions)
        if key not in build.shared:
            build.shared[key] = self._make_table().to(build.device)
        self.table = build.shared[key]

    def _make_table(self) -> torch.Tensor:
        half = self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        inv_freq = self.theta ** (-2.0 * i / self.rotary_dim)
        ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        return torch.cat([torch.cos(ang), torch.sin(ang)], dim=1).to(torch.float32).contiguous()

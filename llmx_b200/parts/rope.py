"""Position encodings.  Rotary: cos/sin tables in 32-bit, rotate-half pairing.

Tables follow the reference's order of operations in float32
(src/model/rope.hpp:25-28 base frequency, :159-188 YaRN blend, :191-217 fill):
    freq_i  = powf(theta, -2 i / D)
    angle   = (float) pos * freq_i
    cos/sin = cosf / sinf (angle) [* attention factor under YaRN]
indexed [pos, i], i < D / 2.  The mixer's kernel pairs (i, i + rot_dim / 2).

Another position encoding provides the same two things: `prepare` (build what
its kernel reads) and the attributes the mixer hands to the kernel
(`cos`, `sin`, both None for "no rotation").
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from .base import Part


class NoPositionEncoding(Part):
    cos = None
    sin = None
    rot_dim = 0


class RotaryEmbedding(Part):
    def __init__(self, head_dim: int, theta: float, rot_dim: Optional[int] = None, yarn=None,
                 max_positions: Optional[int] = None):
        self.head_dim = int(head_dim)
        self.rot_dim = int(rot_dim if rot_dim is not None else head_dim)
        if self.rot_dim % 2 or self.rot_dim > self.head_dim or self.rot_dim <= 0:
            raise ValueError("the rotated width must be even, positive and at most the head width")
        self.theta = float(theta)
        self.yarn = yarn
        self.max_positions = max_positions
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def frequencies(self) -> np.ndarray:
        dim, half = self.rot_dim, self.rot_dim // 2
        i = np.arange(half, dtype=np.float32)
        theta = np.float32(self.theta)
        if self.yarn is None:
            return np.power(theta, np.float32(-2.0) * i / np.float32(dim)).astype(np.float32)
        y = self.yarn

        def correction(rotations: float) -> float:
            return dim * math.log(y.original_max_position_embeddings / (rotations * 2 * math.pi)) / (2 * math.log(self.theta))

        low = max(math.floor(correction(y.beta_fast)), 0.0)
        high = min(math.ceil(correction(y.beta_slow)), float(dim - 1))
        if low == high:
            high += 0.001
        power = np.power(theta, (np.float32(2.0) * i) / np.float32(dim)).astype(np.float32)
        extra = np.float32(1.0) / power
        inter = np.float32(1.0) / (np.float32(y.factor) * power)
        ramp = np.clip((i - np.float32(low)) / np.float32(high - low), np.float32(0), np.float32(1)).astype(np.float32)
        extrapolate = np.float32(1.0) - ramp
        return (inter * (np.float32(1.0) - extrapolate) + extra * extrapolate).astype(np.float32)

    def tables(self, positions: int):
        freq = self.frequencies()
        pos = np.arange(positions, dtype=np.float32)[:, None]
        angle = (pos * freq[None, :]).astype(np.float32)
        cos, sin = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
        if self.yarn is not None:
            scale = np.float32(self.yarn.attention_factor)
            cos, sin = cos * scale, sin * scale
        return cos, sin

    def prepare(self, max_positions: int, device) -> None:
        n = max_positions if self.max_positions is None else min(max_positions, self.max_positions)
        if self.cos is not None and self.cos.shape[0] >= n and self.cos.device == torch.device(device):
            return
        cos, sin = self.tables(n)
        self.cos = torch.from_numpy(cos).to(device).contiguous()
        self.sin = torch.from_numpy(sin).to(device).contiguous()

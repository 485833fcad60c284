"""Position-encoding parts. Interface:

    Position(params, rt)
    fused() -> dict or None      tables for the fused q/k kernel: {"inv_freq": float32 [rotary/2],
                                 "rotary_dim": int}; None means the mixer must call apply()
    apply(q, k, positions, tokens)   in-place encoding of q [T, Hq, d] and k [T, Hkv, d] views

Keys are cached after encoding, so an encoding must be a pure function of the absolute position.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from .registry import register_part
from .runtime import Runtime


@register_part("position", "rope_split_half")
class SplitHalfRope:
    """Rotary embedding over pairs (i, i + rotary/2): angle = position * theta^(-2i/rotary).
    Frequencies are computed in double and rounded to float32, the angle product and
    sin/cos are float32, as celeg's CPU kernel does (src/backend/cpu/kernels/rope.cpp:74-79;
    include/celeg/model/position.hpp:77-78)."""

    def __init__(self, params: Mapping, rt: Runtime):
        self.theta = float(params["theta"])
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        half = self.rotary_dim // 2
        exponents = torch.arange(half, dtype=torch.float64) * (-2.0 / self.rotary_dim)
        self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), exponents).to(
            torch.float32).to(rt.device)

    def fused(self) -> Optional[dict]:
        return {"inv_freq": self.inv_freq, "rotary_dim": self.rotary_dim}


@register_part("position", "none")
class NoPosition:
    def __init__(self, params: Mapping, rt: Runtime):
        pass

    def fused(self) -> Optional[dict]:
        return {"inv_freq": None, "rotary_dim": 0}

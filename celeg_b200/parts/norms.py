"""Norm parts. Interface of a norm:

    Norm(params, weights, rt)
    add_norm(residual, delta, out, n_rows, rows=None)
        residual: float32 [T, width] (updated in place with ``delta`` when ``rows`` is None)
        delta:    activation-type [T, width] or None
        out:      activation-type [n_rows, width]
        rows:     int32 row list to gather (then the residual is left untouched)
    as_prologue() -> (weight, eps) or None      optional: a plain RMSNorm, which the runtime may split
                                                between the products before and after it
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from .. import kernels
from .registry import register_part
from .runtime import Runtime


@register_part("norm", "rmsnorm")
class RmsNorm:
    """y = x / sqrt(mean(x^2) + eps) * w, the weight a direct scale
    (celeg src/backend/cpu/kernels/elementwise.cpp:56-76)."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], rt: Runtime):
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.weight = rt.vector(weights["weight"])
        if self.weight.shape != (self.width,):
            raise ValueError(f"rmsnorm weight has shape {tuple(self.weight.shape)}, expected ({self.width},)")

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor, n_rows: int,
                 rows: Optional[torch.Tensor] = None) -> None:
        kernels.add_rmsnorm(residual, delta, self.weight, out, self.eps, rows=rows, n_rows=n_rows)

    def as_prologue(self):
        return self.weight, self.eps

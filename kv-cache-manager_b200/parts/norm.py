"""RMSNorm with the residual add that precedes it fused in.

out = w * round(x * rsqrt(mean(x^2) + eps)); statistics in float32 over the float32 residual
stream (the reference's kernel, ``src/cuda/kernels.cu:34-49``; its separate residual kernel,
``:84-88``, is folded into this one).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import library as K
from .base import NORMS, Norm


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, hidden: int, eps: float, init=("ones",)) -> None:
        super().__init__()
        self.hidden, self.eps = hidden, float(eps)
        self.declare("weight", (hidden,), init, "vector")

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        K.rmsnorm(x, pending, self.param("weight"), out, self.eps, rows)


@NORMS.register("rmsnorm_output")
class OutputRMSNorm(Norm):
    """The norm of a block that normalises what a sublayer RETURNS, not what it reads:
    x += mult * w * y / sqrt(mean(y^2) + eps), statistics and sum in float32.  ``forward(x, y, out)``
    adds into the float32 residual ``x`` and, when ``out`` is given, writes the new rows of x in the
    storage dtype for the next sublayer to read."""

    def __init__(self, hidden: int, eps: float, mult: float = 1.0, init=("ones",)) -> None:
        super().__init__()
        self.hidden, self.eps, self.mult = hidden, float(eps), float(mult)
        self.declare("weight", (hidden,), init, "vector")

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], out: Optional[torch.Tensor],
                rows: Optional[torch.Tensor] = None) -> None:
        if rows is not None or pending is None:
            raise ValueError("rmsnorm_output: needs the sublayer's output for every row")
        K.rms_scale_add(x, pending, self.param("weight"), out, self.eps, self.mult)

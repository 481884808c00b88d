"""The gated delta rule: a mixer with a fixed-size state per request instead of a cache of keys.

Per value head (its query/key head is ``head // (heads // qk_heads)``) a float32 matrix S [dk, dv],
zero at a request's start, is carried from token to token:

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

(the read-out sees the current token's write).  q, k, v are projections of the layer's input that
pass a short causal convolution over time per channel (``taps`` taps, no bias, zeros before the
start) and SiLU; q and k are then scaled to unit length per head, x / sqrt(sum x^2 + 1e-6), q also
by dk^-1/2; beta = sigmoid(W_b h); g = exp(-exp(A_log) softplus(W_a h + dt_bias)), one per head.
Each head's o is divided by its root mean square over dv, multiplied by a weight [dv] shared by
the heads and by SiLU of a gate projection, and the heads go through the output projection.

State of a request, one float32 row per call site: S of every head, then the last ``taps - 1``
inputs of the convolution.  Everything after the projections runs in float32 in both storage
dtypes (csrc/cuda/delta_rule.cu).
"""
from __future__ import annotations

import torch

from ..kernels import library as K
from .base import MIXERS, Mixer, SiteCache, StateSpec, StepContext
from .linear import Linear


@MIXERS.register("gated_delta")
class GatedDeltaMixer(Mixer):
    def __init__(self, hidden: int, heads: int, qk_heads: int, dk: int, dv: int, taps: int, norm_eps: float) -> None:
        super().__init__()
        if qk_heads < 1 or heads % qk_heads:
            raise ValueError(f"gated_delta: {heads} heads are not a multiple of {qk_heads} query/key heads")
        if taps < 1:
            raise ValueError("gated_delta: the convolution needs at least one tap")
        self.hidden, self.heads, self.qk_heads, self.dk, self.dv, self.taps = hidden, heads, qk_heads, dk, dv, taps
        self.norm_eps = float(norm_eps)
        self.channels = 2 * qk_heads * dk + heads * dv               # what the convolution sees: q | k | v
        std = hidden ** -0.5
        # one product for q | k | v | gate (storage dtype) and a small one for b | a (float32 results)
        self.qkvg = self.add_child("qkvg", Linear(hidden, self.channels + heads * dv, std))
        self.ba = self.add_child("ba", Linear(hidden, 2 * heads, std))
        self.o = self.add_child("o", Linear(heads * dv, hidden, (heads * dv) ** -0.5))
        self.declare("conv", (self.channels, taps), ("normal", 0.5), "vector")
        self.declare("A_log", (heads,), ("normal", 0.5), "vector")
        self.declare("dt_bias", (heads,), ("normal", 0.5), "vector")
        self.declare("norm", (dv,), ("ones",), "vector")
        self._f32 = {}

    def state_spec(self) -> StateSpec:
        return StateSpec((self.heads * self.dk * self.dv + (self.taps - 1) * self.channels,), torch.float32)

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        if self.dk > K.delta_scan_max_dk():
            raise ValueError(f"gated_delta: key size {self.dk} exceeds the recurrence kernel's {K.delta_scan_max_dk()}")
        self._f32 = {n: self.param(n).to(device=device, dtype=torch.float32).contiguous()
                     for n in ("conv", "A_log", "dt_bias", "norm")}

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        M, H, C = h.shape[0], self.heads, self.channels
        proj = self.qkvg.forward(h, ctx)
        ba = self.ba.forward(h, ctx, out_dtype=torch.float32)
        qkv = torch.empty((M, C), dtype=torch.float32, device=h.device)
        K.delta_conv(proj, self._f32["conv"], site.state, H * self.dk * self.dv, ctx, qkv)
        K.delta_prepare(qkv, ba, self._f32["A_log"], self._f32["dt_bias"], H, self.qk_heads, self.dk)
        o = torch.zeros((M, H * self.dv), dtype=torch.float32, device=h.device)   # padding rows stay zero
        K.delta_scan(qkv, ba, site.state, ctx, o, H, self.qk_heads, self.dk, self.dv)
        gated = torch.empty((M, H * self.dv), dtype=h.dtype, device=h.device)
        K.gated_rms(o, proj[:, C:], self._f32["norm"], gated, H, self.dv, self.norm_eps)
        return self.o.forward(gated, ctx, out_dtype=torch.float32)

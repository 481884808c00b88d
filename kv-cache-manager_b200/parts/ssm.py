"""The selective state-space mixer in its matrix-state form (state-space duality): per head a float32
matrix S [state, vdim], zero at a request's start, carried from token to token,

    S <- exp(-exp(A_log) dt) S + dt B x^T;     y = S^T C + D x

with x [vdim] per head, B and C [state] per group of heads (head h uses group h // (heads // groups))
and dt = softplus(raw + dt_bias) per head (no clamp).  One input product gives
[z: inner | x: inner | B: groups*state | C: groups*state | raw dt: heads], inner = heads * vdim; x, B
and C go through a causal convolution of a few taps along time, channel by channel (with a bias), and SiLU.  The heads'
outputs, side by side, are multiplied by SiLU(z) and THEN normalised in ``norm_groups`` equal parts
(every part by the root mean square of its own elements) and scaled by a weight over inner; output product.

State of a request, one float32 row per call site: S of every head, then the last ``taps - 1`` inputs
of the convolution.  The recurrence is the engine's matrix-state scan in its linear form
(csrc/cuda/delta_rule.cu: k = B, q = C, step = dt, v = x); everything after the input product is
float32 in both storage dtypes.
"""
from __future__ import annotations

import torch

from ..kernels import library as K
from .base import MIXERS, Mixer, SiteCache, StateSpec, StepContext
from .linear import Linear


@MIXERS.register("mamba2")
class Mamba2Mixer(Mixer):
    def __init__(self, hidden: int, heads: int, vdim: int, state: int, groups: int, taps: int, norm_groups: int,
                 norm_eps: float) -> None:
        super().__init__()
        if groups < 1 or heads % groups:
            raise ValueError(f"mamba2: {heads} heads are not a multiple of {groups} groups")
        inner = heads * vdim
        if norm_groups < 1 or inner % norm_groups:
            raise ValueError(f"mamba2: {inner} inner channels do not split into {norm_groups} equal parts")
        if taps < 1:
            raise ValueError("mamba2: the convolution needs at least one tap")
        self.hidden, self.heads, self.vdim, self.state, self.groups, self.taps = hidden, heads, vdim, state, groups, taps
        self.norm_groups, self.norm_eps, self.inner = norm_groups, float(norm_eps), inner
        self.conv_channels = inner + 2 * groups * state
        self.inp = self.add_child("inp", Linear(hidden, 2 * inner + 2 * groups * state + heads, hidden ** -0.5))
        self.o = self.add_child("o", Linear(inner, hidden, inner ** -0.5))
        self.declare("conv", (self.conv_channels, taps), ("normal", 0.5), "vector")
        self.declare("conv_bias", (self.conv_channels,), ("normal", 0.2), "vector")
        self.declare("dt_bias", (heads,), ("normal", 0.5), "vector")
        self.declare("A_log", (heads,), ("normal", 0.5), "vector")
        self.declare("D", (heads,), ("normal", 0.5), "vector")
        self.declare("norm", (inner,), ("ones_jitter", 0.1), "vector")
        self._f32 = {}

    def state_spec(self) -> StateSpec:
        return StateSpec((self.heads * self.state * self.vdim + (self.taps - 1) * self.conv_channels,), torch.float32)

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        if self.state > K.delta_scan_max_dk():
            raise ValueError(f"mamba2: state size {self.state} exceeds the recurrence kernel's {K.delta_scan_max_dk()}")
        self._f32 = {n: self.param(n).to(device=device, dtype=torch.float32).contiguous() for n in self.param_specs()}

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        T, H, inner, C, f = h.shape[0], self.heads, self.inner, self.conv_channels, self._f32
        GN = self.groups * self.state
        proj = self.inp.forward(h, ctx)
        xbc = torch.empty((T, C), dtype=torch.float32, device=h.device)
        K.delta_conv(proj[:, inner:inner + C], f["conv"], site.state, H * self.state * self.vdim, ctx, xbc, f["conv_bias"])
        steps = torch.empty((T, 2 * H), dtype=torch.float32, device=h.device)            # [dt | decay]
        K.ssm_prepare(proj[:, inner + C:], f["A_log"], f["dt_bias"], steps, H)
        y = torch.empty((T, inner), dtype=torch.float32, device=h.device)                # (the scan zeroes padding rows)
        K.state_scan(K.SCAN_LINEAR, xbc, (inner + GN, inner, 0), steps[:, :H], steps[:, H:], None, site.state, ctx, y,
                     H, self.groups, self.state, self.vdim)
        gated = torch.empty((T, inner), dtype=h.dtype, device=h.device)
        K.group_rms_gate(y, proj[:, :inner], f["norm"], gated, inner // self.norm_groups, self.norm_eps, True, "silu",
                         skip=xbc, skip_coef=f["D"], head=self.vdim)
        return self.o.forward(gated, ctx, out_dtype=torch.float32)

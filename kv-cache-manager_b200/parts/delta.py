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
from .linear import Linear, matmul_nt


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
        o = torch.empty((M, H * self.dv), dtype=torch.float32, device=h.device)   # (the scan zeroes padding rows)
        K.delta_scan(qkv, ba, site.state, ctx, o, H, self.qk_heads, self.dk, self.dv)
        gated = torch.empty((M, H * self.dv), dtype=h.dtype, device=h.device)
        K.gated_rms(o, proj[:, C:], self._f32["norm"], gated, H, self.dv, self.norm_eps)
        return self.o.forward(gated, ctx, out_dtype=torch.float32)


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


@MIXERS.register("gated_delta_channel")
class ChannelDecayDeltaMixer(Mixer):
    """The gated delta rule with channel-wise decays (a factor for every key channel of every head):

        S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q        (g [dk] per head)

    q, k (``qk_heads`` x dk) and v (``heads`` x dv) pass the short causal convolution and SiLU and q, k
    become unit vectors as in ``gated_delta``; beta = sigmoid(W_b h);
    g = exp(-exp(A_log[head]) softplus(W_a2 (W_a1 h) + dt_bias)), the decay's projection going through
    ``decay_rank`` numbers; each head's o is divided by its root mean square over dv, multiplied by a
    weight [dv] shared by the heads and by sigmoid(W_g2 (W_g1 h)), the gate's projection going through
    ``gate_rank`` numbers.  State as in ``gated_delta``.

    The three small projections that read h (W_a1, W_g1, W_b) are one product whose sections are
    padded with zero rows to multiples of 8 (so that the second-stage products read aligned slices of
    its result; W_a2 and W_g2 get matching zero columns); the padded copies are made once after loading."""

    def __init__(self, hidden: int, heads: int, qk_heads: int, dk: int, dv: int, taps: int, decay_rank: int,
                 gate_rank: int, norm_eps: float) -> None:
        super().__init__()
        if qk_heads < 1 or heads % qk_heads:
            raise ValueError(f"gated_delta_channel: {heads} heads are not a multiple of {qk_heads} query/key heads")
        if taps < 1:
            raise ValueError("gated_delta_channel: the convolution needs at least one tap")
        self.hidden, self.heads, self.qk_heads, self.dk, self.dv, self.taps = hidden, heads, qk_heads, dk, dv, taps
        self.decay_rank, self.gate_rank, self.norm_eps = decay_rank, gate_rank, float(norm_eps)
        self.channels = 2 * qk_heads * dk + heads * dv
        std = hidden ** -0.5
        self.qkv = self.add_child("qkv", Linear(hidden, self.channels, std))
        self.a1 = self.add_child("a1", Linear(hidden, decay_rank, std))
        self.a2 = self.add_child("a2", Linear(decay_rank, heads * dk, decay_rank ** -0.5))
        self.g1 = self.add_child("g1", Linear(hidden, gate_rank, std))
        self.g2 = self.add_child("g2", Linear(gate_rank, heads * dv, gate_rank ** -0.5))
        self.b = self.add_child("b", Linear(hidden, heads, std))
        self.o = self.add_child("o", Linear(heads * dv, hidden, (heads * dv) ** -0.5))
        self.declare("conv", (self.channels, taps), ("normal", 0.5), "vector")
        self.declare("A_log", (heads,), ("normal", 0.5), "vector")
        self.declare("dt_bias", (heads * dk,), ("normal", 0.5), "vector")
        self.declare("norm", (dv,), ("ones_jitter", 0.1), "vector")
        self._f32 = {}
        self._low = self._a2 = self._g2 = None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.heads * self.dk * self.dv + (self.taps - 1) * self.channels,), torch.float32)

    def prepare(self, device, dtype) -> None:
        super().prepare(device, dtype)
        if self.dk > K.delta_scan_max_dk():
            raise ValueError(f"gated_delta_channel: key size {self.dk} exceeds the recurrence kernel's {K.delta_scan_max_dk()}")
        self._f32 = {n: self.param(n).to(device=device, dtype=torch.float32).contiguous() for n in self.param_specs()}
        ra, rg, hb = _pad8(self.decay_rank), _pad8(self.gate_rank), _pad8(self.heads)
        a1, g1, b = self.a1.param("weight"), self.g1.param("weight"), self.b.param("weight")
        low = torch.zeros((ra + rg + hb, self.hidden), dtype=a1.dtype, device=a1.device)
        low[:self.decay_rank] = a1
        low[ra:ra + self.gate_rank] = g1
        low[ra + rg:ra + rg + self.heads] = b
        a2 = torch.zeros((self.heads * self.dk, ra), dtype=a1.dtype, device=a1.device)
        a2[:, :self.decay_rank] = self.a2.param("weight")
        g2 = torch.zeros((self.heads * self.dv, rg), dtype=a1.dtype, device=a1.device)
        g2[:, :self.gate_rank] = self.g2.param("weight")
        self._low, self._a2, self._g2 = low, a2, g2

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache) -> torch.Tensor:
        T, H, C = h.shape[0], self.heads, self.channels
        ra, rg = self._a2.shape[1], self._g2.shape[1]
        proj = self.qkv.forward(h, ctx)
        low = matmul_nt(h, self._low, h.dtype, ctx.options)
        decay = matmul_nt(low[:, :ra], self._a2, torch.float32, ctx.options)          # becomes g in place
        gate = matmul_nt(low[:, ra:ra + rg], self._g2, h.dtype, ctx.options)
        qkv = torch.empty((T, C), dtype=torch.float32, device=h.device)
        K.delta_conv(proj, self._f32["conv"], site.state, H * self.dk * self.dv, ctx, qkv)
        beta = torch.empty((T, H), dtype=torch.float32, device=h.device)
        K.delta_prepare_channel(qkv, low[:, ra + rg:ra + rg + H], beta, decay, self._f32["A_log"], self._f32["dt_bias"],
                                H, self.qk_heads, self.dk)
        o = torch.empty((T, H * self.dv), dtype=torch.float32, device=h.device)       # (the scan zeroes padding rows)
        K.state_scan(K.SCAN_DELTA_CHANNEL, qkv, (0, self.qk_heads * self.dk, 2 * self.qk_heads * self.dk), beta, None, decay,
                     site.state, ctx, o, H, self.qk_heads, self.dk, self.dv)
        gated = torch.empty((T, H * self.dv), dtype=h.dtype, device=h.device)
        K.group_rms_gate(o, gate, self._f32["norm"], gated, self.dv, self.norm_eps, False, "sigmoid")
        return self.o.forward(gated, ctx, out_dtype=torch.float32)


@MIXERS.register("side_by_side")
class SideBySideMixer(Mixer):
    """Two mixers that read the same input; the result is left_scale * left + right_scale * right.  At most
    one of them may keep paged keys and values and at most one fixed-size state (they share the call site).
    The sum is not formed here: the two float32 outputs are returned as (tensor, scale) pairs for the
    block to hand to the next norm kernel, which adds them into the stream."""

    def __init__(self, left: Mixer, right: Mixer, left_scale: float = 1.0, right_scale: float = 1.0) -> None:
        super().__init__()
        self.left, self.right = self.add_child("left", left), self.add_child("right", right)
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        specs = [m.cache_spec() for m in (left, right)]
        states = [m.state_spec() for m in (left, right)]
        if all(s is not None for s in specs) or all(s is not None for s in states):
            raise ValueError("side_by_side: both mixers want the call site's cache (or its state)")

    def cache_spec(self):
        return self.left.cache_spec() or self.right.cache_spec()

    def state_spec(self):
        return self.left.state_spec() or self.right.state_spec()

    def forward(self, h: torch.Tensor, ctx: StepContext, site: SiteCache):
        out = []
        for m, s in ((self.left, self.left_scale), (self.right, self.right_scale)):
            y = m.forward(h, ctx, site)
            out += [(t, c * s) for t, c in y] if isinstance(y, (list, tuple)) else [(y, s)]
        return out

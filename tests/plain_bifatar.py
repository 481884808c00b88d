"""Bifatar restated plainly in float64 torch: whole sequences, one function per mechanism, loops
where a loop is the clearest form.  It shares no code with the engine; the tests hold the engine's
kernels, cache, state and batching to it.

Notation: T tokens, D width; ``cfg`` is the model's config as a dict, ``W`` a dict name -> tensor.
Linear weights are [out, in] and applied as x @ W.T.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def lin(x, w, b=None):
    y = x @ w.to(F64).T
    return y if b is None else y + b.to(F64)


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def dyt(x, w, b, alpha):
    """Dynamic tanh norm: no statistics at all."""
    return torch.tanh(alpha.to(F64) * x) * w.to(F64) + b.to(F64)


def rotate(x, base, dims):
    """x [T, heads, dim]; the first ``dims`` dimensions turn, pair (i, i + dims/2), angle p * base^(-2i/dims)."""
    T = x.shape[0]
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    f = torch.tensor(float(base), dtype=F64) ** (-2.0 * i / dims)
    a = torch.arange(T, dtype=F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def causal_conv(x, w, b=None):
    """x [T, C], w [C, taps]: the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    w = w.to(F64)
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1 - j)
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y if b is None else y + b.to(F64)


def softmax_attention(q, k, v, scale, window=0, softcap=0.0, sink=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H*dv].  Row i sees j <= i (and i - j < window
    when a window is given); ``sink`` [H]: one more term exp(sink_h) in the denominator only."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        ok = j <= i
        if window:
            ok = ok & (i - j < window)
        s = s.masked_fill(~ok, -math.inf)
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].to(F64).expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h].to(F64) - m)
        out[:, h] = (e / den) @ v[:, g]
    return out.reshape(T, -1)


def attention_mixer(h, W, p, m, eps, first_v=None):
    """Windowed attention with per-head q/k norm after the rotation, capped scores, a sink, and value
    mixing.  Returns (output, this layer's values before mixing or None)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(h, W[p + "q"]).view(T, H, dk)
    k = lin(h, W[p + "k"]).view(T, G, dk)
    v = lin(h, W[p + "v"]).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q, k = rotate(q, rot["base"], rot["dims"]), rotate(k, rot["base"], rot["dims"])
    q, k = rms(q, eps), rms(k, eps)
    v_own = v
    if m.get("v_mix") and first_v is not None:
        lam = W[p + "vmix"].to(F64)
        v = (1 - lam) * v + lam * first_v
    window = (m.get("mask") or {}).get("size", 0)
    o = softmax_attention(q, k, v, m["scale"], window, m.get("softcap", 0.0), W[p + "sink"])
    return lin(o, W[p + "o"]), (v_own if m.get("v_mix") else None)


def mamba2_mixer(h, W, p, m, eps):
    T = h.shape[0]
    Hn, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hn * P
    zxbcdt = lin(h, W[p + "in"])
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(T, Hn, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"].to(F64))
    A = -torch.exp(W[p + "A_log"].to(F64))
    Dskip = W[p + "D"].to(F64)
    y = torch.zeros(T, Hn, P, dtype=F64)
    for hd in range(Hn):
        g = hd // (Hn // G)
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = torch.exp(A[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + Dskip[hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * W[p + "norm"].to(F64)
    return lin(y, W[p + "o"])


def left_mixer(h, W, p, m, eps):
    """Causal softmax attention with biased projections and a norm over the whole q (and k) projection."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(lin(h, W[p + "q"], W[p + "q.b"]), eps) * W[p + "q.norm"].to(F64)
    k = rms(lin(h, W[p + "k"], W[p + "k.b"]), eps) * W[p + "k.norm"].to(F64)
    v = lin(h, W[p + "v"], W[p + "v.b"]).view(T, G, dv)
    q, k = q.view(T, H, dk), k.view(T, G, dk)
    rot = m.get("rot")
    if rot:
        q, k = rotate(q, rot["base"], rot["dims"]), rotate(k, rot["base"], rot["dims"])
    return lin(softmax_attention(q, k, v, m["scale"]), W[p + "o"])


def right_mixer(h, W, p, m, eps):
    """Gated delta rule with channel-wise decays."""
    T = h.shape[0]
    Hn, Hk, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(lin(h, W[p + "q"]), W[p + "q.conv"])).view(T, Hk, dk)
    k = silu(causal_conv(lin(h, W[p + "k"]), W[p + "k.conv"])).view(T, Hk, dk)
    v = silu(causal_conv(lin(h, W[p + "v"]), W[p + "v.conv"])).view(T, Hn, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(h, W[p + "b"]))
    a = lin(lin(h, W[p + "a1"]), W[p + "a2"]) + W[p + "dt_bias"].to(F64)
    A = torch.exp(W[p + "A_log"].to(F64))
    g = torch.exp(-A[None, :, None] * softplus(a).view(T, Hn, dk))
    gate = torch.sigmoid(lin(lin(h, W[p + "g1"]), W[p + "g2"])).view(T, Hn, dv)
    o = torch.zeros(T, Hn, dv, dtype=F64)
    for hd in range(Hn):
        kh = hd // (Hn // Hk)
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = g[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            o[t, hd] = S.T @ q[t, kh]
    o = rms(o, eps) * W[p + "norm"].to(F64) * gate
    return lin(o.reshape(T, Hn * dv), W[p + "o"])


def parallel_mixer(h, W, p, m, eps):
    return m["left_scale"] * left_mixer(h, W, p + "left.", m["left"], eps) + \
        m["right_scale"] * right_mixer(h, W, p + "right.", m["right"], eps)


def dense_ff(h, W, p):
    return lin(torch.relu(lin(h, W[p + "up"])) ** 2, W[p + "down"])


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = W["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)]
    first_v = None
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        n = f"l{i}.norm1"
        h = dyt(x, W[n], W[n + ".b"], W[n + ".alpha"])
        p, m, kind = f"l{i}.mix.", layer["mixer"], layer["type"]
        if kind == "attention":
            y, v_own = attention_mixer(h, W, p, m, eps, first_v)
            if first_v is None and v_own is not None:
                first_v = v_own
        elif kind == "mamba2":
            y = mamba2_mixer(h, W, p, m, eps)
        elif kind == "parallel":
            y = parallel_mixer(h, W, p, m, eps)
        else:
            raise ValueError(kind)
        if layer.get("mlp") is not None:
            y = y + dense_ff(h, W, f"l{i}.mlp.")
        x = x + y
        streams.append(x)
    h = dyt(x, W["final.norm"], W["final.norm.b"], W["final.norm.alpha"])
    logits = lin(h, W["head"])
    return (logits, torch.stack(streams)) if return_layers else logits

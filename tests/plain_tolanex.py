"""Plain, slow restatement of the Tolanex design in float64 torch on the CPU: whole sequences, no
cache, no batching, one function per mechanism.  It shares no code with the engine; the tests
compare the engine's logits with it.

Notation: n tokens, width D.  Weights are a dict name -> float64 tensor, linear weights [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


# ------------------------------------------------------------------------------- embedding

def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets)
    return rows


def embed(cfg, w, tokens: List[int]):
    n = len(tokens)
    x = w["embed"][tokens].clone()
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        x = x + w["bigram"][bigram_rows(tokens, big["buckets"], big["mul_prev"], big["mul_cur"])]
    if "pos" in w:
        x = x + w["pos"][:n]
    return x


# ----------------------------------------------------------------------------- delta mixer

def causal_conv(x, taps_w):
    """x [n, C], taps_w [C, K]: y[t, c] = sum_j taps_w[c, j] * x[t - (K - 1 - j), c], zeros before 0."""
    n, C = x.shape
    K = taps_w.shape[1]
    y = torch.zeros_like(x)
    for j in range(K):
        back = K - 1 - j
        if back < n:
            y[back:] += taps_w[:, j] * x[: n - back]
    return y


def delta_rule(q, k, v, beta, g):
    """One head.  q, k [n, dk]; v [n, dv]; beta, g [n].  Returns o [n, dv] and the last state."""
    n, dk = q.shape
    dv = v.shape[1]
    S = torch.zeros(dk, dv, dtype=q.dtype)
    o = torch.zeros(n, dv, dtype=q.dtype)
    for t in range(n):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o, S


def delta_mixer(m, w, p, h, eps):
    """m: the layer's mixer sizes; p: tensor prefix ('l3.mix.'); h [n, D]."""
    n = h.shape[0]
    H, Hk, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(n, Hk, dk)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(n, Hk, dk)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(n, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                         # [n, H]
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    gate = silu(h @ w[p + "g"].T).reshape(n, H, dv)
    rep = H // Hk
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for i in range(H):
        o, _ = delta_rule(q[:, i // rep], k[:, i // rep], v[:, i], beta[:, i], g[:, i])
        out[:, i] = rms_unit(o, eps) * w[p + "norm"] * gate[:, i]
    return out.reshape(n, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------------ latent attention

def latent_of(m, w, p, h, eps):
    return rms_unit(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]


def latent_attention(m, w, p, h, c):
    """h [n, D] (queries), c [n, R] the latents of the same positions."""
    n = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(n, H, dk)
    k = (c @ w[p + "uk"].T).reshape(n, H, dk)
    v = (c @ w[p + "uv"].T).reshape(n, H, dv)
    mask = torch.tril(torch.ones(n, n, dtype=torch.bool))
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for i in range(H):
        s = (q[:, i] @ k[:, i].T) * m["scale"]
        s = s.masked_fill(~mask, -math.inf)
        out[:, i] = torch.softmax(s, dim=-1) @ v[:, i]
    return out.reshape(n, H * dv) @ w[p + "o"].T


# ---------------------------------------------------------------------------- feed-forward

def gated_expert(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(r, z):
    """r: router constants; z [n, E] logits.  Returns (chosen [n, top], weights [n, top])."""
    s = torch.softmax(z, dim=-1)
    n, E = s.shape
    groups = r.get("groups") or {"count": 1, "keep": 1}
    G, keep = groups["count"], groups["keep"]
    per = E // G
    best = s.reshape(n, G, per).max(dim=-1).values
    kept = best.topk(keep, dim=-1).indices                                          # [n, keep]
    allowed = torch.zeros(n, G, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    allowed = allowed[:, :, None].expand(n, G, per).reshape(n, E)
    masked = torch.where(allowed, s, torch.full_like(s, -1.0))
    chosen = masked.topk(r["top"], dim=-1).indices
    return chosen, s.gather(1, chosen) * r["scale"]


def moe(mlp, w, p, h):
    r = mlp["router"]
    chosen, weights = route(r, h @ w[p + "router"].T)
    y = torch.zeros_like(h)
    for e in range(r["experts"]):
        hit = (chosen == e)
        rows = hit.any(dim=-1).nonzero().flatten()
        if rows.numel():
            wt = (weights * hit)[rows].sum(-1, keepdim=True)
            y[rows] += wt * gated_expert(w, f"{p}e{e}.", h[rows])
    if mlp.get("shared"):
        y = y + torch.sigmoid(h @ w[p + "shared.sg"].T) * gated_expert(w, p + "shared.", h)
    return y


# ------------------------------------------------------------------------------- the model

def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None):
    """float64 logits [n, vocab]; ``layers_out`` receives the residual stream after every layer."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = embed(cfg, w, tokens)
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "delta":
            y = delta_mixer(m, w, p, x, eps)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                latents[i] = latent_of(m, w, p, x, eps)
                c = latents[i]
            else:
                c = latents[m["kv_from"]]
            y = latent_attention(m, w, p, x, c)
        else:
            raise ValueError(layer["type"])
        x = x + mult * rms_unit(y, eps) * w[f"l{i}.norm1"]
        if layer.get("mlp"):
            y = moe(layer["mlp"], w, f"l{i}.mlp.", x)
            x = x + mult * rms_unit(y, eps) * w[f"l{i}.norm2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms_unit(x, eps) * w["final.norm"]) @ w["head"].T

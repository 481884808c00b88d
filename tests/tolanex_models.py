"""Small Tolanex configurations for the tests, their model folders and the plain implementation's
logits.  The configurations differ from each other in every size and constant, put the layer
kinds in different orders, and avoid values that would hide a mix-up (heads equal to query/key
heads, key size equal to value size, one group, one tap, a multiplier of 1).

tlx-a: delta (2 query/key heads under 4 heads, 4 taps, experts in 3 groups of which 2 are kept,
       a shared expert), latent attention without a feed-forward, latent attention that reads
       layer 1's pages (top-1 experts, no groups, no shared expert).
tlx-b: latent attention first (rank 48: the tensor-core attention kernels take it), delta with as
       many query/key heads as heads and 2 taps, a second latent of another rank, and a layer that
       reads layer 0's pages across two layers in between.
tlx-c: a rank the tensor-core kernels do not take, key sizes 12 and 20, one tap, 5 experts.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

import plain_tolanex as P


def _moe(ff, experts, top, scale, groups=None, shared=None):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


CONFIGS = {
    "tlx-a": dict(
        seed=21, block_size=16, sharpen=6.0,
        cfg={"architecture": "Tolanex", "vocab": 211, "width": 72, "max_positions": 320,
             "norm": {"eps": 1e-5}, "residual_mult": 0.7,
             "embedding": {"bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 7}},
             "layers": [
                 {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "conv": 4},
                  "mlp": _moe(48, 6, 2, 1.5, groups=(3, 2), shared=56)},
                 {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "vdim": 24, "kv_rank": 32, "scale": 0.3},
                  "mlp": None},
                 {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "vdim": 16, "kv_rank": 32, "scale": 0.5,
                                                        "kv_from": 1},
                  "mlp": _moe(40, 4, 1, 1.0)},
             ]}),
    "tlx-b": dict(
        seed=22, block_size=8, sharpen=5.0,
        cfg={"architecture": "Tolanex", "vocab": 150, "width": 64, "max_positions": 280,
             "norm": {"eps": 3e-6}, "residual_mult": 0.4,
             "embedding": {"bigram": {"buckets": 53, "mul_prev": 5, "mul_cur": 113}},
             "layers": [
                 {"type": "latent_attention", "mixer": {"heads": 2, "dim": 24, "vdim": 8, "kv_rank": 48, "scale": 0.2},
                  "mlp": _moe(32, 8, 3, 2.5, groups=(4, 2), shared=24)},
                 {"type": "delta", "mixer": {"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 33, "conv": 2},
                  "mlp": _moe(24, 4, 2, 0.8, groups=(2, 1))},
                 {"type": "latent_attention", "mixer": {"heads": 4, "dim": 8, "vdim": 12, "kv_rank": 16, "scale": 0.35},
                  "mlp": None},
                 {"type": "latent_attention", "mixer": {"heads": 5, "dim": 12, "vdim": 20, "kv_rank": 48, "scale": 0.25,
                                                        "kv_from": 0},
                  "mlp": _moe(16, 3, 3, 1.2, shared=40)},
             ]}),
    "tlx-c": dict(
        seed=23, block_size=16, sharpen=4.0,
        cfg={"architecture": "Tolanex", "vocab": 97, "width": 40, "max_positions": 200,
             "norm": {"eps": 1e-6}, "residual_mult": 1.3,
             "embedding": {"bigram": {"buckets": 29, "mul_prev": 211, "mul_cur": 3}},
             "layers": [
                 {"type": "delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 12, "vdim": 20, "conv": 1}, "mlp": None},
                 {"type": "latent_attention", "mixer": {"heads": 3, "dim": 20, "vdim": 12, "kv_rank": 40, "scale": 0.15},
                  "mlp": _moe(56, 5, 2, 3.0, shared=16)},
             ]}),
}

TORCH_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def write_model(name: str, dtype: str, folder: str) -> str:
    """Random weights through the package's own writer, then the query maps of the latent layers
    are scaled up so that the softmax is sharp: single keys, also far ones, then carry weight and
    a missed or doubled key shows in the logits."""
    import kvcm
    from safetensors import safe_open
    from safetensors.torch import save_file
    c = CONFIGS[name]
    cfg = kvcm.config.config_from_dict(c["cfg"])
    kvcm.write_random_model(folder, cfg, c["seed"], TORCH_DT[dtype], norm_jitter=0.1)
    path = os.path.join(folder, "model.safetensors")
    w = {}
    with safe_open(path, framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).clone()
    for i, layer in enumerate(c["cfg"]["layers"]):
        if layer["type"] == "latent_attention":
            w[f"l{i}.mix.q"] = (w[f"l{i}.mix.q"].float() * c["sharpen"]).to(w[f"l{i}.mix.q"].dtype)
    decisive_routers(c["cfg"], w, c["seed"])
    save_file(w, path, metadata={"format": "pt"})
    return folder


def decisive_routers(cfg: dict, w: Dict[str, torch.Tensor], seed: int) -> None:
    """Makes every router's choice a clear one, so that a rounding of the 16-bit path cannot turn it
    (two experts of nearly equal score are no fault of the engine, but they move a position's logits
    by much).  Every routed layer gets residual coordinates of its own, one per expert.  On them the
    token table holds a permutation of 0, 1, 2, ... per token, the other tables hold zero and the
    norms' weights are zero, so no layer writes there; the router reads exactly these coordinates.
    A row's logits are then a permutation of 0 .. experts-1 that depends on its token: gaps of 1.
    The tables are also scaled up to a spread of about 0.5."""
    g = torch.Generator().manual_seed(seed)
    for name in ("embed", "bigram", "pos"):
        w[name] = (w[name].float() * 25.0).to(w[name].dtype)
    at = 0
    for i, layer in enumerate(cfg["layers"]):
        if not layer.get("mlp"):
            continue
        E = layer["mlp"]["router"]["experts"]
        cols = slice(at, at + E)
        at += E
        assert at <= cfg["width"]
        codes = torch.stack([torch.randperm(E, generator=g) for _ in range(cfg["vocab"])]).float()
        w["embed"][:, cols] = codes.to(w["embed"].dtype)
        w["bigram"][:, cols] = 0
        w["pos"][:, cols] = 0
        for name in w:
            if name.endswith(".norm1") or name.endswith(".norm2"):
                w[name][cols] = 0
        router = torch.zeros_like(w[f"l{i}.mlp.router"])
        router[:, cols] = torch.eye(E, dtype=router.dtype)
        w[f"l{i}.mlp.router"] = router


def read_model(folder: str):
    """(config dict, weights as float64)."""
    from safetensors import safe_open
    cfg = json.load(open(os.path.join(folder, "config.json")))
    w: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).double()
    return cfg, w


def plain_logits(folder: str, tokens: List[int]) -> torch.Tensor:
    cfg, w = read_model(folder)
    return P.forward(cfg, w, list(tokens))

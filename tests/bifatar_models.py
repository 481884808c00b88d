"""Small Bifatar configurations for the tests, their model folders and the plain implementation's
logits.  The configurations differ from each other in every size and constant, put the layer kinds
in different orders, and avoid values that would hide a mix-up: key size equal to value size, rotary
width equal to the head size, as many query/key heads as heads, one group, norm parts equal to groups,
scales of 1.

bif-a: attention (partial rotation, window 37, values kept for later layers), the state-space mixer (3 groups
       under 6 heads, 4 norm parts, no feed-forward), attention beside the delta rule (one KV head under 4
       heads; 2 query/key heads under 4 delta heads; ranks 10 and 6), attention that mixes layer 0's values,
       attention without value mixing and with a window shorter than a page.
bif-b: sizes that the tensor-core kernels take (heads of 64 on pages of 32; state 64), the side-by-side layer
       first, then two value-mixing attention layers around a state-space layer.
bif-c: no rotation, no window, no cap (the optional keys are absent), one tap, head sizes 20 and 12.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

import plain_bifatar as P


def _attn(heads, kv, dim, vdim, scale, rot=None, window=None, cap=None, v_mix=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if window:
        m["mask"] = {"size": window}
    if cap:
        m["softcap"] = cap
    if v_mix is not None:
        m["v_mix"] = v_mix
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


CONFIGS = {
    "bif-a": dict(seed=31, block_size=16, cfg={
        "architecture": "Bifatar", "vocab": 211, "width": 72, "norm": {"eps": 2e-5},
        "layers": [
            {"type": "attention", "mixer": _attn(4, 2, 24, 40, 0.3, (10000.0, 16), 37, 5.0, True), "mlp": _dense(100)},
            {"type": "mamba2", "mixer": {"heads": 6, "vdim": 12, "state": 20, "groups": 3, "conv": 3, "norm_groups": 4},
             "mlp": None},
            {"type": "parallel", "mixer": {
                "left": _attn(4, 1, 16, 24, 0.2, (500.0, 8)),
                "right": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "conv": 4, "decay_rank": 10, "gate_rank": 6},
                "left_scale": 0.7, "right_scale": 1.6}, "mlp": _dense(56)},
            {"type": "attention", "mixer": _attn(2, 2, 32, 40, 0.25, (300.0, 32), 50, 8.0, True), "mlp": _dense(64)},
            {"type": "attention", "mixer": _attn(3, 1, 16, 16, 0.4, (2000.0, 4), 9, 3.0, False), "mlp": None},
        ]}),
    "bif-b": dict(seed=32, block_size=32, cfg={
        "architecture": "Bifatar", "vocab": 150, "width": 128, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "parallel", "mixer": {
                "left": _attn(4, 2, 32, 48, 0.15, (1000000.0, 32)),
                "right": {"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 64, "conv": 2, "decay_rank": 16, "gate_rank": 8},
                "left_scale": 1.3, "right_scale": 0.6}, "mlp": _dense(160)},
            {"type": "attention", "mixer": _attn(4, 1, 64, 64, 0.1, (50000.0, 64), 70, 12.0, True), "mlp": _dense(96)},
            {"type": "mamba2", "mixer": {"heads": 4, "vdim": 32, "state": 64, "groups": 1, "conv": 4, "norm_groups": 1},
             "mlp": _dense(64)},
            {"type": "attention", "mixer": _attn(2, 1, 64, 64, 0.12, (777.0, 32), 129, 30.0, True), "mlp": None},
        ]}),
    "bif-c": dict(seed=33, block_size=8, cfg={
        "architecture": "Bifatar", "vocab": 97, "width": 40, "norm": {"eps": 1e-4},
        "layers": [
            {"type": "mamba2", "mixer": {"heads": 2, "vdim": 10, "state": 8, "groups": 2, "conv": 1, "norm_groups": 5},
             "mlp": _dense(24)},
            {"type": "attention", "mixer": _attn(3, 3, 20, 12, 0.35), "mlp": None},
            {"type": "parallel", "mixer": {
                "left": _attn(2, 2, 12, 20, 0.45),
                "right": {"heads": 3, "kv_heads": 1, "dim": 20, "vdim": 12, "conv": 1, "decay_rank": 3, "gate_rank": 5},
                "left_scale": 2.0, "right_scale": 0.3}, "mlp": None},
        ]}),
}

TORCH_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def write_model_from(cfg_dict: dict, seed: int, dtype: str, folder: str, table_scale: float = 25.0) -> str:
    """Random weights through the package's own writer; the token table is scaled up to a spread of
    about 0.5 so that the tanh norms work in their curved part."""
    import kvcm
    from safetensors import safe_open
    from safetensors.torch import save_file
    cfg = kvcm.config.config_from_dict(cfg_dict)
    kvcm.write_random_model(folder, cfg, seed, TORCH_DT[dtype], norm_jitter=0.1)
    path = os.path.join(folder, "model.safetensors")
    w = {}
    with safe_open(path, framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).clone()
    w["embed"] = (w["embed"].float() * table_scale).to(w["embed"].dtype)
    save_file(w, path, metadata={"format": "pt"})
    return folder


def write_model(name: str, dtype: str, folder: str) -> str:
    c = CONFIGS[name]
    return write_model_from(c["cfg"], c["seed"], dtype, folder)


def read_model(folder: str):
    """(config dict, weights as float64)."""
    from safetensors import safe_open
    cfg = json.load(open(os.path.join(folder, "config.json")))
    w: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).double()
    return cfg, w


def save_weights(folder: str, w: Dict[str, torch.Tensor], dtype: str) -> None:
    from safetensors.torch import save_file
    save_file({n: t.to(TORCH_DT[dtype]).contiguous() for n, t in w.items()}, os.path.join(folder, "model.safetensors"),
              metadata={"format": "pt"})


def plain_logits(folder: str, tokens: List[int]) -> torch.Tensor:
    cfg, w = read_model(folder)
    return P.forward(cfg, w, list(tokens))

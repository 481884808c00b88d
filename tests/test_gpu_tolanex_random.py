"""Tolanex configurations drawn at random (fixed seeds): odd widths and head sizes, ranks the
tensor-core attention kernels do not take, expert sizes that are no multiple of 8 (the plain expert
kernels), every layer order, layers without a feed-forward, routers that choose every expert of
the kept groups.  Each model runs whole, in portions and token by token, in float32 and bfloat16,
against the plain implementation.

float32: every position within the float32 bound.  bfloat16: these models are not tuned to be well
conditioned (a mixer output that nearly cancels is blown up by the norm on it, a softmax may sit
between two keys), so single positions can move by tens of percent under 16-bit rounding with the
plain kernels and the tensor-core kernels alike; what is held here is that the typical position is
within 3 % of the spread and at least 85 % are within 6 %: a size the kernels mishandle, a lost key
or a wrong state moves nearly every position by the order of the spread."""
import random

import pytest
import torch

import helpers
import tolanex_models as TM
from test_gpu_tolanex import close


def close_typical(got, ref, what):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / ref.std().item()
    assert err.median().item() <= 0.03 and (err <= 0.06).double().mean().item() >= 0.85, \
        f"{what}: median {err.median().item():.3f}, {int((err > 0.06).sum())} of {err.numel()} beyond 6 %"

pytestmark = pytest.mark.gpu


def draw(seed: int) -> dict:
    r = random.Random(seed)
    n_layers = r.randint(1, 5)
    layers, owners, experts_total = [], {}, 0
    for i in range(n_layers):
        kind = r.choice(["delta", "latent_attention", "latent_attention"])
        if kind == "delta":
            qk = r.choice([1, 2, 3])
            mixer = {"heads": qk * r.choice([1, 2, 3]), "kv_heads": qk, "dim": r.choice([4, 9, 16, 20, 33, 64, 72]),
                     "vdim": r.choice([5, 8, 24, 40, 65]), "conv": r.choice([1, 2, 3, 4, 5])}
        else:
            rank = r.choice([8, 16, 24, 32, 40, 48, 64, 100])
            mixer = {"heads": r.randint(1, 6), "dim": r.choice([4, 10, 16, 32, 48]), "vdim": r.choice([6, 16, 32, 40]),
                     "kv_rank": rank, "scale": round(r.uniform(0.05, 0.6), 3)}
            same = [j for j, rk in owners.items() if rk == rank]
            if same and r.random() < 0.5:
                mixer["kv_from"] = r.choice(same)
            else:
                owners[i] = rank
        mlp = None
        if r.random() < 0.75:
            count = r.choice([1, 1, 2, 3, 4])
            per = r.randint(1, 4)
            keep = r.randint(1, count)
            E = count * per
            top = r.randint(1, per * keep)
            experts_total += E
            mlp = TM._moe(r.choice([8, 12, 24, 36, 50]), E, top, round(r.uniform(0.5, 3.0), 2),
                          groups=(count, keep) if (count > 1 or r.random() < 0.5) else None,
                          shared=r.choice([None, 8, 20, 48]))
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    width = max(r.choice([24, 40, 52, 66, 88, 130]), experts_total + 8)
    return {"architecture": "Tolanex", "vocab": r.choice([61, 100, 257]), "width": width, "max_positions": 160,
            "norm": {"eps": r.choice([1e-6, 1e-5, 3e-5])}, "residual_mult": round(r.uniform(0.3, 1.5), 2),
            "embedding": {"bigram": {"buckets": r.choice([7, 31, 1021]), "mul_prev": r.randint(1, 500),
                                     "mul_cur": r.randint(1, 500)}},
            "layers": layers}


@pytest.mark.parametrize("seed", range(10))
def test_random_configuration(seed, tmp_path):
    cfg = draw(seed)
    name = f"tlx-random-{seed}"
    # (queries are not sharpened here: with scales up to 0.6 and key sizes up to 48 the softmax is already
    # close to a choice of one key, and sharper still a bfloat16 rounding turns near-ties between keys)
    TM.CONFIGS[name] = dict(seed=100 + seed, block_size=16, sharpen=1.0, cfg=cfg)
    toks = helpers.random_tokens(75, cfg["vocab"], 500 + seed)
    for dtype in ("float32", "bfloat16"):
        folder = TM.write_model(name, dtype, str(tmp_path / dtype))
        ref = TM.plain_logits(folder, toks)
        r = helpers.Replayer(folder, dtype, 256, 16, max_live=3)
        whole = r.step([dict(id="w", tokens=toks, want=list(range(75)))], end=["w"])
        check = (lambda g, w: close(g, ref, dtype, w)) if dtype == "float32" else (lambda g, w: close_typical(g, ref, w))
        check(whole, f"seed {seed} whole ({cfg['layers']})")
        outs, at = [], 0
        for k in (1, 2, 30, 1, 17, 2, 1, 1, 20):
            outs.append(r.step([dict(id="p", tokens=toks[at:at + k], want=list(range(k)))]))
            at += k
        assert at == 75
        check(torch.cat(outs), f"seed {seed} in portions")

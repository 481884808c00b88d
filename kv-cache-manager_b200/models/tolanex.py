"""Tolanex assembled from parts (registered as ``Tolanex``).

Embedding = token row + hashed (previous token, token) row + learned position row.  Every layer
is an output-norm block, x += m * norm1(mixer(x)); x += m * norm2(ff(x)), whose mixer is the
gated delta rule ("delta") or attention over a cached latent ("latent_attention", optionally
reading an earlier layer's latent pages), and whose feed-forward is absent or a set of routed
experts with an optional gated shared expert.  Final RMSNorm, output head.  Which parts a layer
gets, and every size, is read from the config's layer list.

Checkpoint names: ``embed``, ``bigram``, ``pos``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``; linear weights [out, in].  Fused at load: q|k|v|g and b|a
of a delta mixer, the three convolutions, q|dkv of a latent mixer, router|shared.sg, and the
experts' gate|up and down matrices stacked expert by expert.
"""
from __future__ import annotations

from ..config.model_config import TolanexConfig
from ..config.registry import register_architecture
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, LayerCall
from ..parts.embedding import LMHead, SummedEmbedding
from .spec import ModelSpec, TensorBinding


def build_tolanex(cfg: TolanexConfig, norm_init=("ones",)) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    embedding = SummedEmbedding(cfg.vocab, D, cfg.bigram_buckets, cfg.bigram_mul_prev, cfg.bigram_mul_cur,
                                cfg.max_positions)
    bindings = [TensorBinding(embedding, "weight", [("embed", (cfg.vocab, D))])]
    if cfg.bigram_buckets:
        bindings.append(TensorBinding(embedding, "pair", [("bigram", (cfg.bigram_buckets + 1, D))]))
    if cfg.max_positions:
        bindings.append(TensorBinding(embedding, "place", [("pos", (cfg.max_positions, D))]))
    blocks, order = [], []
    for i, layer in enumerate(cfg.layers):
        m, p = layer["mixer"], f"l{i}.mix."
        cache_of = None
        if layer["type"] == "delta":
            H, Hk, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            mixer = MIXERS.build("gated_delta", hidden=D, heads=H, qk_heads=Hk, dk=dk, dv=dv, taps=taps, norm_eps=eps)
            bindings += [
                TensorBinding(mixer.qkvg, "weight", [(p + "q", (Hk * dk, D)), (p + "k", (Hk * dk, D)),
                                                     (p + "v", (H * dv, D)), (p + "g", (H * dv, D))]),
                TensorBinding(mixer.ba, "weight", [(p + "b", (H, D)), (p + "a", (H, D))]),
                TensorBinding(mixer, "conv", [(p + "q.conv", (Hk * dk, taps)), (p + "k.conv", (Hk * dk, taps)),
                                              (p + "v.conv", (H * dv, taps))]),
                TensorBinding(mixer, "A_log", [(p + "A_log", (H,))]),
                TensorBinding(mixer, "dt_bias", [(p + "dt_bias", (H,))]),
                TensorBinding(mixer, "norm", [(p + "norm", (dv,))]),
                TensorBinding(mixer.o, "weight", [(p + "o", (D, H * dv))]),
            ]
        else:                                   # latent_attention (the config has been validated)
            H, dk, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            own = m.get("kv_from") is None
            mixer = MIXERS.build("latent_attention", hidden=D, heads=H, dk=dk, dv=dv, rank=R, scale=m["scale"],
                                 norm_eps=eps, own_latent=own)
            if own:
                bindings += [TensorBinding(mixer.q_dkv, "weight", [(p + "q", (H * dk, D)), (p + "dkv", (R, D))]),
                             TensorBinding(mixer, "latent_norm", [(p + "dkv.norm", (R,))])]
            else:
                bindings.append(TensorBinding(mixer.q_dkv, "weight", [(p + "q", (H * dk, D))]))
                cache_of = int(m["kv_from"])    # one call site per layer: the site's index is the layer's
            bindings += [TensorBinding(mixer.uk, "weight", [(p + "uk", (H * dk, R))]),
                         TensorBinding(mixer.uv, "weight", [(p + "uv", (H * dv, R))]),
                         TensorBinding(mixer.o, "weight", [(p + "o", (D, H * dv))])]
        norm1 = NORMS.build("rmsnorm_output", hidden=D, eps=eps, mult=cfg.residual_mult, init=norm_init)
        bindings.append(TensorBinding(norm1, "weight", [(f"l{i}.norm1", (D,))]))
        norm2 = ffn = None
        mlp = layer.get("mlp")
        if mlp is not None:
            r, q = mlp["router"], f"l{i}.mlp."
            E, F = r["experts"], mlp["expert"]["ff"]
            groups = r.get("groups") or {"count": 1, "keep": 1}
            shared_ff = (mlp.get("shared") or {}).get("ff", 0)
            ffn = FEED_FORWARDS.build("routed_experts", hidden=D, experts=E, expert_ff=F, top=r["top"],
                                      scale=r.get("scale", 1.0), groups=groups["count"], keep=groups["keep"],
                                      shared_ff=shared_ff)
            bindings += [
                TensorBinding(ffn, "router", [(q + "router", (E, D))] + ([(q + "shared.sg", (1, D))] if shared_ff else [])),
                TensorBinding(ffn, "gate_up", [(f"{q}e{e}.{n}", (F, D)) for e in range(E) for n in ("gate", "up")]),
                TensorBinding(ffn, "down", [(f"{q}e{e}.down", (D, F)) for e in range(E)]),
            ]
            if shared_ff:
                bindings += [TensorBinding(ffn.shared.gate_up, "weight", [(q + "shared.gate", (shared_ff, D)),
                                                                          (q + "shared.up", (shared_ff, D))]),
                             TensorBinding(ffn.shared.down, "weight", [(q + "shared.down", (D, shared_ff))])]
            norm2 = NORMS.build("rmsnorm_output", hidden=D, eps=eps, mult=cfg.residual_mult, init=norm_init)
            bindings.append(TensorBinding(norm2, "weight", [(f"l{i}.norm2", (D,))]))
        blocks.append(BLOCKS.build("output_norm", norm1=norm1, mixer=mixer, norm2=norm2, ffn=ffn))
        order.append(LayerCall(i, cache_of))
    final_norm = NORMS.build("rmsnorm", hidden=D, eps=eps, init=norm_init)
    bindings.append(TensorBinding(final_norm, "weight", [("final.norm", (D,))]))
    head = LMHead(D, cfg.vocab)
    bindings.append(TensorBinding(head, "weight", [("head", (cfg.vocab, D))]))
    return ModelSpec(cfg, embedding, blocks, order, final_norm, head, bindings)


register_architecture("Tolanex", TolanexConfig, build_tolanex, replace=True)

"""Bifatar assembled from parts (registered as ``Bifatar``).

Embedding; every layer is a parallel block, x += mixer(h) + ff(h) with h = tanh-norm(x); the mixer is,
by the layer's ``type``,

* "attention": windowed grouped-query attention with (partial) rotary encoding, q and k of every head scaled
  to unit root mean square after the rotation, capped scores, a sink per head, and values mixed with
  those of the first such layer (``attention_general``);
* "mamba2": the selective state-space mixer (``mamba2``);
* "parallel": two mixers side by side, left a causal grouped-query attention with biased projections and
  a norm over the whole q and k projections before the rotation, right the gated delta rule with a
  decay per key channel (``side_by_side`` of ``attention_general`` and ``gated_delta_channel``);

the feed-forward is absent or dense with a squared ReLU.  Final tanh-norm, output head.  Which parts a
layer gets, and every size, comes from the config's layer list; the ranks of the right mixer's two-stage
projections are the shapes of their tensors (``tensor_shapes``, from the checkpoint's header) or, when a
model is made without a checkpoint, the optional mixer keys ``decay_rank`` and ``gate_rank``.

Checkpoint names: ``embed``, ``l<i>.norm1[.b|.alpha]``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``,
``final.norm[.b|.alpha]``, ``head``; linear weights [out, in].  Fused at load: q|k|v (and their biases) of
an attention mixer, q|k|v and the three convolutions of the right mixer.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

from ..config.model_config import BifatarConfig, ConfigError
from ..config.registry import register_architecture
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LayerCall
from ..parts.embedding import Embedding, LMHead
from .spec import ModelSpec, TensorBinding


def _position(m: dict):
    rot = m.get("rot")
    if rot is None:
        return POSITION_ENCODINGS.build("none")
    return POSITION_ENCODINGS.build("rope", head_dim=m["dim"], theta=rot["base"], rotary_dim=rot["dims"])


def _norm(bindings, name: str, D: int, init):
    norm = NORMS.build("dyt", hidden=D, init=init)
    bindings += [TensorBinding(norm, "weight", [(name, (D,))]), TensorBinding(norm, "bias", [(name + ".b", (D,))]),
                 TensorBinding(norm, "alpha", [(name + ".alpha", ())])]
    return norm


def _attention_bindings(bindings, mixer, p: str, D: int, m: dict, bias: bool):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    bindings += [TensorBinding(mixer.qkv, "weight", [(p + "q", (H * dk, D)), (p + "k", (G * dk, D)), (p + "v", (G * dv, D))]),
                 TensorBinding(mixer.o, "weight", [(p + "o", (D, H * dv))])]
    if bias:
        bindings.append(TensorBinding(mixer, "bias", [(p + "q.b", (H * dk,)), (p + "k.b", (G * dk,)), (p + "v.b", (G * dv,))]))


def _rank(m: dict, key: str, name: str, shapes: Optional[Dict[str, Tuple[int, ...]]]) -> int:
    if shapes is not None and name in shapes and len(shapes[name]) == 2:
        return int(shapes[name][0])
    if isinstance(m.get(key), int) and m[key] > 0:
        return m[key]
    raise ConfigError(f"Bifatar: the rank of '{name}' is given neither by a tensor's shape nor by mixer key '{key}'")


def build_bifatar(cfg: BifatarConfig, norm_init=("ones",), tensor_shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    embedding = Embedding(cfg.vocab, D)
    bindings = [TensorBinding(embedding, "weight", [("embed", (cfg.vocab, D))])]
    blocks, order = [], []
    mix_source_seen = False
    for i, layer in enumerate(cfg.layers):
        m, p, kind = layer["mixer"], f"l{i}.mix.", layer["type"]
        if kind == "attention":
            H, G = m["heads"], m["kv_heads"]
            mix = None
            if m.get("v_mix"):
                mix = "mix" if mix_source_seen else "source"
                mix_source_seen = True
            mixer = MIXERS.build("attention_general", hidden=D, num_heads=H, num_kv_heads=G, dk=m["dim"], dv=m["vdim"],
                                 position=_position(m), scale=m["scale"], window=(m.get("mask") or {}).get("size", 0),
                                 softcap=m.get("softcap") or 0.0, sink=True, head_norm=True, norm_eps=eps, value_mix=mix)
            _attention_bindings(bindings, mixer, p, D, m, bias=False)
            bindings.append(TensorBinding(mixer, "sink", [(p + "sink", (H,))]))
            if mix is not None:
                bindings.append(TensorBinding(mixer, "vmix", [(p + "vmix", ())]))
        elif kind == "mamba2":
            Hn, P, N, Gr, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            mixer = MIXERS.build("mamba2", hidden=D, heads=Hn, vdim=P, state=N, groups=Gr, taps=taps,
                                 norm_groups=m["norm_groups"], norm_eps=eps)
            C = mixer.conv_channels
            bindings += [TensorBinding(mixer.inp, "weight", [(p + "in", (2 * Hn * P + 2 * Gr * N + Hn, D))]),
                         TensorBinding(mixer, "conv", [(p + "conv", (C, taps))]),
                         TensorBinding(mixer, "conv_bias", [(p + "conv.b", (C,))]),
                         TensorBinding(mixer, "dt_bias", [(p + "dt_bias", (Hn,))]),
                         TensorBinding(mixer, "A_log", [(p + "A_log", (Hn,))]),
                         TensorBinding(mixer, "D", [(p + "D", (Hn,))]),
                         TensorBinding(mixer, "norm", [(p + "norm", (Hn * P,))]),
                         TensorBinding(mixer.o, "weight", [(p + "o", (D, Hn * P))])]
        else:                                       # "parallel" (the config has been validated)
            lm, rm = m["left"], m["right"]
            left = MIXERS.build("attention_general", hidden=D, num_heads=lm["heads"], num_kv_heads=lm["kv_heads"],
                                dk=lm["dim"], dv=lm["vdim"], position=_position(lm), scale=lm["scale"], bias=True,
                                proj_norm=True, norm_eps=eps)
            pl = p + "left."
            _attention_bindings(bindings, left, pl, D, lm, bias=True)
            bindings += [TensorBinding(left, "q_norm", [(pl + "q.norm", (lm["heads"] * lm["dim"],))]),
                         TensorBinding(left, "k_norm", [(pl + "k.norm", (lm["kv_heads"] * lm["dim"],))])]
            pr = p + "right."
            Hn, Hk, dk, dv, taps = rm["heads"], rm["kv_heads"], rm["dim"], rm["vdim"], rm["conv"]
            ra, rg = _rank(rm, "decay_rank", pr + "a1", tensor_shapes), _rank(rm, "gate_rank", pr + "g1", tensor_shapes)
            right = MIXERS.build("gated_delta_channel", hidden=D, heads=Hn, qk_heads=Hk, dk=dk, dv=dv, taps=taps,
                                 decay_rank=ra, gate_rank=rg, norm_eps=eps)
            bindings += [
                TensorBinding(right.qkv, "weight", [(pr + "q", (Hk * dk, D)), (pr + "k", (Hk * dk, D)), (pr + "v", (Hn * dv, D))]),
                TensorBinding(right, "conv", [(pr + "q.conv", (Hk * dk, taps)), (pr + "k.conv", (Hk * dk, taps)),
                                              (pr + "v.conv", (Hn * dv, taps))]),
                TensorBinding(right.b, "weight", [(pr + "b", (Hn, D))]),
                TensorBinding(right, "A_log", [(pr + "A_log", (Hn,))]),
                TensorBinding(right, "norm", [(pr + "norm", (dv,))]),
                TensorBinding(right.a1, "weight", [(pr + "a1", (ra, D))]),
                TensorBinding(right.a2, "weight", [(pr + "a2", (Hn * dk, ra))]),
                TensorBinding(right, "dt_bias", [(pr + "dt_bias", (Hn * dk,))]),
                TensorBinding(right.g1, "weight", [(pr + "g1", (rg, D))]),
                TensorBinding(right.g2, "weight", [(pr + "g2", (Hn * dv, rg))]),
                TensorBinding(right.o, "weight", [(pr + "o", (D, Hn * dv))]),
            ]
            mixer = MIXERS.build("side_by_side", left=left, right=right, left_scale=m["left_scale"],
                                 right_scale=m["right_scale"])
        norm1 = _norm(bindings, f"l{i}.norm1", D, norm_init)
        ffn = None
        mlp = layer.get("mlp")
        if mlp is not None:
            ffn = FEED_FORWARDS.build("dense_mlp", hidden=D, intermediate=mlp["ff"], activation="relu2")
            bindings += [TensorBinding(ffn.up, "weight", [(f"l{i}.mlp.up", (mlp["ff"], D))]),
                         TensorBinding(ffn.down, "weight", [(f"l{i}.mlp.down", (D, mlp["ff"]))])]
        blocks.append(BLOCKS.build("parallel", norm1=norm1, mixer=mixer, ffn=ffn))
        order.append(LayerCall(i))
    final_norm = _norm(bindings, "final.norm", D, norm_init)
    head = LMHead(D, cfg.vocab)
    bindings.append(TensorBinding(head, "weight", [("head", (cfg.vocab, D))]))
    return ModelSpec(cfg, embedding, blocks, order, final_norm, head, bindings)


register_architecture("Bifatar", BifatarConfig, build_bifatar, replace=True)

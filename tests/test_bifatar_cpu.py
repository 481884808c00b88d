"""Bifatar without a GPU: the configuration reader and its refusals, the builder's tensor names and
shapes, and the plain implementation's own pieces against each other."""
import copy

import pytest
import torch

import bifatar_models as BM
import plain_bifatar as P


def test_config_is_read_and_written_back():
    import kvcm
    for name, c in BM.CONFIGS.items():
        cfg = kvcm.config.config_from_dict(c["cfg"])
        assert cfg.architecture == "Bifatar" and cfg.width == c["cfg"]["width"]
        assert kvcm.config.config_from_dict(cfg.to_json_dict()) == cfg


@pytest.mark.parametrize("edit,word", [
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "unknown type"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 26), "within"),
    (lambda d: d["layers"][1]["mixer"].__setitem__("norm_groups", 5), "norm_groups"),
    (lambda d: d["layers"][2]["mixer"].pop("left_scale"), "left_scale"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("vdim", 24), "mix values"),
    (lambda d: d["layers"][0].__setitem__("mlp", {"kind": "moe"}), "dense"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_config_refusals_name_the_key(edit, word):
    import kvcm
    d = copy.deepcopy(BM.CONFIGS["bif-a"]["cfg"])
    edit(d)
    with pytest.raises(kvcm.config.ConfigError) as e:
        kvcm.config.config_from_dict(d)
    assert word in str(e.value)


def test_builder_names_every_tensor_once_and_takes_ranks_from_shapes():
    import kvcm
    from kvcm.engine.model_io import build_spec
    d = copy.deepcopy(BM.CONFIGS["bif-a"]["cfg"])
    cfg = kvcm.config.config_from_dict(d)
    spec = build_spec(cfg)
    names = [n for b in spec.bindings for n, _ in b.sources]
    assert len(names) == len(set(names))
    for want in ("embed", "l0.norm1.alpha", "l0.mix.sink", "l0.mix.vmix", "l1.mix.conv.b", "l1.mix.D", "l2.mix.left.q.b",
                 "l2.mix.left.k.norm", "l2.mix.right.a2", "l2.mix.right.dt_bias", "l3.mix.vmix", "final.norm.b", "head"):
        assert want in names, want
    assert "l4.mix.vmix" not in names and "l1.mlp.up" not in names
    shapes = dict(s for b in spec.bindings for s in b.sources)
    assert shapes["l2.mix.right.a1"] == (10, 72) and shapes["l2.mix.right.dt_bias"] == (4 * 12,)
    # without the optional keys the ranks come from the checkpoint's shapes
    for k in ("decay_rank", "gate_rank"):
        d["layers"][2]["mixer"]["right"].pop(k)
    cfg2 = kvcm.config.config_from_dict(d)
    with pytest.raises(kvcm.config.ConfigError):
        build_spec(cfg2)
    spec2 = build_spec(cfg2, {"l2.mix.right.a1": (7, 72), "l2.mix.right.g1": (5, 72)})
    shapes2 = dict(s for b in spec2.bindings for s in b.sources)
    assert shapes2["l2.mix.right.a2"] == (48, 7) and shapes2["l2.mix.right.g2"] == (80, 5)
    # the cache of a head is as wide as the wider of key and value, in a size the attention kernels take
    assert spec.blocks[0].mixer.cache_spec().head_dim == 48 and spec.blocks[0].mixer.cache_spec().window == 37
    assert spec.blocks[2].mixer.cache_spec().window == 0 and spec.blocks[2].mixer.state_spec() is not None


def test_plain_pieces():
    g = torch.Generator().manual_seed(0)
    # a window as large as the sequence is no window; a very negative sink is no sink
    q, k, v = (torch.randn(30, 4, 8, generator=g, dtype=torch.float64), torch.randn(30, 2, 8, generator=g, dtype=torch.float64),
               torch.randn(30, 2, 6, generator=g, dtype=torch.float64))
    a = P.softmax_attention(q, k, v, 0.3)
    assert torch.allclose(a, P.softmax_attention(q, k, v, 0.3, window=30, sink=torch.full((4,), -80.0)))
    assert not torch.allclose(a, P.softmax_attention(q, k, v, 0.3, window=29))
    assert torch.allclose(P.softmax_attention(q, k, v, 0.3, window=1).view(30, 4, 6)[:, 1], v[:, 0])
    # a sink of zero with one visible key halves that key's weight
    assert torch.allclose(P.softmax_attention(q[:1], k[:1], v[:1], 0.0, sink=torch.zeros(4)).view(4, 6)[3], v[0, 1] / 2)
    # the rotation keeps lengths and leaves the dimensions beyond `dims` alone; position 0 is not turned
    x = torch.randn(5, 2, 12, generator=g, dtype=torch.float64)
    y = P.rotate(x, 100.0, 8)
    assert torch.allclose(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1)) and not torch.allclose(y[1:, :, :8], x[1:, :, :8])
    # the convolution's last column weighs the current token
    w = torch.zeros(3, 4, dtype=torch.float64)
    w[:, -1] = 2.0
    z = torch.randn(6, 3, generator=g, dtype=torch.float64)
    assert torch.allclose(P.causal_conv(z, w), 2 * z)
    w2 = torch.zeros(3, 4, dtype=torch.float64)
    w2[:, 0] = 1.0
    assert torch.allclose(P.causal_conv(z, w2)[3:], z[:3]) and P.causal_conv(z, w2)[:3].abs().max() == 0


def test_plain_logits_of_a_prefix_do_not_depend_on_what_follows(tmp_path):
    folder = BM.write_model("bif-c", "float32", str(tmp_path / "m"))
    cfg, w = BM.read_model(folder)
    toks = torch.randint(0, 97, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    assert torch.allclose(P.forward(cfg, w, toks)[:25], P.forward(cfg, w, toks[:25]), atol=1e-12)

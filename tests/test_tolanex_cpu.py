"""CPU-side checks for Tolanex: the configuration reader and its refusals, the builder's tensor
names, the previous tokens the batch builder packs, and the plain implementation's own pieces
against each other (a recurrence cut in two equals the whole; the router's group limit)."""
import copy

import pytest
import torch

import plain_tolanex as P
import tolanex_models as TM


def test_config_round_trip_and_registry():
    import kvcm
    from kvcm.config import config_from_dict
    for name, c in TM.CONFIGS.items():
        cfg = config_from_dict(c["cfg"])
        assert cfg.architecture == "Tolanex" and cfg.vocab == c["cfg"]["vocab"] and len(cfg.layers) == len(c["cfg"]["layers"])
        assert config_from_dict(cfg.to_json_dict()) == cfg
        assert cfg.bigram_buckets == c["cfg"]["embedding"]["bigram"]["buckets"]
    assert "Tolanex" in kvcm.registered_architectures()
    plural = dict(TM.CONFIGS["tlx-c"]["cfg"])
    plural["architectures"] = [plural.pop("architecture")]
    assert config_from_dict(plural) == config_from_dict(TM.CONFIGS["tlx-c"]["cfg"])


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "conv_only", "unknown type"),
    (("layers", 0, "mixer", "kv_heads"), 3, "multiple"),
    (("layers", 2, "mixer", "kv_from"), 0, "kv_from"),          # layer 0 is no latent layer
    (("layers", 2, "mixer", "kv_from"), 2, "kv_from"),          # not an earlier layer
    (("layers", 0, "mlp", "router", "top"), 5, "cannot choose"),  # 2 groups kept x 2 experts < 5
    (("layers", 0, "mlp", "kind"), "dense", "kind 'moe'"),
    (("norm", "eps"), 0.0, "eps"),
    (("width",), 0, "width"),
])
def test_config_refusals(path, value, word):
    from kvcm.config import ConfigError, config_from_dict
    d = copy.deepcopy(TM.CONFIGS["tlx-a"]["cfg"])
    at = d
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_builder_names_every_tensor_once():
    from kvcm.config import config_from_dict
    from kvcm.config.registry import get_architecture
    cfg = config_from_dict(TM.CONFIGS["tlx-a"]["cfg"])
    spec = get_architecture("Tolanex").build(cfg)
    names = [n for b in spec.bindings for n, _ in b.sources]
    assert len(names) == len(set(names))
    assert {"embed", "bigram", "pos", "final.norm", "head", "l0.mix.q.conv", "l0.mix.A_log", "l0.mlp.e5.down",
            "l0.mlp.shared.sg", "l1.mix.dkv.norm", "l2.mix.uk", "l2.mlp.router"} <= set(names)
    assert "l2.mix.dkv" not in names and "l1.norm2" not in names and "l2.mlp.shared.sg" not in names
    assert [c.cache_of for c in spec.order] == [None, None, 1]
    shapes = dict(s for b in spec.bindings for s in b.sources)
    assert shapes["bigram"] == (98, 72) and shapes["l0.mix.v.conv"] == (160, 4) and shapes["l0.mix.b"] == (4, 72)


def test_batch_builder_packs_previous_tokens():
    from kvcm.cache import core
    b = core.BatchBuilder(4, 8, 1, 64)
    seqs = []
    for n, toks in enumerate(([5, 6, 7, 8, 9], [11, 12, 13])):
        s = core.Sequence()
        s.id = n
        s.tokens = list(toks)
        s.tables = [[n * 2, n * 2 + 1]]
        seqs.append(s)
    buf = torch.zeros(int(b.capacity_for(16, 4, 16)), dtype=torch.int32)
    L = b.build([(seqs[0], 2, 3, []), (seqs[1], 0, 1, [0])], buf.data_ptr(), buf.numel())
    toks = buf[L.off_tokens:L.off_tokens + L.rows].tolist()
    prev = buf[L.off_prev_tokens:L.off_prev_tokens + L.rows].tolist()
    assert toks == [11, 7, 8, 9] and prev == [-1, 6, 7, 8]      # the single-token entry is laid out first
    padded = b.build([(seqs[1], 2, 1, [0])], buf.data_ptr(), buf.numel(), 2, 2, 2)
    assert buf[padded.off_prev_tokens:padded.off_prev_tokens + 2].tolist() == [12, -1]


def test_plain_recurrence_cut_in_two_equals_the_whole():
    g = torch.Generator().manual_seed(0)
    n, dk, dv = 23, 6, 5
    q, k = torch.randn(n, dk, generator=g, dtype=P.F), torch.randn(n, dk, generator=g, dtype=P.F)
    v = torch.randn(n, dv, generator=g, dtype=P.F)
    beta, gd = torch.rand(n, generator=g, dtype=P.F), torch.rand(n, generator=g, dtype=P.F)
    o, S = P.delta_rule(q, k, v, beta, gd)
    # by hand for the first token: S = k u^T with u = beta v, o = (q . k) u
    assert torch.allclose(o[0], (q[0] @ k[0]) * beta[0] * v[0])
    # a key the state has seen once with beta = 1 and g = 1 reads back its value
    o2, _ = P.delta_rule(torch.stack([k[3], k[3]]) / (k[3] @ k[3]), torch.stack([k[3], k[3]]) / k[3].norm(),
                         torch.stack([v[3], v[3]]), torch.ones(2, dtype=P.F), torch.ones(2, dtype=P.F))
    assert torch.allclose(o2[1] * k[3].norm(), v[3])


def test_plain_router_group_limit():
    r = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    z = torch.log(torch.tensor([[0.05, 0.30, 0.25, 0.20, 0.10, 0.10]], dtype=P.F))
    chosen, weights = P.route(r, z)                              # best group is {0, 1}: its best expert scores 0.30
    assert sorted(chosen[0].tolist()) == [0, 1]
    assert torch.allclose(weights.sort().values, torch.tensor([[0.10, 0.60]], dtype=P.F))
    r["groups"]["keep"] = 3
    assert sorted(P.route(r, z)[0][0].tolist()) == [1, 2]
    assert P.causal_conv(torch.arange(4, dtype=P.F)[:, None], torch.tensor([[1.0, 10.0, 100.0]], dtype=P.F)).flatten().tolist() \
        == [0.0, 100.0, 210.0, 321.0]

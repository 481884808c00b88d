"""Tolanex in the engine against the plain implementation (``plain_tolanex.py``, float64, whole
sequences): every way of cutting the work, every kind of layer alone, pages and state slots
that are used again, keys far away and at page borders, the first tokens, long decoding, and
greedy generation through the engine's own entry point and scheduler.

float32 engine: every position within 1e-4 (relative to max(1, |logit|)) of the plain logits.
bfloat16 engine: per position, the root mean square of the difference (mean taken off) is held
against the spread of the plain logits.  Unit roundoff 2^-9, some dozens of roundings on the way
to a logit: about 2 % of the spread; the bound is 6 %.  A rounding can also turn a router's choice
between two experts of nearly equal score, which moves that position by much more without being
a fault, so up to 3 % of the positions may exceed the bound (a lost key, a wrong state or a stale
page moves most positions by the order of the spread itself).
"""
import itertools
import json
import os

import pytest
import torch

import helpers
import plain_tolanex as P
import tolanex_models as TM

pytestmark = pytest.mark.gpu

NAMES = ("tlx-a", "tlx-b", "tlx-c")
LENGTHS = {"tlx-a": [1, 9, 47, 130, 300], "tlx-b": [3, 64, 150, 257], "tlx-c": [2, 33, 190]}
CASES = [(n, d) for n in NAMES for d in ("float32", "bfloat16")]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = TM.write_model(name, dtype, str(tmp_path_factory.mktemp(f"{name}_{dtype}")))
        return made[(name, dtype)]
    return get


@pytest.fixture(scope="module")
def oracle(folders):
    cache = {}

    def get(name, dtype, i):
        if (name, dtype, i) not in cache:
            cache[(name, dtype, i)] = TM.plain_logits(folders(name, dtype), tokens_of(name, i))
        return cache[(name, dtype, i)]
    return get


def tokens_of(name, i):
    return helpers.random_tokens(LENGTHS[name][i], TM.CONFIGS[name]["cfg"]["vocab"], 300 + i)


def replayer(folders, name, dtype, max_tokens, **kw):
    return helpers.Replayer(folders(name, dtype), dtype, max_tokens, TM.CONFIGS[name]["block_size"], **kw)


def close(got, ref, dtype, what):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    if dtype == "float32":
        helpers.assert_logits_close(got, ref, "float32", what)
        return
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / ref.std().item()
    over = int((err > 0.06).sum())
    assert over <= max(1, int(0.03 * err.numel())), \
        f"{what}: {over} of {err.numel()} positions beyond 6 % of the spread (worst {err.max().item():.3f} at {int(err.argmax())})"


# ------------------------------------------------------------------------ ways of cutting the work

@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_requests(name, dtype, folders, oracle):
    r = replayer(folders, name, dtype, 320)
    for i, n in enumerate(LENGTHS[name]):
        toks = tokens_of(name, i)
        got = r.step([dict(id=f"r{i}", tokens=toks, want=list(range(n)))], end=[f"r{i}"])
        close(got, oracle(name, dtype, i), dtype, f"{name} whole request {i}")
    assert r.kv.blocks_in_use() == 0 and r.slots.num_taken() == 0
    assert r.stray_writes() == []


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_against_token_by_token(name, dtype, folders, oracle):
    """The second request token by token from its first token on (the state starts at zero and the
    first tokens have no earlier inputs for the convolution, no previous token for the pair table);
    the longest mostly as one portion, then 40 single tokens."""
    r = replayer(folders, name, dtype, 320)
    toks, ref = tokens_of(name, 1), oracle(name, dtype, 1)
    outs = [r.step([dict(id="x", tokens=[t], want=[0])]) for t in toks]
    close(torch.cat(outs), ref, dtype, f"{name} token by token")
    r.session.release("x")
    i = len(LENGTHS[name]) - 1
    toks, ref = tokens_of(name, i), oracle(name, dtype, i)
    head = len(toks) - 40
    outs = [r.step([dict(id="y", tokens=toks[:head], want=list(range(head)))])]
    outs += [r.step([dict(id="y", tokens=[t], want=[0])]) for t in toks[head:]]
    close(torch.cat(outs), ref, dtype, f"{name} prefill then 40 single tokens")


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_down_to_two_tokens(name, dtype, folders, oracle):
    r = replayer(folders, name, dtype, 320)
    sizes = itertools.cycle([7, 2, 13, 2, 1, 5, 31, 3, 2, 17, 64, 1, 1, 2])
    for i, n in enumerate(LENGTHS[name]):
        toks = tokens_of(name, i)
        outs, at = [], 0
        while at < n:
            k = min(next(sizes), n - at)
            outs.append(r.step([dict(id="p", tokens=toks[at:at + k], want=list(range(k)))]))
            at += k
        r.session.release("p")
        close(torch.cat(outs), oracle(name, dtype, i), dtype, f"{name} request {i} in portions")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_requests_together_with_pages_and_slots_used_again(name, dtype, folders, oracle):
    """Up to three live requests in a pool that cannot hold all requests at once and with three
    state slots: portions of some beside single tokens of others; a request that ends gives its
    pages and its slot to the next one, which must start from zero state."""
    B = TM.CONFIGS[name]["block_size"]
    lens = LENGTHS[name]
    todo = list(range(len(lens))) + [1, 0]                       # two of them a second time
    pool = helpers.roundup(max(lens), B) + 2 * helpers.roundup(sorted(lens)[-2], B)
    r = replayer(folders, name, dtype, pool, max_live=3)
    cuts = itertools.cycle([11, 1, 2, 29, 1, 1, 5, 64, 3, 1])
    live, got, step_no = {}, {}, 0
    slots_seen = []
    while todo or live:
        held = sum(helpers.roundup(len(tokens_of(name, i)), B) for i, _ in live.values())
        while todo and len(live) < 3 and held + helpers.roundup(lens[todo[0]], B) <= pool:
            i = todo.pop(0)
            held += helpers.roundup(lens[i], B)
            live[f"q{step_no}_{i}"] = (i, 0)
            got[f"q{step_no}_{i}"] = []
        entries, ends = [], []
        for rid, (i, at) in list(live.items()):
            toks = tokens_of(name, i)
            k = min(next(cuts), len(toks) - at)
            entries.append(dict(id=rid, tokens=toks[at:at + k], want=list(range(k))))
            live[rid] = (i, at + k)
            if at + k == len(toks):
                ends.append(rid)
        out = r.step(entries, end=())
        slots_seen += [r.live[e["id"]].state_slot for e in entries]
        row = 0
        for e in entries:
            got[e["id"]].append(out[row:row + len(e["tokens"])])
            row += len(e["tokens"])
        for rid in ends:
            r.session.release(rid)
            del live[rid]
        step_no += 1
    for rid, parts in got.items():
        i = int(rid.split("_")[1])
        close(torch.cat(parts), oracle(name, dtype, i), dtype, f"{name} request {rid} among others")
    assert set(slots_seen) <= {0, 1, 2} and r.slots.num_taken() == 0 and r.kv.blocks_in_use() == 0
    assert len(set(r.pages_seen)) < len(r.pages_seen)            # pages were handed out more than once


# ------------------------------------------------------------------------------ each layer kind alone

def one_layer_model(tmp_path, layer, dtype="float32", **top):
    import kvcm
    cfg = {"architecture": "Tolanex", "vocab": 120, "width": 48, "max_positions": 200, "norm": {"eps": 2e-6},
           "residual_mult": 0.9, "layers": [layer]}
    cfg.update(top)
    folder = str(tmp_path / "m")
    kvcm.write_random_model(folder, kvcm.config.config_from_dict(cfg), 7, TM.TORCH_DT[dtype], norm_jitter=0.2)
    return folder


@pytest.mark.parametrize("layer", [
    {"type": "delta", "mixer": {"heads": 6, "kv_heads": 2, "dim": 10, "vdim": 36, "conv": 3}, "mlp": None},
    {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 70, "vdim": 7, "conv": 5}, "mlp": None},
    {"type": "latent_attention", "mixer": {"heads": 5, "dim": 12, "vdim": 28, "kv_rank": 24, "scale": 0.4}, "mlp": None},
], ids=["delta", "delta-one-wide-head", "latent"])
def test_one_mixer_alone(tmp_path, layer):
    folder = one_layer_model(tmp_path, layer, embedding={"bigram": {"buckets": 11, "mul_prev": 3, "mul_cur": 5}})
    toks = helpers.random_tokens(90, 120, 5)
    ref = TM.plain_logits(folder, toks)
    r = helpers.Replayer(folder, "float32", 128, 16)
    whole = r.step([dict(id="a", tokens=toks, want=list(range(90)))], end=["a"])
    close(whole, ref, "float32", "one mixer, whole")
    parts = [r.step([dict(id="b", tokens=toks[a:b], want=list(range(b - a)))]) for a, b in ((0, 1), (1, 3), (3, 50), (50, 51), (51, 90))]
    close(torch.cat(parts), ref, "float32", "one mixer, in portions")


@pytest.mark.parametrize("mlp", [
    TM._moe(20, 9, 4, 1.7, groups=(3, 2), shared=12),
    TM._moe(33, 2, 1, 0.5),
    TM._moe(8, 12, 2, 2.0, groups=(6, 1)),
], ids=["groups-shared", "two-experts", "one-group-kept"])
def test_routed_experts_alone(tmp_path, mlp):
    """A layer whose mixer is as small as it gets, so that the feed-forward carries the logits; the
    plain router's choices are checked to use several experts and every group."""
    layer = {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "conv": 1}, "mlp": mlp}
    folder = one_layer_model(tmp_path, layer)
    toks = helpers.random_tokens(150, 120, 6)
    cfg, w = TM.read_model(folder)
    ref = P.forward(cfg, w, toks)
    r = helpers.Replayer(folder, "float32", 160, 16)
    got = r.step([dict(id="a", tokens=toks, want=list(range(150)))])
    close(got, ref, "float32", "routed experts")
    # the router itself against the plain one, on rows of its own
    from kvcm.kernels import library as K
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    g = mlp["router"].get("groups") or {"count": 1, "keep": 1}
    h = torch.randn(64, 48, dtype=torch.float32, device="cuda")
    wr = torch.randn(E, 48, dtype=torch.float32, device="cuda")
    idx = torch.empty((64, top), dtype=torch.int32, device="cuda")
    wt = torch.empty((64, top), dtype=torch.float32, device="cuda")
    K.moe_route(h, wr, E, g["count"], g["keep"], top, mlp["router"]["scale"], idx, wt, None)
    chosen, weights = P.route(mlp["router"], h.double().cpu() @ wr.double().cpu().T)
    assert torch.equal(idx.cpu().long().sort(dim=-1).values, chosen.sort(dim=-1).values)
    assert torch.allclose(wt.cpu().double().sort(dim=-1).values, weights.sort(dim=-1).values, rtol=1e-5, atol=1e-7)
    assert len(set(chosen.flatten().tolist())) > min(E, 4) // 2


def test_pair_table_and_positions_of_the_embedding():
    """The embedding kernel alone: rows of the pair table by (previous token, token), the extra row
    for a first token, multipliers large enough to overflow 32 bits, positions added unscaled."""
    from kvcm.kernels import library as K
    V, D, buckets, mp, mc = 50000, 24, 1009, 91813, 77773
    g = torch.Generator().manual_seed(3)
    table, pair, place = (torch.randn(n, D, generator=g) for n in (V, buckets + 1, 40))
    ids = torch.tensor([49999, 3, 49998, 7, 0, 49999], dtype=torch.int32)
    prev = torch.tensor([-1, 49999, 3, -1, 7, 0], dtype=torch.int32)
    pos = torch.tensor([0, 1, 2, 0, 1, 39], dtype=torch.int32)
    x = torch.empty(6, D, dtype=torch.float32, device="cuda")
    K.embed_sum(ids.cuda(), prev.cuda(), pos.cuda(), table.cuda(), pair.cuda(), place.cuda(), x, None, buckets, mp, mc)
    rows = [buckets if p < 0 else (p * mp + t * mc) % buckets for p, t in zip(prev.tolist(), ids.tolist())]
    want = table[ids.long()].double() + pair[rows].double() + place[pos.long()].double()
    assert (x.cpu().double() - want).abs().max().item() < 1e-6
    assert P.bigram_rows([49999, 3], buckets, mp, mc) == rows[:2]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [
    {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 48, "conv": 4}, "mlp": None},
    {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "conv": 2}, "mlp": None},
    {"type": "delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 200, "vdim": 36, "conv": 3}, "mlp": None},
    {"type": "latent_attention", "mixer": {"heads": 4, "dim": 32, "vdim": 24, "kv_rank": 64, "scale": 0.2}, "mlp": None},
    {"type": "latent_attention", "mixer": {"heads": 6, "dim": 64, "vdim": 64, "kv_rank": 128, "scale": 0.125}, "mlp": None},
    {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "vdim": 16, "kv_rank": 256, "scale": 0.25}, "mlp": None},
], ids=["delta-64", "delta-128", "delta-200", "latent-64", "latent-128", "latent-256"])
def test_mixers_at_the_sizes_of_the_fast_kernels(tmp_path, layer, dtype):
    """Key sizes that take the other forms of the recurrence kernel (8 lanes a column; more rows of
    S per thread) and ranks that take the tensor-core attention kernels with all heads on one shared
    head (tcgen05 for 64 and 128, mma.sync for 256): 300 tokens whole, then a prompt with 40 single
    tokens behind it."""
    folder = one_layer_model(tmp_path, layer, dtype, width=96, max_positions=320,
                             embedding={"bigram": {"buckets": 11, "mul_prev": 3, "mul_cur": 5}})
    toks = helpers.random_tokens(300, 120, 17)
    ref = TM.plain_logits(folder, toks)
    r = helpers.Replayer(folder, dtype, 640, 16)
    whole = r.step([dict(id="a", tokens=toks, want=list(range(300)))], end=["a"])
    close(whole, ref, dtype, "whole")
    outs = [r.step([dict(id="b", tokens=toks[:260], want=list(range(260)))])]
    outs += [r.step([dict(id="b", tokens=[t], want=[0])]) for t in toks[260:]]
    close(torch.cat(outs), ref, dtype, "prompt, then single tokens")


@pytest.mark.parametrize("heads,rank", [(2, 80), (3, 96), (2, 112), (2, 160), (1, 192), (2, 224), (20, 64), (33, 32)])
def test_latent_ranks_and_head_counts_in_bfloat16(tmp_path, heads, rank):
    """Every rank the tensor-core attention kernels take besides those of the other tests, and more
    heads on the one shared latent head than a block of the decode kernel holds (16): a prompt in two
    portions, then 24 single tokens, two requests side by side."""
    layer = {"type": "latent_attention", "mixer": {"heads": heads, "dim": 16, "vdim": 8, "kv_rank": rank, "scale": 0.2},
             "mlp": None}
    folder = one_layer_model(tmp_path, layer, "bfloat16", width=64, max_positions=256)
    a, b = helpers.random_tokens(200, 120, 31), helpers.random_tokens(150, 120, 32)
    ra, rb = TM.plain_logits(folder, a), TM.plain_logits(folder, b)
    r = helpers.Replayer(folder, "bfloat16", 512, 16)
    oa = [r.step([dict(id="a", tokens=a[:100], want=list(range(100)))])]
    both = r.step([dict(id="a", tokens=a[100:176], want=list(range(76))), dict(id="b", tokens=b[:126], want=list(range(126)))])
    oa.append(both[:76])
    ob = [both[76:]]
    for k in range(24):
        out = r.step([dict(id="a", tokens=[a[176 + k]], want=[0]), dict(id="b", tokens=[b[126 + k]], want=[0])])
        oa.append(out[:1])
        ob.append(out[1:])
    close(torch.cat(oa), ra, "bfloat16", f"rank {rank}, {heads} heads, first request")
    close(torch.cat(ob), rb, "bfloat16", f"rank {rank}, {heads} heads, second request")


# ------------------------------------------------------------------ keys far away, at page borders

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_key_that_stands_out(tmp_path, dtype):
    """Latent attention with one planted position: the queries of all later positions are made to
    point at the latent of position ``far`` (its token appears once), so nearly all attention
    weight lies on that one key among hundreds.  Losing it, or taking a neighbour for it, changes
    the logits completely.  The planted key is tried just before and just behind page borders, as
    first key, and far back; the asking positions are in a prompt's portion and decoded alone."""
    import kvcm
    from safetensors.torch import save_file
    layer = {"type": "latent_attention", "mixer": {"heads": 2, "dim": 16, "vdim": 16, "kv_rank": 32, "scale": 1.0}, "mlp": None}
    folder = one_layer_model(tmp_path, layer, dtype)
    cfg, w = TM.read_model(folder)
    # token 119 has an embedding along one direction e; dkv maps e to a latent l; uk maps l to k; q maps
    # every token's embedding (which has a common component m) to a multiple of k.
    D, R, H, dk = 48, 32, 2, 16
    g = torch.Generator().manual_seed(9)
    e = torch.zeros(D, dtype=torch.float64); e[0] = 6.0
    m = torch.zeros(D, dtype=torch.float64); m[1] = 2.0
    w["embed"] = torch.randn(120, D, generator=g, dtype=torch.float64) * 0.3
    w["embed"][:, :2] = 0
    w["embed"] += m
    w["embed"][119] = e
    w["pos"] = torch.zeros_like(w["pos"])
    w["l0.mix.dkv"] = torch.randn(R, D, generator=g, dtype=torch.float64) * 0.2
    w["l0.mix.dkv.norm"] = torch.ones(R, dtype=torch.float64)
    lat = P.rms_unit(w["l0.mix.dkv"] @ e, cfg["norm"]["eps"])
    k = (w["l0.mix.uk"] @ lat).reshape(H, dk)
    wq = torch.zeros(H * dk, D, dtype=torch.float64)
    wq[:, 1] = (k / k.norm(dim=-1, keepdim=True)).reshape(-1) * 3.0
    w["l0.mix.q"] = wq
    save_file({n: t.to(TM.TORCH_DT[dtype]).contiguous() for n, t in w.items()}, os.path.join(folder, "model.safetensors"),
              metadata={"format": "pt"})
    cfg, w = TM.read_model(folder)
    n = 200
    for far in (0, 15, 16, 17, 31, 32, 100):
        toks = helpers.random_tokens(n, 119, 40 + far)
        toks[far] = 119
        lo = []
        ref = P.forward(cfg, w, toks, lo)
        r = helpers.Replayer(folder, dtype, 256, 16)
        head = 170
        outs = [r.step([dict(id="f", tokens=toks[:far + 1], want=list(range(far + 1)))])]
        if far + 1 < head:
            outs.append(r.step([dict(id="f", tokens=toks[far + 1:head], want=list(range(head - far - 1)))]))
        outs += [r.step([dict(id="f", tokens=[t], want=[0])]) for t in toks[head:]]
        got = torch.cat(outs)
        close(got, ref, dtype, f"planted key at {far}")
        # the plant works: without that key the plain logits are far from the reference
        toks2 = list(toks); toks2[far] = 5
        assert (P.forward(cfg, w, toks2)[far + 1:] - ref[far + 1:]).abs().max().item() > 0.5 * ref.std().item()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, folders, oracle):
    """A short prompt, then 260 tokens one by one: the delta state is read and written 260 times,
    the latent pages grow across many page borders."""
    name = "tlx-a"
    toks, ref = tokens_of(name, 4), oracle(name, dtype, 4)
    r = replayer(folders, name, dtype, 320)
    outs = [r.step([dict(id="d", tokens=toks[:40], want=list(range(40)))])]
    outs += [r.step([dict(id="d", tokens=[t], want=[0])]) for t in toks[40:]]
    close(torch.cat(outs), ref, dtype, "long decoding")


# -------------------------------------------------------------- the engine's own entry point

@pytest.mark.parametrize("name", ["tlx-a", "tlx-b"])
def test_greedy_generation_through_the_engine(name, folders):
    """Scheduler with chunked prefill and few sequences at a time; every generated token must be the
    plain implementation's choice given the tokens before it (ties within 2e-4 allowed)."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    folder = folders(name, "float32")
    cfg, w = TM.read_model(folder)
    B = TM.CONFIGS[name]["block_size"]
    prompts = [helpers.random_tokens(n, cfg["vocab"], 70 + i) for i, n in enumerate([21, 4, 50, 13, 1, 33])]

    def run(graphs):
        ec = EngineConfig(kv=KVManagerConfig(num_blocks=256 // B, block_size=B, max_seq_len=96, watermark_blocks=0),
                          sched=SchedulerConfig(max_num_seqs=3, max_batched_tokens=24), dtype="float32", cuda_graphs=graphs)
        eng = kvcm.Engine.from_folder(folder, ec)
        return eng, kvcm.generate(eng, prompts, 20)

    eng, outs = run(True)
    assert eng.graphs is not None and eng.graphs.replays > 10         # decode steps were replayed from CUDA graphs
    for p, o in zip(prompts, outs):
        assert len(o) == 20
        logits = P.forward(cfg, w, list(p) + list(o))
        for k, tok in enumerate(o):
            row = logits[len(p) - 1 + k]
            assert row.max().item() - row[tok].item() <= 2e-4, (len(p), k, tok, int(row.argmax()))
    assert eng.kv.blocks_in_use(0) == 0 and eng.sched.slots_taken() == 0
    eng2, outs2 = run(False)
    assert eng2.graphs is None and outs2 == outs


def test_generation_in_bfloat16_with_eviction(folders):
    """So few pages that running requests are evicted and computed again from their first token:
    the state slot is reset, the previous token of the pair table is found again.  Same tokens as
    with room for all."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    folder = folders("tlx-a", "bfloat16")
    prompts = [helpers.random_tokens(n, 211, 90 + i) for i, n in enumerate([30, 44, 25, 38])]

    def run(blocks):
        ec = EngineConfig(kv=KVManagerConfig(num_blocks=blocks, block_size=16, max_seq_len=96, watermark_blocks=0),
                          sched=SchedulerConfig(max_num_seqs=4, max_batched_tokens=64), dtype="bfloat16")
        eng = kvcm.Engine.from_folder(folder, ec)
        outs = kvcm.generate(eng, prompts, 30)
        return eng, outs

    roomy, outs = run(64)
    tight, outs2 = run(11)
    assert all(len(o) == 30 for o in outs)
    assert tight.sched.counters().preemptions > 0
    assert outs2 == outs


def test_trace_tool_on_a_model_folder(tmp_path, folders, oracle):
    name, dtype = "tlx-b", "float32"
    toks, ref = tokens_of(name, 2), oracle(name, dtype, 2)
    other = tokens_of(name, 1)
    steps = [dict(step=0, entries=[dict(id="a", tokens=toks[:70], want=[0, 69])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=toks[70:72], want=[1]), dict(id="b", tokens=other, want=[63])], end=["b"]),
             dict(step=2, entries=[dict(id="a", tokens=toks[72:], want=[len(toks) - 73])], end=["a"])]
    out = helpers.run_trace_tool(folders(name, dtype), dtype, steps, 320, str(tmp_path / "out"), vocab_key="vocab")
    close(torch.from_numpy(out[0]), ref[[0, 69]], dtype, "trace tool step 0")
    close(torch.from_numpy(out[1][:1]), ref[[71]], dtype, "trace tool step 1")
    close(torch.from_numpy(out[1][1:]), oracle(name, dtype, 1)[[63]], dtype, "trace tool step 1, second request")
    close(torch.from_numpy(out[2]), ref[[len(toks) - 1]], dtype, "trace tool step 2")


@pytest.mark.parametrize("T,E,top,F,D", [(300, 8, 2, 192, 320), (5, 16, 4, 72, 136), (1, 3, 3, 264, 64), (700, 4, 1, 40, 520)])
def test_expert_products_on_tensor_cores_against_float64(T, E, top, F, D):
    """The experts' products alone: bfloat16 rows through the tensor-core kernels and through the
    plain kernels, both against float64 on the same bfloat16 values.  Experts that get no row, tiles
    of fewer than 128 pairs beside full ones, sizes that are no multiple of the tile."""
    from kvcm.kernels import library as K
    g = torch.Generator().manual_seed(T + E)
    h = (torch.randn(T, D, generator=g) * 0.5).to(torch.bfloat16).cuda()
    wgu = (torch.randn(E, 2 * F, D, generator=g) * D ** -0.5).to(torch.bfloat16).cuda()
    wd = (torch.randn(E, D, F, generator=g) * F ** -0.5).to(torch.bfloat16).cuda()
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if E > 3:
        idx[idx == 1] = 0 if top == 1 else idx[idx == 1]          # (top 1: expert 1 gets no row at all)
    idx = idx.cuda()
    wt = torch.rand(T, top, generator=g).cuda()
    hd, gud, dd = h.double().cpu(), wgu.double().cpu(), wd.double().cpu()
    ref = torch.zeros(T, D, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            a = P.silu(gud[e, :F] @ hd[t]) * (gud[e, F:] @ hd[t])
            ref[t] += wt[t, k].double().cpu() * (dd[e] @ a)
    outs = []
    for tensor_cores in (True, False):
        work = torch.empty(K.moe_work_ints(T, top, E), dtype=torch.int32, device="cuda")
        act = torch.empty(T * top, F, dtype=torch.bfloat16, device="cuda")
        y = torch.empty(T * top, D, dtype=torch.float32, device="cuda")
        xs = torch.empty(T * top, D, dtype=torch.bfloat16, device="cuda") if tensor_cores else None
        out = torch.empty(T, D, dtype=torch.float32, device="cuda")
        K.moe_experts(h, wgu, wd, idx, work, act, y, xs)
        K.moe_combine(y, work, wt, E, None, None, out)
        torch.cuda.synchronize()
        K.check_errors()
        outs.append(out.cpu().double())
        # what remains is the rounding of act to bfloat16 (unit roundoff 2^-8) in a sum over F whose terms have
        # heavy tails; the largest of some 10^5 such errors stays below 4 % of the spread, a fault is of its order
        assert (outs[-1] - ref).abs().max().item() <= 0.04 * ref.std().item(), ("tensor cores" if tensor_cores else "plain")
    assert (outs[0] - outs[1]).abs().max().item() <= 0.04 * ref.std().item()


def test_score_borrows_a_state_slot(folders, oracle):
    """``Engine.score`` on a model with per-request state: teacher-forced logits of a whole sequence,
    twice (the slot is zeroed each time) and with requests running beside it."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    name = "tlx-a"
    B = TM.CONFIGS[name]["block_size"]
    eng = kvcm.Engine.from_folder(folders(name, "float32"), EngineConfig(
        kv=KVManagerConfig(num_blocks=40, block_size=B, max_seq_len=160, watermark_blocks=0),
        sched=SchedulerConfig(max_num_seqs=3, max_batched_tokens=64), dtype="float32"))
    toks, ref = tokens_of(name, 3), oracle(name, "float32", 3)
    close(eng.score(toks), ref, "float32", "score")
    eng.add_request(tokens_of(name, 2), max_new_tokens=5)
    eng.step()
    close(eng.score(toks), ref, "float32", "score beside a running request")
    eng.run_until_idle()
    assert eng.sched.slots_taken() == 0 and eng.kv.blocks_in_use(0) == 0

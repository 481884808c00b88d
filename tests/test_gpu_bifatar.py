"""Bifatar in the engine against the plain implementation (``plain_bifatar.py``, float64, whole
sequences): every way of cutting the work, every kind of layer alone, pages and state slots that are
used again, keys far away, at page borders and at a window's edge, the first tokens, long decoding,
and greedy generation through the engine's own entry point and scheduler.

float32 engine: every position within 1e-4 (relative to max(1, |logit|)) of the plain logits.
bfloat16 engine: per position, the root mean square of the difference (mean taken off) is held
against the spread of the plain logits.  Unit roundoff 2^-9, some dozens of roundings on the way to a
logit: about 2 % of the spread; the bound is 6 % and up to 3 % of the positions may exceed it (a lost
key, a wrong state or a stale page moves most positions by the order of the spread itself).
"""
import itertools
import json
import os

import pytest
import torch

import bifatar_models as BM
import helpers
import plain_bifatar as P

pytestmark = pytest.mark.gpu

NAMES = ("bif-a", "bif-b", "bif-c")
LENGTHS = {"bif-a": [1, 9, 47, 130, 300], "bif-b": [3, 64, 150, 257], "bif-c": [2, 33, 190]}
CASES = [(n, d) for n in NAMES for d in ("float32", "bfloat16")]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = BM.write_model(name, dtype, str(tmp_path_factory.mktemp(f"{name}_{dtype}")))
        return made[(name, dtype)]
    return get


@pytest.fixture(scope="module")
def oracle(folders):
    cache = {}

    def get(name, dtype, i):
        if (name, dtype, i) not in cache:
            cache[(name, dtype, i)] = BM.plain_logits(folders(name, dtype), tokens_of(name, i))
        return cache[(name, dtype, i)]
    return get


def tokens_of(name, i):
    return helpers.random_tokens(LENGTHS[name][i], BM.CONFIGS[name]["cfg"]["vocab"], 500 + i)


def replayer(folders, name, dtype, max_tokens, **kw):
    return helpers.Replayer(folders(name, dtype), dtype, max_tokens, BM.CONFIGS[name]["block_size"], **kw)


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
    if name == "bif-c":                     # (a group with a window gives pages back inside a step: its record of
        assert r.stray_writes() == []       # pages held is incomplete, so only the windowless model is checked)


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_against_token_by_token(name, dtype, folders, oracle):
    """The second request token by token from its first token on (the states start at zero, the first
    tokens have no earlier inputs for the convolutions and fewer keys than a window holds); the
    longest mostly as one portion, then 60 single tokens (windows pass over decoded tokens)."""
    r = replayer(folders, name, dtype, 320)
    toks, ref = tokens_of(name, 1), oracle(name, dtype, 1)
    outs = [r.step([dict(id="x", tokens=[t], want=[0])]) for t in toks]
    close(torch.cat(outs), ref, dtype, f"{name} token by token")
    r.session.release("x")
    i = len(LENGTHS[name]) - 1
    toks, ref = tokens_of(name, i), oracle(name, dtype, i)
    head = len(toks) - 60
    outs = [r.step([dict(id="y", tokens=toks[:head], want=list(range(head)))])]
    outs += [r.step([dict(id="y", tokens=[t], want=[0])]) for t in toks[head:]]
    close(torch.cat(outs), ref, dtype, f"{name} prefill then 60 single tokens")


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
    """Up to three live requests in a pool that cannot hold all requests at once and with three state
    slots: some requests bring a portion while others bring one token; a request that ends gives its pages and its
    slot to the next one, which must start from zero state."""
    B = BM.CONFIGS[name]["block_size"]
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

def one_layer_model(tmp_path, layer, dtype="float32", width=48, vocab=120, eps=3e-6, seed=5):
    cfg = {"architecture": "Bifatar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": [layer]}
    return BM.write_model_from(cfg, seed, dtype, str(tmp_path / "m"))


ALONE = [
    {"type": "attention", "mixer": BM._attn(4, 2, 12, 20, 0.5, (100.0, 6), 21, 4.0, True), "mlp": None},
    {"type": "attention", "mixer": BM._attn(2, 1, 16, 8, 0.3, None, None, None, None), "mlp": BM._dense(40)},
    {"type": "mamba2", "mixer": {"heads": 4, "vdim": 6, "state": 10, "groups": 2, "conv": 4, "norm_groups": 3}, "mlp": None},
    {"type": "mamba2", "mixer": {"heads": 3, "vdim": 8, "state": 36, "groups": 1, "conv": 2, "norm_groups": 1},
     "mlp": BM._dense(16)},
    {"type": "parallel", "mixer": {"left": BM._attn(3, 1, 8, 12, 0.4, (50.0, 8)),
                                   "right": {"heads": 2, "kv_heads": 1, "dim": 10, "vdim": 14, "conv": 3, "decay_rank": 4,
                                             "gate_rank": 9},
                                   "left_scale": 0.5, "right_scale": 1.5}, "mlp": None},
]


@pytest.mark.parametrize("layer", ALONE, ids=lambda l: l["type"])
def test_one_layer_alone(tmp_path, layer):
    """One layer of each kind (and the feed-forward with it or without) in float32: whole, and in portions
    with single tokens at the end."""
    folder = one_layer_model(tmp_path, layer)
    cfg, w = BM.read_model(folder)
    toks = helpers.random_tokens(90, 120, 77)
    ref = P.forward(cfg, w, toks)
    r = helpers.Replayer(folder, "float32", 128, 16)
    close(r.step([dict(id="a", tokens=toks, want=list(range(90)))], end=["a"]), ref, "float32", "whole")
    outs = [r.step([dict(id="b", tokens=toks[:2], want=[0, 1])]), r.step([dict(id="b", tokens=toks[2:41], want=list(range(39)))]),
            r.step([dict(id="b", tokens=toks[41:80], want=list(range(39)))])]
    outs += [r.step([dict(id="b", tokens=[t], want=[0])]) for t in toks[80:]]
    close(torch.cat(outs), ref, "float32", "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [
    {"type": "attention", "mixer": BM._attn(8, 2, 128, 128, 0.05, (10000.0, 64), 100, 15.0, True), "mlp": None},
    {"type": "attention", "mixer": BM._attn(4, 4, 64, 48, 0.08, (10000.0, 64), 300, None, None), "mlp": None},
    {"type": "attention", "mixer": BM._attn(20, 1, 32, 32, 0.2, (10000.0, 16), 64, 50.0, None), "mlp": None},
    {"type": "mamba2", "mixer": {"heads": 8, "vdim": 64, "state": 128, "groups": 2, "conv": 4, "norm_groups": 2}, "mlp": None},
    {"type": "parallel", "mixer": {"left": BM._attn(4, 2, 128, 96, 0.06, (10000.0, 32)),
                                   "right": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 24,
                                             "gate_rank": 20},
                                   "left_scale": 1.0, "right_scale": 1.0}, "mlp": BM._dense(512)},
], ids=["attn128", "attn64_48", "attn20heads", "ssm128", "side_by_side128"])
def test_mixers_at_the_sizes_of_the_fast_kernels(tmp_path, layer, dtype):
    """Head and state sizes that take the tensor-core attention kernels and the wide forms of the
    recurrence kernel, in a prompt of three portions and 70 decoded tokens, beside a second request."""
    folder = one_layer_model(tmp_path, layer, dtype, width=256, vocab=200)
    cfg, w = BM.read_model(folder)
    toks, other = helpers.random_tokens(420, 200, 3), helpers.random_tokens(150, 200, 4)
    ref, ref2 = P.forward(cfg, w, toks), P.forward(cfg, w, other)
    r = helpers.Replayer(folder, dtype, 640, 16)
    outs = [r.step([dict(id="a", tokens=toks[:200], want=list(range(200)))]),
            r.step([dict(id="a", tokens=toks[200:203], want=[0, 1, 2]), dict(id="b", tokens=other[:100], want=list(range(100)))])]
    o2 = [outs[1][3:]]
    outs[1] = outs[1][:3]
    outs.append(r.step([dict(id="a", tokens=toks[203:350], want=list(range(147)))]))
    for k, t in enumerate(toks[350:]):
        e = [dict(id="a", tokens=[t], want=[0])]
        if k < 50:
            e.append(dict(id="b", tokens=[other[100 + k]], want=[0]))
        out = r.step(e)
        outs.append(out[:1])
        if k < 50:
            o2.append(out[1:])
    close(torch.cat(outs), ref, dtype, "first request")
    close(torch.cat(o2), ref2, dtype, "second request")


# ------------------------------------------------------------ one key that carries all the weight

def plant(tmp_path, dtype, kind, window):
    """A one-layer model in which every query points at the key of ONE token (id 119, used once per
    prompt): the key direction lives in head dimensions that the rotation leaves alone, so the score of
    that key is the largest possible at every distance and all others are near zero.  Losing the key,
    or seeing it one position too long, changes the logits completely."""
    D, H, G, dk, dv = 48, 2, 1, 16, 12
    if kind == "attention":
        layer = {"type": "attention", "mixer": BM._attn(H, G, dk, dv, 1.0, (100.0, 8), window, 40.0, True), "mlp": None}
        p = "l0.mix."
    else:
        layer = {"type": "parallel", "mixer": {"left": BM._attn(H, G, dk, dv, 1.0, (100.0, 8)),
                                               "right": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 2,
                                                         "decay_rank": 4, "gate_rank": 4},
                                               "left_scale": 1.0, "right_scale": 0.05}, "mlp": None}
        p = "l0.mix.left."
    folder = one_layer_model(tmp_path, layer, dtype)
    cfg, w = BM.read_model(folder)
    g = torch.Generator().manual_seed(9)
    w["embed"] = torch.randn(120, D, generator=g, dtype=torch.float64) * 0.3
    w["embed"][:, :2] = 0
    w["embed"][:, 1] = 2.0                       # every token has the common component along coordinate 1
    w["embed"][119] = 0
    w["embed"][119, 0] = 6.0                     # the planted token lies along coordinate 0
    w["l0.norm1"] = torch.ones(D, dtype=torch.float64)
    w["l0.norm1.b"] = torch.zeros(D, dtype=torch.float64)
    w["l0.norm1.alpha"] = torch.tensor(0.5, dtype=torch.float64)
    wk = torch.randn(G * dk, D, generator=g, dtype=torch.float64) * 0.02
    wk[:, :2] = 0
    wk[12:16] = 0                                # no other token's key reaches into dimensions 12..15 (not rotated) ...
    wk[12:16, 0] = 1.0                           # ... which hold the planted token's key
    wq = torch.zeros(H * dk, D, dtype=torch.float64)
    for h in range(H):
        wq[h * dk + 12:h * dk + 16, 1] = 1.0     # every query: the same dimensions
    w[p + "q"], w[p + "k"] = wq, wk
    if kind != "attention":
        for n in ("q.b", "k.b", "v.b"):
            w[p + n] = torch.zeros_like(w[p + n])
        w[p + "q.norm"] = torch.ones_like(w[p + "q.norm"])
        w[p + "k.norm"] = torch.ones_like(w[p + "k.norm"])
    BM.save_weights(folder, w, dtype)
    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind,window", [("attention", 40), ("attention", 33), ("parallel", 0)])
def test_one_key_that_stands_out(tmp_path, dtype, kind, window):
    """The planted key is tried as first key, just before, at and behind page borders, and far back; the
    asking positions are in a prompt's portion and decoded alone.  With a window the positions just
    inside it (distance window - 1) and just outside (distance window) are among them, in the portion
    for some plants and among the decoded tokens for others; the check that the plant works compares
    exactly these two positions in the plain implementation."""
    folder = plant(tmp_path, dtype, kind, window)
    cfg, w = BM.read_model(folder)
    n, head = 200, 120
    for far in (0, 15, 16, 17, 31, 32, 79, 81, 100, 150):
        toks = helpers.random_tokens(n, 119, 40 + far)
        toks[far] = 119
        ref = P.forward(cfg, w, toks)
        r = helpers.Replayer(folder, dtype, 256, 16)
        outs = [r.step([dict(id="f", tokens=toks[:far + 1], want=list(range(far + 1)))])]
        if far + 1 < head:
            outs.append(r.step([dict(id="f", tokens=toks[far + 1:head], want=list(range(head - far - 1)))]))
        outs += [r.step([dict(id="f", tokens=[t], want=[0])]) for t in toks[max(head, far + 1):]]
        close(torch.cat(outs), ref, dtype, f"planted key at {far}")
        spread = ref.std().item()
        toks2 = list(toks)
        toks2[far] = 5
        without = P.forward(cfg, w, toks2)
        last_in = min(n - 1, far + window - 1) if window else n - 1
        if last_in > far:                         # the key is seen up to here and carries the weight
            assert (without[last_in] - ref[last_in]).abs().max().item() > 0.5 * spread
        if window and far + window < n:           # and not one position later
            assert (without[far + window] - ref[far + window]).abs().max().item() < 1e-6 * max(1.0, spread)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, folders, oracle):
    """A short prompt, then 260 tokens one by one: the states are read and written 260 times, the pages
    grow across many borders and every window passes over decoded tokens."""
    name = "bif-a"
    toks, ref = tokens_of(name, 4), oracle(name, dtype, 4)
    r = replayer(folders, name, dtype, 320)
    outs = [r.step([dict(id="d", tokens=toks[:40], want=list(range(40)))])]
    outs += [r.step([dict(id="d", tokens=[t], want=[0])]) for t in toks[40:]]
    close(torch.cat(outs), ref, dtype, "long decoding")


# --------------------------------------------------------------------------------- kernels alone

def test_tanh_norm_kernel_with_three_pending_outputs():
    from kvcm.kernels import library as K
    g = torch.Generator().manual_seed(1)
    for hidden in (40, 37):
        x = torch.randn(9, hidden, generator=g).cuda()
        pend = [(torch.randn(9, hidden, generator=g).cuda(), s) for s in (0.7, 1.0, -1.3)]
        w, b = torch.randn(hidden, generator=g).cuda(), torch.randn(hidden, generator=g).cuda()
        alpha = torch.tensor([0.8]).cuda()
        for dtype in (torch.float32, torch.bfloat16):
            xs, out = x.clone(), torch.empty(9, hidden, dtype=dtype, device="cuda")
            K.dyt_norm(xs, pend, w, b, alpha, out)
            total = x.double() + sum(s * t.double() for t, s in pend)
            ref = P.dyt(total.cpu(), w.cpu(), b.cpu(), alpha.cpu()[0])
            assert (xs.double().cpu() - total.cpu()).abs().max().item() < 1e-5
            assert (out.double().cpu() - ref).abs().max().item() < (1e-5 if dtype == torch.float32 else 0.03)
            rows = torch.tensor([7, 2], dtype=torch.int32, device="cuda")
            xs2, out2 = x.clone(), torch.empty(2, hidden, dtype=dtype, device="cuda")
            K.dyt_norm(xs2, pend, w, b, alpha, out2, rows)
            assert torch.equal(xs2, x) and torch.equal(out2, out[[7, 2]])


def test_squared_relu_in_the_streaming_product():
    """The up product of a decode step applies the activation in its epilogue: the same bits as the product
    followed by the activation kernel."""
    from kvcm.kernels import library as K
    g = torch.Generator().manual_seed(2)
    for M, N, Kd in ((1, 336, 128), (8, 1000, 256), (13, 64, 512)):
        x = torch.randn(M, Kd, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(N, Kd, generator=g) * Kd ** -0.5).to(torch.bfloat16).cuda()
        if not K.stream_gemm_supported(M, N, Kd):
            continue
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        K.gemm_stream(x, w, y)
        K.relu_sq(y, y)
        z = torch.empty_like(y)
        K.gemm_stream_relu_sq(x, w, z)
        assert torch.equal(y, z)
        ref = torch.relu(x.double() @ w.double().T) ** 2
        assert (z.double() - ref).abs().max().item() < 0.05 * max(1.0, ref.abs().max().item())


def test_capped_attention_with_a_sink_in_every_kernel():
    """The tensor-core attention kernels (decode in one block, split over a cluster, split through scratch
    memory; prefill) against the plain kernel, with a cap, a sink and a window."""
    from kvcm.kernels import library as K
    import bifatar_models  # noqa: F401
    layer = {"type": "attention", "mixer": BM._attn(8, 2, 64, 64, 0.2, (10000.0, 64), 700, 6.0, None), "mlp": None}
    import tempfile
    folder = BM.write_model_from({"architecture": "Bifatar", "vocab": 64, "width": 64, "norm": {"eps": 1e-6}, "layers": [layer]},
                                 3, "bfloat16", tempfile.mkdtemp())
    toks = helpers.random_tokens(900, 64, 8)
    outs = {}
    for options in ({"attention": "plain"}, {"attn_parts": 1}, {"attn_parts": 4}, {"attn_parts": 4, "attn_merge": "kernel"},
                    {"attn_prefill": "mma"}):
        r = helpers.Replayer(folder, "bfloat16", 1024, 16, options=options)
        o = [r.step([dict(id="a", tokens=toks[:880], want=[100, 500, 879])])]
        o += [r.step([dict(id="a", tokens=[t], want=[0])]) for t in toks[880:]]
        outs[json.dumps(options)] = torch.cat(o)
    base = outs.pop(json.dumps({"attention": "plain"}))
    for name, o in outs.items():
        close(o, base, "bfloat16", name)


# -------------------------------------------------------------- the engine's own entry point

@pytest.mark.parametrize("name", ["bif-a", "bif-c"])
def test_greedy_generation_through_the_engine(name, folders):
    """Scheduler with chunked prefill and few sequences at a time; every generated token must be the
    plain implementation's choice given the tokens before it (ties within 2e-4 allowed)."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    folder = folders(name, "float32")
    cfg, w = BM.read_model(folder)
    B = BM.CONFIGS[name]["block_size"]
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
    """So few pages that running requests are evicted and computed again from their first token: the
    state slot is reset.  Same tokens as with room for all."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    folder = folders("bif-a", "bfloat16")
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
    name, dtype = "bif-b", "float32"
    toks, ref = tokens_of(name, 2), oracle(name, dtype, 2)
    other = tokens_of(name, 1)
    steps = [dict(step=0, entries=[dict(id="a", tokens=toks[:70], want=[0, 69])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=toks[70:72], want=[1]), dict(id="b", tokens=other, want=[63])], end=["b"]),
             dict(step=2, entries=[dict(id="a", tokens=toks[72:], want=[len(toks) - 73])], end=["a"])]
    out = helpers.run_trace_tool(folders(name, dtype), dtype, steps, 512, str(tmp_path / "out"), vocab_key="vocab")
    got = torch.cat([torch.from_numpy(out[0]), torch.from_numpy(out[1][:1]), torch.from_numpy(out[2])])
    close(got, ref[[0, 69, 71, len(toks) - 1]], dtype, "trace tool")
    close(torch.from_numpy(out[1][1:]), oracle(name, dtype, 1)[[63]], dtype, "trace tool, second request")

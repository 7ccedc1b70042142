"""Rakizen through the engine against the plain implementation (tests/plain/rakizen_plain.py): whole prompts, decoding
token by token, portions down to two tokens, unequal requests in one batch over pages that are used again, long decoding
across pages, windows and blocks of positions, the first tokens, keys far back and at the edges of every mask, greedy
generation through `LLM`, the replay program and the command line.  The configurations are made here; they differ from
each other in every size."""
import json
import os
import random
import subprocess

import numpy as np
import pytest
import torch

from conftest import ROOT
from plain import rakizen_plain as P

pytestmark = pytest.mark.gpu


def _two_map(heads, kv_heads, dim, vdim, size, diff, scale, softcap):
    return {"type": "attention", "mixer": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, diff=diff, scale=scale,
                                               softcap=softcap, mask=dict(size=size))}


def _windowed(heads, kv_heads, dim, vdim, size, rot_dims, base, scale, softcap):
    return {"type": "attention_2", "mixer": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, softcap=softcap,
                                                 mask=dict(size=size), rot=dict(dims=rot_dims, base=base))}


def _dense(layer, ff):
    return dict(layer, mlp={"kind": "dense", "ff": ff})


def _moe(layer, ff, experts, top, count=None, keep=None, scale=1.0):
    router = {"experts": experts, "top": top, "scale": scale}
    if count:
        router["groups"] = {"count": count, "keep": keep}
    return dict(layer, mlp={"kind": "moe", "expert": {"ff": ff}, "router": router})


def _none(layer):
    return dict(layer, mlp=None)


CONFIGS = {
    # the first two layers run twice; a layer without a feed-forward; a block of positions as long as a page, another that
    # is no multiple of it; a window shorter than three pages; groups of two experts; three query heads on one key head
    "A": dict(block_size=16, config={
        "architecture": "Rakizen", "vocab": 173, "width": 80, "norm": {"eps": 1e-5}, "loop": {"start": 0, "stop": 2, "times": 2},
        "layers": [_dense(_two_map(4, 2, 24, 40, 50, 0.25, 0.2, 20.0), 120),
                   _moe(_windowed(3, 1, 32, 16, 37, 8, 1000.0, 0.15, 12.0), 40, 8, 2, 4, 2, 1.5),
                   _none(_two_map(2, 2, 16, 16, 16, 0.1, 0.3, 8.0))]}),
    # no loop; head sizes the tensor-core kernels take; as many key heads as heads; every element rotated; experts without
    # groups; a window of one page; values as wide as keys in a two-map layer and narrower in a windowed one
    "B": dict(block_size=64, config={
        "architecture": "Rakizen", "vocab": 384, "width": 128, "norm": {"eps": 1e-6},
        "layers": [_moe(_windowed(4, 4, 64, 32, 64, 64, 10000.0, 0.125, 30.0), 64, 6, 3, None, None, 2.5),
                   _dense(_two_map(2, 1, 64, 64, 100, 0.5, 0.11, 50.0), 192),
                   _dense(_windowed(2, 1, 128, 64, 7, 2, 500000.0, 0.09, 5.0), 128),
                   _moe(_two_map(4, 4, 32, 96, 33, 0.8, 0.2, 15.0), 48, 4, 1, 4, 4)]}),
    # one head; nothing rotated; a window of one position (a token sees itself alone) and blocks of two; every expert a
    # group of its own, so a group's score is its one expert's; one expert chosen; the loop runs to the last layer three times
    "C": dict(block_size=32, config={
        "architecture": "Rakizen", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "loop": {"start": 1, "stop": 3, "times": 3},
        "layers": [_moe(_windowed(1, 1, 40, 24, 1, 0, 100.0, 0.15, 25.0), 48, 5, 1, 5, 3, 0.7),
                   _dense(_two_map(1, 1, 36, 20, 2, 0.3, 0.25, 6.0), 64),
                   _moe(_windowed(6, 2, 16, 16, 90, 16, 777.0, 0.3, 40.0), 33, 6, 3, 3, 2, 2.0)]}),
    # sizes that are no multiples of 8: width, vocabulary, head sizes, feed-forward and expert widths; the whole model is one
    # loop that runs twice; pages of 16 under a window of 17 and blocks of 15
    "D": dict(block_size=16, config={
        "architecture": "Rakizen", "vocab": 211, "width": 100, "norm": {"eps": 1e-6}, "loop": {"start": 0, "stop": 2, "times": 2},
        "layers": [_moe(_two_map(5, 5, 12, 28, 15, 0.35, 0.3, 9.0), 30, 9, 2, 3, 2, 1.2),
                   _dense(_windowed(3, 3, 20, 12, 17, 10, 3000.0, 0.22, 14.0), 150)]}),
}
NAMES = sorted(CONFIGS)
DTYPES = ["float32", "bfloat16"]
KEPT_FLOAT = ("norm", ".lq", ".lk", "router")


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: random_folders(tmp_path_factory.mktemp(f"rakizen_{name}"), spec["config"], 51 + k)
            for k, (name, spec) in enumerate(sorted(CONFIGS.items()))}


_models, _truth = {}, {}


def tokens_for(name, n, salt=0):
    g = torch.Generator().manual_seed(7001 * (NAMES.index(name) + 1) + salt)
    return torch.randint(0, CONFIGS[name]["config"]["vocab"], (n,), generator=g).tolist()


def as_held(w, dtype):
    """The weights as the engine holds them: matrices rounded to bfloat16 on that path; norms, the two-map factor's
    vectors and the routers stay float."""
    if dtype == "float32":
        return w
    return {k: (v if any(s in k for s in KEPT_FLOAT) or not v.dtype.is_floating_point else v.to(torch.bfloat16).to(v.dtype))
            for k, v in w.items()}


CLOSE_CALL = 0.02     # a router's choice that scores moved by this much would turn over is not held against bfloat16
TIE = 1e-6            # ... and one that this much would turn over not against 32 bits either


class Rows(np.ndarray):
    """Logits with, per row, whether some router's choice there was a close call (`unsure`) and how far rounding what the
    sublayers read and return to 16 bits moves the row, as a share of its spread (`moved`)."""


def to_16_bits(t):
    return t.to(torch.bfloat16).to(t.dtype)


def plain_logits(cfg, w, tokens):
    margins = []
    exact = P.forward(cfg, w, tokens, torch.float64, margins=margins).numpy()
    out = exact.view(Rows)
    least = torch.stack(margins).min(0).values.numpy() if margins else np.ones(len(tokens))
    out.unsure = least < CLOSE_CALL
    # a tie in 32 bits (two scores that only float64 tells apart, as where both sigmoids are all but 1): from that row on
    # the two runs may have taken different experts, and later rows read what that row left
    ties = np.nonzero(least < TIE)[0]
    out.sure_rows = int(ties[0]) if len(ties) else len(tokens)
    rounded = P.forward(cfg, w, tokens, torch.float64, noise=to_16_bits).numpy()
    out.moved = np.sqrt(((rounded - exact) ** 2).mean(-1)) / exact.std(-1)
    return out


# A random router's scores lie close together, and rounding to bfloat16 turns a choice over every few dozen tokens; the
# other expert's output then goes into keys that later tokens read.  So the two precisions get folders of their own,
# equal but for the routers' matrices: times five for the 32-bit runs (choices that differ from token to token, held
# exactly), times 0.02 for bfloat16 (all scores near one half: what is held there is the arithmetic in 16 bits, and
# rows where the plain run calls a choice close are left out).  tests/test_gpu_rakizen_parts.py routes varied tokens in
# bfloat16 too, on inputs that both sides share.
ROUTER_FACTOR = {"float32": 5.0, "bfloat16": 0.02}


def random_folders(folder, config, seed):
    """{dtype: folder} of one random model."""
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    from vllm_oxide_b200.weights.safetensors_io import write_safetensors
    out = {}
    for dtype, factor in ROUTER_FACTOR.items():
        out[dtype] = os.path.join(str(folder), dtype)
        write_random_model_folder(out[dtype], config, seed, "fan_in", torch.float32)
        _, w = P.read_folder(out[dtype])
        write_safetensors(os.path.join(out[dtype], "model.safetensors"),
                          {k: (factor * v if k.endswith("router") else v) for k, v in w.items()})
    return out


def truth(folders, name, tokens, dtype):
    key = (name, tuple(tokens), dtype)
    if key not in _truth:
        if (name, dtype) not in _models:
            cfg, w = P.read_folder(folders[name][dtype])
            _models[(name, dtype)] = (cfg, as_held(w, dtype))
        _truth[key] = plain_logits(*_models[(name, dtype)], tokens)
    return _truth[key]


def close(got, want, dtype, what):
    """float32: within 1e-4 of the logits' spread, row by row (rounding alone stays near 1e-6; a wrong key, gate, expert or
    mask moves a row by percents).  bfloat16: within 0.1 of it, wider where the plain run itself moves when its sublayers
    round to 16 bits, and except for rows where the plain run says that a router's choice was a close call."""
    unsure, moved, sure_rows = getattr(want, "unsure", None), getattr(want, "moved", None), getattr(want, "sure_rows", None)
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, what
    err = np.sqrt(((got - want) ** 2).mean(-1)) / want.std(-1)
    if dtype == "float32":
        if sure_rows is not None and len(unsure) == len(err):
            err = err[:sure_rows]
        if len(err) == 0:
            return
        assert err.max() < 1e-4, f"{what}: row {int(err.argmax())} is {err.max():.3e} of the spread off"
        return
    sure = np.ones(len(err), bool) if unsure is None or len(unsure) != len(err) else ~unsure
    bound = 0.1 + 5.0 * moved if moved is not None and len(moved) == len(err) else np.full(len(err), 0.1)
    worst = np.where(sure, err / bound, 0.0)
    assert worst.max() < 1.0, f"{what}: row {int(worst.argmax())} is {err[worst.argmax()]:.3e} of the spread off"
    if len(err) >= 8:
        assert np.median(err) < 0.04, f"{what}: half of the rows are more than {np.median(err):.3e} of the spread off"
        assert np.median(bound) < 0.3, f"{what}: the plain run itself does not hold under rounding"


def pick(rows, which):
    out = np.asarray(rows)[which].view(Rows)
    out.unsure, out.moved = rows.unsure[which], rows.moved[which]
    return out


def runner(folders, name, dtype, max_tokens, max_live=4):
    from vllm_oxide_b200.engine.trace import TraceRunner
    return TraceRunner(folders[name][dtype], dtype, max_tokens, CONFIGS[name]["block_size"], max_live=max_live)


def feed(r, rid, tokens, cuts):
    """Feeds `tokens` in portions of the sizes `cuts` (cycled); logits at every position."""
    rows, at, k = [], 0, 0
    while at < len(tokens):
        n = min(cuts[k % len(cuts)], len(tokens) - at)
        k += 1
        end = [rid] if at + n == len(tokens) else []
        rows.append(r.step([{"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))}], end))
        at += n
    return np.concatenate(rows, 0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_then_decoded_then_in_portions(folders, name, dtype):
    toks = tokens_for(name, 150)
    want = truth(folders, name, toks, dtype)
    r = runner(folders, name, dtype, 256)
    whole = feed(r, "w", toks, [len(toks)])
    close(whole, want, dtype, f"{name} {dtype} whole")
    decoded = feed(r, "d", toks, [len(toks) - 60] + [1] * 60)
    close(decoded, want, dtype, f"{name} {dtype} last 60 tokens one by one")
    for cuts in ([2], [3, 1, 17, 2, 64, 5], [CONFIGS[name]["block_size"]], [1, 2]):
        got = feed(r, "p", toks, cuts)
        close(got, want, dtype, f"{name} {dtype} portions {cuts}")
        if dtype == "float32":
            assert np.abs(got - whole).max() <= 1e-5 * np.abs(whole).max(), f"{name} portions {cuts} against whole"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first(folders, name, dtype):
    toks = tokens_for(name, 120, salt=5)
    r = runner(folders, name, dtype, 128)
    close(feed(r, "t", toks, [1]), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} every token alone")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_of_a_sequence(folders, name, dtype):
    r = runner(folders, name, dtype, 64)
    for n in (1, 2, 3, 4, 6):
        toks = tokens_for(name, n, salt=40 + n)
        close(feed(r, f"f{n}", toks, [n]), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} a prompt of {n}")
        close(feed(r, f"g{n}", toks, [1]), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} {n} single tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_requests_in_one_batch_over_pages_used_again(folders, name, dtype):
    """Nine requests, at most three live, over a pool that holds far less than all of them: portions of some beside single
    tokens of others; a finished request's pages go to the next one."""
    rng = random.Random(NAMES.index(name))
    bs = CONFIGS[name]["block_size"]
    lengths = [70, 1, 33, 130, 2, 64, 97, 18, 150]
    reqs = {f"q{i}": tokens_for(name, n, salt=100 + i) for i, n in enumerate(lengths)}
    live_cap = 3
    pool = sum(sorted(((n + bs - 1) // bs * bs for n in lengths), reverse=True)[:live_cap])
    r = runner(folders, name, dtype, pool, max_live=live_cap)
    free_pages = lambda: [r.manager.num_free_blocks(g) for g in range(r.manager.num_groups)]
    free_at_start = free_pages()
    waiting, live, at, got = list(reqs), [], {}, {k: [] for k in reqs}
    while waiting or live:
        while waiting and len(live) < live_cap:
            live.append(waiting.pop(0))
            at[live[-1]] = 0
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                              # left out of this step, goes on later
            left = len(reqs[rid]) - at[rid]
            n = min(left, rng.choice([1, 1, 2, 3, 7, bs, bs + 5, 40]))
            entries.append({"id": rid, "tokens": reqs[rid][at[rid]:at[rid] + n], "want": list(range(n))})
            at[rid] += n
            if at[rid] == len(reqs[rid]):
                end.append(rid)
                live.remove(rid)
        if not entries:
            continue
        out = r.step(entries, end)
        k = 0
        for e in entries:
            got[e["id"]].append(out[k:k + len(e["tokens"])])
            k += len(e["tokens"])
    assert free_pages() == free_at_start, "every page came back"
    for rid, toks in reqs.items():
        close(np.concatenate(got[rid], 0), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} request {rid} in mixed batches")


def random_configuration(seed):
    """A configuration drawn from a seeded generator: two to four layers of either kind in any order, head counts, key and
    value sizes (equal, unequal, multiples of 16 or not), masks shorter and longer than a page, any part of a head
    rotated, every kind of feed-forward, a loop or none."""
    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(2, 4)):
        kv = rng.choice([1, 2, 3])
        heads = kv * rng.choice([1, 2, 4])
        dim = rng.choice([8, 16, 24, 32, 48, 64])
        vdim = rng.choice([dim, dim, 2 * dim, rng.choice([8, 16, 40, 64])])
        size, scale, cap = rng.choice([1, 5, 16, 23, 64, 100, 400]), rng.choice([0.05, 0.15, 0.3]), rng.choice([0.0, 4.0, 20.0, 50.0])
        if rng.random() < 0.5:
            layer = _two_map(heads, kv, dim, vdim, size, rng.choice([0.1, 0.4, 0.7]), scale, cap)
        else:
            layer = _windowed(heads, kv, dim, vdim, size, rng.choice([0, 2, dim // 2, dim]), rng.choice([100.0, 1e4, 1e6]), scale, cap)
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            layer = _none(layer)
        elif kind == "dense":
            layer = _dense(layer, rng.choice([24, 64, 100]))
        else:
            count = rng.choice([None, 1, 2, 3])
            per = rng.choice([1, 2, 3])
            experts = (count or 1) * per if count else rng.choice([3, 5, 8])
            keep = rng.randint(1, count) if count else None
            top = rng.randint(1, max(1, min(3, per * keep if count else experts)))
            layer = _moe(layer, rng.choice([8, 24, 40]), experts, top, count, keep, rng.choice([1.0, 2.5]))
        layers.append(layer)
    cfg = {"architecture": "Rakizen", "vocab": rng.choice([61, 128, 300]), "width": rng.choice([32, 48, 72, 128]),
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.6:
        start = rng.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": start, "stop": rng.randint(start + 1, len(layers)), "times": rng.randint(1, 3)}
    return cfg, rng.choice([16, 32, 64])


@pytest.mark.parametrize("seed", range(24))
def test_random_configurations(seed, tmp_path):
    from vllm_oxide_b200.engine.trace import TraceRunner
    cfg, page = random_configuration(1000 + seed)
    dirs = random_folders(tmp_path, cfg, seed)
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, cfg["vocab"], (140,), generator=g).tolist()
    for dtype in DTYPES:
        c, w = P.read_folder(dirs[dtype])
        want = plain_logits(c, as_held(w, dtype), toks)
        r = TraceRunner(dirs[dtype], dtype, 192, page, max_live=2)
        for cuts in ([len(toks)], [len(toks) - 30] + [1] * 30, [3, 1, 17, 2, 40]):
            close(feed(r, "x", toks, cuts), want, dtype, f"random configuration {seed}, {dtype}, cuts {cuts[:5]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_across_pages_windows_and_blocks(folders, dtype):
    for name in ("A", "C"):
        toks = tokens_for(name, 330, salt=9)
        r = runner(folders, name, dtype, 384)
        close(feed(r, "l", toks, [6] + [1] * 324), truth(folders, name, toks, dtype), dtype, f"{name} {dtype} 324 decoded tokens")


def _loud_model(tmp_path, layer, seed):
    """A model of one layer in which token 45's key and token 46's query point the same way and tower over the rest (both
    tokens appear where the test puts them and nowhere else): the row behind a query token hangs on whether a key token is
    visible to it."""
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    from vllm_oxide_b200.weights.safetensors_io import write_safetensors
    cfg = {"architecture": "Rakizen", "vocab": 50, "width": 64, "norm": {"eps": 1e-6}, "layers": [_none(layer)]}
    write_random_model_folder(str(tmp_path), cfg, seed, "fan_in", torch.float32)
    cfg, w = P.read_folder(str(tmp_path))
    g = torch.Generator().manual_seed(seed + 5)
    d_key, d_query = torch.nn.functional.normalize(torch.randn(2, 64, generator=g), dim=-1)
    w["embed"][45], w["embed"][46] = 8.0 * d_key, 8.0 * d_query
    w["l0.norm1"].fill_(1.0)
    w["l0.norm1.b"].zero_()
    m = layer["mixer"]
    row = m["dim"] - 1                        # the last element of the first head (of its first map): never rotated here
    w["l0.mix.k"][row], w["l0.mix.q"][row] = 3.0 * d_key, 3.0 * d_query
    if "l0.mix.q.norm" in w:
        w["l0.mix.q.norm"].fill_(1.0)
        w["l0.mix.k.norm"].fill_(1.0)
    write_safetensors(str(tmp_path / "model.safetensors"), w)
    return cfg, w


def _edge_case(cfg, w, dtype, toks, query_at, key_at, seen, what):
    """The plain model's row at `query_at` moves when the token at `key_at` is another one if and only if `seen`."""
    want = P.forward(cfg, as_held(w, dtype), toks, torch.float64).numpy()
    other = list(toks)
    other[key_at] = 44
    gap = np.abs(P.forward(cfg, as_held(w, dtype), other, torch.float64).numpy()[query_at] - want[query_at]).max()
    if seen:
        assert gap > 0.2 * want[query_at].std(), f"{what}: the plain row hangs on the key"
    else:
        assert gap == 0.0, f"{what}: the plain row does not see the key"
    return want


@pytest.mark.parametrize("kind", ["window", "block"])
def test_keys_far_away_and_at_the_edges_of_a_mask(kind, tmp_path):
    """The loud key sits just inside and just outside the window or the block of the loud query, far back inside it, and
    at a page border; the query comes in a prompt's portion or decoded alone.  The engine follows the plain model in every
    cut (a key one position off would move the row by more than a fifth of its spread)."""
    from vllm_oxide_b200.engine.trace import TraceRunner
    size, page = (300, 64) if kind == "window" else (320, 64)
    layer = (_windowed(2, 1, 64, 48, size, 16, 10000.0, 1.0, 30.0) if kind == "window"
             else _two_map(2, 1, 64, 48, size, 0.2, 1.0, 30.0))
    cfg, w = _loud_model(tmp_path, layer, 3 if kind == "window" else 4)
    n = 700 if kind == "window" else 2 * size + 280
    query_at = n - 1 if kind == "window" else 2 * size + 250      # the block case: position 250 of the third block
    first = query_at - size + 1 if kind == "window" else 2 * size
    cases = [(first, True, "the first key that is seen"), (first - 1, False, "the key before it"),
             (first + 37, True, "far back, seen"), (first - 1 - page, False, "a page further out"),
             (query_at - 1, True, "the key next to the query")]
    if kind == "window":
        cases.append((first // page * page + page, True, "the first key of a page inside the window"))
    for dtype in DTYPES:
        r = TraceRunner(str(tmp_path), dtype, 1024, page, max_live=2)
        for key_at, seen, what in cases:
            toks = [1 + (i % 40) for i in range(n)]
            toks[key_at], toks[query_at] = 45, 46
            want = _edge_case(cfg, w, dtype, toks, query_at, key_at, seen, f"{kind} {what}")
            for cuts in ([n], [query_at, 1] + [n], [100, 2, 64], [key_at + 1, query_at - key_at - 1, 1, n], [query_at - 1, 2, n]):
                cuts = [c for c in cuts if c > 0]
                close(feed(r, "x", toks, cuts), want, dtype, f"{kind}, {what}, {dtype}, cuts {cuts}")


def test_the_cap_bends_large_scores(tmp_path):
    """With a small cap the loud score is bent far below its plain value: a kernel that left the cap out would put all
    weight on one key; with it the other keys keep a share."""
    from vllm_oxide_b200.engine.trace import TraceRunner
    cfg, w = _loud_model(tmp_path, _windowed(2, 1, 64, 32, 64, 0, 1.0, 1.0, 2.0), 9)
    toks = [1 + (i % 40) for i in range(60)]
    toks[20], toks[-1] = 45, 46
    want = P.forward(cfg, w, toks, torch.float64).numpy()
    uncapped = json.loads(json.dumps(cfg))
    uncapped["layers"][0]["mixer"]["softcap"] = 0.0
    assert np.abs(P.forward(uncapped, w, toks, torch.float64).numpy()[-1] - want[-1]).max() > 0.2 * want[-1].std()
    for dtype in DTYPES:
        wt = P.forward(cfg, as_held(w, dtype), toks, torch.float64).numpy()
        r = TraceRunner(str(tmp_path), dtype, 128, 16, max_live=2)
        for cuts in ([60], [59, 1], [7]):
            close(feed(r, "x", toks, cuts), wt, dtype, f"cap, {dtype}, cuts {cuts}")


def plain_greedy(folders, name, prompt, new):
    toks = list(prompt)
    for _ in range(new):
        toks.append(int(truth(folders, name, toks, "float32")[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_engine(folders, name):
    """`LLM.generate`: the scheduler cuts prompts to its token budget, batches them with decoding requests and preempts
    when the pool runs dry; the tokens are the plain implementation's."""
    from vllm_oxide_b200 import LLM, EngineOptions, SamplingParams
    bs = CONFIGS[name]["block_size"]
    llm = LLM(folders[name]["float32"], EngineOptions(dtype="float32", block_size=bs, num_kv_blocks=max(6, 320 // bs), max_num_seqs=3,
                                                      max_num_batched_tokens=48, max_model_len=256))
    prompts = [tokens_for(name, n, salt=300 + n) for n in (5, 61, 1, 100, 17)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders, name, p, 10), f"{name}: a prompt of {len(p)}"
    outs = llm.generate(prompts[:2], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders, name, p, 10)[:4]


def test_bfloat16_generation_runs_from_graphs_and_agrees_where_the_plain_run_is_sure(folders):
    from vllm_oxide_b200 import LLM, EngineOptions, SamplingParams
    name = "B"
    llm = LLM(folders[name]["bfloat16"], EngineOptions(dtype="bfloat16", block_size=64, num_kv_blocks=16, max_num_seqs=4, max_model_len=512))
    prompts = [tokens_for(name, n, salt=500 + n) for n in (9, 70, 130)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))
    assert llm.core.graph_replays > 0
    for p, o in zip(prompts, outs):
        toks = list(p)
        for t in o.token_ids:
            row = truth(folders, name, toks, "bfloat16")[-1]
            top = np.sort(row)[-2:]
            if top[1] - top[0] < 0.1 * row.std():
                break                                  # too close to call in bfloat16: the runs may part here
            assert t == int(row.argmax())
            toks.append(t)


def test_the_replay_program(folders, tmp_path):
    name = "A"
    toks = tokens_for(name, 50, salt=77)
    other = tokens_for(name, 21, salt=78)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[30:32], "want": []}, {"id": "b", "tokens": other, "want": [20]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[32:], "want": [17]}], "end": ["a"]}]
    for dtype in DTYPES:
        out = tmp_path / dtype
        p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name][dtype], "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "128", "--block-size", "16"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=1200)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        want = truth(folders, name, toks, dtype)
        close(np.fromfile(out / "0.f32", "<f4").reshape(2, -1), pick(want, [0, 29]), dtype, "step 0")
        close(np.fromfile(out / "1.f32", "<f4").reshape(1, -1), pick(truth(folders, name, other, dtype), [20]), dtype, "step 1")
        close(np.fromfile(out / "2.f32", "<f4").reshape(1, -1), pick(want, [49]), dtype, "step 2")


def test_the_command_line(folders):
    name = "C"
    prompt = tokens_for(name, 9, salt=900)
    p = subprocess.run([os.path.join(ROOT, "bin", "vllm-oxide"), "-m", folders[name]["float32"], "--token-ids", " ".join(map(str, prompt)),
                        "--max-tokens", "6", "--dtype", "float32", "--ignore-eos", "--max-model-len", "128", "--block-size", "32",
                        "--num-kv-blocks", "16"], capture_output=True, text=True, timeout=1200)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.split()] == plain_greedy(folders, name, prompt, 6)

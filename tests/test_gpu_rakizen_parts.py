"""The mechanisms of Rakizen one by one: each part is built alone, given a cache of its own and stepped in portions, and
compared with its plain form (tests/plain/rakizen_plain.py).  Where random numbers would hide a fault the inputs are made
to show it: one key made so loud that a query sees almost nothing else, placed just inside and just outside a window or
a block of positions and at page borders; scores large enough for the cap to bend them; a router whose groups decide."""
import math

import pytest
import torch

from helpers import DEV, Alone, assert_close, held, in_portions, load, rand
from plain import rakizen_plain as P

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


# ---------------------------------------------------------------- the stream and its one norm
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("D", [64, 50, 33, 344, 4096, 8200])
def test_layer_norm_step(D, dt):
    from vllm_oxide_b200 import kernels
    n, eps = 7, 1e-5
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    x, y1, y2 = rand((n, D), 1, 3.0) + 2.0, held(rand((n, D), 2, 0.7), dt), held(rand((n, D), 3, 0.4), dt)
    w, b = 1.0 + 0.1 * rand((D,), 4), 0.3 * rand((D,), 5)
    f32 = lambda t: t.float().to(DEV).contiguous()
    act = lambda t: t.to(dt).to(DEV).contiguous()
    stream, out = f32(x), torch.empty((n, D), dtype=dt, device=DEV)
    kernels.layer_norm_step(stream, eps, err, y1=act(y1), y2=act(y2), w=f32(w), b=f32(b), out=out)
    want = x.float().double() + (y1 + y2)
    assert_close(stream, want, torch.float32, "the stream")
    norm = lambda t: P.layer_norm(t, w.float().double(), b.float().double(), eps)
    assert_close(out, norm(want), dt, "the layer's input")
    assert (norm(want) - P.layer_norm(want, w.float().double(), 0 * b, eps)).abs().max() > 0.1, "the bias shows"
    # one pending output, and none
    s1 = f32(x)
    kernels.layer_norm_step(s1, eps, err, y1=act(y1), w=f32(w), out=out)
    assert_close(s1, x.float().double() + y1, torch.float32, "one output")
    assert_close(out, P.layer_norm(x.float().double() + y1, w.float().double(), 0 * b, eps), dt, "no bias")
    s0 = f32(x)
    kernels.layer_norm_step(s0, eps, err, w=f32(w), b=f32(b), out=out)
    assert torch.equal(s0, f32(x))
    assert_close(out, norm(x.float().double()), dt, "the norm alone")
    # the start of a stream: what was there does not count
    s2 = torch.full((n, D), 7.0, dtype=torch.float32, device=DEV)
    kernels.layer_norm_step(s2, eps, err, y1=act(y1), w=f32(w), b=f32(b), out=out, init=True)
    assert_close(s2, y1, torch.float32, "a stream that begins")
    assert_close(out, norm(y1), dt, "its norm")
    # chosen rows only: nothing is stored
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    before, picked = stream.clone(), torch.empty((3, D), dtype=dt, device=DEV)
    kernels.layer_norm_step(stream, eps, err, y1=act(y1), y2=act(y2), w=f32(w), b=f32(b), out=picked, rows=rows, n_out=3)
    assert torch.equal(before, stream)
    assert_close(picked, norm(want + (y1 + y2))[[5, 0, 5]], dt, "rows")
    assert int(err.item()) == 0


# ---------------------------------------------------------------- attention
def capped_part(dt, D, kind, m):
    from vllm_oxide_b200.parts import PartSpec, build_part
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions, params = {}, dict(hidden_size=D, num_heads=H, num_kv_heads=G, dim=d, vdim=e, scale=m["scale"], softcap=m["softcap"],
                                 eps=1e-6, prefix="m.")
    maps = 2 if kind == "attention" else 1
    if kind == "attention":
        params.update(maps=2, diff=m["diff"], gate=True, chunk=m["mask"]["size"])
    else:
        rot = m.get("rot")
        if rot and rot["dims"]:
            positions["r"] = build_part("position", PartSpec("rope", dict(head_dim=d, rotary_dim=rot["dims"], max_position=1 << 30,
                                                                         theta=rot["base"], interleaved=True, table=False)), device=DEV)
        params.update(row_norm=True, position="r" if positions else None, window=m["mask"]["size"])
    part = build_part("mixer", PartSpec("attention_capped", params), positions=positions, dtype=dt, device=DEV)
    w = {"m.q": rand((H * maps * d, D), 1, D ** -0.5), "m.k": rand((G * maps * d, D), 2, D ** -0.5),
         "m.v": rand((G * e, D), 3, D ** -0.5), "m.o": rand((D, H * e), 4, (H * e) ** -0.5)}
    if kind == "attention":
        w["m.g"] = rand((H * e, D), 5, D ** -0.5)
        for i, nme in enumerate(("lq1", "lk1", "lq2", "lk2")):
            w["m." + nme] = rand((d,), 6 + i, 0.3)
    else:
        w["m.q.norm"], w["m.k.norm"] = 1.0 + 0.2 * rand((H * d,), 10), 1.0 + 0.2 * rand((G * d,), 11)
    return part, w


def hold(w, dt):
    return {k: (v.float().double() if k.endswith((".norm", "lq1", "lk1", "lq2", "lk2")) else held(v, dt)) for k, v in w.items()}


CASES = {
    # two maps, blocks of 50 positions over pages of 16, values wider than keys, two heads a key head
    "two maps": ("attention", 40, dict(heads=4, kv_heads=2, dim=24, vdim=40, diff=0.3, scale=0.25, softcap=15.0, mask={"size": 50})),
    # one key head for three, values narrower than keys, a block as long as a page
    "two maps, one key head": ("attention", 48, dict(heads=3, kv_heads=1, dim=32, vdim=16, diff=0.1, scale=0.2, softcap=8.0, mask={"size": 16})),
    # as many key heads as heads, equal sizes, a block of one position more than two pages, no cap
    "two maps, no cap": ("attention", 32, dict(heads=2, kv_heads=2, dim=16, vdim=16, diff=0.5, scale=0.3, softcap=0.0, mask={"size": 33})),
    # a window of 37 over pages of 16, a quarter of the head rotated
    "window": ("attention_2", 40, dict(heads=3, kv_heads=1, dim=32, vdim=16, scale=0.5, softcap=10.0, mask={"size": 37},
                                       rot={"dims": 8, "base": 1000.0})),
    # the whole head rotated, values wider than keys, a window of one page
    "window, whole head rotated": ("attention_2", 64, dict(heads=4, kv_heads=2, dim=16, vdim=48, scale=0.7, softcap=30.0, mask={"size": 16},
                                                           rot={"dims": 16, "base": 50000.0})),
    # equal sizes that the tensor-core kernels take, nothing rotated, a window of one key
    "window of one": ("attention_2", 64, dict(heads=2, kv_heads=2, dim=64, vdim=64, scale=0.3, softcap=5.0, mask={"size": 1},
                                              rot={"dims": 0, "base": 1.0})),
    # equal head sizes of 64 and 128: in bfloat16 the tensor-core kernels run these (two key maps over one value head, blocks
    # that end inside a page and inside a 64-key tile; a window longer than two tiles)
    "two maps, 64 wide": ("attention", 64, dict(heads=4, kv_heads=2, dim=64, vdim=64, diff=0.3, scale=0.2, softcap=12.0, mask={"size": 50})),
    "two maps, 128 wide": ("attention", 48, dict(heads=3, kv_heads=1, dim=128, vdim=128, diff=0.6, scale=0.15, softcap=25.0, mask={"size": 72})),
    "window, 128 wide": ("attention_2", 64, dict(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.12, softcap=9.0, mask={"size": 141},
                                                 rot={"dims": 64, "base": 1e4})),
    # equal head sizes that the mma.sync kernels take in bfloat16: by cp.async (32, 96) and by TMA (192)
    "two maps, 32 wide": ("attention", 40, dict(heads=2, kv_heads=1, dim=32, vdim=32, diff=0.2, scale=0.3, softcap=10.0, mask={"size": 21})),
    "two maps, 192 wide": ("attention", 48, dict(heads=2, kv_heads=2, dim=192, vdim=192, diff=0.4, scale=0.1, softcap=18.0, mask={"size": 64})),
    "window, 96 wide": ("attention_2", 56, dict(heads=4, kv_heads=2, dim=96, vdim=96, scale=0.14, softcap=7.0, mask={"size": 45},
                                                rot={"dims": 48, "base": 2e4})),
    "window, 64 wide": ("attention_2", 64, dict(heads=4, kv_heads=1, dim=64, vdim=64, scale=0.4, softcap=20.0, mask={"size": 70},
                                                rot={"dims": 32, "base": 1e6})),
}
# Key and value sizes that the bfloat16 path pads to every other multiple of 16 up to 256 (the tensor-core kernels are
# compiled for one head size each), two maps and windows in turn.
for _i, (_d, _e) in enumerate([(100, 200), (72, 144), (110, 110), (150, 75), (170, 96), (220, 64), (230, 230), (90, 96), (250, 256)]):
    if _i % 2:
        CASES[f"padded {_d}/{_e}"] = ("attention_2", 40, dict(heads=2, kv_heads=1, dim=_d, vdim=_e, scale=_d ** -0.5, softcap=11.0,
                                                            mask={"size": 41 + _i}, rot={"dims": 2 * (_d // 4), "base": 3e3}))
    else:
        CASES[f"padded {_d}/{_e}"] = ("attention", 40, dict(heads=2, kv_heads=2, dim=_d, vdim=_e, diff=0.25, scale=_d ** -0.5,
                                                          softcap=14.0, mask={"size": 37 + _i}))


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("case", sorted(CASES))
def test_capped_attention_alone_with_loud_tokens(case, dt):
    kind, D, m = CASES[case]
    part, w = capped_part(dt, D, kind, m)
    load(part, w, dt)
    wh = hold(w, dt)
    bs, n, size = 16, 150, m["mask"]["size"]
    x = rand((n, D), 33)
    # loud tokens at the first position, on both sides of page borders, and on both sides of the mask's edges as seen from
    # the last query and from a query in the middle
    for j in {0, 15, 16, 31, 32, max(0, n - size - 1), max(0, n - size), (n - 1) // size * size, max(0, (n - 1) // size * size - 1),
              max(0, 100 - size), max(0, 101 - size)}:
        x[j] *= 4.0
    x = held(x, dt)
    plain = P.two_map_attention if kind == "attention" else P.window_attention
    want = plain(x, wh, "m.", m, 1e-6, torch.float64)
    # the plain form itself: the mask and the cap show
    wider = dict(m, mask={"size": size + 1})
    assert (plain(x, wh, "m.", wider, 1e-6, torch.float64) - want).abs().max() > 1e-3 * want.abs().max(), "one key more shows"
    if m["softcap"] and size > 1:      # one visible key: its weight is 1 whatever its score
        assert (plain(x, wh, "m.", dict(m, softcap=0.0), 1e-6, torch.float64) - want).abs().max() > 1e-3 * want.abs().max(), "the cap shows"
    tol = 2e-4 if dt == torch.float32 else 0.08
    alone = Alone([part], dt, block_size=bs, pages=4 * (n // bs + 1), slots=3)
    for cuts, what in (([n], "whole"), ([n - 60] + [1] * 60, "decoded"), ([2, 5, 1, 30, 3], "portions"), ([bs], "pages"), ([1], "alone"),
                       ([size, 1], "cut at the mask's size")):
        assert_close(in_portions(alone, 7, x, cuts), want, dt, f"{case}: {what}", tol)
    other = held(rand((120, D), 34), dt)
    o_want = plain(other, wh, "m.", m, 1e-6, torch.float64)
    a = alone.step([(1, x[:90]), (2, other[:119])])[0]
    b = alone.step([(2, other[119:]), (1, x[90:])], end=[1, 2])[0]
    assert_close(torch.cat([a[:90], b[1:]]), want, dt, f"{case}: beside another request", tol)
    assert_close(torch.cat([a[90:], b[:1]]), o_want, dt, f"{case}: the other request", tol)
    # every page came back (those behind a window or a block went back on the way)
    assert alone.m.num_free_blocks(0) == 4 * (n // bs + 1)


@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_one_key_inside_or_outside_the_mask_decides(kind):
    """Query and key projections are made so that the last query's score with ONE earlier token towers over the rest.  That
    token is placed just inside and just outside the window or block: inside, the output is that token's value row;
    outside, it is not."""
    dt, D, size = torch.float32, 32, 20
    m = dict(heads=1, kv_heads=1, dim=8, vdim=8, diff=0.0, scale=1.0, softcap=50.0, mask={"size": size}, rot={"dims": 0, "base": 1.0})
    part, w = capped_part(dt, D, kind, m)
    e_key, e_query = torch.zeros(D, dtype=torch.float64), torch.zeros(D, dtype=torch.float64)
    e_key[0], e_query[1] = 1.0, 1.0
    w["m.q"] *= 0.0
    w["m.k"] *= 0.0
    w["m.q"][0], w["m.k"][0] = 40.0 * e_query, 40.0 * e_key       # row 0 of the first map: the query token answers the key token
    load(part, w, dt)
    wh = hold(w, dt)
    plain = P.two_map_attention if kind == "attention" else P.window_attention
    n = 3 * size + 5                                       # the last query is at n - 1
    lo = (n - 1) // size * size if kind == "attention" else n - size
    for at, inside in ((lo, True), (lo - 1, False), (lo + 1, True)):
        x = 0.1 * rand((n, D), 50)
        x[:, :2] = 0.0
        x[at, 0], x[n - 1, 1] = 1.0, 1.0
        x = held(x, dt)
        want = plain(x, wh, "m.", m, 1e-6, torch.float64)
        moved = x.clone()
        moved[at, 2:] = -moved[at, 2:]                     # another value at the loud key
        differs = (plain(moved, wh, "m.", m, 1e-6, torch.float64)[-1] - want[-1]).abs().max() > 0.05 * want[-1].abs().max()
        assert bool(differs) == inside, f"{kind}: the plain form at {at}"
        alone = Alone([part], dt, block_size=16, pages=12, slots=2)
        for cuts in ([n], [n - 1, 1], [at + 1, n - at - 2, 1], [7]):
            assert_close(in_portions(alone, 3, x, cuts), want, dt, f"{kind}: loud key at {at}, cuts {cuts}", 2e-4)


# ---------------------------------------------------------------- routing and the experts
def experts_part(dt, D, I, E, top, count, keep, scale):
    from vllm_oxide_b200.parts import PartSpec, build_part
    part = build_part("feed_forward", PartSpec("routed_experts", dict(
        hidden_size=D, expert_size=I, experts=E, top=top, groups=count, keep=keep, prefix="f.", activation="silu_gated",
        scores="sigmoid", correction=False, group_top=2, normalise=True, weight_scale=scale)), dtype=dt, device=DEV)
    w = {"f.router": rand((E, D), 1, 2.0 * D ** -0.5)}
    for e in range(E):
        w[f"f.e{e}.gate"], w[f"f.e{e}.up"] = rand((I, D), 10 + 3 * e, D ** -0.5), rand((I, D), 11 + 3 * e, D ** -0.5)
        w[f"f.e{e}.down"] = rand((D, I), 12 + 3 * e, I ** -0.5)
    return part, w


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("D, I, E, top, count, keep, scale, n", [
    (64, 24, 12, 2, 3, 2, 2.0, 40),        # groups decide
    (48, 16, 6, 3, 1, 1, 1.0, 9),          # no groups
    (40, 8, 5, 1, 5, 2, 0.5, 5),           # every expert a group of its own: a group counts by its one score
    (128, 64, 8, 4, 4, 3, 2.5, 300),       # enough pairs for the tensor-core products in bfloat16
    (72, 33, 4, 2, 2, 2, 1.0, 3),          # an odd expert width
])
def test_routed_gated_experts(D, I, E, top, count, keep, scale, n, dt):
    from vllm_oxide_b200 import kernels
    from helpers import make_context
    from vllm_oxide_b200.cache.paged_cache import PagedCache
    part, w = experts_part(dt, D, I, E, top, count, keep, scale)
    load(part, w, dt)
    wh = {k: (v.float().double() if k.endswith("router") else held(v, dt)) for k, v in w.items()}
    x = held(rand((n, D), 77), dt)
    mlp = {"router": {"experts": E, "top": top, "groups": {"count": count, "keep": keep}, "scale": scale}}
    margins = []
    idx, wt = P.route(x, wh, "f.", mlp["router"], torch.float64, margins)
    # the router alone: same experts in the same order, same weights
    xs = x.to(dt).to(DEV).contiguous()
    ids = torch.empty((n, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((n, top), dtype=torch.float32, device=DEV)
    kernels.moe_route(xs, part.router, None, ids, weights, n, top, count, keep, sigmoid_scores=True, group_top=2, normalise=True,
                      weight_scale=scale)
    sure = margins[0] > 1e-4
    assert sure.sum() >= n // 2
    assert torch.equal(ids.cpu()[sure].long(), idx[sure])
    assert_close(weights.cpu()[sure], wt[sure], torch.float32, "weights", 1e-4)
    # the whole feed-forward
    cache = PagedCache([None], [None], dt, DEV, 16, 2 + n // 16, 1)
    assert cache.manager.add_request(0) and cache.manager.ensure(0, 0, n)
    ctx = make_context(cache.manager, [(0, 0, [0] * n, [])], dt)
    got = part.forward(xs, ctx)
    want = P.moe_ff(x, wh, "f.", mlp, torch.float64)
    assert int(ctx.err.item()) == 0
    assert_close(got[sure.to(DEV)], want[sure], dt, "experts", 2e-5 if dt == torch.float32 else 0.04)


def test_groups_shut_out_the_best_expert():
    """Six experts in three groups of two: the single best expert sits beside a weak one, and the two groups whose two
    scores together are larger are kept; the kernel follows the plain rule."""
    from vllm_oxide_b200 import kernels
    s = torch.tensor([[0.55, 0.6, 0.95, 0.01, 0.5, 0.52]], dtype=torch.float64)
    z = torch.log(s / (1 - s))
    router = torch.eye(6, dtype=torch.float32, device=DEV)
    ids = torch.empty((1, 2), dtype=torch.int32, device=DEV)
    weights = torch.empty((1, 2), dtype=torch.float32, device=DEV)
    kernels.moe_route(z.float().to(DEV), router, None, ids, weights, 1, 2, 3, 2, sigmoid_scores=True, group_top=2, normalise=True,
                      weight_scale=3.0)
    idx, wt = P.route(z, {"r.router": torch.eye(6, dtype=torch.float64)}, "r.", {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2},
                                                                              "scale": 3.0}, torch.float64)
    assert idx.tolist() == [[1, 0]] and ids.cpu().tolist() == [[1, 0]]
    assert_close(weights.cpu(), wt, torch.float32, "weights", 1e-5)
    assert abs(float(weights.sum()) - 3.0) < 1e-5
    # with groups that count by their best score alone (another design's rule) the best expert's group is kept
    kernels.moe_route(z.float().to(DEV), router, None, ids, weights, 1, 2, 3, 2, sigmoid_scores=True, group_top=1)
    assert ids.cpu().tolist() == [[2, 1]]

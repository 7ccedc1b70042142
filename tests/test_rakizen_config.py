"""Rakizen without a GPU: configuration, plan, tensor names, the cache manager's blocks of positions, and closed forms of
the plain mechanisms (tests/plain/rakizen_plain.py)."""
import math

import pytest
import torch

from plain import rakizen_plain as P
from vllm_oxide_b200 import host
from vllm_oxide_b200.config import ConfigError, RakizenConfig
from vllm_oxide_b200.models import CausalLM, resolve


def two_map(heads=4, kv=2, dim=24, vdim=40, size=50, diff=0.25, scale=0.2, softcap=20.0):
    return {"type": "attention", "mixer": dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, diff=diff, scale=scale, softcap=softcap,
                                               mask={"size": size})}


def windowed(heads=3, kv=1, dim=32, vdim=16, size=37, dims=8, base=1000.0, scale=0.15, softcap=12.0):
    return {"type": "attention_2", "mixer": dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, softcap=softcap,
                                                 mask={"size": size}, rot={"dims": dims, "base": base})}


def config(layers, **more):
    return dict({"architecture": "Rakizen", "vocab": 90, "width": 48, "norm": {"eps": 1e-5}, "layers": layers}, **more)


MOE = {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}, "scale": 1.5}}


def test_the_plan_follows_the_configuration():
    layers = [dict(two_map(), mlp={"kind": "dense", "ff": 64}), dict(windowed(), mlp=MOE), dict(windowed(dims=0), mlp=None)]
    cfg, plan = resolve(config(layers, loop={"start": 1, "stop": 3, "times": 3}))
    assert isinstance(cfg, RakizenConfig) and cfg.runs() == [0, 1, 2, 1, 2, 1, 2]
    assert [(s.layer, s.plane) for s in plan.order] == [(0, 0), (1, 1), (2, 2), (1, 3), (2, 4), (1, 5), (2, 6)]
    assert [l.kind for l in plan.layers] == ["parallel"] * 3 and plan.final_norm.kind == "layernorm_stream"
    a, b, c = (l.params["mixer"].params for l in plan.layers)
    assert (a["maps"], a["chunk"], a["gate"], a["diff"], a["softcap"]) == (2, 50, True, 0.25, 20.0)
    assert (b["row_norm"], b["window"], b["position"]) == (True, 37, "l1.rot") and c["position"] is None
    assert list(plan.positions) == ["l1.rot"] and plan.positions["l1.rot"].params["interleaved"] is True
    ff = plan.layers[1].params["feed_forward"].params
    assert (ff["activation"], ff["scores"], ff["group_top"], ff["normalise"], ff["weight_scale"], ff["correction"]) == \
        ("silu_gated", "sigmoid", 2, True, 1.5, False)
    assert plan.layers[2].params["feed_forward"] is None
    model = CausalLM(plan, torch.bfloat16, "cpu")
    names = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert names["l0.mix.q"] == (4 * 2 * 24, 48) and names["l0.mix.k"] == (2 * 2 * 24, 48) and names["l0.mix.v"] == (2 * 40, 48)
    assert names["l0.mix.g"] == (160, 48) and names["l0.mix.o"] == (48, 160) and names["l0.mix.lq2"] == (24,)
    assert names["l1.mix.q.norm"] == (96,) and names["l1.mix.k.norm"] == (32,) and names["l1.mix.v"] == (16, 48)
    assert names["l1.mlp.e5.gate"] == (20, 48) and names["l1.mlp.router"] == (6, 48) and "l1.mlp.correction" not in names
    assert names["l0.norm1.b"] == (48,) and names["final.norm.b"] == (48,) and "l2.mlp.gate" not in names
    # the 32-bit model holds keys and values in their own sizes; the bfloat16 model pads both to one size that the
    # tensor-core attention kernels take (the next multiple of 16 of the larger)
    specs = CausalLM(plan, torch.float32, "cpu").cache_specs()
    assert (specs[0].kv_heads, specs[0].head_dim, specs[0].value_shape(), specs[0].chunk, specs[0].window) == (4, 24, (2, 40), 50, 0)
    assert (specs[1].kv_heads, specs[1].head_dim, specs[1].value_shape(), specs[1].chunk, specs[1].window) == (1, 32, (1, 16), 0, 37)
    specs = model.cache_specs()
    assert (specs[0].kv_heads, specs[0].head_dim, specs[0].value_shape(), specs[0].chunk, specs[0].window) == (4, 48, (2, 48), 50, 0)
    assert (specs[1].kv_heads, specs[1].head_dim, specs[1].value_shape(), specs[1].chunk, specs[1].window) == (1, 32, (1, 32), 0, 37)
    assert RakizenConfig.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("bad, word", [
    (lambda c: c["layers"][0].update(type="delta"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "choices"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "choices"),
    (lambda c: c.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_what_cannot_be_is_an_error(bad, word):
    import copy
    c = config([dict(two_map(), mlp=None), dict(windowed(), mlp=copy.deepcopy(MOE))])
    bad(c)
    with pytest.raises(ConfigError, match=word):
        RakizenConfig.from_dict(c)


def test_pages_behind_a_block_of_positions_are_given_back():
    """A group whose queries read only their own block of 40 positions, pages of 16: once position 40 is next, the pages
    that lie wholly before it go back to the pool; a window group beside it keeps its own rule."""
    m = host.KvCacheManager([host.GroupSpec(16, 12, 0, 40), host.GroupSpec(16, 12, 20, 0), host.GroupSpec(16, 12)], 2, False)
    assert m.add_request(1) and m.ensure(1, 0, 39)
    m.advance(1, 39)
    assert [p >= 0 for p in m.block_table(1, 0)] == [True, True, True]
    assert m.ensure(1, 39, 2)
    m.advance(1, 41)                 # the next query is in the block that starts at 40: pages 0 and 1 end before it
    assert [p >= 0 for p in m.block_table(1, 0)] == [False, False, True]
    assert [p >= 0 for p in m.block_table(1, 1)] == [False, True, True]        # the window reads from 41 - 20 + 1 = 22
    assert all(p >= 0 for p in m.block_table(1, 2))
    assert m.num_free_blocks(0) == 11 and m.num_free_blocks(2) == 9
    assert m.ensure(1, 41, 80 - 41)
    m.advance(1, 80)                 # 80 starts a block: everything before it may go
    assert [p >= 0 for p in m.block_table(1, 0)] == [False] * 5
    m.free_request(1)
    assert [m.num_free_blocks(g) for g in range(3)] == [12, 12, 12]


# ---------------------------------------------------------------- the plain mechanisms against closed forms
def test_masks():
    b = P.block_mask(10, 4)
    assert b[5].tolist() == [False] * 4 + [True, True] + [False] * 4 and b[4].sum() == 1 and b[3].sum() == 4 and b[0].sum() == 1
    w = P.window_mask(10, 3)
    assert w[5].tolist() == [False] * 3 + [True] * 3 + [False] * 4 and w[1].sum() == 2 and w[9].sum() == 3
    assert P.window_mask(6, 1).sum() == 6 and P.block_mask(6, 1).sum() == 6


def test_rotation_turns_neighbours_and_keeps_lengths():
    x = torch.randn(5, 2, 12, dtype=torch.float64)
    pos = torch.arange(5)
    y = P.rotate_pairs(x, {"dims": 8, "base": 100.0}, pos)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.equal(y[0], x[0])
    for i in range(4):
        a = 3 * 100.0 ** (-2.0 * i / 8)
        u, v = x[3, 1, 2 * i], x[3, 1, 2 * i + 1]
        assert abs(y[3, 1, 2 * i] - (u * math.cos(a) - v * math.sin(a))) < 1e-12
        assert abs(y[3, 1, 2 * i + 1] - (v * math.cos(a) + u * math.sin(a))) < 1e-12
    # scores depend on the distance only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    rot = {"dims": 8, "base": 50.0}
    s = lambda i, j: (P.rotate_pairs(q, rot, torch.tensor([i])) * P.rotate_pairs(k, rot, torch.tensor([j]))).sum()
    assert abs(s(9, 4) - s(105, 100)) < 1e-9


def test_route_by_hand():
    """Six experts in three groups of two, two groups kept, two experts taken.  Scores (sigmoids of the logits) are set
    through a router that reads one input element per expert."""
    s = torch.tensor([[0.9, 0.1, 0.6, 0.55, 0.7, 0.05]], dtype=torch.float64)
    z = torch.log(s / (1 - s))
    w = {"r.router": torch.eye(6, dtype=torch.float64)}
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}, "scale": 2.0}
    idx, wt = P.route(z, w, "r.", r, torch.float64)
    # group sums 1.0, 1.15, 0.75: the last group, which holds the second best expert, is shut out
    assert idx.tolist() == [[0, 2]]
    assert torch.allclose(wt, torch.tensor([[0.9, 0.6]], dtype=torch.float64) / 1.5 * 2.0)
    r1 = {"experts": 6, "top": 3}
    idx, wt = P.route(z, w, "r.", r1, torch.float64)
    assert idx.tolist() == [[0, 4, 2]] and abs(float(wt.sum()) - 1.0) < 1e-12


def test_two_maps_reduce_to_one_when_the_factor_vanishes():
    """With lq, lk and diff chosen so that lam = 0 the second map drops out: the head is the unit-normed first map."""
    torch.manual_seed(0)
    n, D, H, G, d, e = 9, 16, 2, 1, 4, 6
    m = dict(heads=H, kv_heads=G, dim=d, vdim=e, diff=0.0, scale=0.5, softcap=0.0, mask={"size": 100})
    w = {"p.q": torch.randn(H * 2 * d, D, dtype=torch.float64), "p.k": torch.randn(G * 2 * d, D, dtype=torch.float64),
         "p.v": torch.randn(G * e, D, dtype=torch.float64), "p.o": torch.eye(H * e, dtype=torch.float64),
         "p.g": torch.zeros(H * e, D, dtype=torch.float64)}
    for nme in ("lq1", "lk1", "lq2", "lk2"):
        w["p." + nme] = torch.zeros(d, dtype=torch.float64)
    h = torch.randn(n, D, dtype=torch.float64)
    out = P.two_map_attention(h, w, "p.", m, 1e-9, torch.float64).reshape(n, H, e)
    q = (h @ w["p.q"].T).reshape(n, H, 2, d)[:, :, 0]
    k = (h @ w["p.k"].T).reshape(n, G, 2, d)[:, 0, 0]
    v = h @ w["p.v"].T
    causal = torch.tril(torch.ones(n, n, dtype=torch.bool))
    for head in range(H):
        s = torch.where(causal, q[:, head] @ k.T * 0.5, torch.tensor(-math.inf, dtype=torch.float64))
        a = torch.softmax(s, -1) @ v
        assert torch.allclose(out[:, head], 0.5 * P.rms(a, 1e-9), atol=1e-9)      # the gate is sigmoid(0)
    assert abs(float((out[:, 0] ** 2).mean(-1)[0]) - 0.25) < 1e-6


def test_layer_runs_and_layer_norm():
    cfg = {"layers": [0, 1, 2, 3], "loop": {"start": 1, "stop": 3, "times": 2}}
    assert P.layer_runs(cfg) == [0, 1, 2, 1, 2, 3] and P.layer_runs({"layers": [0, 1]}) == [0, 1]
    x = torch.randn(3, 10, dtype=torch.float64)
    y = P.layer_norm(x, torch.full((10,), 2.0, dtype=torch.float64), torch.full((10,), 0.5, dtype=torch.float64), 0.0)
    assert torch.allclose(y.mean(-1), torch.full((3,), 0.5, dtype=torch.float64)) and torch.allclose(((y - 0.5) ** 2).mean(-1), torch.full((3,), 4.0, dtype=torch.float64))

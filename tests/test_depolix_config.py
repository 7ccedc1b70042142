"""Depolix without a GPU: configuration, plan, tensor names, sizes that are read from a checkpoint's tensors, the cache
manager's kept first pages, and closed forms of the plain mechanisms (tests/plain/depolix_plain.py)."""
import math

import pytest
import torch

from plain import depolix_plain as P
from vllm_oxide_b200 import host
from vllm_oxide_b200.config import ConfigError, DepolixConfig
from vllm_oxide_b200.models import CausalLM, resolve
from vllm_oxide_b200.parts.conv_attention import distance_bucket
from vllm_oxide_b200.parts.rope import scaled_frequencies


def latent(heads=3, dim=24, rot_dim=8, vdim=20, q_rank=28, kv_rank=40, scale=0.2, base=5000.0, dims=None, scaling=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "latent_attention", "mixer": dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank,
                                                      scale=scale, rot=rot)}


def sides(**more):
    left = dict(heads=3, kv_heads=1, dim=24, vdim=40, conv=3, scale=0.25, bias_max=90.0, mask={"size": 21, "keep_first": 5})
    right = dict(heads=4, kv_heads=2, dim=16, vdim=24, conv=4)
    left.update({k[5:]: v for k, v in more.items() if k.startswith("left_")})
    right.update({k[6:]: v for k, v in more.items() if k.startswith("right_")})
    return {"type": "parallel", "mixer": {"left": left, "right": right}}


def config(layers, **more):
    return dict({"architecture": "Depolix", "vocab": 90, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.5},
                 "residual_mult": 0.5, "logit_scale": 0.7, "layers": layers}, **more)


MOE = {"kind": "moe", "expert": {"ff": 20, "limit": 2.0}, "router": {"experts": 6, "top": 2}}
YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}


def test_the_plan_follows_the_configuration():
    layers = [dict(latent(scaling=YARN), mlp={"kind": "dense", "ff": 64, "limit": 1.5}), dict(sides(), mlp=MOE), dict(latent(dims=0), mlp=None)]
    cfg, plan = resolve(config(layers))
    assert isinstance(cfg, DepolixConfig) and (cfg.embedding_scale, cfg.residual_mult, cfg.logit_scale) == (3.5, 0.5, 0.7)
    assert [(s.layer, s.plane) for s in plan.order] == [(0, 0), (1, 1), (2, 2)]
    assert [l.kind for l in plan.layers] == ["parallel"] * 3 and plan.final_norm.kind == "rmsnorm_parallel_stream"
    n = plan.layers[0].params["norm"].params
    assert (n["one_plus"], n["mult"], n["open_scale"]) == (True, 0.5, 3.5) and plan.final_norm.params["out_scale"] == 0.7
    a, b, c = (l.params["mixer"] for l in plan.layers)
    assert a.kind == "latent_attention" and (a.params["gate"], a.params["position"], a.params["window"]) == (True, "l0.rot", None)
    assert c.params["position"] is None and list(plan.positions) == ["l0.rot"]
    rope = plan.positions["l0.rot"].params
    assert (rope["interleaved"], rope["table"], rope["scaling"], rope["rotary_dim"]) == (False, False, YARN, 8)
    assert b.kind == "side_by_side" and b.params["left"].kind == "attention_conv" and b.params["right"].kind == "gated_delta"
    l, r = b.params["left"].params, b.params["right"].params
    assert (l["window"], l["keep_first"], l["bias_rows"], l["bias_max"], l["taps"], l["unit_norm"], l["gate"]) == (21, 5, -1, 90.0, 3, True, True)
    assert (r["decay_rank"], r["gate_rank"], r["gate"], r["taps"]) == (-1, -1, "sigmoid", 4)
    ff = plan.layers[1].params["feed_forward"].params
    assert (ff["activation"], ff["limit"], ff["scores"], ff["normalise"], ff["correction"], ff["router_bias"]) == \
        ("glu_clamped", 2.0, "softmax", True, False, True)
    assert plan.layers[0].params["feed_forward"].kind == "glu_clamped" and plan.layers[2].params["feed_forward"] is None
    model = CausalLM(plan, torch.bfloat16, "cpu")
    names = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert names["l0.mix.dq"] == (28, 48) and names["l0.mix.uq"] == (3 * 32, 28) and names["l0.mix.dkv"] == (48, 48)
    assert names["l0.mix.uk"] == (72, 40) and names["l0.mix.uv"] == (60, 40) and names["l0.mix.g"] == (60, 48) and names["l0.mix.o"] == (48, 60)
    assert names["l0.mlp.gate.b"] == (64,) and names["l0.mlp.down.b"] == (48,) and names["l0.norm1"] == (48,)
    assert names["l1.mix.left.q"] == (72, 48) and names["l1.mix.left.k.conv"] == (24, 3) and names["l1.mix.left.v"] == (40, 48)
    assert names["l1.mix.left.g"] == (3, 48) and names["l1.mix.left.o"] == (48, 120) and names["l1.mix.left.out"] == (48,)
    # sizes that the configuration does not state are read from the checkpoint's tensors
    assert names["l1.mix.left.rel"] == (-1, 3) and names["l1.mix.right.a1"] == (-1, 48) and names["l1.mix.right.a2"] == (64, -1)
    assert names["l1.mix.right.g2"] == (96, -1) and names["l1.mix.right.dt_bias"] == (64,) and names["l1.mix.right.A_log"] == (4,)
    assert names["l1.mix.right.b"] == (4, 48) and names["l1.mix.right.norm"] == (24,) and names["l1.mix.right.v.conv"] == (96, 4)
    assert names["l1.mlp.e5.gate"] == (20, 48) and names["l1.mlp.router.b"] == (6,) and "l2.mlp.gate" not in names
    assert names["final.norm"] == (48,) and names["head"] == (90, 48)
    specs, states = CausalLM(plan, torch.float32, "cpu").cache_specs(), model.state_specs()
    assert (specs[0].kv_heads, specs[0].head_dim, specs[0].tensors, specs[0].window) == (1, 48, 1, 0)
    assert (specs[1].kv_heads, specs[1].head_dim, specs[1].value_shape(), specs[1].window, specs[1].keep_first) == (1, 24, (1, 40), 21, 5)
    # the pair's state: the left filters' inputs, then the right side's matrices and filters' inputs
    assert states[0] is None and states[1].shape == (2 * (72 + 24 + 40) + 4 * 16 * 24 + 3 * (2 * 32 + 96),)
    assert DepolixConfig.from_dict(cfg.to_dict()) == cfg


def test_stated_sizes_make_a_random_model_and_unstated_ones_cannot_be_drawn(tmp_path):
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    with pytest.raises(ValueError, match="read from a checkpoint"):
        write_random_model_folder(str(tmp_path / "a"), config([dict(sides(), mlp=None)]), 1)
    stated = config([dict(sides(left_bias_rows=12, right_decay_rank=6, right_gate_rank=5), mlp=MOE)])
    write_random_model_folder(str(tmp_path / "b"), stated, 1)
    cfg, w = P.read_folder(str(tmp_path / "b"))
    assert w["l0.mix.left.rel"].shape == (12, 3) and w["l0.mix.right.a1"].shape == (6, 48) and w["l0.mix.right.g2"].shape == (96, 5)
    assert P.forward(cfg, w, [1, 2, 3, 4, 5]).shape == (5, 90)


@pytest.mark.parametrize("bad", [
    lambda c: c["layers"][0].update(type="attention"),
    lambda c: c["layers"][0]["mixer"].pop("kv_rank"),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10),
    lambda c: c["layers"][1]["mixer"]["left"].update(heads=4, kv_heads=3),
    lambda c: c["layers"][1]["mixer"].pop("right"),
    lambda c: c["layers"][1]["mixer"]["left"]["mask"].update(keep_first=-1),
    lambda c: c["layers"][0]["mlp"].pop("limit"),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=7),
    lambda c: c.pop("norm"),
])
def test_what_cannot_be_is_an_error(bad):
    c = config([dict(latent(), mlp={"kind": "dense", "ff": 64, "limit": 1.5}), dict(sides(), mlp={**MOE, "router": dict(MOE["router"])})])
    bad(c)
    with pytest.raises(ConfigError):
        resolve(c)


def test_kept_first_pages_stay_while_a_window_gives_the_others_back():
    m = host.KvCacheManager([host.GroupSpec(4, 12, 6, 0, 5), host.GroupSpec(4, 12, 6), host.GroupSpec(4, 12)], 2, False)
    assert m.add_request(1) and m.ensure(1, 0, 30)
    m.advance(1, 30)
    # positions 0..4 are kept: pages 0 and 1; the window of 6 before position 30 starts at 25: pages 6 and 7
    assert list(m.block_table(1, 0)) == [0, 1, -1, -1, -1, -1, 6, 7]
    assert list(m.block_table(1, 1)) == [-1] * 6 + [6, 7] and list(m.block_table(1, 2)) == list(range(8))
    assert m.ensure(1, 30, 10)
    m.advance(1, 40)
    assert [p >= 0 for p in m.block_table(1, 0)] == [True, True] + [False] * 6 + [True, True]
    assert m.check_invariants() == ""
    # a request shorter than the kept span gives nothing back, and a second request gets pages of its own
    assert m.add_request(2) and m.ensure(2, 0, 3)
    m.advance(2, 3)
    assert [p >= 0 for p in m.block_table(2, 0)] == [True]
    m.free_request(1)
    m.free_request(2)
    assert [m.num_free_blocks(g) for g in range(3)] == [12, 12, 12] and m.check_invariants() == ""


def test_distance_buckets():
    rows, far = 24, 300.0
    got = [distance_bucket(n, rows, far) for n in range(400)]
    assert got[:12] == list(range(12)) and got[12] == 12 and got[299] == 23 and got[300] == 23 and got[399] == 23
    assert all(b >= a for a, b in zip(got, got[1:])) and set(got) == set(range(24))
    assert got == [P.distance_bucket(n, rows, far) for n in range(400)]
    # the boundary of bucket 12 + j lies where 12 * 25^(j / 12) is reached
    for j in range(1, 12):
        edge = 12.0 * 25.0 ** (j / 12.0)
        assert got[math.ceil(edge)] >= 12 + j > got[math.floor(edge) - 1]


def test_stretched_frequencies_and_rotation_of_halves():
    stretch = {"factor": 3.0, "original": 1024, "fast": 24.0, "slow": 2.0}
    f, amp = scaled_frequencies(24, 250000.0, stretch, precise=True)
    want, want_amp = P.stretched_frequencies(24, 250000.0, stretch)
    assert torch.allclose(f.double(), want, rtol=1e-7, atol=0) and amp == pytest.approx(want_amp) == pytest.approx(0.1 * math.log(3.0) + 1.0)
    # the fastest wave is left alone, the slowest is slowed by the whole factor
    assert float(want[0]) == 1.0 and float(want[-1]) == pytest.approx(250000.0 ** (-22.0 / 24.0) / 3.0)
    x = torch.arange(12.0, dtype=torch.float64).reshape(1, 12)
    y = P.rotate_halves(x, torch.tensor([3]), torch.tensor([0.5, 0.25], dtype=torch.float64), 2.0)
    c, s = 2.0 * math.cos(1.5), 2.0 * math.sin(1.5)
    assert y[0, 0] == pytest.approx(0.0 * c - 2.0 * s) and y[0, 2] == pytest.approx(2.0 * c + 0.0 * s)
    assert y[0, 1] == pytest.approx(1.0 * 2.0 * math.cos(0.75) - 3.0 * 2.0 * math.sin(0.75)) and torch.equal(y[0, 4:], x[0, 4:])


def test_plain_mechanisms_in_closed_form():
    dt = torch.float64
    # the clamped gate: beyond the limit the gate stands still and the up branch is cut on both sides
    g, u = torch.tensor([0.5, 9.0, -9.0], dtype=dt), torch.tensor([9.0, -9.0, 0.25], dtype=dt)
    y = P.clamped_glu(g, u, 2.0)
    sig = lambda z: 1.0 / (1.0 + math.exp(-z))
    assert y.tolist() == pytest.approx([0.5 * sig(0.851) * 3.0, 2.0 * sig(3.404) * -1.0, -9.0 * sig(-15.318) * 1.25])
    # the convolution: zeros before the start, the last tap is the current token's
    conv = P.causal_conv(torch.tensor([[1.0], [2.0], [4.0]], dtype=dt), torch.tensor([[100.0, 10.0, 1.0]], dtype=dt))
    assert conv[:, 0].tolist() == [1.0, 12.0, 124.0]
    # the router: weights are the softmax over the chosen logits alone
    W = {"r.router": torch.eye(4, dtype=dt), "r.router.b": torch.tensor([0.0, 0.0, 5.0, 0.0], dtype=dt)}
    idx, w, margin = P.route(torch.tensor([[3.0, 1.0, -3.0, 0.0]], dtype=dt), W, "r.", 2, dt)
    assert idx.tolist() == [[0, 2]] and w[0].tolist() == pytest.approx([math.e / (1 + math.e), 1 / (1 + math.e)]) and margin.tolist() == [1.0]
    # the delta rule with one head and a decay of one: writing (k, v) and reading with q = k returns beta * v, a second write
    # along the same key moves the stored value toward the new one
    n, dk, dv = 2, 4, 3
    W = {"d." + k: v for k, v in {
        "q": torch.zeros(dk, 2, dtype=dt), "k": torch.zeros(dk, 2, dtype=dt), "v": torch.zeros(dv, 2, dtype=dt),
        "q.conv": torch.ones(dk, 1, dtype=dt), "k.conv": torch.ones(dk, 1, dtype=dt), "v.conv": torch.ones(dv, 1, dtype=dt),
        "b": torch.zeros(1, 2, dtype=dt), "a1": torch.zeros(1, 2, dtype=dt), "a2": torch.zeros(dk, 1, dtype=dt),
        "dt_bias": torch.full((dk,), -50.0, dtype=dt), "A_log": torch.zeros(1, dtype=dt), "norm": torch.ones(dv, dtype=dt),
        "g1": torch.zeros(1, 2, dtype=dt), "g2": torch.zeros(dv, 1, dtype=dt), "o": torch.eye(dv, dtype=dt)}.items()}
    W["d.q"][0, 0] = W["d.k"][0, 0] = 50.0        # SiLU(50) = 50: q and k along the first channel, unit after the norm
    W["d.v"][:, 1] = torch.tensor([1.0, 2.0, 3.0], dtype=dt)
    h = torch.tensor([[1.0, 1.0], [1.0, -1.0]], dtype=dt)
    out = P.delta_rule(h, W, "d.", dict(heads=1, kv_heads=1, dim=dk, vdim=dv), 0.0, dt)
    v1, v2 = P.silu(torch.tensor([1.0, 2.0, 3.0], dtype=dt)), P.silu(torch.tensor([-1.0, -2.0, -3.0], dtype=dt))
    o1 = 0.5 * v1 * dk ** -0.5                    # beta = sigmoid(0) = 1/2; q carries dim^(-1/2)
    o2 = (0.5 * v1 + 0.5 * (v2 - 0.5 * v1)) * dk ** -0.5
    unit = lambda o: o / torch.sqrt((o * o).mean())
    assert torch.allclose(out[0], unit(o1) * 0.5, atol=1e-5) and torch.allclose(out[1], unit(o2) * 0.5, atol=1e-5)

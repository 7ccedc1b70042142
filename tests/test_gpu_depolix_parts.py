"""Every mechanism of Depolix alone, as a part with pages and state slots of its own, against its plain function
(tests/plain/depolix_plain.py): the stream's RMS norm step, the pair norm, the clamped gate, attention through a latent with
rotated halves and an output gate, attention behind short convolutions (bias by distance, window, kept first tokens, a gate
a head) on the plain and on the tensor-core kernels, the delta rule with a decay per key channel at every width of its scan,
the router and the experts in all three products."""
import math

import pytest
import torch

from helpers import DEV, Alone, assert_close, held, make_context, rand
from plain import depolix_plain as P

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
FLOAT_NAMES = (".conv", "A_log", "dt_bias", ".rel", "norm", "router", "router.b")


def load(part, w, dt):
    """Gives a part the tensors it lists, each in the type the engine keeps it in."""
    from vllm_oxide_b200.weights.loader import kept_dtype
    part.load({s.name: w[s.name].to(kept_dtype(s.role, dt)).to(DEV).contiguous() for s in part.tensor_specs()})


def draw(part, seed, scale_of=None):
    """Random tensors for everything the part lists (float64): matrices by their fan-in, the rest small."""
    w = {}
    for i, s in enumerate(part.tensor_specs()):
        if s.role == "matrix":
            w[s.name] = rand(s.shape, seed + i, (s.fan_in or s.shape[-1]) ** -0.5)
        elif s.role == "norm":
            w[s.name] = 1.0 + 0.2 * rand(s.shape, seed + i)
        else:
            w[s.name] = rand(s.shape, seed + i, 0.5 if s.name.endswith((".conv", "dt_bias", ".rel")) else 0.2)
    for k, f in (scale_of or {}).items():
        w[k] = w[k] * f
    return w


def hold(part, w, dt):
    """The same tensors as the plain functions should see them: what the engine keeps in float as it is, the rest rounded."""
    from vllm_oxide_b200.weights.loader import kept_dtype
    roles = {s.name: s.role for s in part.tensor_specs()}
    return {k: (v.float().double() if kept_dtype(roles[k], dt) == torch.float32 else held(v, dt)) for k, v in w.items()}


# ---------------------------------------------------------------- the stream's step with its norm
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("D", [8, 30, 64, 257, 1024, 4100])
def test_rms_norm_step(D, dt):
    from vllm_oxide_b200 import kernels
    n, eps, mult, open_scale = 7, 1e-5, 0.3, 3.7
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    emb, y1, y2 = (held(rand((n, D), s), dt) for s in (1, 2, 3))
    w = 0.2 * rand((D,), 4).float().double()
    dev = lambda t, d=dt: t.to(d).to(DEV).contiguous()
    stream = torch.full((n, D), 99.0, dtype=torch.float32, device=DEV)
    out = torch.empty((n, D), dtype=dt, device=DEV)
    norm = lambda x, off: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (off + w)
    # the stream begins: x = embedded * open_scale, whatever the buffer held
    kernels.rms_norm_step(stream, eps, err, y1=dev(emb), w=dev(w, torch.float32), out=out, init=True, mult=mult, open_scale=open_scale,
                          gain_offset=1.0)
    x = (emb.float() * torch.tensor(open_scale, dtype=torch.float32)).double()
    assert_close(stream, x, torch.float32, "the stream's first rows", 1e-6)
    assert_close(out, norm(x, 1.0), dt, "the first norm")
    # a layer's two outputs enter together, times the factor
    kernels.rms_norm_step(stream, eps, err, y1=dev(y1), y2=dev(y2), w=dev(w, torch.float32), out=out, mult=mult, gain_offset=1.0)
    x = x + mult * (y1 + y2)
    assert_close(stream, x, torch.float32, "the stream after a layer", 1e-6)
    assert_close(out, norm(x, 1.0), dt, "the next norm")
    # one output alone, a plain gain; then chosen rows only, nothing stored
    kernels.rms_norm_step(stream, eps, err, y1=dev(y2), w=dev(w, torch.float32), out=out, mult=mult, gain_offset=0.0)
    x = x + mult * y2
    assert_close(out, norm(x, 0.0), dt, "a plain gain")
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    some = torch.empty((3, D), dtype=dt, device=DEV)
    before = stream.clone()
    kernels.rms_norm_step(stream, eps, err, y1=dev(y1), y2=dev(y2), w=dev(w, torch.float32), out=some, rows=rows, n_out=3, mult=mult,
                          gain_offset=0.7)
    assert torch.equal(stream, before) and int(err.item()) == 0
    assert_close(some, norm(x + mult * (y1 + y2), 0.7)[[5, 0, 5]], dt, "chosen rows")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("D, I", [(48, 24), (100, 37), (256, 512)])
def test_pair_norm_clamped_gate_and_bias(D, I, dt):
    from vllm_oxide_b200 import kernels
    n, eps = 9, 1e-5
    dev = lambda t, d=dt: t.to(d).to(DEV).contiguous()
    a, b = held(rand((n, D), 1, 3.0), dt), held(rand((n, D), 2, 0.1), dt)
    wa, wb = ((1.0 + 0.3 * rand((D,), s)).float().double() for s in (3, 4))
    out = torch.empty((n, D), dtype=dt, device=DEV)
    kernels.pair_norm_mean(dev(a), dev(b), dev(wa, torch.float32), dev(wb, torch.float32), out, eps)
    assert_close(out, 0.5 * (P.rms(a, eps) * wa + P.rms(b, eps) * wb), dt, "pair norm")
    gu, bias = held(rand((n, 2 * I), 5, 2.0), dt), rand((2 * I,), 6).float().double()
    act = torch.empty((n, I), dtype=dt, device=DEV)
    for bs, limit in ((bias, 1.5), (None, 0.4), (bias, 30.0)):
        kernels.clamped_glu(dev(gu), None if bs is None else dev(bs, torch.float32), act, limit)
        z = gu if bs is None else gu + bs
        assert_close(act, P.clamped_glu(z[:, :I], z[:, I:], limit), dt, f"clamped gate, limit {limit}")
    x = dev(a)
    kernels.add_bias(x, dev(wa, torch.float32))
    assert_close(x, a + wa, dt, "bias")
    x, g = dev(gu[:, :I]), dev(gu[:, I:])
    kernels.sigmoid_gate_mul(x, g, I)
    assert_close(x, gu[:, :I] * P.sigmoid(gu[:, I:]), dt, "gate an element")


# ---------------------------------------------------------------- mixers alone
def run_cuts(alone, part_index, x, cuts_list, want, dt, what, tol=None):
    """Feeds x [n, D] in several cuts (each as a request of its own, ended afterwards) and holds every cut to `want`."""
    for k, cuts in enumerate(cuts_list):
        rid, at, rows, i = 100 + k, 0, [], 0
        while at < x.shape[0]:
            n = min(cuts[i % len(cuts)], x.shape[0] - at)
            i += 1
            rows.append(alone.step([(rid, x[at:at + n])], end=[rid] if at + n == x.shape[0] else [])[part_index])
            at += n
        assert_close(torch.cat(rows), want, dt, f"{what}, cuts {cuts[:4]}", tol)


LATENT = {
    "three heads, stretched": dict(D=48, m=dict(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=12, kv_rank=20, scale=0.3,
                                                rot={"dims": 8, "base": 1000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}})),
    "part of the shared key unrotated": dict(D=40, m=dict(heads=2, dim=8, rot_dim=12, vdim=8, q_rank=16, kv_rank=24, scale=0.4,
                                                         rot={"dims": 6, "base": 50.0})),
    "a row the tensor-core kernels take whole": dict(D=64, m=dict(heads=4, dim=32, rot_dim=32, vdim=32, q_rank=24, kv_rank=96, scale=0.2,
                                                                 rot={"dims": 32, "base": 10000.0})),
}


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("case", sorted(LATENT))
def test_latent_attention_with_rotated_halves_and_a_gate(case, dt):
    from vllm_oxide_b200.parts import PartSpec, build_part
    D, m = LATENT[case]["D"], LATENT[case]["m"]
    positions = {"r": build_part("position", PartSpec("rope", dict(head_dim=m["rot_dim"], rotary_dim=m["rot"]["dims"], max_position=1 << 30,
                                                                    theta=m["rot"]["base"], interleaved=False, table=False, precise=True,
                                                                    scaling=m["rot"].get("scaling"))), device=DEV)}
    part = build_part("mixer", PartSpec("latent_attention", dict(
        hidden_size=D, num_heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], q_rank=m["q_rank"], kv_rank=m["kv_rank"],
        scale=m["scale"], eps=1e-5, window=None, position="r", prefix="m.", gate=True)), positions=positions, dtype=dt, device=DEV)
    w = draw(part, 11)
    load(part, w, dt)
    x = held(rand((90, D), 5), dt)
    want = P.latent_attention(x, hold(part, w, dt), "m.", m, 1e-5, torch.float64)
    run_cuts(Alone([part], dt, block_size=16), 0, x, [[90], [60] + [1] * 30, [7, 2, 33], [2]], want, dt, case)


WINDOW = {
    # (D, left sizes): plain kernel in 32 bits; in bfloat16 padded to 48 (cp.async), 64 and 128 (TMA), 32 (cp.async)
    "values wider than keys": (40, dict(heads=4, kv_heads=2, dim=24, vdim=40, conv=3, scale=0.3, bias_max=50.0, rows=10, mask=dict(size=19, keep_first=4))),
    "64 wide, keeps more than a page": (64, dict(heads=4, kv_heads=1, dim=64, vdim=64, conv=4, scale=0.15, bias_max=300.0, rows=24, mask=dict(size=44, keep_first=21))),
    "128 wide, window of one tile": (48, dict(heads=2, kv_heads=2, dim=128, vdim=128, conv=2, scale=0.1, bias_max=100.0, rows=16, mask=dict(size=64, keep_first=3))),
    "nothing kept": (32, dict(heads=2, kv_heads=1, dim=32, vdim=32, conv=3, scale=0.25, bias_max=30.0, rows=8, mask=dict(size=23, keep_first=0))),
    "kept beyond the window, one tap": (32, dict(heads=2, kv_heads=2, dim=16, vdim=32, conv=1, scale=0.3, bias_max=9.0, rows=4, mask=dict(size=5, keep_first=70))),
    "no window": (32, dict(heads=3, kv_heads=1, dim=16, vdim=16, conv=2, scale=0.3, bias_max=20.0, rows=6, mask=None)),
}


def window_part(dt, D, m):
    from vllm_oxide_b200.parts import PartSpec, build_part
    mask = m.get("mask") or {}
    return build_part("mixer", PartSpec("attention_conv", dict(
        hidden_size=D, num_heads=m["heads"], num_kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], scale=m["scale"], taps=m["conv"],
        eps=1e-5, prefix="m.", window=mask.get("size"), keep_first=mask.get("keep_first", 0), bias_rows=m["rows"], bias_max=m["bias_max"])),
        dtype=dt, device=DEV)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("case", sorted(WINDOW))
def test_attention_behind_convolutions_alone(case, dt):
    from vllm_oxide_b200 import kernels
    D, m = WINDOW[case]
    part = window_part(dt, D, m)
    w = draw(part, 21)
    load(part, w, dt)
    x = held(rand((200, D), 6), dt)
    want = P.window_attention(x, hold(part, w, dt), "m.", m, 1e-5, torch.float64)
    kernels.enable_kernel_timers(True)
    kernels.kernel_timer_report()
    try:
        run_cuts(Alone([part], dt, block_size=16), 0, x, [[200], [150] + [1] * 50, [7, 2, 33, 64], [2]], want, dt, case)
        ran = set(kernels.kernel_timer_report())
    finally:
        kernels.enable_kernel_timers(False)
    if dt == torch.bfloat16:
        # the tensor-core kernels ran it, for portions and for single tokens, and the plain kernel did not
        assert "attention_prefill_window_bias" in ran and "attention_decode_window_bias" in ran, ran
        assert "paged_attention_generic" not in ran, ran
    else:
        assert "paged_attention_generic" in ran


@pytest.mark.parametrize("dt", DTYPES)
def test_pages_and_slots_used_again_by_the_pair(dt):
    """Two mixers side by side over a pool of few pages and two slots: requests come and go, pages behind the window go back
    while a request runs (but for the kept ones), and a new request finds a slot that another has used."""
    from vllm_oxide_b200.parts import PartSpec, build_part
    D = 48
    left = PartSpec("attention_conv", dict(hidden_size=D, num_heads=2, num_kv_heads=1, dim=16, vdim=16, scale=0.3, taps=3, eps=1e-5,
                                           prefix="m.left.", window=20, keep_first=18, bias_rows=8, bias_max=40.0))
    right = PartSpec("gated_delta", dict(hidden_size=D, num_heads=2, num_kv_heads=1, dim=16, vdim=8, taps=4, eps=1e-5, prefix="m.right.",
                                         decay_rank=3, gate_rank=4, gate="sigmoid"))
    part = build_part("mixer", PartSpec("side_by_side", dict(left=left, right=right, hidden_size=D, eps=1e-5, left_norm="m.left.out",
                                                             right_norm="m.right.out")), positions={}, dtype=dt, device=DEV)
    w = draw(part, 31, {"m.right.A_log": 0.0})
    w["m.right.A_log"] = w["m.right.A_log"] - 3.0
    load(part, w, dt)
    wh = hold(part, w, dt)
    m = {"left": dict(heads=2, kv_heads=1, dim=16, vdim=16, conv=3, scale=0.3, bias_max=40.0, mask=dict(size=20, keep_first=18)),
         "right": dict(heads=2, kv_heads=1, dim=16, vdim=8, conv=4)}
    alone = Alone([part], dt, block_size=16, pages=12, slots=2)
    xs = {rid: held(rand((n, D), 40 + rid), dt) for rid, n in ((1, 100), (2, 37), (3, 64), (4, 5), (5, 90))}
    got = {rid: [] for rid in xs}
    plan = [[(1, 50)], [(1, 1), (2, 30)], [(1, 49), (2, 7)], [(3, 64)], [(4, 5), (5, 2)], [(5, 88)]]
    at = {rid: 0 for rid in xs}
    for portions in plan:
        batch = [(rid, xs[rid][at[rid]:at[rid] + n]) for rid, n in portions if n > 0]
        done = [rid for rid, n in portions if at[rid] + n == xs[rid].shape[0]]
        out = alone.step(batch, end=done)[0]
        k = 0
        for rid, rows in batch:
            got[rid].append(out[k:k + rows.shape[0]])
            at[rid] += rows.shape[0]
            k += rows.shape[0]
    assert alone.m.num_free_blocks(0) == 12 and alone.m.num_free_state_slots == 2
    for rid, x in xs.items():
        want = P.side_by_side(x, wh, "m.", m, 1e-5, torch.float64)
        assert_close(torch.cat(got[rid]), want, dt, f"request {rid}", 3e-5 if dt == torch.float32 else 0.04)


# (the last: ranks and a width that the weight-streaming product takes, so that a decoding step's second, small products read
# their low-rank inputs as columns of the first product's row and write theirs behind it)
DELTA = [(8, 4, 16, 8, 2, 64, 64), (2, 1, 16, 8, 4, 3, 5), (4, 4, 24, 20, 2, 8, 2), (2, 2, 64, 16, 5, 16, 16), (3, 1, 128, 12, 4, 4, 6), (1, 1, 200, 36, 3, 7, 9), (2, 2, 8, 40, 1, 2, 3)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("heads, kv, dim, vdim, taps, decay_rank, gate_rank", DELTA)
def test_delta_rule_with_a_decay_per_key_channel(heads, kv, dim, vdim, taps, decay_rank, gate_rank, dt):
    from vllm_oxide_b200.parts import PartSpec, build_part
    D = 128 if decay_rank == 64 else 40
    part = build_part("mixer", PartSpec("gated_delta", dict(hidden_size=D, num_heads=heads, num_kv_heads=kv, dim=dim, vdim=vdim, taps=taps,
                                                            eps=1e-5, prefix="m.", decay_rank=decay_rank, gate_rank=gate_rank, gate="sigmoid")),
                      dtype=dt, device=DEV)
    w = draw(part, 51, {"m.a2": 3.0})
    w["m.A_log"] = w["m.A_log"] - 2.0             # heads that forget slowly, channels that forget at rates of their own
    load(part, w, dt)
    x = held(rand((120, D), 8), dt)
    want = P.delta_rule(x, hold(part, w, dt), "m.", dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim), 1e-5, torch.float64)
    run_cuts(Alone([part], dt, block_size=16, slots=2), 0, x, [[120], [90] + [1] * 30, [3, 1, 17, 2, 40], [2]], want, dt,
             f"delta rule {heads}/{kv} heads of {dim} x {vdim}", 5e-5 if dt == torch.float32 else 0.04)


# ---------------------------------------------------------------- the router and the experts
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("D, I, E, top, limit, n", [
    (64, 24, 12, 2, 1.0, 40),        # few pairs: the experts' rows are streamed pair by pair in bfloat16
    (48, 16, 6, 6, 0.5, 9),          # every expert chosen
    (40, 8, 5, 1, 0.7, 5),           # one expert: its weight is one
    (128, 64, 8, 4, 2.0, 300),       # enough pairs for the tcgen05 products in bfloat16
    (72, 33, 4, 2, 1.5, 3),          # an odd expert width: the float-accumulating tile kernel
])
def test_router_with_bias_and_clamped_experts(D, I, E, top, limit, n, dt):
    from vllm_oxide_b200 import kernels
    from vllm_oxide_b200.cache.paged_cache import PagedCache
    from vllm_oxide_b200.parts import PartSpec, build_part
    part = build_part("feed_forward", PartSpec("routed_experts", dict(
        hidden_size=D, expert_size=I, experts=E, top=top, prefix="f.", activation="glu_clamped", limit=limit, scores="softmax",
        correction=False, normalise=True, router_bias=True)), dtype=dt, device=DEV)
    w = draw(part, 61, {"f.router": 8.0})
    w["f.router.b"] = rand((E,), 62, 1.0)        # biases as large as the logits: they turn choices over
    load(part, w, dt)
    wh = hold(part, w, dt)
    x = held(rand((n, D), 77, 2.0), dt)            # inputs large enough to reach the clamp
    idx, wt, margin = P.route(x, wh, "f.", top, torch.float64)
    without = torch.topk(x @ wh["f.router"].T, top, dim=-1).indices
    assert E == top or n < 30 or (without != idx).any(), "the bias decides some choices"
    xs = x.to(dt).to(DEV).contiguous()
    ids = torch.empty((n, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((n, top), dtype=torch.float32, device=DEV)
    kernels.moe_route(xs, part.router, None, ids, weights, n, top, 1, 1, normalise=True, router_bias=part.router_b)
    sure = margin > 1e-4
    assert sure.sum() >= n // 2
    assert torch.equal(ids.cpu()[sure].long(), idx[sure])
    assert_close(weights.cpu()[sure], wt[sure], torch.float32, "weights", 1e-4)
    cache = PagedCache([None], [None], dt, DEV, 16, 2 + n // 16, 1)
    assert cache.manager.add_request(0) and cache.manager.ensure(0, 0, n)
    ctx = make_context(cache.manager, [(0, 0, [0] * n, [])], dt)
    got = part.forward(xs, ctx)
    want = P.moe_ff(x, wh, "f.", {"router": {"experts": E, "top": top}, "expert": {"ff": I, "limit": limit}}, torch.float64)
    unclamped = P.moe_ff(x, wh, "f.", {"router": {"experts": E, "top": top}, "expert": {"ff": I, "limit": 1e9}}, torch.float64)
    assert (unclamped - want).abs().max() > 0.05 * want.abs().max(), "the clamp is reached"
    assert int(ctx.err.item()) == 0
    assert_close(got[sure.to(DEV)], want[sure], dt, "experts", 2e-5 if dt == torch.float32 else 0.04)

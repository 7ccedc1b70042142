"""Plain, slow Depolix forward pass: whole sequences, no cache, one function per mechanism.

The oracle for the engine's Depolix model.  It shares no code with the package: it reads a model folder with its own
few lines (or takes a dict of tensors), works on one whole sequence at a time and keeps nothing between calls.  Every
function works in the dtype `dt` it is given (float64 for an oracle); nothing is rounded below `dt`.

Notation: n tokens, D the model width, m the residual factor.  A layer is  h = N(x);  x += m (mixer(h) + ff(h))  with
ONE RMS norm whose gain is stored around zero (x / rms * (1 + w)).  The mixer is `latent_attention` (low-rank queries,
one latent and one rotated key part a token, rotation of halves with stretched frequencies, an output gate an element)
or `parallel`: two mixers side by side over the same h, each normed over the width, half their sum.  The left one is
attention behind short convolutions with unit-RMS q and k, a learned bias by distance, a sliding window that keeps the
first tokens, and a gate a head; the right one is a gated delta rule with one decay per head and key channel.  The
feed-forward is a clamped gated layer with biases, or a mixture of such experts (without biases) weighted by the
softmax over the chosen logits.
"""
import json
import math
import struct

import torch

_ST = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
       "I32": torch.int32, "I64": torch.int64}


def read_folder(path):
    with open(f"{path}/config.json") as f:
        cfg = json.load(f)
    with open(f"{path}/model.safetensors", "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    head = json.loads(blob[8:8 + n])
    out = {}
    for name, meta in head.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(blob[8 + n + a:8 + n + b]), dtype=_ST[meta["dtype"]])
        out[name] = t.reshape(meta["shape"]).clone()
    return cfg, out


# ---------------------------------------------------------------- small functions
def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def clamped_glu(g, u, limit):
    """min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u) + 1)."""
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, -limit, limit)
    return g * sigmoid(1.702 * g) * (u + 1.0)


def causal_conv(u, w):
    """y[t] = sum_j w[:, j] u[t - taps + 1 + j], zeros before the start.  u [n, C], w [C, taps]."""
    n, taps = u.shape[0], w.shape[1]
    pad = torch.cat([u.new_zeros((taps - 1, u.shape[1])), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + n] * w[:, j]
    return y


# ---------------------------------------------------------------- rotation
def stretched_frequencies(dims, base, scaling, dt=torch.float64):
    """f_i of pair i (i < dims / 2) and the amplitude of cos and sin."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=dt)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    where = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=dt)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_halves(x, positions, freq, amp):
    """x [n, ..., dims]: element i pairs with i + dims/2."""
    half = freq.shape[0]
    ang = positions.to(freq.dtype)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = (torch.cos(ang) * amp).reshape(shape), (torch.sin(ang) * amp).reshape(shape)
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)


# ---------------------------------------------------------------- attention through a latent
def latent_attention(h, W, p, m, eps, dt):
    n = h.shape[0]
    H, dk, dr, dv, rk = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    g = lambda name: W[p + name].to(dt)
    cq = rms(h @ g("dq").T, eps) * g("dq.norm")
    q = (cq @ g("uq").T).reshape(n, H, dk + dr)
    down = h @ g("dkv").T
    c = rms(down[:, :rk], eps) * g("dkv.norm")
    shared = down[:, rk:rk + dr]
    rot = m["rot"]
    freq, amp = stretched_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"), dt)
    pos = torch.arange(n)
    q_rot = rotate_halves(q[:, :, dk:], pos, freq, amp)
    k_rot = rotate_halves(shared, pos, freq, amp)
    k = (c @ g("uk").T).reshape(n, H, dk)
    v = (c @ g("uv").T).reshape(n, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q[:, :, :dk], k) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    mask = torch.tril(torch.ones((n, n), dtype=torch.bool))
    s = s.masked_fill(~mask, float("-inf"))
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", a, v).reshape(n, H * dv)
    o = o * sigmoid(h @ g("g").T)
    return o @ g("o").T


# ---------------------------------------------------------------- the left side: windowed attention with a distance bias
def distance_bucket(nn, B, D):
    half = B // 2
    if nn < half:
        return nn
    return min(B - 1, half + int(math.floor(math.log(nn / half) / math.log(D / half) * (B - half))))


def window_attention(h, W, p, m, eps, dt):
    n = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    g = lambda name: W[p + name].to(dt)
    q = causal_conv(h @ g("q").T, g("q.conv")).reshape(n, H, dk)
    k = causal_conv(h @ g("k").T, g("k.conv")).reshape(n, G, dk)
    v = causal_conv(h @ g("v").T, g("v.conv")).reshape(n, G, dv)
    q, k = rms(q, eps), rms(k, eps)
    rel = g("rel") if p + "rel" in W else None
    B, D = (rel.shape[0], float(m["bias_max"])) if rel is not None else (0, 0.0)
    mk = m.get("mask") or {}
    size, keep = int(mk.get("size") or 0), int(mk.get("keep_first") or 0)
    kh = torch.arange(H) // (H // G)
    s = torch.einsum("ihd,jhd->hij", q, k[:, kh]) * float(m["scale"])
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    mask = (j <= i) & ((i - j < size) | (j < keep)) if size else (j <= i)
    if rel is not None:
        bucket_of = torch.tensor([distance_bucket(d, B, D) for d in range(n)])
        s = s + rel[bucket_of[(i - j).clamp(min=0)]].permute(2, 0, 1)          # [H, n, n]
    s = s.masked_fill(~mask, float("-inf"))
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", a, v[:, kh])
    o = o * sigmoid(h @ g("g").T)[:, :, None]
    return o.reshape(n, H * dv) @ g("o").T


# ---------------------------------------------------------------- the right side: gated delta rule, a decay per key channel
def delta_rule(h, W, p, m, eps, dt):
    n = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    g = lambda name: W[p + name].to(dt)
    q = silu(causal_conv(h @ g("q").T, g("q.conv"))).reshape(n, G, dk)
    k = silu(causal_conv(h @ g("k").T, g("k.conv"))).reshape(n, G, dk)
    v = silu(causal_conv(h @ g("v").T, g("v.conv"))).reshape(n, H, dv)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(q) * dk ** -0.5, unit(k)
    beta = sigmoid(h @ g("b").T)                                             # [n, H]
    a = (h @ g("a1").T) @ g("a2").T + g("dt_bias")
    decay = torch.exp(-torch.exp(g("A_log"))[None, :, None] * softplus(a.reshape(n, H, dk)))      # [n, H, dk]
    out = torch.zeros((n, H, dv), dtype=dt)
    for hh in range(H):
        kh = hh // (H // G)
        S = torch.zeros((dk, dv), dtype=dt)
        for t in range(n):
            S = decay[t, hh][:, None] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            out[t, hh] = S.T @ q[t, kh]
    out = rms(out, eps) * g("norm")
    out = out * sigmoid((h @ g("g1").T) @ g("g2").T).reshape(n, H, dv)
    return out.reshape(n, H * dv) @ g("o").T


def side_by_side(h, W, p, m, eps, dt):
    left = rms(window_attention(h, W, p + "left.", m["left"], eps, dt), eps) * W[p + "left.out"].to(dt)
    right = rms(delta_rule(h, W, p + "right.", m["right"], eps, dt), eps) * W[p + "right.out"].to(dt)
    return 0.5 * (left + right)


# ---------------------------------------------------------------- feed-forwards
def dense_ff(h, W, p, mlp, dt):
    g = lambda name: W[p + name].to(dt)
    y = clamped_glu(h @ g("gate").T + g("gate.b"), h @ g("up").T + g("up.b"), float(mlp["limit"]))
    return y @ g("down").T + g("down.b")


def route(h, W, p, top, dt):
    """(chosen experts [n, top], weights [n, top], margin [n]: how far the last chosen logit lies above the best one left out)."""
    z = h @ W[p + "router"].to(dt).T + W[p + "router.b"].to(dt)
    vals, idx = torch.topk(z, top, dim=-1)
    if top < z.shape[-1]:
        margin = vals[:, -1] - torch.topk(z, top + 1, dim=-1).values[:, -1]
    else:
        margin = torch.full((z.shape[0],), float("inf"), dtype=dt)
    return idx, torch.softmax(vals, dim=-1), margin


def expert_ff(h, W, p, limit, dt):
    g = lambda name: W[p + name].to(dt)
    return clamped_glu(h @ g("gate").T, h @ g("up").T, limit) @ g("down").T


def moe_ff(h, W, p, mlp, dt, margins=None):
    top, limit = int(mlp["router"]["top"]), float(mlp["expert"]["limit"])
    idx, w, margin = route(h, W, p, top, dt)
    if margins is not None:
        margins.append(margin)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] = out[t] + w[t, j] * expert_ff(h[t:t + 1], W, f"{p}e{e}.", limit, dt)[0]
    return out


# ---------------------------------------------------------------- the model
def forward(cfg, W, tokens, dt=torch.float64, layers_out=None, margins=None, noise=None):
    """Logits [n, vocab] of one whole sequence; `layers_out` (a list) receives the stream after every layer, `margins` (a
    list) every router's margins [n]; `noise` (a function) is applied to what the sublayers read and return (rounding to 16
    bits there shows how far a row moves under it)."""
    noise = noise or (lambda t: t)
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x = W["embed"].to(dt)[torch.as_tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = noise(rms(x, eps) * (1.0 + W[p + "norm1"].to(dt)))
        if layer["type"] == "latent_attention":
            y = latent_attention(h, W, p + "mix.", layer["mixer"], eps, dt)
        elif layer["type"] == "parallel":
            y = side_by_side(h, W, p + "mix.", layer["mixer"], eps, dt)
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        y = noise(y)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + noise(dense_ff(h, W, p + "mlp.", mlp, dt) if mlp["kind"] == "dense" else moe_ff(h, W, p + "mlp.", mlp, dt, margins))
        x = x + mult * y
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps) * (1.0 + W["final.norm"].to(dt))
    return (x @ W["head"].to(dt).T) * float(cfg.get("logit_scale", 1.0))

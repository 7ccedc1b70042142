"""Plain, slow Rakizen forward pass: whole sequences, no cache, one function per mechanism.

The oracle for the engine's Rakizen model.  It shares no code with the package: it reads a model folder with its own
few lines (or takes a dict of tensors), works on one whole sequence at a time and keeps nothing between calls.  Every
function works in the dtype `dt` it is given (float64 for an oracle); nothing is rounded below `dt`.

Notation: n tokens, D the model width.  A layer is  h = LN(x);  x += mixer(h) + ff(h)  with ONE layer norm (gain and
bias) that both sublayers read.  The mixer is `attention` (two softmax maps per head over shared values, subtracted with
a learned factor, scores capped by a tanh, keys visible inside blocks of positions, a unit norm per head, an output gate)
or `attention_2` (an RMS norm over the whole q and the whole k projection, the front of each head rotated in
neighbouring pairs, capped scores, a sliding window).  The feed-forward is a gated SiLU layer, a mixture of such layers
chosen by sigmoid scores among groups, or absent.  A stretch of layers may run several times with the same weights.
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
def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def cap(s, softcap):
    return softcap * torch.tanh(s / softcap) if softcap else s


# ---------------------------------------------------------------- masks
def block_mask(n, size):
    """[n, n] bool: query i sees key j <= i of the same block of `size` positions (blocks counted from position 0)."""
    pos = torch.arange(n)
    return (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))


def window_mask(n, size):
    """[n, n] bool: query i sees itself and the size - 1 positions before it."""
    pos = torch.arange(n)
    d = pos[:, None] - pos[None, :]
    return (d >= 0) & (d < size)


def masked_softmax(s, mask):
    s = torch.where(mask, s, torch.full_like(s, -math.inf))
    return torch.softmax(s, dim=-1)


# ---------------------------------------------------------------- rotation
def rotate_pairs(x, rot, positions):
    """x [n, heads, dim]: of every head's first rot.dims elements, element 2i turns with element 2i + 1 by the angle
    position * base^(-2i/dims); the rest pass."""
    dims, base = int(rot["dims"]), float(rot["base"])
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = torch.as_tensor(base, dtype=x.dtype) ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    front = torch.stack([u * c - v * s, v * c + u * s], dim=-1).reshape(*x.shape[:-1], dims)
    return torch.cat([front, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------- mixers
def two_map_attention(h, w, p, m, eps, dt):
    """`attention`: each head has two query/key maps over the same values; out = a1 - lam a2, unit norm per head times
    (1 - diff), gated by sigmoid(W_g h), then W_o."""
    n = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    q = (h @ w[p + "q"].to(dt).T).reshape(n, H, 2, d)
    k = (h @ w[p + "k"].to(dt).T).reshape(n, G, 2, d)
    v = (h @ w[p + "v"].to(dt).T).reshape(n, G, e)
    lam = (torch.exp((w[p + "lq1"].to(dt) * w[p + "lk1"].to(dt)).sum())
           - torch.exp((w[p + "lq2"].to(dt) * w[p + "lk2"].to(dt)).sum()) + diff)
    mask = block_mask(n, int(m["mask"]["size"]))
    out = torch.zeros(n, H, e, dtype=dt)
    for head in range(H):
        g = head // (H // G)
        maps = []
        for j in range(2):
            s = cap((q[:, head, j] @ k[:, g, j].T) * float(m["scale"]), float(m.get("softcap") or 0.0))
            maps.append(masked_softmax(s, mask) @ v[:, g])
        out[:, head] = rms(maps[0] - lam * maps[1], eps) * (1.0 - diff)
    gate = torch.sigmoid(h @ w[p + "g"].to(dt).T)
    return (out.reshape(n, H * e) * gate) @ w[p + "o"].to(dt).T


def window_attention(h, w, p, m, eps, dt):
    """`attention_2`: q and k each pass an RMS norm over their whole width (with a gain), the front of each head turns
    with the position, scores are capped, a query sees a sliding window."""
    n = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms(h @ w[p + "q"].to(dt).T, eps) * w[p + "q.norm"].to(dt)
    k = rms(h @ w[p + "k"].to(dt).T, eps) * w[p + "k.norm"].to(dt)
    v = (h @ w[p + "v"].to(dt).T).reshape(n, G, e)
    pos = torch.arange(n)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q, k = rotate_pairs(q.reshape(n, H, d), rot, pos), rotate_pairs(k.reshape(n, G, d), rot, pos)
    mask = window_mask(n, int(m["mask"]["size"]))
    out = torch.zeros(n, H, e, dtype=dt)
    for head in range(H):
        g = head // (H // G)
        s = cap((q[:, head] @ k[:, g].T) * float(m["scale"]), float(m.get("softcap") or 0.0))
        out[:, head] = masked_softmax(s, mask) @ v[:, g]
    return out.reshape(n, H * e) @ w[p + "o"].to(dt).T


# ---------------------------------------------------------------- feed-forwards
def gated_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def dense_ff(h, w, p, dt):
    return gated_ff(h, w[p + "gate"].to(dt), w[p + "up"].to(dt), w[p + "down"].to(dt))


def route(h, w, p, r, dt, margins=None):
    """(chosen experts [n, top], their weights [n, top]).  Scores are sigmoids of the router's logits; a group of
    neighbouring experts scores the sum of its two largest; the `top` largest scores among the experts of the `keep`
    best groups are chosen; the weights are those scores over their sum, times the router's scale.  `margins` (a list):
    a tensor [n] is appended, the smallest gap that decided a token's choice (between groups, and between experts)."""
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    per = E // count
    s = torch.sigmoid(h @ w[p + "router"].to(dt).T)
    group_score = s.reshape(-1, count, per).topk(min(2, per), dim=-1).values.sum(-1)      # [n, count]
    kept = torch.zeros_like(group_score, dtype=torch.bool)
    kept.scatter_(1, group_score.topk(keep, dim=-1).indices, True)
    allowed = kept[:, :, None].expand(-1, -1, per).reshape(-1, E)
    choice = torch.where(allowed, s, torch.full_like(s, -math.inf))
    idx = choice.topk(top, dim=-1).indices
    if margins is not None:
        gap = torch.full((h.shape[0],), math.inf, dtype=dt)
        if keep < count:
            o = group_score.sort(-1, descending=True).values
            gap = torch.minimum(gap, o[:, keep - 1] - o[:, keep])
        if top < per * keep:
            o = choice.sort(-1, descending=True).values
            gap = torch.minimum(gap, o[:, top - 1] - o[:, top])
        margins.append(gap)
    chosen = s.gather(1, idx)
    return idx, chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))


def moe_ff(h, w, p, mlp, dt, margins=None):
    idx, weight = route(h, w, p, mlp["router"], dt, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            q = f"{p}e{int(idx[t, j])}."
            y = gated_ff(h[t:t + 1], w[q + "gate"].to(dt), w[q + "up"].to(dt), w[q + "down"].to(dt))[0]
            out[t] = out[t] + weight[t, j] * y
    return out


# ---------------------------------------------------------------- the model
def layer_runs(cfg):
    """The layers in the order they run: the stretch start..stop-1 runs `times` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, w, tokens, dt=torch.float64, return_layers=False, margins=None, noise=None):
    """Logits [n, vocab] for one whole sequence; with `return_layers` also the residual stream after every layer run.
    `margins` (a list): every run of a routed feed-forward appends its tokens' margins (see `route`).  `noise` (a
    function of a tensor): applied to what the sublayers read and return, e.g. a rounding to 16 bits."""
    eps = float(cfg["norm"]["eps"])
    noise = noise or (lambda t: t)
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"].to(dt)[ids]
    after = []
    for i in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        h = noise(layer_norm(x, w[p + "norm1"].to(dt), w[p + "norm1.b"].to(dt), eps))
        mix = two_map_attention if layer["type"] == "attention" else window_attention
        y = noise(mix(h, w, p + "mix.", layer["mixer"], eps, dt))
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + noise(dense_ff(h, w, p + "mlp.", dt) if mlp["kind"] == "dense"
                          else moe_ff(h, w, p + "mlp.", mlp, dt, margins))
        x = x + y
        after.append(x)
    logits = noise(layer_norm(x, w["final.norm"].to(dt), w["final.norm.b"].to(dt), eps)) @ w["head"].to(dt).T
    return (logits, torch.stack(after)) if return_layers else logits

"""Typed model configuration, read from the architecture's own config.json keys.

`Qwen3Config` holds exactly what a Qwen3 (dense) config.json gives; no size of the model
lives anywhere else in the package.  The keys and their defaults follow the reference's
`Qwen3Config` (vllm-oxide, crates/vllm-oxide/src/models/qwen3.rs:26-58) with three
deliberate differences, each an error instead of a silent change of model:

* `attention_bias` defaults to False (the reference defaults it to true and thereby drops
  q_norm/k_norm, qwen3.rs:52-54,124-139; every published Qwen3 config says false);
* `hidden_act` must be "silu" (the reference requires the key and never reads it, :40);
* `rope_scaling` must be absent or null; the window keys (`use_sliding_window`,
  `sliding_window`, `max_window_layers`), which the reference ignores, are honoured.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Optional


class ConfigError(ValueError):
    """config.json is missing a key, has a value of the wrong type, or asks for something unsupported."""


_DTYPE_NAMES = {
    # crates/vllm-oxide/src/config.rs:90-105
    "bfloat16": "bfloat16", "bf16": "bfloat16",
    "float16": "float16", "fp16": "float16", "half": "float16",
    "float32": "float32", "fp32": "float32", "float": "float32",
    "float64": "float64", "fp64": "float64", "double": "float64",
}


def _need(d: dict, key: str, typ, where: str):
    if key not in d or d[key] is None:
        raise ConfigError(f"{where}: required key '{key}' is missing")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{where}: '{key}' must be an integer, got {v!r}")
        if v <= 0:
            raise ConfigError(f"{where}: '{key}' must be positive, got {v}")
    elif typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{where}: '{key}' must be a number, got {v!r}")
        v = float(v)
    return v


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    eos_token_id: Optional[int] = None

    architecture = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "Qwen3Config":
        hidden = _need(d, "hidden_size", int, where)
        heads = _need(d, "num_attention_heads", int, where)
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"{where}: no 'head_dim' and hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads}")
            head_dim = hidden // heads  # qwen3.rs:48-51
        elif isinstance(head_dim, bool) or not isinstance(head_dim, int) or head_dim <= 0:
            raise ConfigError(f"{where}: 'head_dim' must be a positive integer, got {head_dim!r}")
        kv = _need(d, "num_key_value_heads", int, where)
        if heads % kv:
            raise ConfigError(f"{where}: num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv}")
        if head_dim % 2:
            raise ConfigError(f"{where}: head_dim {head_dim} must be even for rotate-half position encoding")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{where}: hidden_act {act!r} is not supported (only 'silu')")
        if d.get("rope_scaling") is not None:
            raise ConfigError(f"{where}: rope_scaling {d['rope_scaling']!r} is not supported")
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if not isinstance(dtype, str) or dtype not in _DTYPE_NAMES:
            raise ConfigError(f"{where}: torch_dtype {dtype!r} is not one of {sorted(set(_DTYPE_NAMES))}")
        use_window = bool(d.get("use_sliding_window", False))
        window = d.get("sliding_window")
        if use_window:
            if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
                raise ConfigError(f"{where}: use_sliding_window needs a positive 'sliding_window', got {window!r}")
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        return cls(
            hidden_size=hidden,
            num_hidden_layers=_need(d, "num_hidden_layers", int, where),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            intermediate_size=_need(d, "intermediate_size", int, where),
            vocab_size=_need(d, "vocab_size", int, where),
            rms_norm_eps=_need(d, "rms_norm_eps", float, where),
            rope_theta=float(d.get("rope_theta", 1_000_000.0)),  # qwen3.rs:22-24
            max_position_embeddings=_need(d, "max_position_embeddings", int, where),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),  # qwen3.rs:55-57
            attention_bias=bool(d.get("attention_bias", False)),
            hidden_act=act,
            torch_dtype=_DTYPE_NAMES[dtype],
            use_sliding_window=use_window,
            sliding_window=int(window) if use_window else None,
            max_window_layers=int(d.get("max_window_layers", 0) or 0),
            eos_token_id=eos,
        )

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "qwen3"
        if not self.use_sliding_window:
            d["sliding_window"] = None
        return d

    def layer_window(self, layer: int) -> Optional[int]:
        """Window of a layer's attention, None for all keys: with `use_sliding_window`,
        layers from `max_window_layers` on see the last `sliding_window` positions."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{folder}: no config.json in the model folder")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def write_config_json(folder: str, config_dict: dict) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config_dict, f, indent=1, sort_keys=True)


# ---------------------------------------------------------------------------------------------------------------
_TOFILORN_MIXERS = ("mingru", "latent_attention", "hgrn2")


def _sub(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: '{key}' must be an object")
    return v


@dataclass(frozen=True)
class TofilornLayer:
    type: str                   # "mingru" | "latent_attention" | "hgrn2"
    mixer: dict                 # the mixer's sizes and constants, as config.json gives them
    ff: Optional[int]           # width of the gated feed-forward, None: the layer has none


@dataclass(frozen=True)
class TofilornConfig:
    """Tofilorn: a decoder whose layers are listed one by one in config.json, each with one of three token mixers
    (a gated recurrence, a matrix-state recurrence, windowed attention through a latent) and an optional gated
    feed-forward, over several float residual streams with learned mixing.  Keys: `vocab`, `width`, `streams`
    (absent: one plain residual stream), `norm.eps`, `layers[i]` = {type, mixer{...}, mlp: null | {kind: "dense", ff}}.
    There is no largest position: rotation angles are computed from the position."""
    vocab: int
    width: int
    streams: Optional[int]
    eps: float
    layers: tuple
    torch_dtype: str = "bfloat16"

    architecture = "Tofilorn"

    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "TofilornConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        streams = d.get("streams")
        if streams is not None:
            streams = _need(d, "streams", int, where)
        out = []
        for i, layer in enumerate(layers):
            w = f"{where}: layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"{w} must be an object")
            kind = layer.get("type")
            if kind not in _TOFILORN_MIXERS:
                raise ConfigError(f"{w}: type {kind!r} is not one of {list(_TOFILORN_MIXERS)}")
            m = _sub(layer, "mixer", w)
            if kind == "mingru":
                _need(m, "width", int, w)
            elif kind == "hgrn2":
                for k in ("heads", "dim", "vdim"):
                    _need(m, k, int, w)
            else:
                for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
                    _need(m, k, int, w)
                _need(m, "scale", float, w)
                rot = _sub(m, "rot", w)
                _need(rot, "dims", int, w + ".rot")
                _need(rot, "base", float, w + ".rot")
                if rot["dims"] % 2 or rot["dims"] > m["rot_dim"]:
                    raise ConfigError(f"{w}: rot.dims {rot['dims']} must be even and at most rot_dim {m['rot_dim']}")
                sc = rot.get("scaling")
                if sc is not None:
                    for k in ("factor", "original", "fast", "slow"):
                        _need(_sub(rot, "scaling", w), k, float, w + ".rot.scaling")
                if m.get("mask") is not None:
                    _need(_sub(m, "mask", w), "size", int, w + ".mask")
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                        raise ConfigError(f"{w}: kv_from {src!r} must name an earlier layer")
                    other = layers[src]
                    if not isinstance(other, dict) or other.get("type") != "latent_attention" or \
                            not isinstance(other.get("mixer"), dict) or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{w}: kv_from {src} must name a latent_attention layer with keys of its own")
                    for k in ("kv_rank", "rot_dim"):
                        if other["mixer"].get(k) != m[k]:
                            raise ConfigError(f"{w}: {k} differs from that of layer {src}, whose keys it reads")
            mlp = layer.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{w}: mlp must be null or of kind 'dense', got {mlp!r}")
                ff = _need(mlp, "ff", int, w + ".mlp")
            out.append(TofilornLayer(kind, dict(m), ff))
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if not isinstance(dtype, str) or dtype not in _DTYPE_NAMES:
            raise ConfigError(f"{where}: torch_dtype {dtype!r} is not one of {sorted(set(_DTYPE_NAMES))}")
        return cls(vocab=_need(d, "vocab", int, where), width=_need(d, "width", int, where), streams=streams,
                   eps=_need(_sub(d, "norm", where), "eps", float, where + ".norm"), layers=tuple(out),
                   torch_dtype=_DTYPE_NAMES[dtype])

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": [{"type": l.type, "mixer": dict(l.mixer), "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}}
                        for l in self.layers]}
        if self.streams is not None:
            d["streams"] = self.streams
        return d


# ---------------------------------------------------------------------------------------------------------------
_KESOZEN_MIXERS = ("attention", "delta")


@dataclass(frozen=True)
class KesozenLayer:
    type: str                   # "attention" | "delta"
    mixer: dict                 # the mixer's sizes and constants, as config.json gives them
    mlp: Optional[dict]         # None, {"kind": "dense", "ff"} or {"kind": "moe", "expert": {"ff"}, "router": {...}}


@dataclass(frozen=True)
class KesozenConfig:
    """Kesozen: a decoder whose layers are listed one by one in config.json, each with a norm before and after both of
    its sublayers around one float residual stream.  The mixer is attention whose keys double as values (a sink in the
    softmax, a gate per head, part of each head rotated) or a gated delta rule behind short convolutions; the
    feed-forward is dense or a mixture of experts chosen among groups, both with the squared relu.  A stretch of the
    layers (`loop`: start, stop, times) may run several times in a row with the same weights, every pass with a cache of
    its own, the normed embedding added back before each pass but the first.  Keys: `vocab`, `width`, `norm.eps`,
    `layers[i]` = {type, mixer{...}, mlp}, `loop`.  There is no largest position."""
    vocab: int
    width: int
    eps: float
    layers: tuple
    loop: Optional[tuple] = None      # (start, stop, times)
    torch_dtype: str = "bfloat16"

    architecture = "Kesozen"

    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "KesozenConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            w = f"{where}: layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"{w} must be an object")
            kind = layer.get("type")
            if kind not in _KESOZEN_MIXERS:
                raise ConfigError(f"{w}: type {kind!r} is not one of {list(_KESOZEN_MIXERS)}")
            m = _sub(layer, "mixer", w)
            for k in ("heads", "kv_heads", "dim", "vdim"):
                _need(m, k, int, w)
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{w}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
            if kind == "attention":
                _need(m, "scale", float, w)
                if m["vdim"] != m["dim"]:
                    raise ConfigError(f"{w}: the values are the keys, so vdim {m['vdim']} must equal dim {m['dim']}")
                rot = m.get("rot")
                if rot is not None:
                    rot = _sub(m, "rot", w)
                    _need(rot, "base", float, w + ".rot")
                    dims = rot.get("dims")
                    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"{w}: rot.dims {dims!r} must be even and between 0 and dim {m['dim']}")
            else:
                _need(m, "conv", int, w)
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"{w}: mlp must be null or of kind 'dense' or 'moe', got {mlp!r}")
                if mlp["kind"] == "dense":
                    _need(mlp, "ff", int, w + ".mlp")
                else:
                    _need(_sub(mlp, "expert", w + ".mlp"), "ff", int, w + ".mlp.expert")
                    r = _sub(mlp, "router", w + ".mlp")
                    E, top = _need(r, "experts", int, w + ".mlp.router"), _need(r, "top", int, w + ".mlp.router")
                    g = r.get("groups")
                    count = keep = 1
                    if g is not None:
                        g = _sub(r, "groups", w + ".mlp.router")
                        count, keep = _need(g, "count", int, w + ".mlp.router.groups"), _need(g, "keep", int, w + ".mlp.router.groups")
                    if E % count or keep > count or top > (E // count) * keep:
                        raise ConfigError(f"{w}: {E} experts in {count} groups of which {keep} are kept cannot give {top} choices")
            out.append(KesozenLayer(kind, dict(m), None if mlp is None else dict(mlp)))
        loop = d.get("loop")
        if loop is not None:
            loop = _sub(d, "loop", where)
            start, stop = loop.get("start"), loop.get("stop")
            times = _need(loop, "times", int, where + ".loop")
            for v in (start, stop):
                if isinstance(v, bool) or not isinstance(v, int):
                    raise ConfigError(f"{where}: loop.start and loop.stop must be integers")
            if not 0 <= start <= stop <= len(out):
                raise ConfigError(f"{where}: loop {start}..{stop} does not lie within the {len(out)} layers")
            loop = (start, stop, times)
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if not isinstance(dtype, str) or dtype not in _DTYPE_NAMES:
            raise ConfigError(f"{where}: torch_dtype {dtype!r} is not one of {sorted(set(_DTYPE_NAMES))}")
        return cls(vocab=_need(d, "vocab", int, where), width=_need(d, "width", int, where),
                   eps=_need(_sub(d, "norm", where), "eps", float, where + ".norm"), layers=tuple(out), loop=loop,
                   torch_dtype=_DTYPE_NAMES[dtype])

    def runs(self):
        """The layers in the order they run: [(layer, first of a pass after the first)]."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        order = [(i, False) for i in range(start)]
        for rep in range(times):
            order += [(i, rep > 0 and i == start) for i in range(start, stop)]
        return order + [(i, False) for i in range(stop, n)]

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": [{"type": l.type, "mixer": dict(l.mixer), "mlp": None if l.mlp is None else dict(l.mlp)}
                        for l in self.layers]}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d


# ---------------------------------------------------------------------------------------------------------------
_RAKIZEN_MIXERS = ("attention", "attention_2")


def _check_moe(mlp: dict, w: str) -> None:
    """`mlp` = null | {kind: dense, ff} | {kind: moe, expert{ff}, router{experts, top, groups{count, keep}}} as the
    layer-list configurations write it."""
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{w}: mlp must be null or of kind 'dense' or 'moe', got {mlp!r}")
    if mlp["kind"] == "dense":
        _need(mlp, "ff", int, w + ".mlp")
        return
    _need(_sub(mlp, "expert", w + ".mlp"), "ff", int, w + ".mlp.expert")
    r = _sub(mlp, "router", w + ".mlp")
    E, top = _need(r, "experts", int, w + ".mlp.router"), _need(r, "top", int, w + ".mlp.router")
    count = keep = 1
    if r.get("groups") is not None:
        g = _sub(r, "groups", w + ".mlp.router")
        count, keep = _need(g, "count", int, w + ".mlp.router.groups"), _need(g, "keep", int, w + ".mlp.router.groups")
    if min(E, top, count, keep) <= 0 or E % count or keep > count or top > (E // count) * keep:
        raise ConfigError(f"{w}: {E} experts in {count} groups of which {keep} are kept cannot give {top} choices")
    if r.get("scale") is not None:
        _need(r, "scale", float, w + ".mlp.router")


@dataclass(frozen=True)
class RakizenLayer:
    type: str                   # "attention" | "attention_2"
    mixer: dict                 # the mixer's sizes and constants, as config.json gives them
    mlp: Optional[dict]         # None, {"kind": "dense", "ff"} or {"kind": "moe", "expert": {"ff"}, "router": {...}}


@dataclass(frozen=True)
class RakizenConfig:
    """Rakizen: a decoder whose layers are listed one by one in config.json.  A layer has ONE layer norm (gain and bias)
    that its mixer and its feed-forward both read; their outputs are added to one float residual stream together.  The
    mixer is `attention` (every head the difference of two softmax maps over shared values, scores capped by a tanh, keys
    visible inside blocks of `mask.size` positions, a unit norm per head, an output gate; nothing is rotated) or
    `attention_2` (q and k normed over their whole projections, the first `rot.dims` elements of each head rotated in
    neighbouring pairs, capped scores, a sliding window of `mask.size` positions).  The feed-forward is a gated SiLU layer,
    a mixture of such layers routed by sigmoid scores among groups, or absent.  A stretch of the layers (`loop`: start,
    stop, times) may run several times in a row with the same weights, every pass with a cache of its own.  Keys: `vocab`,
    `width`, `norm.eps`, `layers[i]` = {type, mixer{...}, mlp}, `loop`.  There is no largest position."""
    vocab: int
    width: int
    eps: float
    layers: tuple
    loop: Optional[tuple] = None      # (start, stop, times)
    torch_dtype: str = "bfloat16"

    architecture = "Rakizen"

    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "RakizenConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            w = f"{where}: layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"{w} must be an object")
            kind = layer.get("type")
            if kind not in _RAKIZEN_MIXERS:
                raise ConfigError(f"{w}: type {kind!r} is not one of {list(_RAKIZEN_MIXERS)}")
            m = _sub(layer, "mixer", w)
            for k in ("heads", "kv_heads", "dim", "vdim"):
                if _need(m, k, int, w) <= 0:
                    raise ConfigError(f"{w}: {k} must be positive")
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{w}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
            _need(m, "scale", float, w)
            if m.get("softcap") is not None and _need(m, "softcap", float, w) < 0:
                raise ConfigError(f"{w}: softcap must not be negative")
            if m.get("mask") is not None and _need(_sub(m, "mask", w), "size", int, w + ".mask") <= 0:
                raise ConfigError(f"{w}: mask.size must be positive")
            if kind == "attention":
                _need(m, "diff", float, w)
            elif m.get("rot") is not None:
                rot = _sub(m, "rot", w)
                _need(rot, "base", float, w + ".rot")
                dims = rot.get("dims")
                if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"{w}: rot.dims {dims!r} must be even and between 0 and dim {m['dim']}")
            mlp = layer.get("mlp")
            if mlp is not None:
                _check_moe(mlp, w)
            out.append(RakizenLayer(kind, dict(m), None if mlp is None else dict(mlp)))
        loop = d.get("loop")
        if loop is not None:
            loop = _sub(d, "loop", where)
            start, stop = loop.get("start"), loop.get("stop")
            times = _need(loop, "times", int, where + ".loop")
            for v in (start, stop):
                if isinstance(v, bool) or not isinstance(v, int):
                    raise ConfigError(f"{where}: loop.start and loop.stop must be integers")
            if not 0 <= start <= stop <= len(out) or times < 1:
                raise ConfigError(f"{where}: loop {start}..{stop} x {times} does not lie within the {len(out)} layers")
            loop = (start, stop, times)
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if not isinstance(dtype, str) or dtype not in _DTYPE_NAMES:
            raise ConfigError(f"{where}: torch_dtype {dtype!r} is not one of {sorted(set(_DTYPE_NAMES))}")
        return cls(vocab=_need(d, "vocab", int, where), width=_need(d, "width", int, where),
                   eps=_need(_sub(d, "norm", where), "eps", float, where + ".norm"), layers=tuple(out), loop=loop,
                   torch_dtype=_DTYPE_NAMES[dtype])

    def runs(self):
        """The layers in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": [{"type": l.type, "mixer": dict(l.mixer), "mlp": None if l.mlp is None else dict(l.mlp)}
                        for l in self.layers]}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d


# ---------------------------------------------------------------------------------------------------------------
_DEPOLIX_MIXERS = ("latent_attention", "parallel")


def _count(d: dict, key: str, where: str, default: int = 0) -> int:
    """A whole number that may be zero."""
    v = d.get(key, default)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"{where}: '{key}' must be a whole number that is not negative, got {v!r}")
    return v


@dataclass(frozen=True)
class DepolixLayer:
    type: str                   # "latent_attention" | "parallel"
    mixer: dict                 # the mixer's sizes and constants, as config.json gives them
    mlp: Optional[dict]         # None, {"kind": "dense", "ff", "limit"} or {"kind": "moe", "expert": {"ff", "limit"}, "router": {...}}


@dataclass(frozen=True)
class DepolixConfig:
    """Depolix: a decoder whose layers are listed one by one in config.json.  A layer has ONE RMS norm with a gain stored
    around zero that its mixer and its feed-forward both read; m times the sum of their outputs is added to one float
    residual stream (`residual_mult`).  The mixer is `latent_attention` (low-rank queries; one latent and one rotated key
    part a token; rotation of halves with stretched frequencies; an output gate an element) or `parallel`: `left`,
    attention behind short convolutions with unit-RMS q and k, a learned bias by distance, a window that keeps the first
    tokens and a gate a head, beside `right`, a gated delta rule with a decay per head and key channel; each side is normed
    over the width and the result is half their sum.  The feed-forward is a clamped gated layer with biases, a mixture of
    such experts weighted by the softmax over the chosen logits, or absent.  Keys: `vocab`, `width`, `norm.eps`,
    `embedding.scale`, `residual_mult`, `logit_scale`, `layers[i]` = {type, mixer{...}, mlp}.  There is no largest position."""
    vocab: int
    width: int
    eps: float
    layers: tuple
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    torch_dtype: str = "bfloat16"

    architecture = "Depolix"

    @staticmethod
    def _check_latent(m: dict, w: str) -> None:
        for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
            _need(m, k, int, w)
        _need(m, "scale", float, w)
        rot = _sub(m, "rot", w)
        _need(rot, "base", float, w + ".rot")
        dims = rot.get("dims")
        if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > m["rot_dim"]:
            raise ConfigError(f"{w}: rot.dims {dims!r} must be even and between 0 and rot_dim {m['rot_dim']}")
        if rot.get("scaling") is not None:
            s = _sub(rot, "scaling", w + ".rot")
            for k in ("factor", "original", "fast", "slow"):
                if _need(s, k, float, w + ".rot.scaling") <= 0:
                    raise ConfigError(f"{w}: rot.scaling.{k} must be positive")

    @staticmethod
    def _check_side(m: dict, w: str) -> None:
        for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
            _need(m, k, int, w)
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{w}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")

    @classmethod
    def from_dict(cls, d: dict, where: str = "config.json") -> "DepolixConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            w = f"{where}: layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"{w} must be an object")
            kind = layer.get("type")
            if kind not in _DEPOLIX_MIXERS:
                raise ConfigError(f"{w}: type {kind!r} is not one of {list(_DEPOLIX_MIXERS)}")
            m = _sub(layer, "mixer", w)
            if kind == "latent_attention":
                cls._check_latent(m, w)
            else:
                left, right = _sub(m, "left", w), _sub(m, "right", w)
                cls._check_side(left, w + ".left")
                cls._check_side(right, w + ".right")
                _need(left, "scale", float, w + ".left")
                if left.get("mask") is not None:
                    mask = _sub(left, "mask", w + ".left")
                    _need(mask, "size", int, w + ".left.mask")
                    _count(mask, "keep_first", w + ".left.mask")
                if left.get("bias_max") is not None:
                    _need(left, "bias_max", float, w + ".left")
            mlp = layer.get("mlp")
            if mlp is not None:
                _check_moe(mlp, w)
                if _need(mlp if mlp["kind"] == "dense" else mlp["expert"], "limit", float, w + ".mlp") <= 0:
                    raise ConfigError(f"{w}: the feed-forward's limit must be positive")
            out.append(DepolixLayer(kind, dict(m), None if mlp is None else dict(mlp)))
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if not isinstance(dtype, str) or dtype not in _DTYPE_NAMES:
            raise ConfigError(f"{where}: torch_dtype {dtype!r} is not one of {sorted(set(_DTYPE_NAMES))}")
        number = lambda key, sub=None: (float((d.get(sub) or {}).get(key, 1.0)) if sub else float(d.get(key, 1.0)))
        return cls(vocab=_need(d, "vocab", int, where), width=_need(d, "width", int, where),
                   eps=_need(_sub(d, "norm", where), "eps", float, where + ".norm"), layers=tuple(out),
                   embedding_scale=number("scale", "embedding"), residual_mult=number("residual_mult"),
                   logit_scale=number("logit_scale"), torch_dtype=_DTYPE_NAMES[dtype])

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult,
                "logit_scale": self.logit_scale,
                "layers": [{"type": l.type, "mixer": dict(l.mixer), "mlp": None if l.mlp is None else dict(l.mlp)}
                           for l in self.layers]}

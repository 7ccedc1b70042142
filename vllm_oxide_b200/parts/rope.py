"""Rotary position encoding: the table of angles and the rule by which a mixer's kernel applies it.

The table is the reference's (vllm-oxide, crates/vllm-oxide/src/layers/rope.rs:50-88):
inv_freq[i] = 1 / theta^(2i/d) with a float32 pow, angle = float32(p) * inv_freq[i], and
[max_pos, d] = cos(angle) || sin(angle), all float32 on both paths.  The rotation itself
(rope.rs:129-159) happens inside the mixer's kernel, which gets the table and the rule from
`rotation_rule()`.  The reference rotates the whole head in halves (d = head_dim, rope.rs asserts it);
`rotary_dim` < head_dim rotates only the first elements of a head and `interleaved` pairs neighbouring
elements instead of halves: parameters an architecture's plan may set, not used by Qwen3.

Two more parameters, for architectures that stretch a trained context.  `scaling` = {factor, original, fast,
slow} slows the long waves down and leaves the short ones alone: with d(t) = rotary_dim * ln(original / (2 pi t))
/ (2 ln theta), the index whose wave makes t turns over `original` positions, a ramp r_i rises from 0 at
lo = max(floor(d(fast)), 0) to 1 at hi = min(ceil(d(slow)), rotary_dim - 1) (its width at least 0.001);
inv_freq[i] becomes inv_freq[i] / factor * r_i + inv_freq[i] * (1 - r_i), and cos and sin are both multiplied by
0.1 ln(factor) + 1 (the "YaRN" interpolation of Peng, Quesnelle, Fan and Shippole).  `table=False` makes no table:
the rule then carries the frequencies and the amplitude, the kernels compute float32(p) * inv_freq[i] where they
rotate, and `max_position` bounds nothing.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding, RotationRule, register_part


def scaled_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict], precise: bool = False):
    """(inv_freq float32 [rotary_dim/2], amplitude) of a rotary encoding, with the stretch of `scaling` if given.
    `precise`: the frequencies are computed in float64 and rounded once (else with a float32 power, as the reference's)."""
    half = rotary_dim // 2
    work = torch.float64 if precise else torch.float32
    i = torch.arange(half, dtype=work)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=work), (2 * i) / rotary_dim)
    if not scaling:
        return inv_freq.to(torch.float32), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if factor <= 0 or original <= 0:
        raise ValueError(f"rotary scaling needs a positive factor and original length, got {scaling!r}")

    def index_of(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))
    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), rotary_dim - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return (inv_freq / factor * ramp + inv_freq * (1.0 - ramp)).to(torch.float32), 0.1 * math.log(factor) + 1.0


class RotaryEmbedding(PositionEncoding):
    def __init__(self, head_dim: int, max_position: int, theta: float, rotary_dim: Optional[int] = None,
                 interleaved: bool = False, scaling: Optional[dict] = None, table: bool = True, device=None,
                 precise: bool = False, **_):
        d = head_dim if rotary_dim is None else int(rotary_dim)
        if d % 2 or not 0 < d <= head_dim:
            raise ValueError(f"rotary position encoding needs an even rotary_dim in (0, head_dim {head_dim}], got {d}")
        self.head_dim, self.rotary_dim, self.interleaved = head_dim, d, bool(interleaved)
        self.max_position, self.theta = max_position, float(theta)
        inv_freq, self.amplitude = scaled_frequencies(d, self.theta, scaling, precise)
        self.cos_sin = self.frequencies = None
        if table:
            t = torch.arange(max_position, dtype=torch.float32)
            freqs = t[:, None] * inv_freq[None, :]
            cos, sin = freqs.cos(), freqs.sin()
            if self.amplitude != 1.0:
                cos, sin = cos * self.amplitude, sin * self.amplitude
            self.cos_sin = torch.cat([cos, sin], dim=-1).contiguous().to(device)
        else:
            self.frequencies = inv_freq.contiguous().to(device)

    def rotation_rule(self) -> RotationRule:
        return RotationRule(self.cos_sin, self.rotary_dim, self.interleaved, self.frequencies, float(self.amplitude))


register_part("position", "rope", RotaryEmbedding)

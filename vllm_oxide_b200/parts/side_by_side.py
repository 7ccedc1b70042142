"""Two token mixers side by side: both read the same input, each output passes an RMS norm over the model width with a
plain gain, and the result is half their sum.

    out = ( RMSNorm(left(x)) * w_left + RMSNorm(right(x)) * w_right ) / 2

`left` and `right` are part specs of any two mixers.  What they keep per request is kept for them: at most one of them may
keep pages (its cache plane is the pair's), and their per-request states lie one behind the other in ONE float row of the
cache manager's state slots, each mixer seeing its own columns.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import CacheSpec, Mixer, PartSpec, StateSpec, build_part, register_part


class SideBySide(Mixer):
    def __init__(self, left: PartSpec, right: PartSpec, hidden_size: int, eps: float, left_norm: str, right_norm: str, **common):
        self.H, self.eps, self.n_left, self.n_right = int(hidden_size), float(eps), left_norm, right_norm
        self.left = build_part("mixer", left, **common)
        self.right = build_part("mixer", right, **common)
        if self.left.cache_spec() is not None and self.right.cache_spec() is not None:
            raise ValueError("two mixers side by side share one cache plane: only one of them may keep pages")
        self._states = []
        off = 0
        for m in (self.left, self.right):
            s = m.state_spec()
            if s is not None and (s.dtype != torch.float32 or len(s.shape) != 1):
                raise ValueError("mixers side by side keep their states as one float row each")
            n = 0 if s is None else int(s.shape[0])
            self._states.append((off, n))
            off += n
        self._state_floats = off
        self.w_left = self.w_right = None
        self.graph_safe = self.left.graph_safe and self.right.graph_safe

    def parts(self):
        return [self.left, self.right]

    def tensor_specs(self) -> List[TensorSpec]:
        return (self.left.tensor_specs() + self.right.tensor_specs()
                + [TensorSpec(self.n_left, (self.H,), "norm"), TensorSpec(self.n_right, (self.H,), "norm")])

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for m in (self.left, self.right):
            m.load({s.name: tensors[s.name] for s in m.tensor_specs()})
        self.w_left, self.w_right = tensors[self.n_left].contiguous(), tensors[self.n_right].contiguous()

    def cache_spec(self) -> Optional[CacheSpec]:
        return self.left.cache_spec() or self.right.cache_spec()

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self._state_floats,), torch.float32) if self._state_floats else None

    def forward(self, x, ctx, cache, state, write_cache: bool = True):
        outs = []
        for m, (off, n) in zip((self.left, self.right), self._states):
            own_cache = cache if m.cache_spec() is not None else None
            own_state = state[:, off:off + n] if n else None
            outs.append(m.forward(x, ctx, own_cache, own_state, write_cache))
        a, b = outs
        if a.data_ptr() == b.data_ptr():
            raise RuntimeError("the two mixers wrote their outputs into the same workspace buffer")
        out = ctx.ws.get("side_by_side_out", x.shape[0], self.H, x.dtype)
        kernels.pair_norm_mean(a, b, self.w_left, self.w_right, out, self.eps)
        return out


register_part("mixer", "side_by_side", SideBySide)

"""One float residual stream around layers whose mixer and feed-forward read the SAME norm ("parallel" layers).

    h = LayerNorm(x) * w + b;      x <- x + (mixer(h) + feed_forward(h))          (feed_forward None: x <- x + mixer(h))

The stream is float on both paths and lives in one workspace buffer [tokens, width]; it is never rounded to 16 bits.
One kernel (`kernels.layer_norm_step`) adds the two outputs of the layer before into the stream and forms this layer's
one norm, so a layer costs one pass over the stream.  Between blocks the convention of the other blocks holds:
`(hidden, residual)` = (the mixer's output, not yet in the stream; the stream); the feed-forward's output, which is
pending beside it, travels in `ctx.pending_second`.

The norm kind `layernorm_stream` (mean taken off, variance as the mean of squared deviations, gain and optional bias)
also serves as a plan's last norm, on the wanted rows.  The norm kind `rmsnorm_parallel_stream` is the same arrangement with
an RMS norm (x / rms(x) * w, or * (1 + w) for a gain stored around zero) and a factor on what enters the stream:
x <- x + mult * (mixer(h) + feed_forward(h)).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Block, Norm, PartSpec, build_part, register_part


class StreamLayerNorm(Norm):
    """(x - mean(x)) / sqrt(var(x) + eps) * w + b on a float residual stream, fused with the stream's update."""
    graph_safe = True

    def __init__(self, size: int, eps: float, weight_name: str, bias_name: Optional[str] = None, **_):
        self.size, self.eps, self.weight_name, self.bias_name = int(size), float(eps), weight_name, bias_name
        self.weight = self.bias = None

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.weight_name, (self.size,), "norm")]
        if self.bias_name:
            specs.append(TensorSpec(self.bias_name, (self.size,), "coefficient", init="small"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()
        self.bias = tensors[self.bias_name].contiguous() if self.bias_name else None

    def enter(self, hidden, stream, ctx, name: str, rows=None, n_rows=None):
        """The pending outputs (`hidden` and `ctx.pending_second`) go into `stream` (None: the stream begins with
        `hidden`), and this norm of the result is returned with the stream."""
        init = stream is None
        # a stream that begins has nothing pending beside the embedded tokens (a context may be walked twice: what the
        # last layer of the walk before left is not this walk's)
        second = None if init else getattr(ctx, "pending_second", None)
        T = hidden.shape[0] if hidden is not None else stream.shape[0]
        dtype = hidden.dtype if hidden is not None else ctx.ws.dtype
        if init:
            stream = ctx.ws.get("residual_stream", T, self.size, torch.float32)
        out = ctx.ws.get(name, T if rows is None else n_rows, self.size, dtype)
        kernels.layer_norm_step(stream, self.eps, ctx.err, y1=hidden, y2=second, w=self.weight, b=self.bias, out=out,
                                rows=rows, n_out=n_rows, init=init)
        if rows is None:
            ctx.pending_second = None
        return out, stream

    def forward(self, x, residual, ctx, rows=None, n_rows=None, name="normed"):
        """As a model's last norm: norm(stream after the pending writes), on the wanted rows."""
        return self.enter(x, residual, ctx, name, rows=rows, n_rows=n_rows)


class StreamRMSNorm(Norm):
    """x / sqrt(mean(x^2) + eps) * (offset + w) on a float residual stream, fused with the stream's update
    x <- x + mult * (mixer + feed-forward); `one_plus`: the gain is stored around zero (offset 1).  `open_scale`: the
    factor on the embedded tokens where the stream begins (applied in float, so the table's values are not rounded twice);
    `out_scale`: a factor on the norm's output."""
    graph_safe = True

    def __init__(self, size: int, eps: float, weight_name: str, one_plus: bool = False, mult: float = 1.0,
                 open_scale: float = 1.0, out_scale: float = 1.0, **_):
        self.size, self.eps, self.weight_name = int(size), float(eps), weight_name
        self.one_plus, self.mult, self.open_scale = bool(one_plus), float(mult), float(open_scale)
        # a factor on the norm's output (a model's last norm: the factor on its logits), folded into the gain in float
        self.out_scale = float(out_scale)
        self.gain_offset = self.out_scale if self.one_plus else 0.0
        self.weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        if self.one_plus:
            return [TensorSpec(self.weight_name, (self.size,), "coefficient", init="small")]
        return [TensorSpec(self.weight_name, (self.size,), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors[self.weight_name]
        self.weight = (w * self.out_scale if self.out_scale != 1.0 else w).contiguous()

    def enter(self, hidden, stream, ctx, name: str, rows=None, n_rows=None):
        init = stream is None
        second = None if init else getattr(ctx, "pending_second", None)
        T = hidden.shape[0] if hidden is not None else stream.shape[0]
        dtype = hidden.dtype if hidden is not None else ctx.ws.dtype
        if init:
            stream = ctx.ws.get("residual_stream", T, self.size, torch.float32)
        out = ctx.ws.get(name, T if rows is None else n_rows, self.size, dtype)
        kernels.rms_norm_step(stream, self.eps, ctx.err, y1=hidden, y2=second, w=self.weight, out=out, rows=rows, n_out=n_rows,
                              init=init, mult=self.mult, open_scale=self.open_scale, gain_offset=self.gain_offset)
        if rows is None:
            ctx.pending_second = None
        return out, stream

    def forward(self, x, residual, ctx, rows=None, n_rows=None, name="normed"):
        """As a model's last norm: norm(stream after the pending writes), on the wanted rows."""
        return self.enter(x, residual, ctx, name, rows=rows, n_rows=n_rows)

    def pending_into(self, x, hidden, second, init: bool, ctx) -> None:
        kernels.rms_norm_step(x, 0.0, ctx.err, y1=hidden, y2=second, init=init, mult=self.mult, open_scale=self.open_scale)


class ParallelBlock(Block):
    def __init__(self, mixer: PartSpec, feed_forward: Optional[PartSpec], norm: PartSpec, size: int, **common):
        self.size = int(size)
        self.norm = build_part("norm", norm, **common)
        self.mixer = build_part("mixer", mixer, **common)
        self.feed_forward = build_part("feed_forward", feed_forward, **common) if feed_forward is not None else None
        if not isinstance(self.norm, (StreamLayerNorm, StreamRMSNorm)):
            raise ValueError("the parallel block fuses its norm into the stream's kernel: it must be of kind "
                             "'layernorm_stream' or 'rmsnorm_parallel_stream'")
        self._parts = [p for p in (self.norm, self.mixer, self.feed_forward) if p is not None]
        self.input_norm = self.norm
        self.graph_safe = all(p.graph_safe for p in self._parts)

    def parts(self):
        return list(self._parts)

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load({s.name: tensors[s.name] for s in p.tensor_specs()})

    def forward(self, hidden, residual, ctx, cache, state, write_cache=True):
        normed, stream = self.norm.enter(hidden, residual, ctx, "normed")
        y = self.mixer.forward(normed, ctx, cache, state, write_cache)
        ctx.pending_second = self.feed_forward.forward(normed, ctx) if self.feed_forward is not None else None
        return y, stream


def stream_value(hidden, stream, ctx, norm=None) -> torch.Tensor:
    """The residual stream [tokens, width] (float, a new tensor) after the pending writes: what the next layer's norm
    would see.  For inspection; no step of the engine needs it.  `norm`: a block's norm that has factors of its own on the
    pending outputs (`StreamRMSNorm`)."""
    if norm is not None and hasattr(norm, "pending_into"):
        x = stream.clone() if stream is not None else torch.zeros((hidden.shape[0], hidden.shape[1]), dtype=torch.float32,
                                                                  device=hidden.device)
        norm.pending_into(x, hidden, None if stream is None else getattr(ctx, "pending_second", None), stream is None, ctx)
        return x
    if stream is None:
        x = torch.zeros((hidden.shape[0], hidden.shape[1]), dtype=torch.float32, device=hidden.device)
        kernels.layer_norm_step(x, 0.0, ctx.err, y1=hidden, y2=getattr(ctx, "pending_second", None), init=True)
        return x
    x = stream.clone()
    kernels.layer_norm_step(x, 0.0, ctx.err, y1=hidden, y2=getattr(ctx, "pending_second", None))
    return x


register_part("norm", "layernorm_stream", StreamLayerNorm)
register_part("norm", "rmsnorm_parallel_stream", StreamRMSNorm)
register_part("block", "parallel", ParallelBlock)

"""SwiGLU feed-forward: down( silu(gate(x)) * up(x) ) with gate and up merged into one product
(vllm-oxide, crates/vllm-oxide/src/models/qwen3.rs:60-87, crates/vllm-oxide/src/layers/activation.rs:17-21)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import FeedForward, register_part
from .linear import linear, linear_into_stream, tc5_product


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str,
                 names=("gate_proj.weight", "up_proj.weight", "down_proj.weight"), **_):
        """`names`: what the checkpoint calls the gate, up and down matrices behind `prefix`."""
        self.H, self.I, self.prefix = hidden_size, intermediate_size, prefix
        self.n_gate, self.n_up, self.n_down = (prefix + n for n in names)
        self.wgu = self.wdown = None
        self.interleaved = False

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.n_gate, (self.I, self.H), "matrix", self.H),
                TensorSpec(self.n_up, (self.I, self.H), "matrix", self.H),
                TensorSpec(self.n_down, (self.H, self.I), "matrix", self.I)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        gate, up = tensors[self.n_gate], tensors[self.n_up]
        self.interleaved = self.I % 8 == 0
        if self.interleaved:
            # groups of eight gate rows followed by the eight up rows of the same outputs: one 16-row tile of the
            # product then holds both halves of eight outputs, and the activation becomes the product's epilogue
            self.wgu = torch.stack([gate.reshape(self.I // 8, 8, self.H), up.reshape(self.I // 8, 8, self.H)],
                                   dim=1).reshape(2 * self.I, self.H).contiguous()
        else:
            # rows of gate, then up (crates/vllm-oxide/src/layers/linear.rs:132-138)
            self.wgu = torch.cat([gate, up], dim=0).contiguous()
        self.wdown = tensors[self.n_down].contiguous()

    adds_into_stream = True

    def forward(self, x, ctx, add_into=None):
        """`add_into`: the residual stream; the down product then adds its result there and nothing is returned."""
        T = x.shape[0]
        act = ctx.ws.get("act", T, self.I, x.dtype)
        if self.interleaved and kernels.gemm_skinny_supported(x, self.wgu):
            # decode-sized steps: the activation is the epilogue of the gate|up product
            kernels.gemm_skinny(x, self.wgu, act, kernels.EPI_SWIGLU, ctx.err)
        elif self.interleaved and tc5_product(x, self.wgu, act, kernels.EPI_SWIGLU, ctx):
            pass
        else:
            gu = linear(x, self.wgu, ctx.ws.get("gate_up", T, 2 * self.I, x.dtype), ctx)
            kernels.silu_mul(gu, act, T, self.interleaved)
        if add_into is not None:
            linear_into_stream(act, self.wdown, add_into)
            return None
        return linear(act, self.wdown, ctx.ws.get("mlp_out", T, self.H, x.dtype), ctx)

    # ---- the same with the residual stream kept inside the products (decode-sized steps)
    def can_forward_on_stream(self, stream, ctx) -> bool:
        act = ctx.ws.get("act", stream.shape[0], self.I, stream.dtype)
        return (self.interleaved and kernels.gemm_skinny_supported(stream, self.wgu)
                and kernels.gemm_skinny_supported(act, self.wdown))

    def forward_on_stream(self, stream, norm, ctx, prenormed=None, emit_norm=None):
        """stream += down(SiLU(gate) * up) of RMSNorm(stream): the norm inside the gate|up product, the sum made by
        the down product.  `prenormed` / `emit_norm` as in the attention part: the norm's arithmetic done by the product
        before, and left behind for the part after."""
        from .attention import leave_prenormed
        act = ctx.ws.get("act", stream.shape[0], self.I, stream.dtype)
        if prenormed is not None:
            kernels.gemm_skinny(prenormed.scaled, self.wgu, act, kernels.EPI_SWIGLU, ctx.err, eps=norm.eps,
                                prenormed=prenormed.parts)
        else:
            kernels.gemm_skinny(stream, self.wgu, act, kernels.EPI_SWIGLU, ctx.err, norm_weight=norm.weight, eps=norm.eps)
        left = leave_prenormed(emit_norm, "after_feed_forward", stream, ctx)
        kernels.gemm_skinny(act, self.wdown, stream, kernels.EPI_ADD, ctx.err,
                            emit=(emit_norm.weight, left.scaled, left.parts) if left else None)
        return left


class ClampedGLU(FeedForward):
    """down( g * sigmoid(1.702 g) * (u + 1) ) with g = min(gate(x), limit) and u = clamp(up(x), -limit, limit); gate and up
    are one product; `bias`: all three projections have biases (<name>.b), which stay float."""
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, prefix: str, bias: bool = True,
                 names=("gate", "up", "down"), **_):
        self.H, self.I, self.limit, self.bias = int(hidden_size), int(intermediate_size), float(limit), bool(bias)
        if not self.limit > 0.0:
            raise ValueError(f"the clamp of a gated feed-forward must be positive, not {limit}")
        self.n_gate, self.n_up, self.n_down = (prefix + n for n in names)
        self.wgu = self.wdown = self.bgu = self.bdown = None

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.n_gate, (self.I, self.H), "matrix", self.H), TensorSpec(self.n_up, (self.I, self.H), "matrix", self.H),
                 TensorSpec(self.n_down, (self.H, self.I), "matrix", self.I)]
        if self.bias:
            specs += [TensorSpec(self.n_gate + ".b", (self.I,), "coefficient", init="small"),
                      TensorSpec(self.n_up + ".b", (self.I,), "coefficient", init="small"),
                      TensorSpec(self.n_down + ".b", (self.H,), "coefficient", init="small")]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.wgu = torch.cat([tensors[self.n_gate], tensors[self.n_up]], dim=0).contiguous()
        self.wdown = tensors[self.n_down].contiguous()
        if self.bias:
            self.bgu = torch.cat([tensors[self.n_gate + ".b"], tensors[self.n_up + ".b"]]).contiguous()
            self.bdown = tensors[self.n_down + ".b"].contiguous()

    def forward(self, x, ctx):
        T = x.shape[0]
        gu = linear(x, self.wgu, ctx.ws.get("gate_up", T, 2 * self.I, x.dtype), ctx)
        act = ctx.ws.get("act", T, self.I, x.dtype)
        kernels.clamped_glu(gu, self.bgu, act, self.limit)
        out = ctx.ws.get("mlp_out", T, self.H, x.dtype)
        if x.dtype == torch.float32:
            kernels.gemm_f32(act, self.wdown, out, bias=self.bdown)
            return out
        linear(act, self.wdown, out, ctx)
        if self.bdown is not None:
            kernels.add_bias(out, self.bdown)
        return out


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "glu_clamped", ClampedGLU)

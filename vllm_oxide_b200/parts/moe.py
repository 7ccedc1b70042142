"""A dense feed-forward with the squared relu, and a mixture of experts chosen among groups.

`ReluSquaredMLP`: down(max(up(x), 0)^2).

`RoutedExperts`: `experts` such feed-forwards (<prefix>e<i>.up, <prefix>e<i>.down), of which a token uses `top`.
Router logits z = W_r x are float (the input may be the model type's rounding of x), scores s = softmax(z) over all
experts; the choice is by s + correction; the experts form `groups` equal groups of neighbours, a group counts by its
best choice score and only experts of the `keep` best groups can be chosen; the chosen experts are weighted by their
plain scores s, not renormalised, and the output is the weighted sum of their outputs.  Nothing outside sees the
experts: the step's (token, choice) pairs are sorted by expert on the device, the experts' products run over the sorted
rows (each expert's rows padded to a row tile), and a last kernel sums a token's rows in order.  No count leaves the
device, so a step launches the same kernels whatever the router decides.

Options of `RoutedExperts`, for designs that route otherwise: `activation` "silu_gated" makes an expert
down(SiLU(gate(x)) * up(x)) (<prefix>e<i>.gate beside up and down; gate and up rows are stored in pairs so that the
activation is the epilogue of ONE product); `scores` "sigmoid" takes s = sigmoid(z) instead of the softmax; `correction`
False has no correction tensor (the choice is by s); `group_top` 2 lets a group count by the sum of its two best choice
scores; `normalise` divides the chosen scores by their sum (+ 1e-20); `weight_scale` multiplies them; `router_bias` adds <prefix>router.b to the logits;
`activation` "glu_clamped" with `limit` makes an expert down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate(x), limit),
u = clamp(up(x), -limit, limit).  The softmax over the chosen logits alone is `scores` "softmax" with `normalise` and no
correction: the chosen shares of the full softmax, divided by their sum.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import FeedForward, register_part
from .linear import linear


# bfloat16 steps with at least this many (token, choice) pairs run the experts' products on the tcgen05 tensor cores (row
# tiles of 128); smaller ones stream the experts' rows pair by pair (moe_gemv).  The 32-bit path, and widths those two
# refuse, take the float-accumulating kernel with row tiles of 64.
TC5_MIN_PAIRS = 256


class ReluSquaredMLP(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str, names=("up", "down"), **_):
        self.H, self.I = int(hidden_size), int(intermediate_size)
        self.n_up, self.n_down = (prefix + n for n in names)
        self.wup = self.wdown = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.n_up, (self.I, self.H), "matrix", self.H), TensorSpec(self.n_down, (self.H, self.I), "matrix", self.I)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.wup, self.wdown = tensors[self.n_up].contiguous(), tensors[self.n_down].contiguous()

    def forward(self, x, ctx):
        T = x.shape[0]
        act = linear(x, self.wup, ctx.ws.get("act", T, self.I, x.dtype), ctx)
        kernels.relu_squared(act, act)
        return linear(act, self.wdown, ctx.ws.get("mlp_out", T, self.H, x.dtype), ctx)


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, expert_size: int, experts: int, top: int, prefix: str, groups: int = 1, keep: int = 1,
                 names=("up", "down", "router", "correction"), activation: str = "relu2", gate_name: str = "gate",
                 scores: str = "softmax", correction: bool = True, group_top: int = 1, normalise: bool = False,
                 weight_scale: float = 1.0, router_bias: bool = False, limit: float = 0.0, **_):
        self.H, self.I, self.E, self.top = int(hidden_size), int(expert_size), int(experts), int(top)
        self.groups, self.keep, self.prefix = int(groups), int(keep), prefix
        if self.E % self.groups or self.keep > self.groups or self.top > (self.E // self.groups) * self.keep:
            raise ValueError(f"{self.E} experts in {self.groups} groups of which {self.keep} are kept cannot give {self.top} choices")
        if activation not in ("relu2", "silu_gated", "glu_clamped") or scores not in ("softmax", "sigmoid") or group_top not in (1, 2):
            raise ValueError(f"unknown choice among activation {activation!r}, scores {scores!r}, group_top {group_top!r}")
        self.n_up, self.n_down, self.n_router, self.n_correction = names
        self.n_gate, self.gated = gate_name, activation in ("silu_gated", "glu_clamped")
        self.limit = float(limit) if activation == "glu_clamped" else 0.0
        if activation == "glu_clamped" and not self.limit > 0.0:
            raise ValueError(f"clamped experts need a positive limit, not {limit}")
        self.has_router_bias = bool(router_bias)
        self.sigmoid_scores, self.has_correction, self.group_top = scores == "sigmoid", bool(correction), int(group_top)
        self.normalise, self.weight_scale = bool(normalise), float(weight_scale)
        self.wup = self.wdown = self.router = self.correction = self.router_b = None

    def _expert(self, e: int, name: str) -> str:
        return f"{self.prefix}e{e}.{name}"

    def tensor_specs(self) -> List[TensorSpec]:
        specs = []
        for e in range(self.E):
            if self.gated:
                specs.append(TensorSpec(self._expert(e, self.n_gate), (self.I, self.H), "matrix", self.H))
            specs += [TensorSpec(self._expert(e, self.n_up), (self.I, self.H), "matrix", self.H),
                      TensorSpec(self._expert(e, self.n_down), (self.H, self.I), "matrix", self.I)]
        specs.append(TensorSpec(self.prefix + self.n_router, (self.E, self.H), "coefficient", self.H, init="normal"))
        if self.has_router_bias:
            specs.append(TensorSpec(self.prefix + self.n_router + ".b", (self.E,), "coefficient", init="small"))
        if self.has_correction:
            specs.append(TensorSpec(self.prefix + self.n_correction, (self.E,), "coefficient", init="small"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        up = torch.stack([tensors[self._expert(e, self.n_up)] for e in range(self.E)])
        if self.gated:
            # rows in pairs (gate row, up row of the same output): the activation becomes the first product's epilogue
            gate = torch.stack([tensors[self._expert(e, self.n_gate)] for e in range(self.E)])
            up = torch.stack([gate, up], dim=2).reshape(self.E, 2 * self.I, self.H)
        self.wup = up.contiguous()
        self.wdown = torch.stack([tensors[self._expert(e, self.n_down)] for e in range(self.E)]).contiguous()
        self.router = tensors[self.prefix + self.n_router].contiguous()
        self.correction = tensors[self.prefix + self.n_correction].contiguous() if self.has_correction else None
        self.router_b = tensors[self.prefix + self.n_router + ".b"].contiguous() if self.has_router_bias else None

    def _route(self, x, ids, weights, T: int) -> None:
        kernels.moe_route(x, self.router, self.correction, ids, weights, T, self.top, self.groups, self.keep,
                          sigmoid_scores=self.sigmoid_scores, group_top=self.group_top, normalise=self.normalise,
                          weight_scale=self.weight_scale, router_bias=self.router_b)

    def forward(self, x, ctx):
        T, top = x.shape[0], self.top
        n = T * top
        # bfloat16 steps of many pairs: the experts' products on the tcgen05 tensor cores, over rows gathered into expert order
        fast = (n >= TC5_MIN_PAIRS and kernels.moe_gemm_tc5_supported(x, self.wup) and self.I % 8 == 0)
        ids = ctx.ws.get_flat("moe_ids", n, torch.int32)
        weights = ctx.ws.get_flat("moe_weights", n, torch.float32)
        if (not fast and x.dtype == torch.bfloat16 and self.I % 8 == 0 and kernels.moe_gemv_supported(x, self.wup, n)):
            # bfloat16 steps of few pairs (decoding): nothing is sorted into tiles; the pairs are listed by expert and each
            # streams its expert's rows
            order = ctx.ws.get_flat("moe_order", n, torch.int32)
            self._route(x, ids, weights, T)
            kernels.moe_order(ids, order, n, self.E)
            act = ctx.ws.get_flat("moe_act", n * self.I, x.dtype).view(n, self.I)
            kernels.moe_gemv(x, self.wup, act, ids, order, n, top, not self.gated, silu_pairs=self.gated, glu_limit=self.limit)
            y = ctx.ws.get_flat("moe_y", n * self.H, torch.float32).view(n, self.H)
            kernels.moe_gemv(act, self.wdown, y, ids, order, n, top, False)
            out = ctx.ws.get("mlp_out", T, self.H, x.dtype)
            kernels.moe_combine(y, None, weights, out, T, top)
            return out
        tile = kernels.moe_tc5_row_tile() if fast else kernels.moe_row_tile()
        # every expert's rows are padded to a row tile: at most tile - 1 rows for each expert that has any
        max_rows = (n + min(self.E, n) * (tile - 1) + tile - 1) // tile * tile
        slot_of = ctx.ws.get_flat("moe_slot_of", n, torch.int32)
        row_token = ctx.ws.get_flat("moe_row_token", max_rows, torch.int32)
        tile_expert = ctx.ws.get_flat("moe_tile_expert", max_rows // kernels.moe_row_tile(), torch.int32)
        self._route(x, ids, weights, T)
        kernels.moe_align(ids, slot_of, row_token, tile_expert, n, top, self.E, pad=tile)
        act = ctx.ws.get_flat("moe_act", max_rows * self.I, x.dtype).view(max_rows, self.I)
        y = ctx.ws.get_flat("moe_y", max_rows * self.H, torch.float32).view(max_rows, self.H)
        if fast:
            rows = ctx.ws.get_flat("moe_rows", max_rows * self.H, x.dtype).view(max_rows, self.H)
            kernels.moe_gather_rows(x, rows, row_token)
            kernels.moe_gemm_tc5(rows, self.wup, act, row_token, tile_expert, not self.gated, ctx.err, silu_pairs=self.gated,
                                 glu_limit=self.limit)
            kernels.moe_gemm_tc5(act, self.wdown, y, row_token, tile_expert, False, ctx.err)
        else:
            kernels.moe_gemm(x, self.wup, act, row_token, tile_expert, relu_squared=not self.gated, gather=True,
                             silu_pairs=self.gated, glu_limit=self.limit)
            kernels.moe_gemm(act, self.wdown, y, row_token, tile_expert, relu_squared=False, gather=False)
        out = ctx.ws.get("mlp_out", T, self.H, x.dtype)
        kernels.moe_combine(y, slot_of, weights, out, T, top)
        return out


register_part("feed_forward", "relu2_mlp", ReluSquaredMLP)
register_part("feed_forward", "routed_experts", RoutedExperts)

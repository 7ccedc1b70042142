"""The gated delta rule as a token mixer: a matrix state per head instead of pages.

With `heads` value heads of size vdim and `kv_heads` query/key heads of size dim (value head h reads query/key head
h / (heads / kv_heads)), and x the mixer's input:

    q, k, v = SiLU(conv(W_q x)), SiLU(conv(W_k x)), SiLU(conv(W_v x))      short causal convolutions over time, one filter
                                                                           a channel (<tensor>.conv [channels, taps], the
                                                                           last tap is the current token's)
    q, k    = unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times dim^(-1/2)
    beta    = sigmoid(W_b x),   g = exp(-exp(A_log) * softplus(W_a x + dt_bias))        one of each per value head
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                      per head, S [dim, vdim]
    out     = W_o [ RMSNorm_vdim(o) * norm * SiLU(W_g x) ]                               norm: one weight for all heads

Options for designs that gate otherwise: `decay_rank` r > 0 gives the decay one number a head AND key channel,
g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 x) + dt_bias)) laid out heads x dim (a1 [r, hidden], a2 [heads * dim, r]), which
multiplies the rows of S; `gate_rank` r > 0 makes the output gate W_g2 (W_g1 x); `gate` "sigmoid" multiplies by
sigmoid(gate) instead of SiLU(gate).

All projections that read x are one product (the low-rank ones are followed by a small second product each).  The state of a request, [heads, dim, vdim] floats followed by the last taps - 1
inputs of every convolution channel, lives in the cache manager's state slots (float; zeroed when a slot is assigned).
Unit vectors, beta, the decay, the recurrence and the norm are float on both paths (csrc/kernels/delta.cu).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Mixer, StateSpec, register_part
from .linear import linear


SHORT_PORTIONS = 8      # up to this many tokens a request, the convolution and its state are one kernel


class GatedDelta(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, taps: int, eps: float,
                 prefix: str, dtype=None, device=None, decay_rank: int = 0, gate_rank: int = 0, gate: str = "silu", **_):
        self.H, self.nh, self.kvh, self.dk, self.dv = int(hidden_size), int(num_heads), int(num_kv_heads), int(dim), int(vdim)
        self.taps, self.eps, self.prefix = int(taps), float(eps), prefix
        if self.nh % self.kvh:
            raise ValueError(f"heads {self.nh} is not a multiple of kv_heads {self.kvh}")
        if self.dk > 256:
            raise ValueError(f"the delta-rule scan keeps a column of the state in registers: dim up to 256, not {self.dk}")
        if not 1 <= self.taps <= 9:
            raise ValueError(f"the short convolution takes 1 to 9 taps, not {self.taps}")
        # a rank of -1 is read from the checkpoint's tensors (a1 [rank, hidden], g1 [rank, hidden]) when they are loaded
        self.decay_rank, self.gate_rank = int(decay_rank), int(gate_rank)
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"the output gate is 'silu' or 'sigmoid', not {gate!r}")
        self.gate_sigmoid = gate == "sigmoid"
        self.channels = 2 * self.kvh * self.dk + self.nh * self.dv
        self.matrix_floats = self.nh * self.dk * self.dv
        self.w_in = self.wo = self.conv_w = self.A_log = self.dt_bias = self.norm_weight = self.w_a2 = self.w_g2 = None
        if self.decay_rank >= 0 and self.gate_rank >= 0:
            self._layout()

    def _layout(self) -> None:
        """Where the parts of a projected row lie."""
        up8 = lambda n: (n + 7) // 8 * 8
        self.channels = 2 * self.kvh * self.dk + self.nh * self.dv           # q | k | v: what the convolutions see
        # then, in the first product's row: the output gate (or its low-rank input), beta, the decay (or its low-rank input)
        self.gate_off = self.channels
        self.b_off = self.gate_off + (self.gate_rank or self.nh * self.dv)
        self.a_off = self.b_off + self.nh
        self.width1 = up8(self.a_off + (self.decay_rank or self.nh))         # rows stay 16-byte aligned
        # and behind it what second, small products make of the low-rank inputs: a decay pre-activation a head and key
        # channel, a gate a head and value channel
        self.a_full = self.width1
        self.g_full = up8(self.a_full + (self.nh * self.dk if self.decay_rank else 0))
        self.width = up8(self.g_full + (self.nh * self.dv if self.gate_rank else 0))

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, qk, vd = self.prefix, self.H, self.kvh * self.dk, self.nh * self.dv
        conv = lambda name, c: TensorSpec(p + name + ".conv", (c, self.taps), "coefficient", self.taps, init="normal")
        specs = [TensorSpec(p + "q", (qk, H), "matrix", H), conv("q", qk), TensorSpec(p + "k", (qk, H), "matrix", H), conv("k", qk),
                 TensorSpec(p + "v", (vd, H), "matrix", H), conv("v", vd), TensorSpec(p + "b", (self.nh, H), "matrix", H),
                 TensorSpec(p + "A_log", (self.nh,), "coefficient", init="normal"), TensorSpec(p + "norm", (self.dv,), "norm")]
        if self.decay_rank:
            r = self.decay_rank
            specs += [TensorSpec(p + "a1", (r, H), "matrix", H), TensorSpec(p + "a2", (self.nh * self.dk, r), "matrix", r),
                      TensorSpec(p + "dt_bias", (self.nh * self.dk,), "coefficient", init="normal")]
        else:
            specs += [TensorSpec(p + "a", (self.nh, H), "matrix", H), TensorSpec(p + "dt_bias", (self.nh,), "coefficient", init="normal")]
        if self.gate_rank:
            r = self.gate_rank
            specs += [TensorSpec(p + "g1", (r, H), "matrix", H), TensorSpec(p + "g2", (vd, r), "matrix", r)]
        else:
            specs.append(TensorSpec(p + "g", (vd, H), "matrix", H))
        return specs + [TensorSpec(p + "o", (H, vd), "matrix", vd)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        if self.decay_rank < 0:
            self.decay_rank = int(tensors[p + "a1"].shape[0])
        if self.gate_rank < 0:
            self.gate_rank = int(tensors[p + "g1"].shape[0])
        self._layout()
        rows = [tensors[p + n] for n in ("q", "k", "v", "g1" if self.gate_rank else "g", "b", "a1" if self.decay_rank else "a")]
        rows.append(rows[0].new_zeros((self.width1 - sum(r.shape[0] for r in rows), self.H)))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_a2 = tensors[p + "a2"].contiguous() if self.decay_rank else None
        self.w_g2 = tensors[p + "g2"].contiguous() if self.gate_rank else None
        self.conv_w = torch.cat([tensors[p + n + ".conv"] for n in ("q", "k", "v")], dim=0).contiguous()
        self.A_log, self.dt_bias = tensors[p + "A_log"].contiguous(), tensors[p + "dt_bias"].contiguous()
        self.norm_weight, self.wo = tensors[p + "norm"].contiguous(), tensors[p + "o"].contiguous()

    def state_spec(self) -> StateSpec:
        return StateSpec((self.matrix_floats + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x, ctx, cache, state, write_cache: bool = True):
        T, B = x.shape[0], ctx.launch_requests
        row = ctx.ws.get("delta_in", T, self.width, x.dtype)
        proj = linear(x, self.w_in, row[:, :self.width1], ctx)
        if self.decay_rank:
            linear(row[:, self.a_off:self.a_off + self.decay_rank], self.w_a2, row[:, self.a_full:self.a_full + self.nh * self.dk], ctx)
        if self.gate_rank:
            linear(row[:, self.gate_off:self.gate_off + self.gate_rank], self.w_g2, row[:, self.g_full:self.g_full + self.nh * self.dv], ctx)
        proj = row
        qkv = ctx.ws.get("delta_qkv", T, self.channels, torch.float32)
        if ctx.max_q <= SHORT_PORTIONS:
            # short portions (decoding): a thread a (request, channel) does the filter and leaves the slot's inputs, one launch
            kernels.short_conv_step(proj, self.channels, self.conv_w, state, self.matrix_floats, ctx.cu_q, ctx.state_slots,
                                    qkv, B, ctx.err)
        else:
            kernels.short_conv_silu(proj, self.channels, self.conv_w, state, self.matrix_floats, ctx.token_req, ctx.cu_q,
                                    ctx.state_slots, qkv, T, ctx.err)
            kernels.short_conv_state(proj, self.channels, self.taps, state, self.matrix_floats, ctx.cu_q, ctx.state_slots, B)
        raw = ctx.ws.get("delta_raw", T, self.nh * self.dv, torch.float32)
        kernels.delta_scan(qkv, proj, self.b_off, self.a_full if self.decay_rank else self.a_off, self.A_log, self.dt_bias, state,
                           ctx.cu_q, ctx.state_slots, raw, B, self.nh, self.kvh, self.dk, self.dv, ctx.err,
                           channel_decay=bool(self.decay_rank))
        out = ctx.ws.get("delta_out", T, self.nh * self.dv, x.dtype)
        kernels.delta_out_norm(raw, proj[:, self.g_full if self.gate_rank else self.gate_off:], self.norm_weight, out, T, self.nh,
                               self.dv, self.eps, gate_sigmoid=self.gate_sigmoid)
        return linear(out, self.wo, ctx.ws.get("mixer_proj", T, self.H, x.dtype), ctx)


register_part("mixer", "gated_delta", GatedDelta)

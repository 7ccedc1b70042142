"""Grouped-query attention behind short convolutions, with a learned bias by distance and a window that keeps the first tokens.

With `heads` query heads and `kv_heads` key/value heads (query head h reads key/value head h / (heads / kv_heads)), head
sizes `dim` (queries, keys) and `vdim` (values), and x the mixer's input:

    q, k, v = conv(W_q x), conv(W_k x), conv(W_v x)     short causal convolutions over time, one filter a channel
                                                        (<tensor>.conv [channels, taps], the last tap is the current token's,
                                                        zeros before the sequence's start), no activation
    q, k    = x / sqrt(mean(x^2) + eps) per head        (`unit_norm`; no gain)
    score   = (q . k) * scale + rel[bucket(i - j), h]   (`bias_rows` > 0) a learned bias by the distance n = i - j: with B rows
                                                        and D = `bias_max`, bucket(n) = n below B/2, else
                                                        min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(D / (B/2)) * (B - B/2)))
    position i sees j <= i with i - j < window, and every j < keep_first whatever the distance
    out     = W_o [ head_h * sigmoid((W_g x)_h) ]       (`gate`: one number a head)

Nothing is rotated: positions enter through the mask and the bias alone.  q, k, v and the gates are one product.  The
request's state is the last taps - 1 projected inputs of every channel (float, in the cache manager's state slots); the cache
plane holds the normed keys and the values, in pages that a window gives back once it has passed them, except the pages of
the kept first tokens.  The bias table is expanded when the weights are loaded into one entry a head and distance (up to D, behind
which every distance falls into the last bucket), so the attention kernels look a distance up and compute no logarithm.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .attention import paged_attend
from .base import CacheSpec, Mixer, StateSpec, register_part
from .delta import SHORT_PORTIONS
from .linear import linear


def distance_bucket(n: int, rows: int, bias_max: float) -> int:
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(bias_max / half) * (rows - half))))


class ConvBiasAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float, taps: int,
                 eps: float, prefix: str, dtype, device, window: Optional[int] = None, keep_first: int = 0, bias_rows: int = 0,
                 bias_max: float = 0.0, unit_norm: bool = True, gate: bool = True, **_):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if not 0 < dim <= 512 or not 0 < vdim <= 512:
            raise ValueError(f"head sizes dim {dim} / vdim {vdim} are not supported by the attention kernels (up to 512)")
        if not 1 <= int(taps) <= 9:
            raise ValueError(f"the short convolution takes 1 to 9 taps, not {taps}")
        self.H, self.nh, self.kvh, self.kd, self.vd = int(hidden_size), int(num_heads), int(num_kv_heads), int(dim), int(vdim)
        self.scale, self.taps, self.eps, self.prefix = float(scale), int(taps), float(eps), prefix
        self.window, self.keep_first = int(window or 0), int(keep_first or 0)
        # bias_rows -1: the table's rows are counted when the checkpoint's tensor is loaded
        self.bias_rows, self.bias_max = int(bias_rows or 0), float(bias_max or 0.0)
        self._check_bias()
        self.unit_norm, self.gate, self.dtype, self.device = bool(unit_norm), bool(gate), dtype, device
        # a head's size in the cache and in the query rows: one size for keys and values, a multiple of 16, where the
        # tensor-core attention kernels take it (bfloat16); the sizes as they are otherwise
        one = (max(self.kd, self.vd) + 15) // 16 * 16
        padded = (PAD_HEADS and dtype == torch.bfloat16 and kernels.has_fast_attention(dtype, one, self.nh // self.kvh)
                  and self.scale > 0.0)
        self.kp, self.vp = (one, one) if padded else (self.kd, self.vd)
        self.channels = (self.nh + self.kvh) * self.kd + self.kvh * self.vd         # q | k | v: what the convolutions see
        self.gate_off = (self.channels + 7) // 8 * 8
        self.width = self.gate_off + ((self.nh + 7) // 8 * 8 if self.gate else 0)   # rows stay 16-byte aligned
        self.w_in = self.wo = self.conv_w = self.dist_bias = None
        self._pairs = None

    def _check_bias(self) -> None:
        if self.bias_rows > 0 and not (self.bias_rows >= 2 and self.bias_max > self.bias_rows // 2):
            raise ValueError(f"a distance bias of {self.bias_rows} rows needs bias_max above {self.bias_rows // 2}, not {self.bias_max}")
        if self.bias_rows and self.bias_max > MAX_BIAS_DISTANCES:
            raise ValueError(f"the distance table is expanded to one entry a head and distance up to bias_max: {self.bias_max} is "
                             f"beyond the {MAX_BIAS_DISTANCES} that are built")

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, q, k, v = self.prefix, self.H, self.nh * self.kd, self.kvh * self.kd, self.kvh * self.vd
        conv = lambda name, c: TensorSpec(p + name + ".conv", (c, self.taps), "coefficient", self.taps, init="normal")
        specs = [TensorSpec(p + "q", (q, H), "matrix", H), TensorSpec(p + "k", (k, H), "matrix", H),
                 TensorSpec(p + "v", (v, H), "matrix", H), conv("q", q), conv("k", k), conv("v", v),
                 TensorSpec(p + "o", (H, self.nh * self.vd), "matrix", self.nh * self.vd)]
        if self.bias_rows:
            specs.append(TensorSpec(p + "rel", (self.bias_rows, self.nh), "coefficient", init="small"))
        if self.gate:
            specs.append(TensorSpec(p + "g", (self.nh, H), "matrix", H))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        rows = [tensors[p + "q"], tensors[p + "k"], tensors[p + "v"]]
        rows.append(rows[0].new_zeros((self.gate_off - self.channels, self.H)))
        if self.gate:
            g = tensors[p + "g"]
            rows += [g, g.new_zeros((self.width - self.gate_off - self.nh, self.H))]
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.conv_w = torch.cat([tensors[p + n + ".conv"] for n in ("q", "k", "v")], dim=0).contiguous()
        wo = tensors[p + "o"]
        if self.vp != self.vd:      # zero columns where the padded heads have zeros
            wide = wo.new_zeros((self.H, self.nh, self.vp))
            wide[:, :, :self.vd] = wo.reshape(self.H, self.nh, self.vd)
            wo = wide.reshape(self.H, self.nh * self.vp)
        self.wo = wo.contiguous()
        if self.bias_rows:
            rel = tensors[p + "rel"].to(torch.float32)
            self.bias_rows = int(rel.shape[0])
            self._check_bias()
            last = int(math.ceil(self.bias_max))      # from here on every distance falls into the last bucket
            rows_of = [distance_bucket(n, self.bias_rows, self.bias_max) for n in range(last)] + [self.bias_rows - 1]
            # [heads, distances]: a query's neighbouring keys read neighbouring floats
            self.dist_bias = rel[torch.as_tensor(rows_of, dtype=torch.long, device=rel.device)].t().contiguous()
        if self.wo.is_cuda:
            self._pairs = kernels.decode_pairs_counter(self.wo.device)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.kvh, self.kp, self.window, value_dim=self.vp, keep_first=self.keep_first if self.window else 0)

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec(((self.taps - 1) * self.channels,), torch.float32) if self.taps > 1 else None

    def forward(self, x, ctx, cache, state, write_cache: bool = True):
        T, B = x.shape[0], ctx.launch_requests
        proj = linear(x, self.w_in, ctx.ws.get("conv_attn_in", T, self.width, x.dtype), ctx)
        qkv = ctx.ws.get("conv_attn_qkv", T, self.channels, torch.float32)
        if state is None:
            # one tap: nothing is kept, and no slot is read; every slot number finds the same empty row
            state = ctx.ws.get_flat("conv_attn_no_state", 1, torch.float32, zero=True).view(1, 1).expand(1 << 30, 1)
        if ctx.max_q <= SHORT_PORTIONS:
            kernels.short_conv_step(proj, self.channels, self.conv_w, state, 0, ctx.cu_q, ctx.state_slots, qkv, B, ctx.err,
                                    activation=False)
        else:
            kernels.short_conv_silu(proj, self.channels, self.conv_w, state, 0, ctx.token_req, ctx.cu_q, ctx.state_slots, qkv, T,
                                    ctx.err, activation=False)
            kernels.short_conv_state(proj, self.channels, self.taps, state, 0, ctx.cu_q, ctx.state_slots, B)
        q = ctx.ws.get("conv_attn_q", T, self.nh * self.kp, x.dtype)
        kernels.unit_qk_kv_write(qkv, ctx.slot_mapping[cache.group], q, cache.k, cache.v, T, self.nh, self.kvh, self.kd, self.vd,
                                 self.eps, self.unit_norm, write_cache, ctx.err)
        heads = ctx.ws.get("conv_attn_heads", T, self.nh * self.vp, x.dtype)
        paged_attend(q, self.nh * self.kp, heads, cache.k, cache.v, cache.group, ctx, T, self.nh, self.kvh, self.kp, self.window,
                     self.scale, self._pairs, gate=proj[:, self.gate_off:] if self.gate else None, gate_stride=self.width,
                     keep_first=self.keep_first if self.window else 0, dist_bias=self.dist_bias)
        return linear(heads, self.wo, ctx.ws.get("conv_attn_proj", T, self.H, x.dtype), ctx)


# The most distances the expanded bias table holds a head (4 MiB of floats a head).
MAX_BIAS_DISTANCES = 1 << 20

# Whether bfloat16 layers pad their heads to one size that the tensor-core kernels take (else the plain kernel runs them).
PAD_HEADS = True


register_part("mixer", "attention_conv", ConvBiasAttention)

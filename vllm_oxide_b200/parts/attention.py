"""Grouped-query attention over the paged cache, with optional per-head q/k norm, bias and window.

The order is the reference's (vllm-oxide, crates/vllm-oxide/src/models/qwen3.rs:160-213):
merged q|k|v product, split, RMSNorm over head_dim of q and of k, rotation of q and k, keys
(after norm and rotation) and values written to the cache, attention with scale
1/sqrt(head_dim), output product.  Unlike the reference's prefill, which reads only the keys of
the current step (crates/vllm-oxide/src/attention/flash_attn.rs:15-37), every query here reads
its keys from the pages, so portions, cache hits, recomputation and decoding are one case.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import NO_ROTATION, CacheSpec, Mixer, Prenormed, register_part
from .linear import linear, linear_into_stream


class Attention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, eps: float,
                 qkv_bias: bool, qk_norm: bool, window: Optional[int], position: Optional[str], prefix: str,
                 positions: dict, dtype, device, **_):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if head_dim % 16 or head_dim > 512:
            raise ValueError(f"head_dim {head_dim} is not supported by the attention kernels "
                             f"(a multiple of 16 up to 512)")
        self.H, self.nh, self.kvh, self.hd = hidden_size, num_heads, num_kv_heads, head_dim
        self.eps, self.qkv_bias, self.qk_norm = float(eps), qkv_bias, qk_norm
        self.window = int(window or 0)
        # the position encoding is named by the plan; None (or a part that rotates nothing) leaves q and k as they are
        if position is not None and position not in positions:
            raise KeyError(f"the plan names position encoding {position!r}, but has only {sorted(positions)}")
        encoding = positions[position] if position is not None else None
        self.rotation = encoding.rotation_rule() if encoding is not None else NO_ROTATION
        self.prefix, self.dtype, self.device = prefix, dtype, device
        self.scale = 1.0 / math.sqrt(head_dim)   # qwen3.rs:204
        self.wqkv = self.wo = self.bqkv = self.wq_norm = self.wk_norm = None
        self._pairs = None      # this layer's counter for decode attention of many requests (made with the weights)

    # ---- tensors
    def _names(self):
        p = self.prefix
        return {k: f"{p}{k}" for k in ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight",
                                       "q_proj.bias", "k_proj.bias", "v_proj.bias", "q_norm.weight", "k_norm.weight")}

    def tensor_specs(self) -> List[TensorSpec]:
        n, q, kv = self._names(), self.nh * self.hd, self.kvh * self.hd
        specs = [TensorSpec(n["q_proj.weight"], (q, self.H), "matrix", self.H),
                 TensorSpec(n["k_proj.weight"], (kv, self.H), "matrix", self.H),
                 TensorSpec(n["v_proj.weight"], (kv, self.H), "matrix", self.H),
                 TensorSpec(n["o_proj.weight"], (self.H, q), "matrix", q)]
        if self.qkv_bias:
            specs += [TensorSpec(n["q_proj.bias"], (q,), "bias"), TensorSpec(n["k_proj.bias"], (kv,), "bias"),
                      TensorSpec(n["v_proj.bias"], (kv,), "bias")]
        if self.qk_norm:
            specs += [TensorSpec(n["q_norm.weight"], (self.hd,), "norm"),
                      TensorSpec(n["k_norm.weight"], (self.hd,), "norm")]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self._names()
        # rows of q, then k, then v (crates/vllm-oxide/src/layers/linear.rs:109-119)
        self.wqkv = torch.cat([tensors[n["q_proj.weight"]], tensors[n["k_proj.weight"]],
                               tensors[n["v_proj.weight"]]], dim=0).contiguous()
        self.wo = tensors[n["o_proj.weight"]].contiguous()
        if self.qkv_bias:
            self.bqkv = torch.cat([tensors[n["q_proj.bias"]], tensors[n["k_proj.bias"]],
                                   tensors[n["v_proj.bias"]]], dim=0).contiguous()
        if self.qk_norm:
            self.wq_norm = tensors[n["q_norm.weight"]].contiguous()
            self.wk_norm = tensors[n["k_norm.weight"]].contiguous()
        if self.wo.is_cuda:
            # a counter of this layer's own, so that no two launches that could overlap ever share one
            self._pairs = kernels.decode_pairs_counter(self.wo.device)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.kvh, self.hd, self.window)

    # ---- one step
    adds_into_stream = True

    def forward(self, x, ctx, cache, state=None, write_cache: bool = True, add_into=None):
        """`add_into`: the residual stream; the output product then adds its result there and nothing is returned."""
        T = x.shape[0]
        width = (self.nh + 2 * self.kvh) * self.hd
        qkv = linear(x, self.wqkv, ctx.ws.get("qkv", T, width, x.dtype), ctx)
        g = cache.group
        kernels.qk_norm_rope_kv_write(qkv, self.bqkv, ctx.positions, ctx.slot_mapping[g], self.wq_norm, self.wk_norm,
                                      self.rotation, cache.k, cache.v, T, self.nh, self.kvh, self.hd, self.eps,
                                      write_cache, ctx.err)
        attn = ctx.ws.get("attn_out", T, self.nh * self.hd, x.dtype)
        self.attend(qkv, width, attn, cache, ctx, T)
        if add_into is not None:
            linear_into_stream(attn, self.wo, add_into)
            return None
        return linear(attn, self.wo, ctx.ws.get("attn_proj", T, self.H, x.dtype), ctx)

    # ---- the same with the residual stream kept inside the products (decode-sized steps)
    def can_forward_on_stream(self, stream, ctx) -> bool:
        T = stream.shape[0]
        attn = ctx.ws.get("attn_out", T, self.nh * self.hd, stream.dtype)
        return (kernels.gemm_skinny_supported(stream, self.wqkv) and kernels.gemm_skinny_supported(attn, self.wo))

    def forward_on_stream(self, stream, norm, ctx, cache, state=None, write_cache: bool = True, prenormed=None,
                          emit_norm=None):
        """stream += attention(RMSNorm(stream)): the norm is applied inside the q|k|v product, the sum made by the
        output product.  `prenormed` (a `Prenormed` of `norm`, left by the product that wrote the stream) spares the
        q|k|v product the norm's arithmetic; with `emit_norm` the output product leaves such a half-done norm behind
        for the part that follows, and it is returned."""
        T = stream.shape[0]
        width = (self.nh + 2 * self.kvh) * self.hd
        qkv = ctx.ws.get("qkv", T, width, stream.dtype)
        if prenormed is not None:
            kernels.gemm_skinny(prenormed.scaled, self.wqkv, qkv, kernels.EPI_BF16, ctx.err, eps=norm.eps,
                                prenormed=prenormed.parts)
        else:
            kernels.gemm_skinny(stream, self.wqkv, qkv, kernels.EPI_BF16, ctx.err, norm_weight=norm.weight, eps=norm.eps)
        g = cache.group
        kernels.qk_norm_rope_kv_write(qkv, self.bqkv, ctx.positions, ctx.slot_mapping[g], self.wq_norm, self.wk_norm,
                                      self.rotation, cache.k, cache.v, T, self.nh, self.kvh, self.hd, self.eps,
                                      write_cache, ctx.err)
        attn = ctx.ws.get("attn_out", T, self.nh * self.hd, stream.dtype)
        self.attend(qkv, width, attn, cache, ctx, T)
        left = leave_prenormed(emit_norm, "after_mixer", stream, ctx)
        kernels.gemm_skinny(attn, self.wo, stream, kernels.EPI_ADD, ctx.err,
                            emit=(emit_norm.weight, left.scaled, left.parts) if left else None)
        return left

    def attend(self, qkv, q_stride, out, cache, ctx, T):
        paged_attend(qkv, q_stride, out, cache.k, cache.v, cache.group, ctx, T, self.nh, self.kvh, self.hd, self.window,
                     self.scale, self._pairs)


class SharedKVAttention(Mixer):
    """Grouped-query attention whose values are its keys as projected: there is no value matrix, and the rotation (of the
    first `rotary_dim` elements of every head, in halves, by angles computed from the position) touches the keys that are
    scored but not the keys that are summed.  Options: `scale` (the score's factor, given, not derived from the head
    size); `sink` (the softmax has a silent extra entry of score 0: weights exp(s) / (1 + sum exp(s))); `gate` (head h's
    output is multiplied by sigmoid((W_g x)_h), W_g [heads, hidden] reading the same input as q and k).  q, k and the gate
    are one product; the cache plane holds the rotated key as its key tensor and the plain key as its value tensor.
    Tensors: <prefix>q, k, g, o."""
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float, position: Optional[str],
                 prefix: str, positions: dict, dtype, device, sink: bool = True, gate: bool = True, window: Optional[int] = None,
                 names=("q", "k", "g", "o"), **_):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if not 0 < head_dim <= 512:
            raise ValueError(f"head_dim {head_dim} is not supported by the attention kernels (up to 512; the tensor-core "
                             f"kernels take multiples of 16 up to 256, the plain kernel the rest)")
        self.H, self.nh, self.kvh, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.scale, self.sink, self.gate, self.window = float(scale), bool(sink), bool(gate), int(window or 0)
        if position is not None and position not in positions:
            raise KeyError(f"the plan names position encoding {position!r}, but has only {sorted(positions)}")
        self.rotation = positions[position].rotation_rule() if position is not None else NO_ROTATION
        if self.rotation.rotary_dim > self.hd:
            raise ValueError(f"the position rule rotates {self.rotation.rotary_dim} dimensions, a head has {self.hd}")
        self.prefix, self.dtype, self.device = prefix, dtype, device
        self.n_q, self.n_k, self.n_g, self.n_o = (prefix + n for n in names)
        self.gate_off = (self.nh + self.kvh) * self.hd             # where the gates' columns begin in a merged row
        self.width = self.gate_off + ((self.nh + 7) // 8 * 8 if self.gate else 0)   # rows stay 16-byte aligned
        self.wqkg = self.wo = None
        self._pairs = None

    def tensor_specs(self) -> List[TensorSpec]:
        q, kv = self.nh * self.hd, self.kvh * self.hd
        specs = [TensorSpec(self.n_q, (q, self.H), "matrix", self.H), TensorSpec(self.n_k, (kv, self.H), "matrix", self.H),
                 TensorSpec(self.n_o, (self.H, q), "matrix", q)]
        if self.gate:
            specs.append(TensorSpec(self.n_g, (self.nh, self.H), "matrix", self.H))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        rows = [tensors[self.n_q], tensors[self.n_k]]
        if self.gate:
            g = tensors[self.n_g]
            rows += [g, g.new_zeros((self.width - self.gate_off - self.nh, self.H))]
        self.wqkg = torch.cat(rows, dim=0).contiguous()
        self.wo = tensors[self.n_o].contiguous()
        if self.wo.is_cuda:
            self._pairs = kernels.decode_pairs_counter(self.wo.device)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.kvh, self.hd, self.window)

    def forward(self, x, ctx, cache, state=None, write_cache: bool = True):
        T = x.shape[0]
        qkg = linear(x, self.wqkg, ctx.ws.get("qkg", T, self.width, x.dtype), ctx)
        kernels.rope_shared_kv_write(qkg, ctx.positions, ctx.slot_mapping[cache.group], self.rotation, cache.k, cache.v, T,
                                     self.nh, self.kvh, self.hd, write_cache, ctx.err)
        attn = ctx.ws.get("attn_out", T, self.nh * self.hd, x.dtype)
        paged_attend(qkg, self.width, attn, cache.k, cache.v, cache.group, ctx, T, self.nh, self.kvh, self.hd, self.window,
                     self.scale, self._pairs, sink=self.sink, gate=qkg[:, self.gate_off:] if self.gate else None,
                     gate_stride=self.width)
        return linear(attn, self.wo, ctx.ws.get("attn_proj", T, self.H, x.dtype), ctx)


def paged_attend(q, q_stride, out, keys, values, group: int, ctx, T: int, nh: int, kvh: int, hd: int, window: int,
                 scale: float, pairs=None, value_dim=None, sink: bool = False, gate=None, gate_stride: int = 0,
                 softcap: float = 0.0, chunk: int = 0, keep_first: int = 0, dist_bias=None) -> int:
    """Attention of every query of the step over the pages of `keys` / `values`; returns the width of a head in `out`.
    bfloat16: decoding requests (one token) go to the split-key tensor-core kernel, requests with a portion to the
    tensor-core kernel for portions.  The 32-bit path, and sizes those kernels refuse, go to the plain kernel.
    `value_dim` (keys and values are one plane whose rows begin with the value): the plain kernel reads and writes only
    that much of a value row; the tensor-core kernels take whole rows, and the caller uses the first `value_dim`
    elements of each head of `out`.  `sink`: the softmax has a silent extra entry of score 0.  `gate`: a view whose element
    [t, h] (rows `gate_stride` apart) is head h's gate of token t; its output is multiplied by the sigmoid of it.
    `softcap` > 0: scores become softcap * tanh(score / softcap); `chunk` > 0: a query sees only keys of its own block of
    `chunk` positions.  `keep_first` > 0: the keys at positions below it are seen by every later query, whatever the window;
    `dist_bias` (float [heads, rows]): entry min(distance, rows - 1) of a head's row is added to the scaled scores, a learned bias by the distance
    between query and key.  Values of another shape than the keys (their own head size, or fewer heads)
    go to the plain kernel; values of the keys' head size in a whole fraction of the keys' heads (key
    head k reads value head k / fraction) stay with the tensor-core kernels."""
    tables = ctx.block_tables[group]
    own_values = tuple(values.shape) != tuple(keys.shape)
    # values of the keys' head size in fewer heads: key heads that are several maps over one value head
    value_div = 1
    if (own_values and values.shape[0] == keys.shape[0] and values.shape[2:] == keys.shape[2:] and values.shape[1] > 0
            and keys.shape[1] % values.shape[1] == 0 and FAST_CAP_AND_CHUNK):
        value_div, own_values = keys.shape[1] // values.shape[1], False
    fast = kernels.has_fast_attention(q.dtype, hd, nh // kvh) and scale > 0.0      # the tcgen05 kernel takes maxima before it scales
    fast = fast and not own_values and (FAST_CAP_AND_CHUNK or not (softcap or chunk))
    fast = fast and (out.dtype == q.dtype or (out.dtype == torch.float32 and FAST_CAP_AND_CHUNK))
    fast = fast and (FAST_KEEP_AND_BIAS or not (keep_first or dist_bias is not None))
    if not fast or ((sink or gate is not None) and not FAST_SINK_AND_GATE):
        kernels.paged_attention_generic(q, q_stride, out, keys, values, tables, ctx.token_req, ctx.positions, T,
                                        nh, kvh, hd, window, scale, ctx.err, value_dim=value_dim, sink=sink, gate=gate,
                                        gate_stride=gate_stride, softcap=softcap, chunk=chunk, keep_first=keep_first,
                                        dist_bias=dist_bias)
        return values.shape[3] if own_values else (hd if value_dim is None else value_dim)
    B = ctx.launch_requests
    if ctx.num_decode > 0:
        n_keys = min(ctx.max_context, chunk or (window + keep_first if window else 0) or ctx.max_context)
        splits = decode_splits(B, kvh, n_keys, kernels.sm_count())
        n = kernels.attention_decode_scratch_floats(hd, B, nh, splits)
        scratch = ctx.ws.get_flat("attention_decode_scratch", n, torch.float32) if n else None
        kernels.attention_decode(q, q_stride, out, keys, values, tables, ctx.cu_q, ctx.context_lens, B, nh,
                                 kvh, hd, window, scale, splits, scratch, ctx.err, pairs=pairs, sink=sink, gate=gate,
                                 gate_stride=gate_stride, softcap=softcap, chunk=chunk, value_div=value_div,
                                 keep_first=keep_first, dist_bias=dist_bias)
    if ctx.max_q > 1:
        kernels.attention_prefill(q, q_stride, out, keys, values, tables, ctx.cu_q, ctx.context_lens, B,
                                  ctx.max_q, nh, kvh, hd, window, scale, ctx.err, sink=sink, gate=gate, gate_stride=gate_stride,
                                  softcap=softcap, chunk=chunk, value_div=value_div, keep_first=keep_first, dist_bias=dist_bias)
    return hd


# Whether the tensor-core attention kernels take a softmax with a sink and a gate on the heads (else the plain kernel does).
FAST_SINK_AND_GATE = True
# Whether they take capped scores, blocks of positions and values with fewer heads than keys (else the plain kernel does).
FAST_CAP_AND_CHUNK = True
# Whether they take kept first keys beside a window and a bias by distance (else the plain kernel does): the mma.sync
# kernels with cp.async copies do, for every head size they are built for.
FAST_KEEP_AND_BIAS = True

DECODE_BLOCKS_PER_SM = 2   # blocks of the decode attention kernel that fit an SM (its shared memory decides)


def leave_prenormed(norm, name: str, stream, ctx) -> Optional[Prenormed]:
    """Buffers for the half-done norm that a product adding into `stream` leaves for `norm` (None: nothing to leave)."""
    if norm is None or getattr(norm, "weight", None) is None:
        return None
    T, H = stream.shape
    scaled = ctx.ws.get("stream_scaled_" + name, T, H, stream.dtype)
    parts = ctx.ws.get_flat("stream_squares_" + name, kernels.gemm_skinny_weight_tiles(H) * 16, torch.float32)
    return Prenormed(norm, scaled, parts)


def decode_splits(num_requests: int, kv_heads: int, max_keys: int, num_sms: int) -> int:
    """Splits of the key range per (request, kv head): as many as keep every block resident at once
    (DECODE_BLOCKS_PER_SM blocks on each of the device's SMs), but at least two 64-key tiles per split.  Up to 8 the blocks of a
    (request, kv head) merge their results as a thread-block cluster, without a second kernel; beyond that a second
    kernel merges them, which pays only for few requests with long contexts (one request of 32,000 keys: 56 us with
    8 splits, 44 us with 16, 37 us with 32), so more than 8 are taken only from 8,192 keys on and only if at least 12
    fit, and 32 only from 16,384 keys on and only if all 32 fit (with 18 of them two requests were slower than with 16)."""
    tiles = -(-max_keys // 64)
    fit = (DECODE_BLOCKS_PER_SM * num_sms) // max(1, num_requests * kv_heads)
    most = 8 if tiles < 128 else (32 if tiles >= 256 and fit >= 32 else 16)
    splits = max(1, min(fit, tiles // 2, most))
    return splits if splits <= 8 or splits >= 12 else 8


register_part("mixer", "attention", Attention)
register_part("mixer", "attention_shared_kv", SharedKVAttention)

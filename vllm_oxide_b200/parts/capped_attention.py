"""Grouped-query attention with capped scores, keys and values of separate sizes, and heads that may be the difference
of two softmax maps.

    score = cap * tanh((q . k) * scale / cap)            (`softcap` 0: the plain scaled score)
    a query at position i sees keys j <= i with i - j < window (`window`), or of its own block of `chunk` positions
    (`chunk`; blocks are counted from position 0 of the sequence), or all of them

Options, each a parameter:

* `dim` / `vdim`: the size of a query or key head and of a value head.
* `row_norm`: q and k each pass an RMS norm over their WHOLE projection (all heads at once) with a gain (<prefix>q.norm,
  <prefix>k.norm), before the rotation.
* `position`: a position part whose rule rotates the front of every q and k head by angles computed from the position
  (a `rope` part made with table=False); None rotates nothing, and positions then enter through the mask alone.
* `maps` = 2: a head has two query maps and its key head two key maps, laid out head by head as [map 1, map 2]; each is
  an attention of its own over the same values, and the head's output is
      o = a1 - lam * a2,   lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff       (one number for the layer),
      o / sqrt(mean(o^2) + eps) * (1 - diff)                                  (over the head's vdim values, no gain).
  The two maps run as 2 * heads plain heads over 2 * kv_heads key heads whose pairs share a value head: the rows of W_q are
  reordered at load time so that the plain rule "query head h reads key head h / group" pairs every map with its keys.
* `gate`: the concatenated heads are multiplied element by element by sigmoid(W_g x) (<prefix>g, reading the mixer's
  input) before the output product.

q, k, v and the gate are one product.  The cache plane holds keys [pages, maps * kv_heads, page, dim] and values
[pages, kv_heads, page, vdim]; a window or a chunk lets the cache manager give back the pages behind it.

The tensor-core attention kernels hold ONE head size, a multiple of 16.  On the bfloat16 path a layer whose `dim` and `vdim`
differ (or are no multiple of 16) therefore pads every head with zeros to one size (`PAD_HEADS`): zero rows are added to
W_q, W_k, W_v and W_g and zero columns to W_o when the weights are loaded, so the products write padded heads by
themselves, a padded query against a padded key is the same score, a padded value adds nothing, and the norms' means
count a head's own elements only.  The cost is the cache and the products of the padding; the 32-bit path pads nothing.
Tensors: <prefix>q, k, v, o (+ q.norm, k.norm; lq1, lk1, lq2, lk2; g).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .attention import paged_attend
from .base import NO_ROTATION, CacheSpec, Mixer, register_part
from .linear import linear


# Whether bfloat16 layers pad their heads to one size that the tensor-core kernels take (else such layers run the plain kernel).
PAD_HEADS = True


def _pad_heads(t: torch.Tensor, size: int, to: int, dim: int = 0) -> torch.Tensor:
    """`t` holds heads of `size` elements along `dim`; every head gets zeros behind it up to `to` elements."""
    if size == to:
        return t
    t = t.movedim(dim, 0)
    heads, rest = t.shape[0] // size, t.shape[1:]
    out = t.new_zeros((heads, to) + tuple(rest))
    out[:, :size] = t.reshape(heads, size, *rest)
    return out.reshape(heads * to, *rest).movedim(0, dim)


class CappedAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float, prefix: str,
                 positions: dict, dtype, device, softcap: float = 0.0, window: Optional[int] = None, chunk: Optional[int] = None,
                 row_norm: bool = False, eps: float = 1e-6, position: Optional[str] = None, maps: int = 1, diff: float = 0.0,
                 gate: bool = False, **_):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if maps not in (1, 2):
            raise ValueError(f"a head has one softmax map or two, not {maps}")
        if not 0 < dim <= 512 or not 0 < vdim <= 512:
            raise ValueError(f"head sizes dim {dim} / vdim {vdim} are not supported by the attention kernels (up to 512)")
        if gate and maps != 2:
            raise ValueError("the output gate is applied where two maps are combined: it needs maps = 2")
        if window and chunk:
            raise ValueError("a layer has a sliding window or blocks of positions, not both")
        self.H, self.nh, self.kvh, self.kd, self.vd = int(hidden_size), int(num_heads), int(num_kv_heads), int(dim), int(vdim)
        self.scale, self.softcap = float(scale), float(softcap or 0.0)
        self.window, self.chunk = int(window or 0), int(chunk or 0)
        self.row_norm, self.eps, self.maps, self.diff, self.gate = bool(row_norm), float(eps), int(maps), float(diff), bool(gate)
        if position is not None and position not in positions:
            raise KeyError(f"the plan names position encoding {position!r}, but has only {sorted(positions)}")
        self.rotation = positions[position].rotation_rule() if position is not None else NO_ROTATION
        if self.rotation.rotary_dim > self.kd:
            raise ValueError(f"the position rule rotates {self.rotation.rotary_dim} dimensions, a head has {self.kd}")
        self.prefix, self.dtype, self.device = prefix, dtype, device
        self.group = self.nh // self.kvh
        # kp, vp: a head's size as the products write it and the cache holds it
        one = (max(self.kd, self.vd) + 15) // 16 * 16
        padded = (PAD_HEADS and dtype == torch.bfloat16 and (self.kd != self.vd or self.kd % 16)
                  and kernels.has_fast_attention(dtype, one, self.group) and self.scale > 0.0)
        self.kp, self.vp = (one, one) if padded else (self.kd, self.vd)
        self.n_q, self.n_k = self.maps * self.nh * self.kp, self.maps * self.kvh * self.kp
        self.n_v, self.n_o = self.kvh * self.vp, self.nh * self.vp
        self.gate_off = self.n_q + self.n_k + self.n_v
        self.width = (self.gate_off + (self.n_o if self.gate else 0) + 7) // 8 * 8        # rows stay 16-byte aligned
        self.w_in = self.wo = self.wq_norm = self.wk_norm = None
        self.lam = 0.0
        self._pairs = None

    # ---- tensors
    def tensor_specs(self) -> List[TensorSpec]:
        p, D = self.prefix, self.H
        n_q, n_k, n_v, n_o = (self.maps * self.nh * self.kd, self.maps * self.kvh * self.kd, self.kvh * self.vd, self.nh * self.vd)
        specs = [TensorSpec(p + "q", (n_q, D), "matrix", D), TensorSpec(p + "k", (n_k, D), "matrix", D),
                 TensorSpec(p + "v", (n_v, D), "matrix", D), TensorSpec(p + "o", (D, n_o), "matrix", n_o)]
        if self.row_norm:
            specs += [TensorSpec(p + "q.norm", (n_q,), "norm"), TensorSpec(p + "k.norm", (n_k,), "norm")]
        if self.maps == 2:
            specs += [TensorSpec(p + n, (self.kd,), "coefficient", init="small") for n in ("lq1", "lk1", "lq2", "lk2")]
        if self.gate:
            specs.append(TensorSpec(p + "g", (self.nh * self.vd, D), "matrix", D))
        return specs

    def _by_map(self, t: torch.Tensor) -> torch.Tensor:
        """Rows (or elements) of q, stored head by head as [map 1, map 2], in the order key head, map, head of the group."""
        if self.maps == 1:
            return t
        rest = t.shape[1:]
        return t.reshape(self.kvh, self.group, 2, self.kd, *rest).transpose(1, 2).reshape(t.shape).contiguous()

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        kd, kp, vd, vp = self.kd, self.kp, self.vd, self.vp
        rows = [_pad_heads(self._by_map(tensors[p + "q"]), kd, kp), _pad_heads(tensors[p + "k"], kd, kp),
                _pad_heads(tensors[p + "v"], vd, vp)]
        if self.gate:
            rows.append(_pad_heads(tensors[p + "g"], vd, vp))
        pad = self.width - sum(r.shape[0] for r in rows)
        if pad:
            rows.append(rows[0].new_zeros((pad, self.H)))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.wo = _pad_heads(tensors[p + "o"], vd, vp, dim=1).contiguous()
        if self.row_norm:
            self.wq_norm = _pad_heads(self._by_map(tensors[p + "q.norm"]), kd, kp).contiguous()
            self.wk_norm = _pad_heads(tensors[p + "k.norm"], kd, kp).contiguous()
        if self.maps == 2:
            f = lambda n: tensors[p + n].to(torch.float32)
            lam = torch.exp((f("lq1") * f("lk1")).sum()) - torch.exp((f("lq2") * f("lk2")).sum()) + self.diff
            self.lam = float(lam.item())
        if self.wo.is_cuda:
            self._pairs = kernels.decode_pairs_counter(self.wo.device)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.maps * self.kvh, self.kp, self.window, value_heads=self.kvh, value_dim=self.vp, chunk=self.chunk)

    # ---- one step
    def forward(self, x, ctx, cache, state=None, write_cache: bool = True):
        T = x.shape[0]
        nh, kvh = self.maps * self.nh, self.maps * self.kvh
        qkv = linear(x, self.w_in, ctx.ws.get("qkvg", T, self.width, x.dtype), ctx)
        kernels.rownorm_rope_kv_write(qkv, ctx.positions, ctx.slot_mapping[cache.group], self.wq_norm, self.wk_norm,
                                      self.rotation, cache.k, cache.v, T, nh, kvh, self.kp, self.eps, write_cache, ctx.err,
                                      kd_norm=self.kd)
        # two maps are subtracted before anything rounds them: their outputs stay float
        a = ctx.ws.get("attn_maps", T, nh * self.vp, torch.float32 if self.maps == 2 else x.dtype)
        paged_attend(qkv, self.width, a, cache.k, cache.v, cache.group, ctx, T, nh, kvh, self.kp, self.window, self.scale,
                     self._pairs, softcap=self.softcap, chunk=self.chunk)
        if self.maps == 2:
            heads = ctx.ws.get("attn_out", T, self.n_o, x.dtype)
            kernels.diff_heads_combine(a, qkv[:, self.gate_off:] if self.gate else None, self.width, heads, T, self.nh,
                                       self.group, self.vp, self.lam, 1.0 - self.diff, self.eps, vd_norm=self.vd)
        else:
            heads = a
        return linear(heads, self.wo, ctx.ws.get("attn_proj", T, self.H, x.dtype), ctx)


register_part("mixer", "attention_capped", CappedAttention)

"""Attention through a latent: queries, keys and values are low-rank, and a token's cache row is one latent.

With H heads, per head `dim` plain and `rot_dim` rotated query/key dimensions, value size `vdim`:

    c_q = norm(W_dq h)                         query latent [q_rank], vector-weight RMSNorm
    q   = W_uq c_q                             per head [dim plain | rot_dim rotated]
    [c' | r'] = W_dkv h;  c = norm(c')         key/value latent [kv_rank];  r = rotate(r') one key part for all heads
    k_h = [W_uk,h c | r],  v_h = W_uv,h c;     score = (q_plain . k_plain + q_rot . r) * scale, window, softmax
    out = W_o [heads side by side]

The cache holds [c | r] and nothing else: one row of kv_rank + rot_dim elements a token, in a plane of one tensor and one "head", padded
with zeros to a multiple of 16 elements (the paged kernels read rows in 16-byte pieces).  Keys and values are never
expanded.  Because k_plain = W_uk c, the plain part of a score is (W_uk,h^T q_plain) . c: every query head is carried
into the latent's space once (`head_linear`), after which attention is multi-query attention whose key row is the cache
row itself and whose value row is its first kv_rank elements, and the package's paged attention kernels do it with the
plane given as keys AND values.  The result, a weighted sum of latents a head, is carried to the value heads by W_uv,h.
This is the cheap order while decoding and for short portions; for long prompts with kv_rank much larger than dim
expanding the keys once a portion would cost fewer operations.

A layer with `borrow=True` has no W_dkv and writes nothing: it reads the plane of the layer that the plan names
(`ExecStep(..., write_cache=False)`), with its own W_uk, W_uv, queries, window and scale.  The plane's window is the
largest window of its writer and readers (`cache_window`).

The rotation pairs neighbouring elements, or halves (element i with i + rotary_dim / 2) if the position rule says so, and
computes its angles from frequencies (a position rule made with `table=False`, see parts/rope.py), so there is no largest
position.  `gate`: the heads side by side are multiplied element by element by sigmoid(W_g h) (<prefix>g, one more block of
rows in the down product) before the output product.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .attention import paged_attend
from .base import NO_ROTATION, CacheSpec, Mixer, register_part
from .linear import linear


FAST_GROUP = 16     # query heads that the tensor-core attention kernels take for one key head
# bfloat16 steps of more than 16 tokens: the per-head products go to the library's batched product (as the package's other
# products of that size do); smaller steps and the 32-bit path use head_linear
LIBRARY_HEAD_PRODUCTS = True


def head_product(x, x_width: int, x_used: int, w, y, y_width: int, T: int) -> None:
    """y[t, h, :O] = x[t, h, :x_used] @ w[h] for w [heads, x_used, O]; x is [T, heads * x_width], y [T, heads * y_width]
    (either may be columns of a wider buffer: their row strides are taken from the tensors)."""
    heads, I, O = w.shape
    if LIBRARY_HEAD_PRODUCTS and x.dtype == torch.bfloat16 and T > 16:
        a = torch.as_strided(x, (heads, T, I), (x_width, x.stride(0), 1))
        out = torch.as_strided(y, (heads, T, O), (y_width, y.stride(0), 1))
        torch.bmm(a, w, out=out)
    else:
        kernels.head_linear(x, x.stride(0), x_width, w, y, y.stride(0), y_width, T)


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int,
                 scale: float, eps: float, window: Optional[int], position: Optional[str], prefix: str, positions: dict,
                 dtype, device, borrow: bool = False, cache_window: Optional[int] = None, gate: bool = False, **_):
        self.H, self.nh, self.dk, self.dr, self.dv = int(hidden_size), int(num_heads), int(dim), int(rot_dim), int(vdim)
        self.q_rank, self.kv_rank, self.scale, self.eps = int(q_rank), int(kv_rank), float(scale), float(eps)
        self.window = int(window or 0)
        self.cache_window = self.window if cache_window is None else int(cache_window or 0)
        if self.cache_window and (not self.window or self.window > self.cache_window):
            raise ValueError("a plane must keep at least the keys that its own layer reads")
        self.borrow, self.prefix, self.dtype, self.device = bool(borrow), prefix, dtype, device
        self.gate, self.gate_off = bool(gate), 0
        if position is not None and position not in positions:
            raise KeyError(f"the plan names position encoding {position!r}, but has only {sorted(positions)}")
        self.rotation = positions[position].rotation_rule() if position is not None else NO_ROTATION
        if self.rotation.rotary_dim > self.dr:
            raise ValueError(f"the position rule rotates {self.rotation.rotary_dim} dimensions, the heads have {self.dr} to rotate")
        self.row = (self.kv_rank + self.dr + 15) // 16 * 16      # elements of a cache row
        if self.row > 512:
            raise ValueError(f"a cache row of {self.row} elements exceeds what the paged attention kernels read (512)")
        self.wdown = self.wuq = self.wuk = self.wuv = self.wo = self.wq_norm = self.wkv_norm = None
        self._pairs = None

    # ---- tensors
    def tensor_specs(self) -> List[TensorSpec]:
        p, H, nh = self.prefix, self.H, self.nh
        specs = [TensorSpec(p + "dq", (self.q_rank, H), "matrix", H), TensorSpec(p + "dq.norm", (self.q_rank,), "norm"),
                 TensorSpec(p + "uq", (nh * (self.dk + self.dr), self.q_rank), "matrix", self.q_rank)]
        if not self.borrow:
            specs += [TensorSpec(p + "dkv", (self.kv_rank + self.dr, H), "matrix", H),
                      TensorSpec(p + "dkv.norm", (self.kv_rank,), "norm")]
        specs += [TensorSpec(p + "uk", (nh * self.dk, self.kv_rank), "matrix", self.kv_rank),
                  TensorSpec(p + "uv", (nh * self.dv, self.kv_rank), "matrix", self.kv_rank),
                  TensorSpec(p + "o", (H, nh * self.dv), "matrix", nh * self.dv)]
        if self.gate:
            specs.append(TensorSpec(p + "g", (nh * self.dv, H), "matrix", H))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        # rows of the query latent, then (a layer with a plane of its own) of the key/value latent and the shared key part
        rows = [tensors[p + "dq"]] + ([] if self.borrow else [tensors[p + "dkv"]])
        # the gate's rows follow, from a column that is a multiple of 8 (its reader takes 16-byte pieces where it can)
        self.gate_off = (sum(r.shape[0] for r in rows) + 7) // 8 * 8
        if self.gate:
            pad = self.gate_off - sum(r.shape[0] for r in rows)
            rows += ([rows[0].new_zeros((pad, self.H))] if pad else []) + [tensors[p + "g"]]
        self.wdown = torch.cat(rows, dim=0).contiguous()
        self.wq_norm = tensors[p + "dq.norm"].contiguous()
        self.wkv_norm = None if self.borrow else tensors[p + "dkv.norm"].contiguous()
        self.wuq = tensors[p + "uq"].contiguous()
        # per head [in, out] with the outputs contiguous, as head_linear reads them: W_uk,h is [dim, kv_rank] as stored
        # (its transpose is applied), W_uv,h [vdim, kv_rank] is turned over
        self.wuk = tensors[p + "uk"].reshape(self.nh, self.dk, self.kv_rank).contiguous()
        self.wuv = tensors[p + "uv"].reshape(self.nh, self.dv, self.kv_rank).transpose(1, 2).contiguous()
        self.wo = tensors[p + "o"].contiguous()
        if self.wo.is_cuda:
            # a counter for every group of heads that goes to the decode kernel on its own (see forward)
            self._pairs = [kernels.decode_pairs_counter(self.wo.device) for _ in range(0, self.nh, FAST_GROUP)]

    def cache_spec(self) -> Optional[CacheSpec]:
        return None if self.borrow else CacheSpec(1, self.row, self.cache_window, tensors=1)

    # ---- one step
    def forward(self, x, ctx, cache, state=None, write_cache: bool = True):
        if write_cache == self.borrow:
            raise ValueError("a latent-attention layer writes its own plane, or borrows one: the plan's order says otherwise")
        T, nh = x.shape[0], self.nh
        down = linear(x, self.wdown, ctx.ws.get("latent_down", T, self.wdown.shape[0], x.dtype), ctx)
        cq = ctx.ws.get("latent_cq", T, self.q_rank, x.dtype)
        kernels.latent_prep(down, self.wq_norm, self.wkv_norm, self.rotation, ctx.positions, ctx.slot_mapping[cache.group], cq,
                            cache.k, T, self.q_rank, self.kv_rank, self.dr, self.eps, write_cache, ctx.err)
        q = linear(cq, self.wuq, ctx.ws.get("latent_q", T, nh * (self.dk + self.dr), x.dtype), ctx)
        # every query head into the latent's space, its rotated part behind: a query row is shaped like a cache row
        qa = ctx.ws.get("latent_qa", T, nh * self.row, x.dtype)
        head_product(q, self.dk + self.dr, self.dk, self.wuk, qa, self.row, T)
        kernels.latent_query_rotate(q, qa, self.rotation, ctx.positions, T, nh, self.dk, self.dr, self.kv_rank, self.row)
        heads = ctx.ws.get("latent_heads", T, nh * self.dv, x.dtype)
        # the tensor-core kernels take up to FAST_GROUP query heads for one key head: more heads go in groups, each with
        # the same plane (the plain kernel takes them all at once)
        fast = kernels.has_fast_attention(x.dtype, self.row, min(nh, FAST_GROUP))
        step = min(nh, FAST_GROUP) if fast else nh
        for k, h0 in enumerate(range(0, nh, step)):
            n = min(step, nh - h0)
            mixed = ctx.ws.get(f"latent_mixed{k}", T, n * self.row, x.dtype)
            w = paged_attend(qa[:, h0 * self.row:(h0 + n) * self.row], nh * self.row, mixed, cache.k, cache.k, cache.group, ctx, T,
                             n, 1, self.row, self.window, self.scale, self._pairs[k] if self._pairs else None,
                             value_dim=self.kv_rank)
            # the plain kernel packs rows of n * w elements into the buffer, the tensor-core kernels fill its rows
            packed = mixed if w == self.row else mixed.reshape(-1)[:T * n * w].view(T, n * w)
            head_product(packed, w, self.kv_rank, self.wuv[h0:h0 + n], heads[:, h0 * self.dv:(h0 + n) * self.dv], self.dv, T)
        if self.gate:
            kernels.sigmoid_gate_mul(heads, down[:, self.gate_off:], nh * self.dv)
        return linear(heads, self.wo, ctx.ws.get("mixer_proj", T, self.H, x.dtype), ctx)


register_part("mixer", "latent_attention", LatentAttention)

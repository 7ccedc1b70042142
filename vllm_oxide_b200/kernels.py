"""ctypes bindings of libvob_kernels.so: one Python function per C entry point.

The library is built in-tree at first use.  There is no fallback: without a CUDA device,
without nvcc or without the built library every call raises `KernelError`.  Tensors are
passed as raw device pointers; every launch goes to torch's current stream, so launches
made inside `torch.cuda.graph(...)` are captured.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build


class KernelError(RuntimeError):
    pass


import os as _os

_lib = None
DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1}

ERR_BITS = {1: "a token id outside the vocabulary", 2: "a position beyond max_position_embeddings",
            4: "a cache slot outside the pool", 8: "a block-table entry that names no page",
            16: "a wanted row outside the batch", 32: "a bounded wait inside a kernel ran out",
            0x100: "(in the weight-streaming product)", 0x200: "(in the tcgen05 product)", 0x400: "(in decode attention)",
            0x800: "(in the attention for portions, mma.sync)", 0x1000: "(in the attention for portions, tcgen05)",
            0x2000: "(in the experts' tcgen05 product)"}


def lib():
    global _lib
    if _lib is None:
        try:
            path = _build.build_kernels()
            _lib = ctypes.CDLL(path)
        except (OSError, _build.BuildError) as e:
            raise KernelError(f"the CUDA kernel library of vllm_oxide_b200 is not available: {e}") from e
        _lib.vob_error_string.restype = ctypes.c_char_p
        _lib.vob_error_string.argtypes = [ctypes.c_int]
    return _lib


_attn_libs = {}


def attention_lib(head_dim: int):
    """The tensor-core attention library for one head size, built at first use."""
    if head_dim not in _attn_libs:
        try:
            L = ctypes.CDLL(_build.build_attention(head_dim))
        except (OSError, _build.BuildError) as e:
            raise KernelError(f"the attention kernels for head size {head_dim} are not available: {e}") from e
        L.vob_attention_decode_scratch_floats.restype = ctypes.c_long
        _attn_libs[head_dim] = L
    return _attn_libs[head_dim]


def has_fast_attention(dtype, head_dim: int, group: int) -> bool:
    """Whether the tensor-core attention kernels take this case; the plain kernel takes the rest."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256 and group <= 16


def sm_count() -> int:
    """The number of SMs of the current device (the library asks the device once)."""
    return int(lib().vob_sm_count())


launch_count = 0   # launches of this package's own kernels since import (bench.py reports the difference)

# Per-kernel-class device timers, off unless asked for (VOB_KERNEL_TIMERS=1 or enable_kernel_timers()): every launch
# of this package's kernels is then bracketed by two CUDA events on its stream, and kernel_timer_report() adds them up
# by entry point.  It serialises nothing, but events cannot be recorded into a CUDA graph: time with
# EngineOptions(enforce_eager=True).  The event before a launch is recorded where the launch asks for its stream,
# which every binding does as the last thing before it calls the library.
_timers = None          # None: off; else a list of (entry point, start event, end event)
_timer_start = None


def enable_kernel_timers(on: bool = True) -> None:
    global _timers, _timer_start
    _timers, _timer_start = ([] if on else None), None


def kernel_timer_report(reset: bool = True):
    """{entry point: (launches, milliseconds on the device)} since the timers were enabled or last reset."""
    global _timers
    if _timers is None:
        raise KernelError("the kernel timers are off: enable_kernel_timers() or VOB_KERNEL_TIMERS=1")
    torch.cuda.synchronize()
    out = {}
    for what, e0, e1 in _timers:
        n, ms = out.get(what, (0, 0.0))
        out[what] = (n + 1, ms + e0.elapsed_time(e1))
    if reset:
        _timers = []
    return out


def _check(code: int, what: str) -> None:
    global launch_count, _timer_start
    launch_count += 1
    if _timers is not None and _timer_start is not None:
        end = torch.cuda.Event(enable_timing=True)
        end.record(torch.cuda.current_stream(torch.cuda.current_device()))
        _timers.append((what, _timer_start, end))
        _timer_start = None
    if code != 0:
        raise KernelError(f"{what}: {lib().vob_error_string(code).decode()} (code {code})")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _stream():
    """The current stream's handle.  torch.cuda.current_stream() without a device spends 15 us looking the device up;
    with the index given it is a plain call."""
    global _timer_start
    stream = torch.cuda.current_stream(torch.cuda.current_device())
    if _timers is not None and not torch.cuda.is_current_stream_capturing():
        _timer_start = torch.cuda.Event(enable_timing=True)
        _timer_start.record(stream)
    return ctypes.c_void_p(stream.cuda_stream)


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODES[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported (float32 or bfloat16)") from None


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("vllm_oxide_b200 kernels run on CUDA tensors only; there is no CPU path")


def describe_error_word(word: int) -> str:
    return "; ".join(msg for bit, msg in ERR_BITS.items() if word & bit) or f"unknown error bits {word}"


def embedding(table, ids, out, num_tokens: int, err, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale."""
    _cuda(table, ids, out)
    V, H = table.shape
    _check(lib().vob_embedding(_p(table), _p(ids), _p(out), num_tokens, H, V, ctypes.c_float(scale), _code(table.dtype),
                               _p(err), _stream()), "embedding")


def softcap(logits, num_rows: int, cap: float) -> None:
    """logits = cap * tanh(logits / cap), in place (float32 rows)."""
    _cuda(logits)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    _check(lib().vob_softcap(_p(logits), ctypes.c_long(logits.stride(0)), num_rows, logits.shape[1], ctypes.c_float(cap),
                             _stream()), "softcap")


def add_rmsnorm(x, residual, weight, y, eps: float, has_residual: bool, err, rows=None, n_out: Optional[int] = None):
    """y = RMSNorm(x + residual) * weight; residual updated in place (unless `rows` selects source rows)."""
    _cuda(x, residual, weight, y, rows)
    assert weight.dtype == torch.float32
    H = x.shape[-1]
    n_src = x.shape[0]
    n = n_src if n_out is None else n_out
    _check(lib().vob_add_rmsnorm(_p(x), _p(residual), _p(weight), _p(y), _p(rows), n, H, n_src,
                                 ctypes.c_float(eps), int(has_residual), _code(x.dtype), _p(err), _stream()),
           "add_rmsnorm")


def silu_mul(gate_up, out, num_tokens: int, interleaved: bool = False) -> None:
    """out = SiLU(gate) * up; gate_up holds [gate | up] per token, or, interleaved, groups of 8 gate + 8 up columns."""
    _cuda(gate_up, out)
    I = out.shape[-1]
    _check(lib().vob_silu_mul(_p(gate_up), _p(out), num_tokens, I, int(interleaved), _code(out.dtype), _stream()),
           "silu_mul")


def qk_norm_rope_kv_write(qkv, bias, positions, slots, wq, wk, rule, kcache, vcache, num_tokens, nh, kvh, hd,
                          eps, write_kv: bool, err) -> None:
    """Bias, per-head norm, rotation and cache write of a merged q|k|v row.  `rule` is the position encoding's
    `RotationRule` (table [max_pos, rotary_dim] float32, rotary_dim, interleaved); a rule with rotary_dim 0 rotates
    nothing."""
    table = rule.table if rule.rotary_dim > 0 else None
    if rule.rotary_dim > 0 and table is None:
        raise KernelError("this kernel rotates by a table of angles; the rule has none (a part made with table=False)")
    _cuda(qkv, positions, slots, table, kcache, vcache)
    if table is not None and (table.dtype != torch.float32 or table.shape[1] != rule.rotary_dim or not table.is_contiguous()):
        raise KernelError(f"the table of angles must be contiguous float32 [max_pos, {rule.rotary_dim}]")
    num_slots = kcache.shape[0] * kcache.shape[2] if kcache is not None else 0
    block_size = kcache.shape[2] if kcache is not None else 1
    max_pos = table.shape[0] if table is not None else 0
    _check(lib().vob_qk_norm_rope_kv_write(_p(qkv), _p(bias), _p(positions), _p(slots), _p(wq), _p(wk), _p(table),
                                           _p(kcache), _p(vcache), num_tokens, nh, kvh, hd, rule.rotary_dim,
                                           int(rule.interleaved), ctypes.c_float(eps), max_pos, ctypes.c_long(num_slots),
                                           block_size, int(write_kv), _code(qkv.dtype), _p(err), _stream()),
           "qk_norm_rope_kv_write")


def paged_attention_generic(q, q_stride, out, kcache, vcache, block_tables, token_req, positions, num_tokens, nh, kvh,
                            hd, window: int, scale: float, err, skip_single_cu_q=None, value_dim: Optional[int] = None,
                            sink: bool = False, gate=None, gate_stride: int = 0, softcap: float = 0.0, chunk: int = 0,
                            keep_first: int = 0, dist_bias=None) -> None:
    """Every token of the batch; with `skip_single_cu_q` (the batch's cu_q) the tokens of requests that
    bring exactly one token are left to the decode kernel.  `value_dim`: only that many leading elements of a value
    row are read and `out` is [tokens, nh * value_dim] (keys and values may then be one and the same plane).
    `sink`: the softmax has a silent extra entry of score 0; `gate` (a view whose element [t * gate_stride + h] is head
    h's number for token t): every head's output is multiplied by the sigmoid of its number.  A value plane
    [pages, value heads, page size, value size] of another shape than the key plane is read by its own shape (neighbouring
    key heads share a value head) and `out` is [tokens, nh * value size]; `softcap` > 0: scores become softcap *
    tanh(score / softcap); `chunk` > 0: a query sees only keys of its own block of `chunk` positions; a float32 `out`
    beside bfloat16 inputs is stored unrounded.  `keep_first` > 0: the keys at positions below it are seen by every later
    query, whatever the window; `dist_bias` (float [nh, rows]): dist_bias[h, min(query position - key position, rows - 1)]
    is added to head h's scaled score."""
    _cuda(q, out, kcache, vcache, block_tables, token_req, positions, gate, dist_bias)
    assert dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.is_contiguous() and dist_bias.shape[0] == nh)
    assert gate is None or gate.dtype == q.dtype
    own_shape = vcache.shape[1] != kcache.shape[1] or vcache.shape[3] != kcache.shape[3]
    if own_shape:
        assert value_dim is None or value_dim == vcache.shape[3]
        value_dim = vcache.shape[3]
    assert vcache.shape[0] == kcache.shape[0] and vcache.shape[2] == kcache.shape[2]
    assert out.dtype in (q.dtype, torch.float32)
    _check(lib().vob_paged_attention_generic(_p(q), ctypes.c_long(q_stride), _p(out), _p(kcache), _p(vcache),
                                             _p(block_tables), block_tables.shape[-1], _p(token_req), _p(positions),
                                             _p(skip_single_cu_q), num_tokens, nh, kvh, hd,
                                             hd if value_dim is None else int(value_dim), kcache.shape[2], window,
                                             ctypes.c_float(scale), ctypes.c_long(kcache.shape[0]), int(bool(sink)), _p(gate),
                                             ctypes.c_long(gate_stride), vcache.shape[1], vcache.shape[3],
                                             ctypes.c_float(softcap), int(chunk), int(out.dtype != q.dtype), int(keep_first),
                                             _p(dist_bias), 0 if dist_bias is None else dist_bias.shape[1], _code(q.dtype),
                                             _p(err), _stream()),
           "paged_attention_generic")


def rownorm_rope_kv_write(qkv, positions, slots, wq, wk, rule, kcache, vcache, num_tokens: int, nh: int, kvh: int, kd: int,
                          eps: float, write_kv: bool, err, kd_norm: Optional[int] = None) -> None:
    """A merged q|k|v row whose keys and values have shapes of their own: q (all heads at once) and k each pass an RMS norm
    with a gain (wq, wk float, both or neither), the front of every q and k head turns by computed angles (`rule` with
    `frequencies`; rotary_dim 0 turns nothing), q is written back in place, k goes to `kcache` [pages, kvh, page size, kd]
    and v as projected to `vcache` [pages, value heads, page size, value size].  `kd_norm`: how many elements of a head
    count in the norms' means (heads that are padded with zeros behind their own elements; default kd)."""
    _cuda(qkv, positions, slots, wq, wk, rule.frequencies, kcache, vcache)
    if rule.rotary_dim > 0 and (rule.frequencies is None or rule.amplitude != 1.0):
        raise KernelError("rownorm_rope_kv_write turns by computed angles: the rule needs `frequencies` and amplitude 1")
    assert qkv.stride(1) == 1 and kcache.dtype == qkv.dtype == vcache.dtype and tuple(kcache.shape[1::2]) == (kvh, kd)
    assert kcache.shape[0] == vcache.shape[0] and kcache.shape[2] == vcache.shape[2]
    for w in (wq, wk):
        assert w is None or (w.dtype == torch.float32 and w.is_contiguous())
    _check(lib().vob_rownorm_rope_kv_write(_p(qkv), ctypes.c_long(qkv.stride(0)), _p(positions), _p(slots), _p(wq), _p(wk),
                                           _p(rule.frequencies), _p(kcache), _p(vcache), num_tokens, nh, kvh, kd,
                                           vcache.shape[1], vcache.shape[3], rule.rotary_dim, int(rule.interleaved),
                                           ctypes.c_float(eps), ctypes.c_long(kcache.shape[0] * kcache.shape[2]),
                                           kcache.shape[2], int(write_kv), _code(qkv.dtype), int(kd_norm or kd), _p(err),
                                           _stream()),
           "rownorm_rope_kv_write")


def diff_heads_combine(a, gate, gate_stride: int, out, num_tokens: int, heads: int, group: int, vd: int, lam: float, post: float,
                       eps: float, vd_norm: Optional[int] = None) -> None:
    """out[t, h] = (a1 - lam * a2) / sqrt(mean((a1 - lam * a2)^2) + eps) * post * sigmoid(gate[t, h]) for heads that are
    two maps: `a` [tokens, 2 * heads * vd] (float32, or out's type) holds, per key/value head, the first maps of its
    `group` heads and then their second maps; `gate` (None: none): a view with rows `gate_stride` apart, heads * vd numbers
    a token; `out` [tokens, heads * vd] in the heads' own order.  `vd_norm`: how many elements of a head count in the mean
    (heads padded with zeros; default vd)."""
    _cuda(a, gate, out)
    assert a.is_contiguous() and out.is_contiguous() and a.dtype in (out.dtype, torch.float32)
    assert gate is None or (gate.dtype == out.dtype and gate.stride(1) == 1)
    _check(lib().vob_diff_heads_combine(_p(a), int(a.dtype == torch.float32), _p(gate), ctypes.c_long(gate_stride), _p(out),
                                        num_tokens, heads, group, vd, ctypes.c_float(lam), ctypes.c_float(post),
                                        ctypes.c_float(eps), _code(out.dtype), int(vd_norm or vd), _stream()), "diff_heads_combine")


def layer_norm_step(stream, eps: float, err, y1=None, y2=None, w=None, b=None, out=None, rows=None, n_out: Optional[int] = None,
                    init: bool = False) -> None:
    """One pass over a float residual stream [tokens, width] around layers whose sublayers share one norm: x = 0 (`init`)
    or the stream's row; x += (y1 + y2); the row is stored; out = LayerNorm(x) * w + b (mean and variance of the row, the
    variance as the mean of squared deviations).  With `rows` (source rows, `n_out` of them) only `out` is computed and
    nothing is stored."""
    _cuda(stream, y1, y2, w, b, out, rows)
    assert stream.dtype == torch.float32 and stream.is_contiguous()
    for t in (w, b):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    act = next((t for t in (out, y1, y2) if t is not None), None)
    for t in (y1, y2, out):
        assert t is None or (t.dtype == act.dtype and t.is_contiguous() and t.shape[1] == stream.shape[1])
    n_src = stream.shape[0]
    n = n_src if rows is None else int(n_out)
    _check(lib().vob_layer_norm_step(_p(stream), _p(y1), _p(y2), _p(w), _p(b), _p(out), _p(rows), n, n_src, stream.shape[1],
                                     ctypes.c_float(eps), int(bool(init)),
                                     _code(act.dtype if act is not None else torch.float32), _p(err), _stream()),
           "layer_norm_step")


def sigmoid_gate_mul(x, gate, width: int) -> None:
    """x[t, i] *= sigmoid(gate[t, i]) for i < width; x and gate may be columns of wider rows."""
    _cuda(x, gate)
    assert x.dtype == gate.dtype and x.stride(1) == 1 and gate.stride(1) == 1 and x.shape[0] == gate.shape[0]
    _check(lib().vob_sigmoid_gate_mul(_p(x), ctypes.c_long(x.stride(0)), _p(gate), ctypes.c_long(gate.stride(0)), x.shape[0], width,
                                      _code(x.dtype), _stream()), "sigmoid_gate_mul")


def rms_norm_step(stream, eps: float, err, y1=None, y2=None, w=None, out=None, rows=None, n_out: Optional[int] = None,
                  init: bool = False, mult: float = 1.0, open_scale: float = 1.0, gain_offset: float = 0.0) -> None:
    """One pass over a float residual stream [tokens, width] around layers whose sublayers share one RMS norm: x = y1 *
    open_scale (`init`: the stream begins with the embedded tokens) or x = the stream's row + mult * (y1 + y2); the row is
    stored; out = x / sqrt(mean(x^2) + eps) * (gain_offset + w).  With `rows` (source rows, `n_out` of them) only `out` is
    computed and nothing is stored."""
    _cuda(stream, y1, y2, w, out, rows)
    assert stream.dtype == torch.float32 and stream.is_contiguous()
    assert w is None or (w.dtype == torch.float32 and w.is_contiguous())
    act = next((t for t in (out, y1, y2) if t is not None), None)
    for t in (y1, y2, out):
        assert t is None or (t.dtype == act.dtype and t.is_contiguous() and t.shape[1] == stream.shape[1])
    n_src = stream.shape[0]
    n = n_src if rows is None else int(n_out)
    _check(lib().vob_rms_norm_step(_p(stream), _p(y1), _p(y2), _p(w), _p(out), _p(rows), n, n_src, stream.shape[1],
                                   ctypes.c_float(eps), int(bool(init)), ctypes.c_float(mult), ctypes.c_float(open_scale),
                                   ctypes.c_float(gain_offset), _code(act.dtype if act is not None else torch.float32), _p(err),
                                   _stream()), "rms_norm_step")


def pair_norm_mean(a, b, wa, wb, out, eps: float) -> None:
    """out = (a / rms(a) * wa + b / rms(b) * wb) / 2, row by row (float sums; a, b, out of one type, wa and wb float)."""
    _cuda(a, b, wa, wb, out)
    assert a.dtype == b.dtype == out.dtype and a.is_contiguous() and b.is_contiguous() and out.is_contiguous()
    assert a.shape == b.shape == out.shape and wa.dtype == wb.dtype == torch.float32
    _check(lib().vob_pair_norm_mean(_p(a), _p(b), _p(wa), _p(wb), _p(out), a.shape[0], a.shape[1], ctypes.c_float(eps),
                                    _code(a.dtype), _stream()), "pair_norm_mean")


def unit_qk_kv_write(x, slots, q_out, kcache, vcache, num_tokens: int, nh: int, kvh: int, dim: int, vdim: int, eps: float,
                     unit: bool, write_kv: bool, err) -> None:
    """x float [tokens, (nh + kvh) * dim + kvh * vdim] (q heads, k heads, v heads) -> q_out [tokens, nh * kd_row] of the
    model's type, k and v into the token's slot of kcache [pages, kvh, page, kd_row] and vcache [pages, kvh, page, vd_row];
    `unit`: every q and k head is divided by its root mean square over `dim` first (no gain).  Heads wider than dim / vdim
    in the planes get zeros behind."""
    _cuda(x, slots, q_out, kcache, vcache)
    assert x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == (nh + kvh) * dim + kvh * vdim
    assert q_out.is_contiguous() and kcache.is_contiguous() and vcache.is_contiguous() and kcache.dtype == vcache.dtype == q_out.dtype
    kd_row, vd_row = kcache.shape[3], vcache.shape[3]
    assert q_out.shape[1] == nh * kd_row and kcache.shape[1] == vcache.shape[1] == kvh
    _check(lib().vob_unit_qk_kv_write(_p(x), _p(slots), _p(q_out), _p(kcache), _p(vcache), num_tokens, nh, kvh, dim, vdim, kd_row,
                                      vd_row, kcache.shape[2], ctypes.c_long(kcache.shape[0] * kcache.shape[2]),
                                      ctypes.c_float(eps), int(bool(unit)), int(bool(write_kv)), _code(q_out.dtype), _p(err),
                                      _stream()), "unit_qk_kv_write")


def clamped_glu(gate_up, bias, out, limit: float, alpha: float = 1.702) -> None:
    """out = g * sigmoid(alpha * g) * (u + 1) with g = min(gate + b, limit), u = clamp(up + b, -limit, limit); gate_up
    [tokens, 2 * I]: the gate's columns, then the up columns; bias float [2 * I] or None."""
    _cuda(gate_up, bias, out)
    I = out.shape[1]
    assert gate_up.stride(1) == 1 and gate_up.shape[1] == 2 * I and out.is_contiguous() and gate_up.dtype == out.dtype
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * I and bias.is_contiguous())
    _check(lib().vob_clamped_glu(_p(gate_up), ctypes.c_long(gate_up.stride(0)), _p(bias), _p(out), out.shape[0], I,
                                 ctypes.c_float(limit), ctypes.c_float(alpha), _code(out.dtype), _stream()), "clamped_glu")


def add_bias(x, bias) -> None:
    """x[t, :] += bias (float bias, in place)."""
    _cuda(x, bias)
    assert x.is_contiguous() and bias.dtype == torch.float32 and bias.numel() == x.shape[1]
    _check(lib().vob_add_bias(_p(x), _p(bias), x.shape[0], x.shape[1], _code(x.dtype), _stream()), "add_bias")


def rope_shared_kv_write(qk, positions, slots, rule, kcache, vcache, num_tokens: int, nh: int, kvh: int, hd: int,
                         write_kv: bool, err) -> None:
    """A merged q|k row of an attention whose values are its keys: query heads rotated in place, every key head written
    as it is into `vcache` and rotated into `kcache` (planes [pages, kvh, page size, hd]).  `rule` must carry
    `frequencies` (a position part made with table=False) and rotate in halves; rotary_dim 0 rotates nothing."""
    _cuda(qk, positions, slots, rule.frequencies, kcache, vcache)
    if rule.rotary_dim > 0 and (rule.frequencies is None or rule.interleaved or rule.amplitude != 1.0):
        raise KernelError("rope_shared_kv_write rotates halves by computed angles: the rule needs `frequencies`, no "
                          "interleaving and amplitude 1")
    assert qk.stride(1) == 1 and kcache.dtype == qk.dtype == vcache.dtype and kcache.shape == vcache.shape
    _check(lib().vob_rope_shared_kv_write(_p(qk), ctypes.c_long(qk.stride(0)), _p(positions), _p(slots), _p(rule.frequencies),
                                          _p(kcache), _p(vcache), num_tokens, nh, kvh, hd, rule.rotary_dim,
                                          ctypes.c_long(kcache.shape[0] * kcache.shape[2]), kcache.shape[2], int(write_kv),
                                          _code(qk.dtype), _p(err), _stream()), "rope_shared_kv_write")


def residual_norm_step(stream, eps: float, err, y=None, w_post=None, inject=None, keep=None, w_pre=None, out=None, rows=None,
                       n_out: Optional[int] = None, init: bool = False) -> None:
    """One pass over a float residual stream [tokens, width] with norms on both sides of a sublayer: x = 0 (`init`) or
    the stream's row; x += RMSNorm(y) * w_post (w_post None: x += y); x += inject; the row is stored (and copied to `keep`);
    out = RMSNorm(x) * w_pre.  With `rows` (source rows, `n_out` of them) only `out` is computed and nothing is stored."""
    _cuda(stream, y, w_post, inject, keep, w_pre, out, rows)
    assert stream.dtype == torch.float32 and stream.is_contiguous()
    for t in (w_post, w_pre, inject, keep):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    act = next((t for t in (out, y) if t is not None), None)
    for t in (y, out):
        assert t is None or (t.dtype == act.dtype and t.is_contiguous() and t.shape[1] == stream.shape[1])
    n_src = stream.shape[0]
    n = n_src if rows is None else int(n_out)
    _check(lib().vob_residual_norm_step(_p(stream), _p(y), _p(w_post), _p(inject), _p(keep), _p(w_pre), _p(out), _p(rows), n,
                                        n_src, stream.shape[1], ctypes.c_float(eps), int(bool(init)),
                                        _code(act.dtype if act is not None else torch.float32), _p(err), _stream()),
           "residual_norm_step")


def short_conv_silu(x, channels: int, taps_w, state, conv_off: int, token_req, cu_q, state_slots, out, num_tokens: int, err,
                    activation: bool = True) -> None:
    """out[t, c] = SiLU(sum_j taps_w[c, j] * x[t - (taps - 1) + j, c]) over every request's tokens of this step (float out
    [tokens, channels]); the inputs before a portion's start come from the request's slot: state [slots, n] float, the
    last taps - 1 inputs of every channel at conv_off.  x: the first `channels` columns of its rows.  `activation` False:
    the filter's output as it is.  `state` may be columns of a wider tensor."""
    _cuda(x, taps_w, state, token_req, cu_q, state_slots, out)
    assert x.stride(1) == 1 and taps_w.dtype == torch.float32 and taps_w.is_contiguous() and taps_w.shape[0] == channels
    assert state.dtype == torch.float32 and state.stride(1) == 1 and out.dtype == torch.float32 and out.is_contiguous()
    _check(lib().vob_short_conv_silu(_p(x), ctypes.c_long(x.stride(0)), _p(taps_w), _p(state), ctypes.c_long(state.stride(0)),
                                     ctypes.c_long(conv_off), _p(token_req), _p(cu_q), _p(state_slots), _p(out), num_tokens,
                                     channels, taps_w.shape[1], ctypes.c_long(state.shape[0]), int(bool(activation)),
                                     _code(x.dtype), _p(err), _stream()), "short_conv_silu")


def short_conv_state(x, channels: int, taps: int, state, conv_off: int, cu_q, state_slots, num_requests: int) -> None:
    """Leaves in every request's slot the last taps - 1 inputs of every channel after this step's portion (from the
    portion, and from what the slot held where the portion is shorter).  Run after short_conv_silu."""
    _cuda(x, state, cu_q, state_slots)
    _check(lib().vob_short_conv_state(_p(x), ctypes.c_long(x.stride(0)), _p(state), ctypes.c_long(state.stride(0)),
                                      ctypes.c_long(conv_off), _p(cu_q), _p(state_slots), num_requests, channels, taps,
                                      ctypes.c_long(state.shape[0]), _code(x.dtype), _stream()), "short_conv_state")


def short_conv_step(x, channels: int, taps_w, state, conv_off: int, cu_q, state_slots, out, num_requests: int, err,
                    activation: bool = True) -> None:
    """short_conv_silu and short_conv_state in one launch, a thread a (request, channel): for steps whose portions are
    short (decoding).  Same numbers."""
    _cuda(x, taps_w, state, cu_q, state_slots, out)
    assert x.stride(1) == 1 and taps_w.dtype == torch.float32 and taps_w.is_contiguous() and taps_w.shape[0] == channels
    assert state.dtype == torch.float32 and state.stride(1) == 1 and out.dtype == torch.float32 and out.is_contiguous()
    _check(lib().vob_short_conv_step(_p(x), ctypes.c_long(x.stride(0)), _p(taps_w), _p(state), ctypes.c_long(state.stride(0)),
                                     ctypes.c_long(conv_off), _p(cu_q), _p(state_slots), _p(out), num_requests, channels,
                                     taps_w.shape[1], ctypes.c_long(state.shape[0]), int(bool(activation)), _code(x.dtype),
                                     _p(err), _stream()), "short_conv_step")


def delta_scan(qkv, ab, b_off: int, a_off: int, A_log, dt_bias, state, cu_q, state_slots, raw, num_requests: int, heads: int,
               kvh: int, dim: int, vdim: int, err, channel_decay: bool = False) -> None:
    """The gated delta rule over every request's tokens of this step, from and to its slot (state [slots, n] float, the
    heads' matrices first, each stored column by column, [heads, vdim, dim]).  qkv float [tokens, 2 kvh dim + heads vdim]; ab: rows whose elements
    b_off + h and a_off + h are head h's pre-activations of beta and of the decay; raw float [tokens, heads * vdim].
    `channel_decay`: the decay has one pre-activation a head and key channel, at a_off + h * dim + d, and dt_bias is
    [heads * dim]; it multiplies row d of the head's matrix."""
    _cuda(qkv, ab, A_log, dt_bias, state, cu_q, state_slots, raw)
    assert qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.shape[1] == 2 * kvh * dim + heads * vdim
    assert raw.dtype == torch.float32 and raw.is_contiguous() and A_log.dtype == dt_bias.dtype == torch.float32
    assert state.dtype == torch.float32 and state.stride(1) == 1 and state.shape[1] >= heads * dim * vdim and ab.stride(1) == 1
    assert dt_bias.numel() == (heads * dim if channel_decay else heads)
    _check(lib().vob_delta_scan(_p(qkv), _p(ab), ctypes.c_long(ab.stride(0)), b_off, a_off, _p(A_log), _p(dt_bias), _p(state),
                                ctypes.c_long(state.stride(0)), _p(cu_q), _p(state_slots), _p(raw), num_requests, heads, kvh,
                                dim, vdim, ctypes.c_long(state.shape[0]), int(bool(channel_decay)), _code(ab.dtype), _p(err),
                                _stream()), "delta_scan")


def delta_out_norm(raw, gate, weight, out, num_tokens: int, heads: int, vdim: int, eps: float, gate_sigmoid: bool = False) -> None:
    """out[t, h] = raw[t, h] / sqrt(mean(raw[t, h]^2) + eps) * weight * SiLU(gate[t, h]) per head over vdim; gate: the
    first heads * vdim columns of its rows.  `gate_sigmoid`: times sigmoid(gate) instead of SiLU(gate)."""
    _cuda(raw, gate, weight, out)
    assert raw.dtype == torch.float32 and raw.is_contiguous() and out.is_contiguous() and gate.stride(1) == 1
    assert weight.dtype == torch.float32 and gate.dtype == out.dtype
    _check(lib().vob_delta_out_norm(_p(raw), _p(gate), ctypes.c_long(gate.stride(0)), _p(weight), _p(out), num_tokens, heads,
                                    vdim, ctypes.c_float(eps), int(bool(gate_sigmoid)), _code(out.dtype), _stream()), "delta_out_norm")


def moe_row_tile() -> int:
    """Rows of a tile of the experts' products: every expert's rows are padded to a multiple of it."""
    return int(lib().vob_moe_row_tile())


def moe_route(h, w_router, correction, ids, weights, num_tokens: int, top: int, groups: int, keep: int,
              sigmoid_scores: bool = False, group_top: int = 1, normalise: bool = False, weight_scale: float = 1.0,
              router_bias=None) -> None:
    """ids, weights [tokens, top]: the experts a token uses and their scores (see csrc/kernels/moe.cu): the softmax over
    all experts or (`sigmoid_scores`) a sigmoid each, chosen by score + `correction` (None: by the score) among the `keep`
    groups that count most, a group by its best choice score or (`group_top` 2) by the sum of its two best; the weights
    are the chosen scores, divided by their sum with `normalise`, times `weight_scale`.  `router_bias` (float [experts]) is
    added to the logits."""
    _cuda(h, w_router, correction, ids, weights, router_bias)
    assert router_bias is None or (router_bias.dtype == torch.float32 and router_bias.is_contiguous())
    E, W = w_router.shape
    assert h.is_contiguous() and h.shape[1] == W and w_router.dtype == torch.float32
    assert correction is None or (correction.dtype == torch.float32 and correction.is_contiguous())
    assert w_router.is_contiguous() and ids.dtype == torch.int32 and weights.dtype == torch.float32 and group_top in (1, 2)
    _check(lib().vob_moe_route(_p(h), _p(w_router), _p(router_bias), _p(correction), _p(ids), _p(weights), num_tokens, W, E, top, groups, keep,
                               int(bool(sigmoid_scores)), int(group_top), int(bool(normalise)), ctypes.c_float(weight_scale),
                               _code(h.dtype), _stream()), "moe_route")


def moe_align(ids, slot_of, row_token, tile_expert, n: int, top: int, experts: int, pad: Optional[int] = None) -> None:
    """Sorts n (token, choice) pairs by expert: slot_of[n] a pair's row, row_token[rows] a row's token or -1, tile_expert
    [rows / moe_row_tile()] the expert of every moe_row_tile() rows or -1.  An expert's rows are padded to `pad` rows (a
    multiple of moe_row_tile(), which is the default)."""
    _cuda(ids, slot_of, row_token, tile_expert)
    _check(lib().vob_moe_align(_p(ids), _p(slot_of), _p(row_token), _p(tile_expert), n, top, experts, row_token.numel(),
                               int(pad or moe_row_tile()), _stream()), "moe_align")


def moe_tc5_row_tile() -> int:
    """Rows of a row tile of the tcgen05 product of the experts."""
    return int(lib().vob_moe_tc5_row_tile())


def moe_gemm_tc5_supported(a, w) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.is_contiguous()
            and w.is_contiguous() and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def moe_gemm_tc5(a, w, c, row_token, tile_expert, relu_squared: bool, err, silu_pairs: bool = False, glu_limit: float = 0.0) -> None:
    """c[row] = f(a[row] @ w[expert of the row]^T) on the tcgen05 tensor cores: a [rows, K] bfloat16 already sorted by
    expert in row tiles of moe_tc5_row_tile(), w [experts, N, K]; c bfloat16 with the squared relu, bfloat16 [rows, N / 2]
    with `silu_pairs` (rows of w in (gate, up) pairs: SiLU(gate) * up), or float."""
    _cuda(a, w, c, row_token, tile_expert)
    E, N, K = w.shape
    assert moe_gemm_tc5_supported(a, w) and a.shape[0] == row_token.numel() and c.stride(1) == 1
    assert c.dtype == (torch.bfloat16 if relu_squared or silu_pairs else torch.float32) and not (relu_squared and silu_pairs)
    map_w, map_x = tensor_map_2d(w.view(E * N, K), 128), tensor_map_2d(a, 128)
    _check(lib().vob_moe_gemm_tc5(map_w, map_x, _p(c), ctypes.c_long(c.stride(0)), _p(row_token), _p(tile_expert), a.shape[0], N, K,
                                  2 if silu_pairs else (0 if relu_squared else 1), ctypes.c_float(glu_limit), _p(err), _stream()),
           "moe_gemm_tc5")


def moe_gather_rows(x, xs, row_token) -> None:
    """xs[row] = x[row_token[row]] for the rows that name a token (bfloat16, width a multiple of 8)."""
    _cuda(x, xs, row_token)
    assert x.dtype == xs.dtype == torch.bfloat16 and x.stride(1) == 1 and xs.is_contiguous() and xs.shape[1] == x.shape[1]
    _check(lib().vob_moe_gather_rows(_p(x), ctypes.c_long(x.stride(0)), _p(xs), _p(row_token), xs.shape[0], x.shape[1],
                                     _stream()), "moe_gather_rows")


def moe_gemm(a, w, c, row_token, tile_expert, relu_squared: bool, gather: bool, silu_pairs: bool = False,
             glu_limit: float = 0.0) -> None:
    """c[row] = f(a[row or its token] @ w[expert of the row]^T), w [experts, N, K]; float accumulation in one chain.  f: the
    squared relu, or (`silu_pairs`: rows of w in (gate, up) pairs, c [rows, N / 2]) SiLU(gate) * up, both with `gather`
    into a's type; or the identity into float.  `glu_limit` > 0 with `silu_pairs`: the clamped form min(gate, limit) *
    sigmoid(1.702 min(gate, limit)) * (clamp(up, -limit, limit) + 1) (also in moe_gemv and moe_gemm_tc5)."""
    _cuda(a, w, c, row_token, tile_expert)
    assert a.stride(1) == 1 and w.is_contiguous() and c.stride(1) == 1 and a.dtype == w.dtype
    first = relu_squared or silu_pairs
    assert c.dtype == (a.dtype if first else torch.float32) and first == gather and not (relu_squared and silu_pairs)
    _check(lib().vob_moe_gemm(_p(a), ctypes.c_long(a.stride(0)), _p(w), _p(c), ctypes.c_long(c.stride(0)), _p(row_token),
                              _p(tile_expert), row_token.numel(), w.shape[1], w.shape[2], 2 if silu_pairs else int(relu_squared),
                              int(gather), int(not first), ctypes.c_float(glu_limit),
                              _code(a.dtype), _stream()), "moe_gemm")


def moe_order(ids, order, n: int, experts: int) -> None:
    """order[n]: the step's (token, choice) pairs listed by expert, without padding (-1 behind the last)."""
    _cuda(ids, order)
    _check(lib().vob_moe_order(_p(ids), _p(order), n, experts, _stream()), "moe_order")


def moe_gemv_supported(a, w, n: int) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.shape[1] <= 48 * 1024
            and a.stride(1) == 1 and (a.stride(0) * 2) % 16 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and w.is_contiguous() and n <= 65535)


def moe_gemv(a, w, c, ids, order, n: int, top: int, relu_squared: bool, silu_pairs: bool = False, glu_limit: float = 0.0) -> None:
    """c[pair] = f(a[pair or its token] @ w[expert of the pair]^T) for the step's pairs, few of them (decoding): bfloat16,
    bound by the experts' rows, which a warp streams with 16-byte loads.  relu_squared: the first product (a by token, c
    bfloat16); else the second (a by pair, c float)."""
    _cuda(a, w, c, ids, order)
    first = relu_squared or silu_pairs          # silu_pairs: rows of w in (gate, up) pairs, c bfloat16 [pairs, N / 2]
    assert moe_gemv_supported(a, w, n) and c.stride(1) == 1 and c.dtype == (torch.bfloat16 if first else torch.float32)
    _check(lib().vob_moe_gemv(_p(a), ctypes.c_long(a.stride(0)), _p(w), _p(c), ctypes.c_long(c.stride(0)), _p(ids), _p(order), n,
                              top, w.shape[1], w.shape[2], 2 if silu_pairs else int(relu_squared), int(first),
                              ctypes.c_float(glu_limit), _stream()), "moe_gemv")


def moe_combine(y, slot_of, weights, out, num_tokens: int, top: int) -> None:
    """out[t] = sum_j weights[t, j] * y[slot_of[t, j]] (float, j in order); slot_of None: pair (t, j) is row t * top + j."""
    _cuda(y, slot_of, weights, out)
    assert y.dtype == torch.float32 and y.is_contiguous() and out.is_contiguous()
    _check(lib().vob_moe_combine(_p(y), _p(slot_of), _p(weights), _p(out), num_tokens, out.shape[1], top, _code(out.dtype),
                                 _stream()), "moe_combine")


def relu_squared(x, out) -> None:
    """out = max(x, 0)^2, element by element (out may be x)."""
    _cuda(x, out)
    assert x.is_contiguous() and out.is_contiguous() and x.dtype == out.dtype
    _check(lib().vob_relu_squared(_p(x), _p(out), ctypes.c_long(x.numel()), _code(x.dtype), _stream()), "relu_squared")


def stream_step(streams, num_streams: int, width: int, eps: float, err, y=None, init=None, mix=None, out_w=None, in_w=None,
                gain=None, normed=None, rows=None, n_out: Optional[int] = None) -> None:
    """One pass over the residual streams (float [tokens, num_streams * width]).  `init` [tokens, width]: every stream
    becomes the embedded token; else with `y` [tokens, width]: new stream t = sum_s mix[s, t] * stream s + out_w[t] * y.
    With `normed` [rows, width]: u = sum_s in_w[s] * stream s, normed = u / sqrt(mean(u^2) + eps) * gain.  Missing
    coefficients are the identity, ones and 1.  With `rows` (source rows, `n_out` of them) only the combination is
    computed, for those rows, and no stream is written."""
    _cuda(streams, y, init, mix, out_w, in_w, gain, normed, rows)
    assert streams.dtype == torch.float32 and streams.is_contiguous() and streams.shape[1] == num_streams * width
    n_src = streams.shape[0]
    n = n_src if rows is None else int(n_out)
    act = next((t for t in (normed, y, init) if t is not None), None)
    for t in (mix, out_w, in_w, gain):
        assert t is None or t.dtype == torch.float32
    for t in (y, init, normed):
        assert t is None or (t.dtype == act.dtype and t.is_contiguous() and t.shape[1] == width)
    _check(lib().vob_stream_step(_p(streams), _p(y), _p(init), _p(mix), _p(out_w), _p(in_w), _p(gain), _p(normed), _p(rows),
                                 n, n_src, num_streams, width, ctypes.c_float(eps),
                                 _code(act.dtype if act is not None else torch.float32), _p(err), _stream()), "stream_step")


def stream_sum(streams, sums, num_streams: int, width: int) -> None:
    """sums [tokens, width] (float) = the sum of a token's streams."""
    _cuda(streams, sums)
    assert streams.dtype == sums.dtype == torch.float32 and streams.is_contiguous() and sums.is_contiguous()
    _check(lib().vob_stream_sum(_p(streams), _p(sums), sums.shape[0], num_streams, width, _stream()), "stream_sum")


def scan_chunks(num_tokens: int, num_requests: int) -> int:
    """Ranges that a scan cuts a request's tokens of a step into, from the step's mean portion: 1 while decoding."""
    mean = num_tokens / max(1, num_requests)
    return 1 if mean <= 4 else (8 if mean <= 256 else 32)


def mingru_scan(zxg, bias_z, bias_x, state, cu_q, state_slots, out, num_requests: int, err, chunks: int = 1) -> None:
    """The gated recurrence s = (1 - z) s + z * candidate over every request's tokens of this step, from and to its
    state slot (float [slots, width]); zxg [tokens, 3 * width] holds the pre-activations z | candidate | output gate.
    `chunks` (1, 8 or 32): ranges of a request's tokens that are folded side by side (see scan_chunks)."""
    _cuda(zxg, bias_z, bias_x, state, cu_q, state_slots, out)
    W = out.shape[1]
    assert zxg.is_contiguous() and out.is_contiguous() and zxg.shape[1] == 3 * W and state.dtype == torch.float32
    assert state.is_contiguous() and state.shape[1] == W and bias_z.dtype == zxg.dtype == bias_x.dtype == out.dtype
    _check(lib().vob_mingru_scan(_p(zxg), _p(bias_z), _p(bias_x), _p(state), _p(cu_q), _p(state_slots), _p(out),
                                 num_requests, W, state.shape[0], int(chunks), _code(out.dtype), _p(err), _stream()),
           "mingru_scan")


def hgrn2_scan(qfv, bias_f, lower, norm_weight, state, cu_q, state_slots, out, num_requests: int, heads: int, dk: int,
               dv: int, eps: float, err, raw=None, chunks: int = 1, scratch=None) -> None:
    """The matrix-state recurrence M = diag(f) M + (1 - f) v^T, o = M^T q, with the per-head norm of o, over every
    request's tokens of this step; state float [slots, heads, dk, dv]; qfv [tokens, heads * (2 dk + dv)].  Without `raw`
    one block a (request, head) does it all (decoding; the head must fit: hgrn2_can_fuse); with `raw` (float [tokens,
    heads * dv]) a head's columns are spread over blocks and the norm is a second kernel (portions).  Same numbers.
    `chunks` > 1 (with `raw`): a request's tokens are cut into that many ranges that are walked side by side, twice,
    with a join in between; `scratch`: float, num_requests * chunks * heads * dk * (dv + 1) elements."""
    _cuda(qfv, bias_f, lower, norm_weight, state, cu_q, state_slots, out, raw)
    T = out.shape[0]
    assert qfv.is_contiguous() and out.is_contiguous() and qfv.shape[1] == heads * (2 * dk + dv) and out.shape[1] == heads * dv
    assert state.dtype == torch.float32 and state.is_contiguous() and state[0].numel() == heads * dk * dv
    assert lower.dtype == torch.float32 and norm_weight.dtype == torch.float32 and bias_f.dtype == qfv.dtype == out.dtype
    assert chunks == 1 or (raw is not None and scratch is not None and scratch.dtype == torch.float32
                           and scratch.numel() >= num_requests * chunks * heads * dk * (dv + 1))
    _check(lib().vob_hgrn2_scan(_p(qfv), _p(bias_f), _p(lower), _p(norm_weight), _p(state), _p(cu_q), _p(state_slots),
                                _p(out), _p(raw), _p(scratch), T, num_requests, int(chunks), heads, dk, dv, ctypes.c_float(eps),
                                state.shape[0], int(raw is None), _code(out.dtype), _p(err), _stream()), "hgrn2_scan")


def hgrn2_can_fuse(dk: int, dv: int) -> bool:
    return bool(lib().vob_hgrn2_can_fuse(dk, dv))


def latent_prep(down, wq, wkv, rule, positions, slots, cq, cache, num_tokens: int, q_rank: int, kv_rank: int, rot: int,
                eps: float, write_kv: bool, err) -> None:
    """A token's down-projected row [query latent | key/value latent | shared key part] -> the normalised query latent in
    `cq`, and, with `write_kv`, [normalised latent | shared part rotated by `rule` | zeros] in the token's row of `cache`
    ([pages, 1, page size, row width])."""
    _cuda(down, wq, wkv, rule.frequencies, positions, slots, cq, cache)
    assert down.stride(1) == 1 and cq.is_contiguous() and wq.dtype == torch.float32
    row_width = num_slots = 0
    if write_kv:
        assert cache.is_contiguous() and cache.shape[1] == 1 and wkv.dtype == torch.float32 and cache.dtype == down.dtype
        row_width, num_slots = cache.shape[3], cache.shape[0] * cache.shape[2]
        if rule.rotary_dim > 0 and rule.frequencies is None:
            raise KernelError("latent_prep rotates by computed angles: the rule needs `frequencies`")
    _check(lib().vob_latent_prep(_p(down), ctypes.c_long(down.stride(0)), _p(wq), _p(wkv), _p(rule.frequencies),
                                 ctypes.c_float(rule.amplitude), _p(positions), _p(slots), _p(cq), _p(cache), num_tokens,
                                 q_rank, kv_rank, rot, rule.rotary_dim, row_width, ctypes.c_long(num_slots),
                                 ctypes.c_float(eps), int(write_kv), int(not rule.interleaved), _code(down.dtype), _p(err),
                                 _stream()), "latent_prep")


def latent_query_rotate(q, qa, rule, positions, num_tokens: int, heads: int, dk: int, rot: int, offset: int,
                        row_width: int) -> None:
    """qa[t, h, offset:offset+rot] = the last `rot` elements of query head h of q [tokens, heads * (dk + rot)], rotated by
    `rule`; zeros behind, up to row_width."""
    _cuda(q, qa, rule.frequencies, positions)
    assert q.is_contiguous() and qa.is_contiguous() and q.dtype == qa.dtype
    if rule.rotary_dim > 0 and rule.frequencies is None:
        raise KernelError("latent_query_rotate needs a rule with `frequencies`")
    _check(lib().vob_latent_query_rotate(_p(q), _p(qa), _p(rule.frequencies), ctypes.c_float(rule.amplitude), _p(positions),
                                         num_tokens, heads, dk, rot, rule.rotary_dim, offset, row_width,
                                         int(not rule.interleaved), _code(q.dtype), _stream()), "latent_query_rotate")


def head_linear(x, x_token_stride: int, x_head_stride: int, w, y, y_token_stride: int, y_head_stride: int, num_tokens: int) -> None:
    """y[t, h, :O] = sum_i w[h, i, :] * x[t, h, i] for per-head matrices w [heads, I, O]; x and y are addressed by token
    and head strides (elements), so either may be a slice of wider rows."""
    _cuda(x, w, y)
    assert w.is_contiguous() and w.dim() == 3 and x.dtype == w.dtype == y.dtype
    heads, I, O = w.shape
    _check(lib().vob_head_linear(_p(x), ctypes.c_long(x_token_stride), ctypes.c_long(x_head_stride), _p(w), _p(y),
                                 ctypes.c_long(y_token_stride), ctypes.c_long(y_head_stride), num_tokens, heads, I, O,
                                 _code(x.dtype), _stream()), "head_linear")


def attention_decode_scratch_floats(head_dim: int, num_requests: int, nh: int, num_splits: int) -> int:
    return int(attention_lib(head_dim).vob_attention_decode_scratch_floats(num_requests, nh, num_splits))


def attention_decode(q, q_stride, out, kcache, vcache, block_tables, cu_q, context_lens, num_requests, nh, kvh, hd,
                     window: int, scale: float, num_splits: int, scratch, err, use_tma: bool = True, pairs=None,
                     sink: bool = False, gate=None, gate_stride: int = 0, softcap: float = 0.0, chunk: int = 0,
                     value_div: int = 1, keep_first: int = 0, dist_bias=None) -> None:
    """Requests that bring exactly one token; the others are skipped.  `pairs`: two int32 zeros on the device that belong
    to this caller (`decode_pairs_counter`); with it, one split and more (request, kv head) pairs than blocks fit the GPU
    run as persistent blocks that draw their pairs from it (the kernel leaves it at zero), without it as one block per
    pair.  Same bits either way.  `sink`, `gate`, `gate_stride`, `softcap`, `chunk`: as for paged_attention_generic.
    `value_div` > 1: `vcache` has kvh // value_div heads, and key head k reads value head k // value_div.  `out` is
    bfloat16 or float32.  `keep_first`, `dist_bias`: as for paged_attention_generic; with either the keys and values come in
    by cp.async (the TMA kernels walk one range of keys and know no bias)."""
    _cuda(q, out, kcache, vcache, block_tables, cu_q, context_lens, scratch, pairs, gate, dist_bias)
    assert dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.is_contiguous() and dist_bias.shape[0] == nh)
    use_tma = use_tma and not keep_first and dist_bias is None
    assert pairs is None or (pairs.dtype == torch.int32 and pairs.numel() >= 2)
    assert q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and (gate is None or gate.dtype == torch.bfloat16)
    L = attention_lib(hd)
    map_k = map_v = None
    if use_tma and L.vob_attention_decode_has_tma() and kcache.is_contiguous() and vcache.is_contiguous():
        # head sizes that are a multiple of 64: keys and values come in by TMA (about twice cp.async's rate)
        bs = kcache.shape[2]
        keys, slices = L.vob_attention_decode_box_keys(bs), L.vob_attention_decode_box_slices(bs)
        map_k, map_v = tensor_map(kcache.view(-1, hd), keys, slices), tensor_map(vcache.view(-1, hd), keys, slices)
    _check(L.vob_attention_decode_ex(
        map_k, map_v, _p(q), ctypes.c_long(q_stride), _p(out), _p(kcache), _p(vcache), _p(block_tables),
        block_tables.shape[-1], _p(cu_q), _p(context_lens), num_requests, nh, kvh, kcache.shape[2], window,
        ctypes.c_float(scale), ctypes.c_long(kcache.shape[0]), num_splits, _p(scratch), _p(pairs if map_k is not None else None),
        int(bool(sink)), _p(gate), ctypes.c_long(gate_stride), ctypes.c_float(softcap), int(chunk), int(value_div), int(out.dtype == torch.float32),
        int(keep_first), _p(dist_bias), 0 if dist_bias is None else dist_bias.shape[1], _p(err), _stream()),
        "attention_decode_tma" if map_k is not None else
        ("attention_decode_window_bias" if keep_first or dist_bias is not None else "attention_decode"))


def decode_pairs_counter(device) -> torch.Tensor:
    """The counter that `attention_decode(pairs=...)` draws (request, kv head) pairs from: one per caller whose launches
    do not overlap in time (the engine keeps one per attention layer)."""
    return torch.zeros(2, dtype=torch.int32, device=device)


def attention_prefill(q, q_stride, out, kcache, vcache, block_tables, cu_q, context_lens, num_requests, max_q, nh, kvh,
                      hd, window: int, scale: float, err, use_tma: bool = True, use_tc5: bool = True,
                      query_tiles: int = 2, tiles_by_tma: bool = True, sink: bool = False, gate=None, gate_stride: int = 0,
                      softcap: float = 0.0, chunk: int = 0, value_div: int = 1, keep_first: int = 0, dist_bias=None) -> None:
    """Requests that bring more than one token; the others are skipped.  Head sizes 64 and 128 run on the tcgen05
    tensor cores (`use_tc5`; `tiles_by_tma` False makes that kernel bring its query tiles in by cp.async and store its
    output row by row also where TMA could), other multiples of 64 on mma.sync with TMA copies (`use_tma`), the rest with
    cp.async.  `sink`, `gate`, `gate_stride`, `softcap`, `chunk`: as for paged_attention_generic; `value_div`: as for
    attention_decode.  `keep_first`, `dist_bias`: as for paged_attention_generic; all three kernels take them."""
    _cuda(q, out, kcache, vcache, block_tables, cu_q, context_lens, gate, dist_bias)
    assert dist_bias is None or (dist_bias.dtype == torch.float32 and dist_bias.is_contiguous() and dist_bias.shape[0] == nh)
    assert q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and (gate is None or gate.dtype == torch.bfloat16)
    L = attention_lib(hd)
    extras = (int(bool(sink)), _p(gate), ctypes.c_long(gate_stride), ctypes.c_float(softcap), int(chunk), int(value_div),
              int(out.dtype == torch.float32))
    map_k = map_v = None
    if use_tma and L.vob_attention_decode_has_tma() and kcache.is_contiguous() and vcache.is_contiguous():
        bs = kcache.shape[2]
        keys, slices = L.vob_attention_decode_box_keys(bs), L.vob_attention_decode_box_slices(bs)
        map_k, map_v = tensor_map(kcache.view(-1, hd), keys, slices), tensor_map(vcache.view(-1, hd), keys, slices)
        if use_tc5 and L.vob_attention_prefill_has_tc5() and q_stride % 8 == 0:
            # the query tiles come and whole output tiles leave by TMA too (a tile holds whole tokens: 128 // group of them)
            box_heads = L.vob_attention_prefill_q_box_heads(nh, kvh) if tiles_by_tma else 0
            map_q = tensor_map_heads(q, q_stride, nh, hd, box_heads, 128 // box_heads) if box_heads > 0 else None
            map_o = (tensor_map_heads(out, nh * hd, nh, hd, box_heads, 128 // box_heads)
                     if box_heads > 0 and out.is_contiguous() and out.data_ptr() % 16 == 0 and out.dtype == torch.bfloat16 else None)
            _check(L.vob_attention_prefill_tc5(
                map_k, map_v, map_q, map_o, _p(q), ctypes.c_long(q_stride), _p(out), _p(block_tables), block_tables.shape[-1], _p(cu_q),
                _p(context_lens), num_requests, max_q, nh, kvh, bs, window, ctypes.c_float(scale),
                ctypes.c_long(kcache.shape[0]), query_tiles, *extras, int(keep_first), _p(dist_bias),
                0 if dist_bias is None else dist_bias.shape[1], _p(err), _stream()),
                "attention_prefill_window_bias" if keep_first or dist_bias is not None else "attention_prefill_tc5")
            return
    _check(L.vob_attention_prefill_ex(
        map_k, map_v, _p(q), ctypes.c_long(q_stride), _p(out), _p(kcache), _p(vcache), _p(block_tables),
        block_tables.shape[-1], _p(cu_q), _p(context_lens), num_requests, max_q, nh, kvh, kcache.shape[2], window,
        ctypes.c_float(scale), ctypes.c_long(kcache.shape[0]), *extras, int(keep_first), _p(dist_bias),
        0 if dist_bias is None else dist_bias.shape[1], _p(err), _stream()),
        ("attention_prefill_window_bias" if keep_first or dist_bias is not None else
         ("attention_prefill_tma" if map_k is not None else "attention_prefill")))


def gemm_f32(a, w, out, bias=None) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in true float32."""
    _cuda(a, w, out)
    assert a.dtype == w.dtype == out.dtype == torch.float32
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape[0] == M and out.shape[1] == N
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(lib().vob_gemm_f32(_p(a), ctypes.c_long(a.stride(0)), _p(w), ctypes.c_long(w.stride(0)), _p(out),
                              ctypes.c_long(out.stride(0)), _p(bias), M, N, K, _stream()), "gemm_f32")


EPI_BF16, EPI_F32, EPI_SWIGLU, EPI_ADD = 0, 1, 2, 3
_tensor_maps = {}


def tensor_map(t: torch.Tensor, box_rows: int, box_slices: int):
    """A TMA descriptor (host memory, cached) of a row-major bfloat16 matrix whose width is a multiple of 64: one copy
    brings `box_slices` column slices (64 columns each) of `box_rows` rows."""
    key = (t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows, box_slices)
    hit = _tensor_maps.get(key)
    if hit is None:
        raw = (ctypes.c_char * 256)()
        addr = (ctypes.addressof(raw) + 63) & ~63
        code = lib().vob_tensor_map_bf16_sliced(ctypes.c_void_p(addr), _p(t), ctypes.c_long(t.shape[0]),
                                                ctypes.c_long(t.shape[1]), ctypes.c_long(t.stride(0)), box_rows, box_slices)
        if code != 0:
            raise KernelError(f"tensor map for a [{t.shape[0]}, {t.shape[1]}] matrix: {lib().vob_error_string(code).decode()}")
        if len(_tensor_maps) > 4096:
            _tensor_maps.clear()
        hit = _tensor_maps[key] = (raw, ctypes.c_void_p(addr))
    return hit[1]


def tensor_map_heads(t: torch.Tensor, token_stride: int, heads: int, head_dim: int, box_heads: int, box_tokens: int):
    """A TMA descriptor (host memory, cached) of token rows that begin with `heads` heads of `head_dim` bfloat16 each: one
    copy brings a 64-column slice of `box_heads` heads for `box_tokens` tokens, as rows in the order (token, head)."""
    key = (t.data_ptr(), t.shape[0], token_stride, heads, head_dim, box_heads, box_tokens, "heads")
    hit = _tensor_maps.get(key)
    if hit is None:
        raw = (ctypes.c_char * 256)()
        addr = (ctypes.addressof(raw) + 63) & ~63
        code = lib().vob_tensor_map_bf16_heads(ctypes.c_void_p(addr), _p(t), ctypes.c_long(t.shape[0]), heads, head_dim,
                                               ctypes.c_long(token_stride), box_heads, box_tokens)
        if code != 0:
            raise KernelError(f"tensor map for {t.shape[0]} token rows of {heads} heads: {lib().vob_error_string(code).decode()}")
        if len(_tensor_maps) > 4096:
            _tensor_maps.clear()
        hit = _tensor_maps[key] = (raw, ctypes.c_void_p(addr))
    return hit[1]


def tensor_map_2d(t: torch.Tensor, box_rows: int):
    """A TMA descriptor (host memory, cached) of a row-major bfloat16 matrix with box [box_rows, 64 columns]."""
    key = (t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows, "2d")
    hit = _tensor_maps.get(key)
    if hit is None:
        raw = (ctypes.c_char * 256)()
        addr = (ctypes.addressof(raw) + 63) & ~63
        code = lib().vob_tensor_map_bf16_2d(ctypes.c_void_p(addr), _p(t), ctypes.c_long(t.shape[0]), ctypes.c_long(t.shape[1]),
                                            ctypes.c_long(t.stride(0)), box_rows)
        if code != 0:
            raise KernelError(f"tensor map for a [{t.shape[0]}, {t.shape[1]}] matrix: {lib().vob_error_string(code).decode()}")
        if len(_tensor_maps) > 4096:
            _tensor_maps.clear()
        hit = _tensor_maps[key] = (raw, ctypes.c_void_p(addr))
    return hit[1]


def gemm_tc5_supported(x, w) -> bool:
    """Whether the tcgen05 product takes x[M,K] @ w[N,K]^T: bfloat16, at most 128 rows of x, K a multiple of 8,
    rows that start on 16-byte boundaries."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= 128
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and (x.stride(0) * 2) % 16 == 0
            and (w.stride(0) * 2) % 16 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc5_cluster(x, w, epilogue: int) -> int:
    """The number of K ranges (blocks of a thread-block cluster) the tcgen05 product chooses for x @ w^T on this device."""
    L = lib()
    return int(L.vob_gemm_tc5_cluster(x.shape[0], ctypes.c_long(w.shape[0]), ctypes.c_long(w.shape[1]), epilogue))


def gemm_tc5(x, w, out, epilogue: int, err, cluster: int = 0) -> None:
    """out = x @ w^T on the tcgen05 tensor cores for at most 128 rows of x; epilogues as gemm_skinny.  The product
    is split along K over the blocks of a thread-block cluster where that fills the GPU better (`cluster` 0: chosen
    by the library; 1 to 8: that many K ranges); the partial tiles meet in shared memory, no scratch is needed."""
    _cuda(x, w, out)
    if not gemm_tc5_supported(x, w):
        raise KernelError("gemm_tc5: this product is not supported (bfloat16, at most 128 rows, K a multiple of 8, "
                          "16-byte aligned rows)")
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(1) == 1 and out.shape[0] == M
    assert out.shape[1] == (N // 2 if epilogue == EPI_SWIGLU else N)
    assert out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16)
    L = lib()
    map_w = tensor_map_2d(w, 128)
    map_x = tensor_map_2d(x, int(L.vob_gemm_tc5_token_box(M)))
    _check(L.vob_gemm_tc5(map_w, map_x, _p(out), ctypes.c_long(out.stride(0)), M, N, K, epilogue, int(cluster),
                          _p(err), _stream()), "gemm_tc5")


def gemm_skinny_supported(x, w) -> bool:
    """Whether the weight-streaming kernel takes x[M,K] @ w[N,K]^T: bfloat16, M <= 16, K a multiple of 64 (the
    column slices of a TMA box), rows that start on 16-byte boundaries."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= 16
            and x.shape[1] % 64 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and (x.stride(0) * 2) % 16 == 0 and (w.stride(0) * 2) % 16 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny_weight_tiles(n_rows: int) -> int:
    """The number of row tiles the weight-streaming product cuts a matrix of `n_rows` rows into."""
    box = int(lib().vob_gemm_skinny_weight_box(ctypes.c_long(n_rows)))
    return (n_rows + box - 1) // box


def gemm_skinny(x, w, out, epilogue: int, err, norm_weight=None, eps: float = 0.0, emit=None, prenormed=None) -> None:
    """out = x @ w^T for at most 16 rows of x (see gemm_skinny_supported); epilogue EPI_BF16 (out bfloat16 [M,N]),
    EPI_F32 (out float32 [M,N], rounded to bfloat16 first), EPI_SWIGLU (the rows of w alternate in groups of
    eight between gate and up; out bfloat16 [M,N/2] = SiLU(gate) * up) or EPI_ADD (out bfloat16 [M,N] += the
    product rounded to bfloat16: out is the residual stream).  With `norm_weight` (float [K]; EPI_BF16 and EPI_SWIGLU)
    the product is that of RMSNorm(x) * norm_weight, the norm computed on the way.

    The same norm in two halves, for a chain of products: `emit=(weight, scaled, parts)` (EPI_ADD) makes the product
    leave bfloat16(out * weight) in `scaled` [M,N] and per-tile sums of the squares of the new `out` in `parts`
    (float, gemm_skinny_weight_tiles(N) * 16 entries are enough) for the norm that follows; `prenormed=parts` (EPI_BF16
    and EPI_SWIGLU, with `eps`) takes x to be such a `scaled` buffer and scales the product by 1/rms from the parts."""
    _cuda(x, w, out, norm_weight)
    if not gemm_skinny_supported(x, w):
        raise KernelError("gemm_skinny: this product is not supported (bfloat16, at most 16 rows, K a multiple of 64, 16-byte aligned rows)")
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(1) == 1 and out.shape[0] == M
    assert out.shape[1] == (N // 2 if epilogue == EPI_SWIGLU else N)
    assert out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16)
    if norm_weight is not None:
        assert epilogue in (EPI_BF16, EPI_SWIGLU) and norm_weight.dtype == torch.float32 and norm_weight.numel() == K
    box_m = 8 if M <= 8 else 16
    ss_parts, ss_count = None, 0
    if prenormed is not None:
        assert norm_weight is None and epilogue in (EPI_BF16, EPI_SWIGLU) and prenormed.dtype == torch.float32
        ss_parts, ss_count = prenormed, gemm_skinny_weight_tiles(K)      # the product before wrote K outputs a token
        assert prenormed.numel() >= ss_count * box_m
    emit_w = emit_xn = emit_ss = None
    if emit is not None:
        emit_w, emit_xn, emit_ss = emit
        _cuda(emit_w, emit_xn, emit_ss)
        assert epilogue == EPI_ADD and emit_w.dtype == torch.float32 and emit_w.numel() == N
        assert emit_xn.dtype == torch.bfloat16 and emit_xn.is_contiguous() and emit_xn.shape == (M, N)
        assert emit_ss.dtype == torch.float32 and emit_ss.numel() >= gemm_skinny_weight_tiles(N) * box_m
    map_w = tensor_map(w, int(lib().vob_gemm_skinny_weight_box(ctypes.c_long(N))), 4)
    map_x = tensor_map(x, box_m, 4)
    _check(lib().vob_gemm_skinny(map_w, map_x, _p(out), ctypes.c_long(out.stride(0)), M, N, K, epilogue, _p(norm_weight),
                                 ctypes.c_float(eps), _p(ss_parts), ss_count, _p(emit_w), _p(emit_xn), _p(emit_ss),
                                 _p(err), _stream()), "gemm_skinny")


def gemm_skinny_set_wait_limit(tries: int, withhold_copies: bool = False) -> None:
    """For tests of the bounded waits: after `tries` attempts a pipeline wait of the weight-streaming product gives up
    (0 restores the default); with `withhold_copies` its producers issue no copy, so the waits are for something that
    never comes.  The kernel then sets the timeout bits of the error word and returns without writing."""
    torch.cuda.synchronize()
    code = lib().vob_gemm_skinny_set_wait_limit(ctypes.c_uint(tries), int(withhold_copies))
    if code != 0:
        raise KernelError(f"gemm_skinny_set_wait_limit: {lib().vob_error_string(code).decode()}")


def sample(logits, temperature, top_k, top_p, keys, out, num_rows: int) -> None:
    _cuda(logits, temperature, top_k, top_p, keys, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    _check(lib().vob_sample(_p(logits), ctypes.c_long(logits.stride(0)), num_rows, logits.shape[1], _p(temperature),
                            _p(top_k), _p(top_p), _p(keys), _p(out), _stream()), "sample")


def apply_penalties(logits, row_of, token, count, presence, frequency, repetition, n: int) -> None:
    _cuda(logits, row_of, token, count)
    _check(lib().vob_apply_penalties(_p(logits), ctypes.c_long(logits.stride(0)), logits.shape[1], _p(row_of),
                                     _p(token), _p(count), _p(presence), _p(frequency), _p(repetition), n, _stream()),
           "apply_penalties")


def copy_pages(cache_plane, pairs, n_pairs: int) -> None:
    _cuda(cache_plane, pairs)
    page_elems = cache_plane[0].numel()
    _check(lib().vob_copy_pages(_p(cache_plane), _p(pairs), n_pairs, ctypes.c_long(page_elems),
                                _code(cache_plane.dtype), _stream()), "copy_pages")


if _os.environ.get("VOB_KERNEL_TIMERS", "") not in ("", "0"):
    enable_kernel_timers()

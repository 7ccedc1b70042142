"""Rakizen: config.json -> plan.

The layers come one by one from the configuration, each a `parallel` block (one float residual stream; ONE layer norm
with gain and bias that the mixer and the feed-forward both read; their outputs enter the stream together,
parts/parallel.py) around the mixer `attention_capped` (parts/capped_attention.py) in one of two settings:

  type `attention`    two softmax maps a head over shared values (`maps` = 2, the learned factor from lq1, lk1, lq2, lk2
                      and `diff`), keys visible inside blocks of `mask.size` positions, an output gate, nothing rotated;
  type `attention_2`  q and k normed over their whole projections, the first `rot.dims` elements of every head rotated in
                      neighbouring pairs by angles computed from the position, a sliding window of `mask.size` positions.

Both cap their scores (`softcap`) and take their factor on the score from the configuration (`scale`).  The feed-forward is
`swiglu` (parts/mlp.py), `routed_experts` (parts/moe.py) with gated SiLU experts, sigmoid scores, groups that count by
their two best scores and normalised, scaled weights, or absent.  Tensors are named embed, l<i>.norm1, l<i>.norm1.b,
l<i>.mix.<name>, l<i>.mlp.<name>, final.norm, final.norm.b, head.

`loop` = {start, stop, times}: layers start..stop-1 run `times` times in a row with the same weights.  Every run of a
layer is an `ExecStep` with a cache plane of its own, numbered in running order.
"""
from __future__ import annotations

from ..config.model_config import RakizenConfig
from ..parts.base import PartSpec
from .plan import ExecStep, ModelPlan

NO_POSITION_LIMIT = 1 << 30     # angles are computed from the position: nothing but int32 bounds it


def rakizen_plan(cfg: RakizenConfig) -> ModelPlan:
    D = cfg.width
    norm = lambda name: PartSpec("layernorm_stream", dict(size=D, eps=cfg.eps, weight_name=name, bias_name=name + ".b"))
    layers, positions = [], {}
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        size = int(m["mask"]["size"]) if m.get("mask") else 0
        common = dict(hidden_size=D, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), dim=int(m["dim"]),
                      vdim=int(m["vdim"]), scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0), eps=cfg.eps,
                      prefix=p + "mix.")
        if layer.type == "attention":
            mixer = PartSpec("attention_capped", dict(common, maps=2, diff=float(m["diff"]), gate=True, chunk=size))
        else:
            rot, position = m.get("rot"), None
            if rot and int(rot["dims"]) > 0:
                position = p + "rot"
                positions[position] = PartSpec("rope", dict(head_dim=int(m["dim"]), rotary_dim=int(rot["dims"]),
                                                            max_position=NO_POSITION_LIMIT, theta=float(rot["base"]),
                                                            interleaved=True, table=False))
            mixer = PartSpec("attention_capped", dict(common, row_norm=True, position=position, window=size))
        ff, mlp = None, layer.mlp
        if mlp is not None and mlp["kind"] == "dense":
            ff = PartSpec("swiglu", dict(hidden_size=D, intermediate_size=int(mlp["ff"]), prefix=p + "mlp.",
                                         names=("gate", "up", "down")))
        elif mlp is not None:
            r = mlp["router"]
            g = r.get("groups") or {"count": 1, "keep": 1}
            ff = PartSpec("routed_experts", dict(hidden_size=D, expert_size=int(mlp["expert"]["ff"]), experts=int(r["experts"]),
                                                 top=int(r["top"]), groups=int(g["count"]), keep=int(g["keep"]),
                                                 prefix=p + "mlp.", activation="silu_gated", scores="sigmoid", correction=False,
                                                 group_top=2, normalise=True, weight_scale=float(r.get("scale", 1.0))))
        layers.append(PartSpec("parallel", dict(mixer=mixer, feed_forward=ff, norm=norm(p + "norm1"), size=D)))
    order = [ExecStep(layer, plane, True) for plane, layer in enumerate(cfg.runs())]
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_position=NO_POSITION_LIMIT,
        embedding_name="embed", lm_head_name="head", final_norm=norm("final.norm"), positions=positions, layers=layers,
        order=order, eos_token_id=None, default_dtype=cfg.torch_dtype)

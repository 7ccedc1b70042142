"""Depolix: config.json -> plan.

The layers come one by one from the configuration, each a `parallel` block (one float residual stream; ONE RMS norm with a
gain stored around zero that the mixer and the feed-forward both read; `residual_mult` times the sum of their outputs enters
the stream, parts/parallel.py) around one of two mixers:

  type `latent_attention`  the mixer `latent_attention` (parts/latent_attention.py) with rotation of halves by stretched
                           frequencies computed from the position (a `rope` part made with table=False) and an output gate
                           an element;
  type `parallel`          the mixer `side_by_side` (parts/side_by_side.py) of `attention_conv` (parts/conv_attention.py:
                           short convolutions, unit-RMS q and k, a bias by distance, a window that keeps the first tokens, a
                           gate a head) and `gated_delta` (parts/delta.py) with a decay per head and key channel through a
                           low-rank projection and a low-rank sigmoid output gate.

The feed-forward is `glu_clamped` (parts/mlp.py) with biases, `routed_experts` (parts/moe.py) with clamped gated experts, a
bias on the router's logits and the softmax over the chosen logits as weights, or absent.  The embedded tokens are multiplied
by `embedding.scale` where the float stream begins, the logits by `logit_scale`.  Tensors are named embed, l<i>.norm1,
l<i>.mix.<name> (l<i>.mix.left.<name>, l<i>.mix.right.<name>, l<i>.mix.left.out, l<i>.mix.right.out), l<i>.mlp.<name>,
final.norm, head.
"""
from __future__ import annotations

from ..config.model_config import DepolixConfig
from ..parts.base import PartSpec
from .plan import ExecStep, ModelPlan

NO_POSITION_LIMIT = 1 << 30     # angles are computed from the position: nothing but int32 bounds it


def depolix_plan(cfg: DepolixConfig) -> ModelPlan:
    D = cfg.width
    norm = lambda name: PartSpec("rmsnorm_parallel_stream", dict(size=D, eps=cfg.eps, weight_name=name, one_plus=True,
                                                                 mult=cfg.residual_mult, open_scale=cfg.embedding_scale))
    layers, positions = [], {}
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == "latent_attention":
            rot, position = m["rot"], None
            if int(rot["dims"]) > 0:
                position = p + "rot"
                positions[position] = PartSpec("rope", dict(head_dim=int(m["rot_dim"]), rotary_dim=int(rot["dims"]),
                                                            max_position=NO_POSITION_LIMIT, theta=float(rot["base"]),
                                                            interleaved=False, scaling=rot.get("scaling"), table=False,
                                                            precise=True))
            mixer = PartSpec("latent_attention", dict(hidden_size=D, num_heads=int(m["heads"]), dim=int(m["dim"]),
                                                      rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]), q_rank=int(m["q_rank"]),
                                                      kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), eps=cfg.eps,
                                                      window=None, position=position, prefix=p + "mix.", gate=True))
        else:
            l, r = m["left"], m["right"]
            mask = l.get("mask") or {}
            # the bias table's rows and the ranks of the low-rank projections are sizes of the checkpoint's tensors (-1), unless
            # the configuration states them (a model with random weights has no tensors to count)
            rel_rows = int(l.get("bias_rows") or -1) if l.get("bias_max") is not None else 0
            left = PartSpec("attention_conv", dict(hidden_size=D, num_heads=int(l["heads"]), num_kv_heads=int(l["kv_heads"]),
                                                   dim=int(l["dim"]), vdim=int(l["vdim"]), scale=float(l["scale"]),
                                                   taps=int(l["conv"]), eps=cfg.eps, prefix=p + "mix.left.",
                                                   window=int(mask.get("size") or 0), keep_first=int(mask.get("keep_first") or 0),
                                                   bias_rows=rel_rows, bias_max=float(l.get("bias_max") or 0.0), unit_norm=True,
                                                   gate=True))
            right = PartSpec("gated_delta", dict(hidden_size=D, num_heads=int(r["heads"]), num_kv_heads=int(r["kv_heads"]),
                                                 dim=int(r["dim"]), vdim=int(r["vdim"]), taps=int(r["conv"]), eps=cfg.eps,
                                                 prefix=p + "mix.right.", decay_rank=int(r.get("decay_rank") or -1),
                                                 gate_rank=int(r.get("gate_rank") or -1), gate="sigmoid"))
            mixer = PartSpec("side_by_side", dict(left=left, right=right, hidden_size=D, eps=cfg.eps,
                                                  left_norm=p + "mix.left.out", right_norm=p + "mix.right.out"))
        ff, mlp = None, layer.mlp
        if mlp is not None and mlp["kind"] == "dense":
            ff = PartSpec("glu_clamped", dict(hidden_size=D, intermediate_size=int(mlp["ff"]), limit=float(mlp["limit"]),
                                              prefix=p + "mlp.", bias=True))
        elif mlp is not None:
            r = mlp["router"]
            ff = PartSpec("routed_experts", dict(hidden_size=D, expert_size=int(mlp["expert"]["ff"]), experts=int(r["experts"]),
                                                 top=int(r["top"]), prefix=p + "mlp.", activation="glu_clamped",
                                                 limit=float(mlp["expert"]["limit"]), scores="softmax", correction=False,
                                                 normalise=True, router_bias=True))
        layers.append(PartSpec("parallel", dict(mixer=mixer, feed_forward=ff, norm=norm(p + "norm1"), size=D)))
    order = [ExecStep(i, i, True) for i in range(len(cfg.layers))]
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_position=NO_POSITION_LIMIT,
        embedding_name="embed", lm_head_name="head",
        final_norm=PartSpec("rmsnorm_parallel_stream", dict(size=D, eps=cfg.eps, weight_name="final.norm", one_plus=True,
                                                            mult=cfg.residual_mult, open_scale=cfg.embedding_scale,
                                                            out_scale=cfg.logit_scale)), positions=positions, layers=layers,
        order=order, eos_token_id=None, default_dtype=cfg.torch_dtype)

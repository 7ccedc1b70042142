"""Decode and prefill throughput of the engine at Qwen3-8B sizes (bf16, random weights, one B200).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step.  The default run has the layer sizes of the 8B configuration, a batch
of 8 requests whose context starts at 2,048 tokens, and prints ONE JSON line:
  value     decoded tokens per second, timed on the device with CUDA events around K steps;
  e2e       the same through the Python entry point (LLM.add_request / LLM.step): pinned host
            buffers in, sampled tokens out, every step;
  prefill   one 2,048-token prompt in one step; frac = flops / time / peak;
  roofline  the decode step's bytes (every weight once + the cache of the live requests) / time
            against the measured copy bandwidth;
  points    decode at batch 1, 16, 32 and 64 with their fractions of the copy bandwidth; the end-to-end rate at batch 1
            and 64 and the host's time per step (end-to-end minus device) at batch 1, 8 and 64; decode at contexts of
            8,192 and 32,768 tokens (batch 1 and 8);
  workloads serving_0_6b: 256 whole requests at Qwen3-0.6B sizes through LLM.generate (continuous batching), with the
            bytes its steps had to move against the copy bandwidth.
The cache that the decode steps read was written by a real prefill of random prompts.  Every timed step reads 15 GB of weights, far more than the 126 MB L2, so nothing stays cached
between iterations.  Peaks come from MEASURED_PEAKS.json beside this file when present.

    python bench.py --workload tofilorn | kesozen | rakizen | depolix [--sizes 2048,4096]

measures the Tofilorn design (residual streams, minGRU, HGRN2, latent attention), the Kesozen design (sandwich norms over
a float stream, attention whose keys are its values, gated delta rule, routed experts) or the Rakizen design (parallel
layers over a float stream, capped scores, two-map heads over blocks of positions, sliding windows, gated experts; also
beside Kesozen, with attention held against arithmetic in prompts and against the keys and values read in decoding) at layer sizes of 1B- and 8B-class
models beside Qwen3 at the same width, depth and feed-forward size (Kesozen also beside Tofilorn): one 2,048-token prompt in one step, decode at batch 8
and 64 from a 2,048-token context (CUDA graphs), and, from an eager engine with the per-kernel timers on, the time of each
of this package's kernels in those steps with the bytes it must move against the copy bandwidth.

    python bench.py --workload serving-0.6b | mixed-32b

runs one of the two other workloads instead (whole requests through LLM.generate, wall clock, a JSON line of its
own): 256 requests with prompts of 16 to 1,024 tokens and 128 new tokens each at Qwen3-0.6B sizes (continuous
batching), or 32 requests with prompts of 512 to 8,192 tokens and 256 new tokens at Qwen3-32B sizes under an
8,192-token step budget and a cache pool too small for all of them (portions, recompute preemption).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1000000.0,
                rms_norm_eps=1e-6, max_position_embeddings=40960, tie_word_embeddings=False, hidden_act="silu",
                attention_bias=False, torch_dtype="bfloat16")
PROMPT_LEN, NEW_TOKENS, CONTEXT, BLOCK = 2048, 256, 4096, 256
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            flat = {}
            def walk(x):
                if isinstance(x, dict):
                    for k, v in x.items():
                        if isinstance(v, (int, float)):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(d)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return dict(hbm_gbs=flat["hbm_gbs"], bf16_tflops=flat["bf16_tflops"],
                            bf16_tflops_sustained=flat.get("bf16_tflops_sustained"), source="measured")
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        self.result = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            self.result = dict(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons))


def model_numbers(c):
    H, L, nh, kvh, hd, I, V = (c["hidden_size"], c["num_hidden_layers"], c["num_attention_heads"], c["num_key_value_heads"],
                               c["head_dim"], c["intermediate_size"], c["vocab_size"])
    per_layer = (nh + 2 * kvh) * hd * H + nh * hd * H + 3 * I * H
    linear_params = L * per_layer
    weight_bytes = 2 * (linear_params + V * H) + 4 * (L * (2 * H + 2 * hd) + H)   # bf16 matrices + lm_head, f32 norms
    kv_bytes_per_token = 2 * L * kvh * hd * 2
    return dict(linear_params=linear_params, weight_bytes=weight_bytes, kv_bytes_per_token=kv_bytes_per_token,
                lm_head_params=V * H, L=L, nh=nh, hd=hd)


def prefill_flops(c, T):
    n = model_numbers(c)
    linear = 2 * T * n["linear_params"] + 2 * n["lm_head_params"]          # lm_head on one row
    attention = n["L"] * 4 * n["nh"] * n["hd"] * (T * (T + 1) // 2)         # causal QK^T and PV
    return linear + attention


def fill_cache(llm, ids, ctx_len, seed):
    """Prompts of `ctx_len` random tokens for the requests `ids`, run through the step function in steps of at most the
    token budget, so that the pages the decode steps will read hold real keys and values."""
    import torch
    from vllm_oxide_b200 import host
    mgr, core = llm.cache.manager, llm.core
    g = torch.Generator().manual_seed(seed)
    budget = llm.options.max_num_batched_tokens
    for rid in ids:
        toks = torch.randint(0, llm.model.vocab_size, (ctx_len,), generator=g).tolist()
        for start in range(0, ctx_len, budget):
            core.run([host.BatchEntry(rid, start, toks[start:start + budget], [])])
    torch.cuda.synchronize()
    core.check_errors()


def decode_run(llm, batch, steps, warmup, start_ctx):
    """K decode steps of `batch` requests whose context starts at `start_ctx` (prefilled), timed on the device."""
    import torch
    from vllm_oxide_b200 import host, kernels
    mgr, core, sampler = llm.cache.manager, llm.core, llm.sampler
    ids = list(range(10_000, 10_000 + batch))
    for rid in ids:
        assert mgr.add_request(rid) and mgr.ensure(rid, 0, start_ctx)
    fill_cache(llm, ids, start_ctx, seed=batch)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, llm.model.vocab_size, (batch, steps + warmup), generator=g).tolist()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    temp, topk, topp, keys = [0.0] * batch, [0] * batch, [1.0] * batch, [0] * batch
    pos = start_ctx
    launches0 = 0
    for i in range(steps + warmup):
        if i == warmup:
            torch.cuda.synchronize()
            launches0 = kernels.launch_count
            ev0.record()
        entries = []
        for b, rid in enumerate(ids):
            assert mgr.ensure(rid, pos, 1)
            entries.append(host.BatchEntry(rid, pos, [toks[b][i]], [0]))
        logits = core.run(entries)
        sampler.forward(logits, temp, topk, topp, keys)
        pos += 1
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / steps
    launches = kernels.launch_count - launches0
    core.check_errors()
    for rid in ids:
        mgr.free_request(rid)
    mean_ctx = start_ctx + warmup + (steps + 1) / 2
    return ms, launches, mean_ctx


def decode_kernel_times(llm, batch, steps, start_ctx):
    """{kernel: milliseconds a step} of this package's kernels in decode steps of an eager engine with the kernel timers on
    (the prompts that fill the cache are not counted)."""
    import torch
    from vllm_oxide_b200 import host, kernels
    mgr, core = llm.cache.manager, llm.core
    ids = list(range(30_000, 30_000 + batch))
    for rid in ids:
        assert mgr.add_request(rid) and mgr.ensure(rid, 0, start_ctx)
    fill_cache(llm, ids, start_ctx, seed=batch)
    for i in range(3 + steps):
        if i == 3:
            kernels.kernel_timer_report()
        for rid in ids:
            assert mgr.ensure(rid, start_ctx + i, 1)
        core.run([host.BatchEntry(rid, start_ctx + i, [1 + i], [0]) for rid in ids])
    times = {k: round(v[1] / steps, 4) for k, v in sorted(kernels.kernel_timer_report().items())}
    for rid in ids:
        mgr.free_request(rid)
    return times


def e2e_run(llm, batch, steps, warmup):
    """The same metric through the public calls: prompts of 2,048 host token ids in, tokens out each step.
    Returns (tokens a second, host-to-device bytes a step, device-to-host bytes a step, milliseconds a step)."""
    import torch
    from vllm_oxide_b200 import SamplingParams
    g = torch.Generator().manual_seed(100 + batch)       # other prompts in every run: nothing comes from the prefix cache
    prompts = torch.randint(0, llm.model.vocab_size, (batch, PROMPT_LEN), generator=g).tolist()
    entered = lambda: llm.scheduler.stats.prefill_tokens + llm.scheduler.stats.prefix_hit_tokens
    before = entered()
    # the first requests decode while the later prompts are still being computed: room for those tokens too
    room = steps + warmup + 16 + batch * PROMPT_LEN // llm.options.max_num_batched_tokens
    for p in prompts:
        llm.add_request(p, SamplingParams(temperature=0.0, max_tokens=room, ignore_eos=True))
    while llm.is_running() and entered() - before < batch * PROMPT_LEN:
        llm.step()                            # prompts, in portions under the token budget
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    h2d = d2h = 0
    for _ in range(steps):
        llm.step()                            # pinned batch arrays in, sampled tokens out
        h2d += llm.core.h2d_bytes_last + 20 * batch
        d2h += 4 * batch + 4
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert llm.scheduler.num_running == batch, "a request finished inside the timed region"
    while llm.is_running():
        llm.step()
    return batch * steps / dt, h2d // steps, d2h // steps, dt / steps * 1e3


def prefill_run(llm, T, reps=3, warmup=2):
    import torch
    from vllm_oxide_b200 import host
    mgr, core = llm.cache.manager, llm.core
    g = torch.Generator().manual_seed(2)
    best = None
    for i in range(reps + warmup):
        toks = torch.randint(0, llm.model.vocab_size, (T,), generator=g).tolist()
        rid = 20_000 + i
        assert mgr.add_request(rid) and mgr.ensure(rid, 0, T)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        core.run([host.BatchEntry(rid, 0, toks, [T - 1])])
        ev1.record()
        torch.cuda.synchronize()
        mgr.free_request(rid)
        if i >= warmup:
            ms = ev0.elapsed_time(ev1)
            best = ms if best is None else min(best, ms)
    core.check_errors()
    return best


WORKLOADS = {
    "serving-0.6b": dict(
        config=dict(num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                    intermediate_size=3072, tie_word_embeddings=True),
        requests=256, prompt=(16, 1024), new=128, seed=2,
        options=dict(max_model_len=2048, block_size=256, max_num_seqs=256, max_num_batched_tokens=8192, num_kv_blocks=2048)),
    "mixed-32b": dict(
        config=dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                    intermediate_size=25600, tie_word_embeddings=False),
        requests=32, prompt=(512, 8192), new=256, seed=3,
        # all 32 contexts together would need about 580 pages of 256 tokens: the pool holds 400
        options=dict(max_model_len=8192 + 256, block_size=256, max_num_seqs=32, max_num_batched_tokens=8192, num_kv_blocks=400)),
}


def workload_run(name: str, pk=None) -> dict:
    """Whole requests through the public entry point (LLM.generate, wall clock).  Returns the record of the run: rates,
    steps, mean number of requests in a step, and the bytes its steps had to move (every weight once a step, the cache
    of every scheduled request's context, and the float logits of every sampled row written by the output product and
    read by the sampler) against the copy bandwidth."""
    import random
    import torch
    from vllm_oxide_b200 import LLM, EngineOptions, SamplingParams
    w = WORKLOADS[name]
    pk = pk or peaks()
    cfg = dict(QWEN3_8B)
    cfg.update(w["config"])
    llm = LLM.from_config(cfg, EngineOptions(dtype="bfloat16", **w["options"]), seed=w["seed"], init_scheme="0.02")
    rng = random.Random(0)
    lo, hi = w["prompt"]
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(lo, hi))] for _ in range(w["requests"])]
    sp = SamplingParams(temperature=0.0, max_tokens=w["new"], ignore_eos=True)
    # warm-up: the same shape of work once with other prompts (libraries, a CUDA graph per batch size met; nothing of the
    # timed prompts may lie in the prefix cache)
    wrng = random.Random(1)
    warm = [[wrng.randrange(cfg["vocab_size"]) for _ in range(len(p))] for p in prompts]
    llm.generate(warm, [sp] * len(warm))
    torch.cuda.synchronize()
    s0 = llm.scheduler.stats
    before = (s0.steps, s0.scheduled_requests, s0.context_tokens, s0.sampled_rows)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, [sp] * len(prompts))
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert all(o.finished and len(o.token_ids) == w["new"] for o in outs)
    st, s1 = llm.last_stats, llm.scheduler.stats
    steps, scheduled, context, rows = (b - a for a, b in zip(before, (s1.steps, s1.scheduled_requests, s1.context_tokens,
                                                                      s1.sampled_rows)))
    n = model_numbers(cfg)
    weight_bytes = n["weight_bytes"]       # the layers and the output matrix (tied or not, it is read once a step)
    moved = steps * weight_bytes + context * n["kv_bytes_per_token"] + rows * cfg["vocab_size"] * 8
    achieved = moved / dt / 1e9
    flops = 2 * st.total_tokens * n["linear_params"] + 2 * rows * n["lm_head_params"]
    return {
        "metric": f"tokens/s over whole requests ({name})", "value": round(st.total_tokens / dt, 1), "unit": "tokens/s",
        "generated_tokens_per_s": round(w["requests"] * w["new"] / dt, 1), "seconds": round(dt, 3), "steps": steps,
        "mean_requests_per_step": round(scheduled / max(steps, 1), 1), "preemptions": st.preemptions,
        "bytes_per_step_gb": round(moved / max(steps, 1) / 1e9, 3),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "linear_tflops": round(flops / dt / 1e12, 1),
        "n_gpus": 1, "dtype": "bf16", "impl": "ours", "data": "synthetic token ids, seeded random weights",
        "config": {"model": name, "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "requests": w["requests"],
                   "prompt_min": lo, "prompt_max": hi, "new_tokens": w["new"], "step_budget": w["options"]["max_num_batched_tokens"],
                   "pool_pages": w["options"]["num_kv_blocks"], "block_size": w["options"]["block_size"]}}


def tofilorn_config(width: int, layers: int) -> dict:
    """Layer sizes of a real model of this width: a block of four layers (latent attention, minGRU, HGRN2, latent attention that
    borrows the first one's keys), each with a gated feed-forward of three times the width, over four residual streams."""
    heads = width // 128
    rot = {"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    att = lambda src: dict(heads=heads, dim=128, rot_dim=64, vdim=128, q_rank=3 * width // 8, kv_rank=192, scale=192 ** -0.5,
                           mask={"size": 1024}, rot=rot, **({} if src is None else {"kv_from": src}))
    mlp = {"kind": "dense", "ff": 3 * width}
    out = []
    for i in range(0, layers, 4):
        out += [{"type": "latent_attention", "mixer": att(None), "mlp": mlp}, {"type": "mingru", "mixer": {"width": 2 * width}, "mlp": mlp},
                {"type": "hgrn2", "mixer": {"heads": heads, "dim": 128, "vdim": 128}, "mlp": mlp},
                {"type": "latent_attention", "mixer": att(i), "mlp": mlp}]
    return {"architecture": "Tofilorn", "vocab": 32768, "width": width, "streams": 4, "norm": {"eps": 1e-6}, "layers": out[:layers]}


def tofilorn_kernel_bytes(cfg: dict, T: int) -> dict:
    """Bytes that each of the design's own kernels must move in a step of T tokens, summed over the layers (weights aside,
    which T tokens share): what its time is held against."""
    D, S = cfg["width"], cfg.get("streams", 1)
    b = {"stream_step": 0, "mingru_scan": 0, "hgrn2_scan": 0, "latent_prep": 0, "head_linear": 0, "latent_query_rotate": 0}
    for l in cfg["layers"]:
        m = l["mixer"]
        subs = 2 if l["mlp"] else 1
        if l["mlp"]:
            b["silu_mul"] = b.get("silu_mul", 0) + T * 3 * l["mlp"]["ff"] * 2
        b["stream_step"] += subs * T * (2 * S * D * 4 + 2 * D * 2)                # streams read and written, y in, normed out
        if l["type"] == "mingru":
            b["mingru_scan"] += T * 4 * m["width"] * 2
            b["silu_mul"] = b.get("silu_mul", 0)
        elif l["type"] == "hgrn2":
            b["hgrn2_scan"] += T * m["heads"] * (2 * m["dim"] + 2 * m["vdim"]) * 2
        else:
            row = (m["kv_rank"] + m["rot_dim"] + 15) // 16 * 16
            b["latent_prep"] += T * (2 * m["q_rank"] + (0 if "kv_from" in m else 2 * row)) * 2
            b["latent_query_rotate"] += T * m["heads"] * 2 * m["rot_dim"] * 2
            b["head_linear"] += (T * m["heads"] * (m["dim"] + 2 * row + m["vdim"]) + 2 * m["heads"] * m["kv_rank"] * (m["dim"] + m["vdim"])) * 2
    return b


def kesozen_config(width: int, layers: int) -> dict:
    """Layer sizes of a real model of this width: a block of four layers (three gated delta rules, then attention whose keys
    are its values); feed-forwards of 16 experts of which a token uses 4 (the four together three times the width), but
    for the second layer of each block, whose feed-forward is dense and three times the width; heads of 128."""
    heads = width // 128
    att = dict(heads=heads, kv_heads=8, dim=128, vdim=128, scale=128 ** -0.5, rot={"dims": 64, "base": 10000.0})
    delta = dict(heads=heads, kv_heads=max(1, heads // 2), dim=128, vdim=128, conv=4)
    moe = {"kind": "moe", "expert": {"ff": 3 * width // 4}, "router": {"experts": 16, "top": 4, "groups": {"count": 4, "keep": 2}}}
    dense = {"kind": "dense", "ff": 3 * width}
    out = []
    for _ in range(0, layers, 4):
        out += [{"type": "delta", "mixer": delta, "mlp": moe}, {"type": "delta", "mixer": delta, "mlp": dense},
                {"type": "delta", "mixer": delta, "mlp": moe}, {"type": "attention", "mixer": att, "mlp": moe}]
    return {"architecture": "Kesozen", "vocab": 32768, "width": width, "norm": {"eps": 1e-6}, "layers": out[:layers]}


def kesozen_kernel_bytes(cfg: dict, T: int) -> dict:
    """Bytes that each of the design's own row-wise kernels must move in a step of T tokens, summed over the layers (weights
    aside): what its time is held against.  The scan and the experts' products are held against arithmetic instead."""
    D = cfg["width"]
    b = {"residual_norm_step": T * (D * 2 + D * 4 + D * 2) + T * D * 4}          # the embedding's norm; the last norm reads the stream
    for l in cfg["layers"]:
        m, mlp = l["mixer"], l["mlp"]
        subs = 2 if mlp else 1
        b["residual_norm_step"] += subs * T * (2 * D * 4 + 2 * D * 2)             # stream read and written, y in, normed out
        if l["type"] == "attention":
            nh, kvh, hd = m["heads"], m["kv_heads"], m["dim"]
            b["rope_shared_kv_write"] = b.get("rope_shared_kv_write", 0) + T * ((nh + kvh) + nh + 2 * kvh) * hd * 2
        else:
            C, V = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"], m["heads"] * m["vdim"]
            b["short_conv_silu"] = b.get("short_conv_silu", 0) + T * C * (2 + 4)
            b["delta_out_norm"] = b.get("delta_out_norm", 0) + T * V * (4 + 2 + 2)
        if mlp and mlp["kind"] == "dense":
            b["relu_squared"] = b.get("relu_squared", 0) + T * mlp["ff"] * 2 * 2
        elif mlp:
            top = mlp["router"]["top"]
            b["moe_gather_rows"] = b.get("moe_gather_rows", 0) + T * top * D * 2 * 2
            b["moe_combine"] = b.get("moe_combine", 0) + T * (top * D * 4 + D * 2)
    return b


def rakizen_config(width: int, layers: int) -> dict:
    """Layer sizes of a real model of this width: a block of four layers (two-map attention over blocks of 1,536 positions,
    two sliding windows of 1,024 with half of every head rotated, two-map attention again), heads of 128 with 8 key heads
    (the two-map layers hold two key maps a key head); feed-forwards of 16 gated experts of which a token uses 4 (the four
    together three times the width), but for the second layer of each block, whose feed-forward is dense and three times
    the width."""
    heads = width // 128
    two = dict(heads=heads, kv_heads=8, dim=128, vdim=128, diff=0.3, scale=128 ** -0.5, softcap=30.0, mask={"size": 1536})
    win = dict(heads=heads, kv_heads=8, dim=128, vdim=128, scale=128 ** -0.5, softcap=30.0, mask={"size": 1024},
               rot={"dims": 64, "base": 10000.0})
    moe = {"kind": "moe", "expert": {"ff": 3 * width // 4}, "router": {"experts": 16, "top": 4, "groups": {"count": 4, "keep": 2},
                                                                     "scale": 2.0}}
    dense = {"kind": "dense", "ff": 3 * width}
    out = []
    for _ in range(0, layers, 4):
        out += [{"type": "attention", "mixer": two, "mlp": moe}, {"type": "attention_2", "mixer": win, "mlp": dense},
                {"type": "attention_2", "mixer": win, "mlp": moe}, {"type": "attention", "mixer": two, "mlp": moe}]
    return {"architecture": "Rakizen", "vocab": 32768, "width": width, "norm": {"eps": 1e-6}, "layers": out[:layers]}


def rakizen_kernel_bytes(cfg: dict, T: int) -> dict:
    """Bytes that each of the design's own row-wise kernels must move in a step of T tokens, summed over the layers (weights
    aside): what its time is held against.  Attention and the experts' products are held against arithmetic instead."""
    D = cfg["width"]
    b = {"layer_norm_step": T * (D * 2 + D * 4 + D * 2)}                          # the stream begins: tokens in, stream and normed out
    for l in cfg["layers"]:
        m, mlp = l["mixer"], l["mlp"]
        maps = 2 if l["type"] == "attention" else 1
        nh, kvh, d, e = maps * m["heads"], maps * m["kv_heads"], m["dim"], m["vdim"]
        b["layer_norm_step"] += T * (2 * D * 4 + (3 if mlp else 2) * D * 2)       # stream read and written, outputs in, normed out
        # q and k read and written back, v read; k and v written to the cache
        b["rownorm_rope_kv_write"] = b.get("rownorm_rope_kv_write", 0) + T * (2 * (nh + kvh) * d + 2 * m["kv_heads"] * e + kvh * d) * 2
        if maps == 2:
            b["diff_heads_combine"] = b.get("diff_heads_combine", 0) + T * m["heads"] * e * (2 * 4 + 2 + 2)
        if mlp and mlp["kind"] == "dense":
            b["silu_mul"] = b.get("silu_mul", 0) + T * 3 * mlp["ff"] * 2
        elif mlp:
            top = mlp["router"]["top"]
            b["moe_gather_rows"] = b.get("moe_gather_rows", 0) + T * top * D * 2 * 2
            b["moe_combine"] = b.get("moe_combine", 0) + T * (top * D * 4 + D * 2)
    return b


def depolix_config(width: int, layers: int) -> dict:
    """Layer sizes of a real model of this width: a block of four layers (attention through a latent of 512 + 64 rotated, heads
    of 128 + 64; two mixers side by side: attention behind filters of 4 taps, heads of 128 over 8 key heads, a window of 1,024
    that keeps the first 64 tokens, a bias by distance of 32 rows up to 4,096; and a gated delta rule with half as many heads,
    a decay per key channel through rank 64; attention through a latent again, twice); feed-forwards of 16 clamped gated experts
    of which a token uses 4 (the four together three times the width), but for the second layer of each block, whose
    feed-forward is dense and three times the width."""
    heads = width // 128
    latent = dict(heads=heads, dim=128, rot_dim=64, vdim=128, q_rank=3 * width // 8, kv_rank=192, scale=192 ** -0.5,
                  rot={"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}})
    sides = {"left": dict(heads=heads, kv_heads=8, dim=128, vdim=128, conv=4, scale=128 ** -0.5, bias_rows=32, bias_max=4096.0,
                          mask={"size": 1024, "keep_first": 64}),
             "right": dict(heads=max(1, heads // 2), kv_heads=max(1, heads // 4), dim=128, vdim=128, conv=4, decay_rank=64, gate_rank=64)}
    moe = {"kind": "moe", "expert": {"ff": 3 * width // 4, "limit": 7.0}, "router": {"experts": 16, "top": 4}}
    dense = {"kind": "dense", "ff": 3 * width, "limit": 7.0}
    out = []
    for _ in range(0, layers, 4):
        out += [{"type": "latent_attention", "mixer": latent, "mlp": moe}, {"type": "parallel", "mixer": sides, "mlp": dense},
                {"type": "latent_attention", "mixer": latent, "mlp": moe}, {"type": "latent_attention", "mixer": latent, "mlp": moe}]
    return {"architecture": "Depolix", "vocab": 32768, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "residual_mult": 0.5, "logit_scale": 1.0, "layers": out[:layers]}


def depolix_kernel_bytes(cfg: dict, T: int) -> dict:
    """Bytes that each of the design's own row-wise kernels must move in a step of T tokens, summed over the layers (weights
    aside): what its time is held against.  Attention, the scan and the experts' products are held against arithmetic."""
    D = cfg["width"]
    b = {"rms_norm_step": T * (D * 2 + D * 4 + D * 2) + T * D * 4}                # the stream begins; the last norm reads it
    for l in cfg["layers"]:
        m, mlp = l["mixer"], l["mlp"]
        b["rms_norm_step"] += T * (2 * D * 4 + (3 if mlp else 2) * D * 2)         # stream read and written, outputs in, normed out
        if l["type"] == "latent_attention":
            row = (m["kv_rank"] + m["rot_dim"] + 15) // 16 * 16
            b["latent_prep"] = b.get("latent_prep", 0) + T * ((m["q_rank"] + m["kv_rank"] + m["rot_dim"]) + m["q_rank"] + row) * 2
            b["latent_query_rotate"] = b.get("latent_query_rotate", 0) + T * m["heads"] * 2 * m["rot_dim"] * 2
            b["sigmoid_gate_mul"] = b.get("sigmoid_gate_mul", 0) + T * m["heads"] * m["vdim"] * 3 * 2
        else:
            le, ri = m["left"], m["right"]
            C = (le["heads"] + le["kv_heads"]) * le["dim"] + le["kv_heads"] * le["vdim"]
            Cr, V = 2 * ri["kv_heads"] * ri["dim"] + ri["heads"] * ri["vdim"], ri["heads"] * ri["vdim"]
            b["short_conv_silu"] = b.get("short_conv_silu", 0) + T * (C + Cr) * (2 + 4)
            b["unit_qk_kv_write"] = b.get("unit_qk_kv_write", 0) + T * C * (4 + 2)
            b["delta_out_norm"] = b.get("delta_out_norm", 0) + T * V * (4 + 2 + 2)
            b["pair_norm_mean"] = b.get("pair_norm_mean", 0) + T * 3 * D * 2
        if mlp and mlp["kind"] == "dense":
            b["clamped_glu"] = b.get("clamped_glu", 0) + T * 3 * mlp["ff"] * 2
        elif mlp:
            top = mlp["router"]["top"]
            b["moe_gather_rows"] = b.get("moe_gather_rows", 0) + T * top * D * 2 * 2
            b["moe_combine"] = b.get("moe_combine", 0) + T * (top * D * 4 + D * 2)
    return b


def attention_flops(cfg: dict, T: int) -> float:
    """Multiply-adds x 2 of the score and value products of one prompt of T tokens, every query over the keys it sees."""
    def seen(size, blocks):
        if not size:
            return T * (T + 1) // 2
        return sum((i % size if blocks else min(i, size - 1)) + 1 for i in range(T))
    if "layers" not in cfg:
        return cfg["num_hidden_layers"] * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * seen(0, False)
    total = 0.0
    for l in cfg["layers"]:
        m = l["mixer"]
        if l["type"] in ("attention", "attention_2") and "dim" in m:
            maps = 2 if (l["type"] == "attention" and "diff" in m) else 1
            size = (m.get("mask") or {}).get("size", 0)
            total += 2.0 * maps * m["heads"] * (m["dim"] + m["vdim"]) * seen(size, maps == 2)
    return total


def attention_decode_bytes(cfg: dict, batch: int, context: int) -> float:
    """Bytes of keys and values that one decode step of `batch` requests at `context` tokens must read (bfloat16)."""
    if "layers" not in cfg:
        return cfg["num_hidden_layers"] * batch * context * 2.0 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    total = 0.0
    for l in cfg["layers"]:
        m = l["mixer"]
        if l["type"] in ("attention", "attention_2") and "dim" in m:
            two = l["type"] == "attention" and "diff" in m
            size = (m.get("mask") or {}).get("size", 0)
            keys = context if not size else (context % size + 1 if two else min(context, size))
            planes = m["dim"] if cfg["architecture"] == "Kesozen" else (2 if two else 1) * m["dim"] + m["vdim"]   # Kesozen: keys are values
            total += batch * keys * m["kv_heads"] * planes * 2.0
    return total


def qwen3_kernel_bytes(cfg: dict, T: int) -> dict:
    """The same for the row-wise kernels of a Qwen3 step: add+norm reads the stream and writes the normed rows (the sum was made
    by the product before), the q/k kernel reads q|k|v, writes q and k back and k, v to the cache, SiLU*up reads 2I and writes I."""
    L, D, I = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"]
    nh, kvh, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    return {"add_rmsnorm": 2 * L * T * D * 2 * 2, "silu_mul": L * T * 3 * I * 2,
            "qk_norm_rope_kv_write": L * T * ((nh + 2 * kvh) + (nh + kvh) + 2 * kvh) * hd * 2}


DESIGNS = {"tofilorn": (tofilorn_config, tofilorn_kernel_bytes), "kesozen": (kesozen_config, kesozen_kernel_bytes),
           "rakizen": (rakizen_config, rakizen_kernel_bytes), "depolix": (depolix_config, depolix_kernel_bytes)}


def float_issue_rate():
    """Float instructions a second the device can issue: SMs x 128 lanes x the largest SM clock (0 if the clock cannot be read)."""
    import torch
    try:
        mhz = float(subprocess.run(["nvidia-smi", "--query-gpu=clocks.max.sm", "--format=csv,noheader,nounits", "-i", "0"],
                                   capture_output=True, text=True, timeout=20).stdout.split()[0])
    except (OSError, ValueError, IndexError, subprocess.SubprocessError):
        mhz = 0.0
    return torch.cuda.get_device_properties(0).multi_processor_count * 128 * mhz * 1e6


def design_run(design: str, widths, pk=None, layers: int = 16) -> dict:
    """One of the listed-layer designs beside Qwen3 (and, for the scan kernels, beside each other) at equal layer sizes."""
    import torch
    from vllm_oxide_b200 import LLM, EngineOptions, kernels
    pk = pk or peaks()
    label = design.capitalize()
    out = {"metric": f"tokens/s, {label} beside Qwen3 at equal layer sizes", "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16",
           "data": "synthetic token ids, seeded random weights", "peaks": pk, "sizes": {}}
    bytes_of = {"qwen3": qwen3_kernel_bytes, **{k: v[1] for k, v in DESIGNS.items()}}
    for width in widths:
        models = {design: DESIGNS[design][0](width, layers),
                  "qwen3": dict(QWEN3_8B, num_hidden_layers=layers, hidden_size=width, num_attention_heads=width // 128,
                                num_key_value_heads=8, intermediate_size=3 * width, vocab_size=32768, max_position_embeddings=8192)}
        if design == "kesozen":
            models["tofilorn"] = tofilorn_config(width, layers)       # its matrix-state scan is the delta rule's like kernel
        if design == "rakizen":
            models["kesozen"] = kesozen_config(width, layers)         # the float stream and the routed experts are its like kernels
        if design == "depolix":
            models["kesozen"] = kesozen_config(width, layers)         # the delta rule, the gated heads and the routed experts
            models["tofilorn"] = tofilorn_config(width, layers)       # attention through a latent
        rec = {}
        for name, cfg in models.items():
            r = {}
            for eager in (False, True):
                opts = EngineOptions(max_model_len=CONTEXT, block_size=BLOCK, num_kv_blocks=64 * 10 + 16, max_num_seqs=64,
                                     max_num_batched_tokens=8192, dtype="bfloat16", enforce_eager=eager)
                llm = LLM.from_config(cfg, opts, seed=0, init_scheme="0.02")
                if not eager:
                    r["weight_gb"] = round(llm.model.weight_bytes() / 1e9, 3)
                    ms = prefill_run(llm, PROMPT_LEN)
                    r["prefill_2048"] = {"ms": round(ms, 3), "tokens_per_s": round(PROMPT_LEN * 1e3 / ms)}
                    for batch in (8, 64):
                        ms, launches, _ = decode_run(llm, batch, 32, 4, PROMPT_LEN)
                        r[f"decode_batch{batch}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(batch * 1e3 / ms), "launches": launches // 32}
                else:
                    # this package's kernels one by one (library products are not among them), milliseconds a step
                    kernels.enable_kernel_timers(True)
                    prefill_run(llm, PROMPT_LEN, reps=1, warmup=1)
                    kernels.kernel_timer_report()
                    prefill_run(llm, PROMPT_LEN, reps=1, warmup=0)
                    r["prefill_2048"]["own_kernels_ms"] = {k: round(v[1], 4) for k, v in sorted(kernels.kernel_timer_report().items())}
                    r["decode_batch8"]["own_kernels_ms"] = decode_kernel_times(llm, 8, 8, PROMPT_LEN)
                    kernels.enable_kernel_timers(False)
                del llm
                torch.cuda.empty_cache()
            if True:
                for key, T in (("prefill_2048", PROMPT_LEN), ("decode_batch8", 8)):
                    ms, by = r[key]["own_kernels_ms"], bytes_of[name](cfg, T)
                    r[key]["own_kernels_frac_of_copy"] = {k: round(by[k] / (ms[k] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                                                          for k in by if ms.get(k)}
                if name == "tofilorn" and r["prefill_2048"]["own_kernels_ms"].get("hgrn2_scan"):
                    # the matrix-state scan is arithmetic, not traffic: float instructions a lane must issue (two walks of a
                    # cut portion: multiply + multiply-add, then multiply + two multiply-adds, per state element and token)
                    # against the device's float issue rate (SMs x 128 lanes x clock)
                    rate = float_issue_rate()
                    work = sum(PROMPT_LEN * l["mixer"]["heads"] * l["mixer"]["dim"] * l["mixer"]["vdim"] * 5
                               for l in cfg["layers"] if l["type"] == "hgrn2")
                    if rate:
                        r["prefill_2048"]["hgrn2_scan_frac_of_float_issue_rate"] = round(
                            work / (r["prefill_2048"]["own_kernels_ms"]["hgrn2_scan"] * 1e-3) / rate, 4)
                if design == "rakizen":
                    # attention over a prompt is arithmetic: the products of the keys a query sees against the measured
                    # bfloat16 product of the library, whichever of the attention kernels ran
                    own = r["prefill_2048"]["own_kernels_ms"]
                    ms = sum(v for k, v in own.items() if "attention" in k)
                    if ms:
                        r["prefill_2048"]["attention_ms"] = round(ms, 4)
                        r["prefill_2048"]["attention_frac_of_bf16_peak"] = round(
                            attention_flops(cfg, PROMPT_LEN) / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
                    ms = sum(v for k, v in r["decode_batch8"]["own_kernels_ms"].items() if "attention" in k)
                    if ms:
                        # a decode step reads the keys and values its queries see, once
                        by = attention_decode_bytes(cfg, 8, PROMPT_LEN)
                        r["decode_batch8"]["attention_ms"] = round(ms, 4)
                        r["decode_batch8"]["attention_frac_of_copy"] = round(by / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                if name == "depolix":
                    # the windowed attention with kept first keys and a bias by distance, against the measured bfloat16
                    # product: every query over the keys it sees (the kernels of the latent layers are counted apart)
                    own = r["prefill_2048"]["own_kernels_ms"]
                    le = [l["mixer"]["left"] for l in cfg["layers"] if l["type"] == "parallel"]
                    seen = sum(min(i, le[0]["mask"]["size"] - 1) + 1 + max(0, min(le[0]["mask"]["keep_first"], i - le[0]["mask"]["size"] + 1))
                               for i in range(PROMPT_LEN)) if le else 0
                    flops = sum(2 * seen * m["heads"] * (m["dim"] + m["vdim"]) for m in le)
                    if own.get("attention_prefill_window_bias") and flops:
                        r["prefill_2048"]["window_attention_ms"] = own["attention_prefill_window_bias"]
                        r["prefill_2048"]["window_attention_frac_of_bf16_peak"] = round(
                            flops / (own["attention_prefill_window_bias"] * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
                    lat = [l["mixer"] for l in cfg["layers"] if l["type"] == "latent_attention"]
                    ms = sum(v for k, v in own.items() if k in ("attention_prefill_tma", "attention_prefill_tc5"))
                    if lat and ms:
                        row = lambda m: (m["kv_rank"] + m["rot_dim"] + 15) // 16 * 16
                        flops = sum(2 * (PROMPT_LEN * (PROMPT_LEN + 1) // 2) * m["heads"] * 2 * row(m) for m in lat)
                        r["prefill_2048"]["latent_attention_ms"] = round(ms, 4)
                        r["prefill_2048"]["latent_attention_frac_of_bf16_peak"] = round(flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
                if name in ("kesozen", "rakizen", "depolix"):
                    own = r["prefill_2048"]["own_kernels_ms"]
                    if own.get("delta_scan"):
                        # the delta rule is arithmetic too: a multiply and three multiply-adds per state element and token
                        rate = float_issue_rate()
                        work = sum(PROMPT_LEN * l["mixer"]["heads"] * l["mixer"]["dim"] * l["mixer"]["vdim"] * 4
                                   for l in cfg["layers"] if l["type"] == "delta")
                        work += sum(PROMPT_LEN * l["mixer"]["right"]["heads"] * l["mixer"]["right"]["dim"] * l["mixer"]["right"]["vdim"] * 4
                                    for l in cfg["layers"] if l["type"] == "parallel")
                        if rate:
                            r["prefill_2048"]["delta_scan_frac_of_float_issue_rate"] = round(work / (own["delta_scan"] * 1e-3) / rate, 4)
                    if own.get("moe_gemm_tc5"):
                        # the experts' products against the measured bfloat16 product of the library
                        # (two products an expert; three where it is gated)
                        flops = sum((6 if name in ("rakizen", "depolix") else 4) * PROMPT_LEN * l["mlp"]["router"]["top"] * cfg["width"] * l["mlp"]["expert"]["ff"]
                                    for l in cfg["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe")
                        r["prefill_2048"]["moe_gemm_tc5_frac_of_bf16_peak"] = round(flops / (own["moe_gemm_tc5"] * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
            rec[name] = r
        out["sizes"][str(width)] = rec
    out["value"] = out["sizes"][str(widths[0])][design]["decode_batch8"]["tokens_per_s"]
    out["config"] = {"layers": layers, "widths": list(widths), "prompt": PROMPT_LEN, "block_size": BLOCK,
                     "l2": "weights of a step exceed L2 at every size"}
    return out


def tofilorn_run(widths, pk=None, layers: int = 16) -> dict:
    return design_run("tofilorn", widths, pk, layers)


def attention_kernels_run(pk) -> dict:
    """The attention kernels alone.  Prefill: Qwen3-8B head shapes, one prompt of 2,048 and of 8,192 tokens, the device
    time of a launch (CUDA events around a graph of 20 launches, so the host's share of a launch is not in it).
    Decode: hundreds of requests with one key split each, 50 launches in a row (caches larger than L2)."""
    import math
    import torch
    from vllm_oxide_b200 import kernels
    dev = "cuda:0"
    nh, kvh, hd = QWEN3_8B["num_attention_heads"], QWEN3_8B["num_key_value_heads"], QWEN3_8B["head_dim"]
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    out = {"only": "attention", "heads": nh, "kv_heads": kvh, "head_dim": hd, "block_size": BLOCK, "launches_per_graph": 20}
    for T in (2048, 8192):
        pages = (T + BLOCK - 1) // BLOCK
        kc = torch.randn(pages, kvh, BLOCK, hd, device=dev).bfloat16()
        vc = torch.randn(pages, kvh, BLOCK, hd, device=dev).bfloat16()
        bt = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
        q = torch.randn(T, nh * hd, device=dev).bfloat16()
        o = torch.empty_like(q)
        cu_q = torch.tensor([0, T], dtype=torch.int32, device=dev)
        ctx = torch.tensor([T], dtype=torch.int32, device=dev)

        def launch():
            kernels.attention_prefill(q, nh * hd, o, kc, vc, bt, cu_q, ctx, 1, T, nh, kvh, hd, 0, 1 / math.sqrt(hd), err)
        for _ in range(3):
            launch()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(20):
                launch()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / 20)
        ms = sorted(times)[len(times) // 2]
        flops = 4 * nh * hd * T * (T + 1) / 2
        tf = flops / ms / 1e9
        out[f"prefill_{T}"] = {"us": round(ms * 1e3, 1), "tflops": round(tf, 1), "frac": round(tf / pk["bf16_tflops"], 3)}
        assert err.item() == 0
        del kc, vc, q, o
    # Decode attention of many requests with one key split each (the serving workload's shape: 16 heads over 8 kv heads,
    # contexts of 300 to 1,000 keys): persistent blocks against one block per (request, kv head).
    nh, g = 16, torch.Generator().manual_seed(1)
    for name, B, lo, hi in (("decode_228x650", 228, 650, 650), ("decode_228x300_1000", 228, 300, 1000), ("decode_512x100_400", 512, 100, 400)):
        ctx_host = torch.randint(lo, hi + 1, (B,), generator=g).int()
        per = (hi + BLOCK - 1) // BLOCK
        kc = torch.randn(B * per, kvh, BLOCK, hd, device=dev).bfloat16()
        vc = torch.randn(B * per, kvh, BLOCK, hd, device=dev).bfloat16()
        bt = torch.randperm(B * per, generator=g).int().view(B, per).to(dev)
        q = torch.randn(B, nh * hd, device=dev).bfloat16()
        o = torch.empty_like(q)
        cu_q = torch.arange(B + 1, dtype=torch.int32, device=dev)
        ctx = ctx_host.to(dev)
        nbytes = float(ctx_host.sum()) * kvh * hd * 2 * 2
        row = {}
        for mode, pairs in (("persistent", kernels.decode_pairs_counter(dev)), ("block_per_pair", None)):

            def launch():
                kernels.attention_decode(q, nh * hd, o, kc, vc, bt, cu_q, ctx, B, nh, kvh, hd, 0, 1 / math.sqrt(hd), 1, None, err,
                                         pairs=pairs)
            for _ in range(5):
                launch()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(50):
                launch()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 50 * 1e3
            row[mode] = {"us": round(us, 1), "gbs": round(nbytes / us / 1e3), "frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
        out[name] = row
        assert err.item() == 0
        del kc, vc
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (reported)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + sorted(DESIGNS), default=None,
                    help="another workload instead of the default run")
    ap.add_argument("--sizes", default="2048,4096", help="--workload tofilorn | kesozen | rakizen | depolix: the widths to measure")
    ap.add_argument("--only", choices=["decode", "prefill", "attention"], default=None,
                    help="run one phase and print its time only (for short profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust crate on candle: no Rust toolchain or "
                          "network here, and pip finds neither setup.py nor pyproject.toml in it"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    if args.workload in DESIGNS:
        print(json.dumps(design_run(args.workload, [int(w) for w in args.sizes.split(",")])))
        return 0
    if args.workload:
        print(json.dumps(workload_run(args.workload)))
        return 0
    if args.only == "attention":
        print(json.dumps(attention_kernels_run(peaks())))
        return 0
    import torch
    from vllm_oxide_b200 import LLM, EngineOptions

    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    cfg = dict(QWEN3_8B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    n = model_numbers(cfg)
    max_batch = 64 if not args.skip_points else args.batch
    pages_per_req = (PROMPT_LEN + NEW_TOKENS + BLOCK - 1) // BLOCK + 1
    opts = EngineOptions(max_model_len=CONTEXT, block_size=BLOCK, num_kv_blocks=max_batch * pages_per_req + 16,
                         max_num_seqs=max(max_batch, 8), max_num_batched_tokens=8192, dtype="bfloat16")
    llm = LLM.from_config(cfg, opts, seed=0, init_scheme="0.02")

    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "ms": prefill_run(llm, PROMPT_LEN, reps=1, warmup=1)}))
        return 0
    if args.only == "decode":
        ms, launches, _ = decode_run(llm, args.batch, steps, warmup, PROMPT_LEN)
        print(json.dumps({"only": "decode", "ms_per_step": ms, "gpu_launches": launches}))
        return 0
    prefill_ms = prefill_run(llm, PROMPT_LEN)
    with ClockSampler() as clocks:
        ms, launches, mean_ctx = decode_run(llm, args.batch, steps, warmup, PROMPT_LEN)
    value = args.batch * 1000.0 / ms

    def hbm_frac(batch, ctx, step_ms):
        return (n["weight_bytes"] + batch * ctx * n["kv_bytes_per_token"]) / (step_ms * 1e-3) / 1e9 / pk["hbm_gbs"]
    achieved = hbm_frac(args.batch, mean_ctx, ms) * pk["hbm_gbs"]
    e2e, h2d, d2h, e2e_ms = e2e_run(llm, args.batch, steps, warmup)
    points, workloads = {}, {}
    if not args.skip_points:
        short = min(steps, 32)
        points[f"host_ms_b{args.batch}"] = round(e2e_ms - ms, 4)
        for b in (1, 16, 32, 64):
            pms, _, ctx = decode_run(llm, b, short, warmup, PROMPT_LEN)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
            points[f"frac_b{b}"] = round(hbm_frac(b, ctx, pms), 4)
            if b in (1, 64):
                rate, _, _, step_ms = e2e_run(llm, b, short, warmup)
                points[f"e2e_b{b}"] = round(rate, 1)
                points[f"host_ms_b{b}"] = round(step_ms - pms, 4)
        # longer contexts: another engine over the same model (its decode steps are shaped for up to 32,768 keys)
        config, model = llm.config, llm.model
        del llm
        torch.cuda.empty_cache()
        long_ctx = 32768
        pages = 8 * (long_ctx // BLOCK + 2) + 8
        opts = EngineOptions(max_model_len=long_ctx + 2 * BLOCK, block_size=BLOCK, num_kv_blocks=pages, max_num_seqs=8,
                             max_num_batched_tokens=8192, dtype="bfloat16")
        llm = LLM("<random weights>", opts, _model=(config, model))
        # a longer prompt in one step (attention is a larger share of it)
        p_ms = prefill_run(llm, 8192, reps=2, warmup=1)
        points["prefill_8192"] = round(8192 * 1000.0 / p_ms, 1)
        points["frac_prefill_8192"] = round(prefill_flops(cfg, 8192) / (p_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
        for ctx0 in (8192, long_ctx):
            for b in (1, 8):
                pms, _, ctx = decode_run(llm, b, 16, warmup, ctx0)
                points[f"decode_b{b}_ctx{ctx0}"] = round(b * 1000.0 / pms, 1)
                points[f"frac_b{b}_ctx{ctx0}"] = round(hbm_frac(b, ctx, pms), 4)
        del llm, model
        torch.cuda.empty_cache()
        w = workload_run("serving-0.6b", pk)
        workloads["serving_0_6b"] = {k: w[k] for k in ("value", "generated_tokens_per_s", "seconds", "steps",
                                                       "mean_requests_per_step", "bytes_per_step_gb", "roofline")}
    flops = prefill_flops(cfg, PROMPT_LEN)
    line = {
        "metric": "decode tok/s (Qwen3-8B sizes, bf16, batch 8, context 2048+)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, seeded random weights",
        "impl": "ours",
        "config": {"model": "Qwen3-8B sizes", "layers": cfg["num_hidden_layers"], "layers_of_config": 36,
                   "hidden": 4096, "heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 12288, "vocab": 151936,
                   "global_batch": args.batch, "seq_len": PROMPT_LEN, "new_tokens": NEW_TOKENS, "context": CONTEXT,
                   "block_size": BLOCK, "parallelism": "single GPU", "l2": "every step reads 15 GB of weights (inputs larger than L2)",
                   "peaks": pk["source"]},
        "clocks": clocks.result,
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(PROMPT_LEN * 1000.0 / prefill_ms, 1), "tokens": PROMPT_LEN, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "workloads": workloads,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Dabevik, or Rasezen, beside the closest other model of the library (the Qwen3 dense decoder) at equal
sizes: prompt and decode throughput of a few layers of real-model size with random weights, and
what each class of kernels takes of a step. `python bench.py --design dabevik` prints the result
as one JSON line.

Equal sizes: the same width, layers, vocabulary, heads, kv heads, head size, feed-forward width
and window (every layer of the Qwen3 twin slides the same window). What differs is the design:
two feed-forward matrices instead of three, biased projections, norms on both sides of a
sublayer, the convolutions of the sublayers' inputs, learned positions instead of rotation, kept
first tokens, and the mix of the heads' weights.

Rasezen (`--design rasezen`, RASEZEN_SIZES): the same width, layers, vocabulary, attention heads,
kv heads, head size, window and dense feed-forward width; what differs is the design: parallel
blocks with one norm a layer, norms over whole projections, a value norm, some layers whose
mixer is a state-space recurrence instead of attention, and feed-forwards that are mixtures of
small experts (their chosen experts and the shared one together about a dense one's size).

Lebelix (`--design lebelix`, LEBELIX_SIZES): the same width, layers, vocabulary, attention heads, kv
heads, head size, dense feed-forward width, and a window on every layer of the twin as long as
Lebelix's chunks and windows; what differs is the design: attention with capped scores, chunks, a
sink and an output gate, layers of latent attention (one of them reading an earlier layer's latent
cache), layers whose mixer is the gated delta rule, a two-matrix GELU feed-forward, and the
per-layer token input.

Vekolix (`--design vekolix`, VEKOLIX_SIZES): the same width, layers, vocabulary, attention heads, kv
heads, head size and dense feed-forward width, no window on either side; what differs is the design:
Dynamic Tanh in place of the norms, a multiplier on every update, layers whose mixer is softmax
attention and linear attention side by side, layers of latent attention with a query latent and a gate
a head, a two-matrix squared-ReLU feed-forward, mixtures of clamped gated experts weighted on their
input with a gated shared expert, and capped logits.
"""
from __future__ import annotations

import statistics
import time

SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, window=1024, keep_first=4, layers=8,
               vocab=32768, taps=4),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, window=2048, keep_first=4, layers=4,
               vocab=32768, taps=4),
}
# Rasezen: layers as (mixer, feed-forward) pairs, "a" attention, "s" state-space; "d" dense, "e" experts
RASEZEN_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, window=1024, vocab=32768,
               ssm=dict(heads=64, vdim=64, state=128, groups=8, conv=4, norm_groups=8),
               moe=dict(ff=1024, experts=16, identity=2, top=4, scale=2.0, shared=2048),
               pattern=["ad", "se", "ae", "ae", "se", "ae", "ad", "se"]),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, window=2048, vocab=32768,
               ssm=dict(heads=128, vdim=64, state=128, groups=8, conv=4, norm_groups=8),
               moe=dict(ff=1536, experts=16, identity=2, top=4, scale=2.0, shared=3072),
               pattern=["ad", "se", "ae", "se"]),
}
# Lebelix: a layer's mixer, "a" attention, "l" latent attention, "L" latent attention that reads the
# first "l" layer's cache, "c" the gated delta rule; every layer has the dense feed-forward
LEBELIX_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, window=1024, vocab=32768, rot=64, softcap=50.0,
               latent=dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512),
               delta=dict(heads=16, kv_heads=8, dim=128, vdim=128, conv=4, decay_rank=64, gate_rank=64),
               side=256, pattern=["l", "a", "a", "c", "L", "a", "c", "a"]),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, window=2048, vocab=32768, rot=64, softcap=50.0,
               latent=dict(heads=32, dim=128, rot_dim=64, vdim=128, kv_rank=512),
               delta=dict(heads=32, kv_heads=16, dim=128, vdim=128, conv=4, decay_rank=128, gate_rank=128),
               side=256, pattern=["l", "a", "c", "L"]),
}
# Vekolix: layers as (mixer, feed-forward) pairs, "p" two mixers side by side, "l" latent attention; "d" dense, "e" experts
VEKOLIX_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, window=0, vocab=32768, rot=64,
               linear=dict(heads=16, dim=128, vdim=128),
               latent=dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=768),
               moe=dict(ff=1024, experts=16, top=4, limit=7.0, shared=2048, shared_limit=7.0),
               pattern=["ld", "pe", "pd", "le", "pd", "pe", "ld", "pe"]),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, window=0, vocab=32768, rot=64,
               linear=dict(heads=32, dim=128, vdim=128),
               latent=dict(heads=32, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=1536),
               moe=dict(ff=1536, experts=16, top=4, limit=7.0, shared=3072, shared_limit=7.0),
               pattern=["ld", "pe", "pd", "le"]),
}
CONTEXT = 4096
PROMPT_TOKENS = 2048
DECODE_PROMPTS = (1024, 2048)


def dabevik_config(s):
    mixer = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
             "scale": s["dim"] ** -0.5, "mask": {"size": s["window"], "keep_first": s["keep_first"]}}
    return {"architecture": "Dabevik", "vocab": s["vocab"], "width": s["width"], "max_positions": CONTEXT,
            "embedding": {"scale": s["width"] ** 0.5}, "norm": {"eps": 1e-6}, "canon": {"taps": s["taps"]},
            "layers": [{"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": s["ff"]}}
                       for _ in range(s["layers"])]}


def rasezen_config(s):
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
            "scale": s["dim"] ** -0.5, "mask": {"size": s["window"]}, "rot": {"base": 1000000.0, "dims": s["dim"]}}
    m = s["moe"]
    experts = {"kind": "moe", "expert": {"ff": m["ff"]}, "shared": {"ff": m["shared"]},
               "router": {"experts": m["experts"], "identity": m["identity"], "scale": m["scale"], "top": m["top"]}}
    layers = [{"type": "attention" if p[0] == "a" else "mamba2", "mixer": attn if p[0] == "a" else dict(s["ssm"]),
               "mlp": {"kind": "dense", "ff": s["ff"]} if p[1] == "d" else experts} for p in s["pattern"]]
    return {"architecture": "Rasezen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "max_positions": CONTEXT, "layers": layers}


def lebelix_config(s):
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
            "scale": s["dim"] ** -0.5, "mask": {"size": s["window"]}, "softcap": s["softcap"],
            "rot": {"base": 500000.0, "dims": s["rot"]}}
    lat = dict(s["latent"], scale=(s["latent"]["dim"] + s["latent"]["rot_dim"]) ** -0.5, mask={"size": s["window"]},
               rot={"base": 1000000.0, "dims": s["latent"]["rot_dim"]})
    first = s["pattern"].index("l") if "L" in s["pattern"] else None
    mixers = {"a": ("attention", attn), "l": ("latent_attention", lat),
              "L": ("latent_attention", dict(lat, kv_from=first)), "c": ("channel_delta", dict(s["delta"]))}
    return {"architecture": "Lebelix", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": s["width"] ** 0.5}, "token_side": {"dim": s["side"]}, "max_positions": CONTEXT,
            "layers": [{"type": mixers[p][0], "mixer": mixers[p][1], "mlp": {"kind": "dense", "ff": s["ff"]}}
                       for p in s["pattern"]]}


def vekolix_config(s):
    left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
            "rot": {"base": 1000000.0, "dims": s["rot"],
                    "scaling": {"factor": 4.0, "original": 2048, "fast": 16.0, "slow": 2.0}}}
    n = s["linear"]["heads"]
    right = dict(s["linear"], decay=[1.0 - 2.0 ** (-2.0 - 8.0 * h / max(n - 1, 1)) for h in range(n)])
    side = {"left": left, "right": right, "left_scale": 0.7, "right_scale": 0.9}
    lat = dict(s["latent"], scale=(s["latent"]["dim"] + s["latent"]["rot_dim"]) ** -0.5,
               rot={"base": 1000000.0, "dims": s["latent"]["rot_dim"]})
    m = s["moe"]
    experts = {"kind": "moe", "expert": {"ff": m["ff"], "limit": m["limit"]},
               "router": {"experts": m["experts"], "top": m["top"]},
               "shared": {"ff": m["shared"], "limit": m["shared_limit"]}}
    layers = [{"type": "parallel" if p[0] == "p" else "latent_attention", "mixer": side if p[0] == "p" else lat,
               "mlp": {"kind": "dense", "ff": s["ff"]} if p[1] == "d" else experts} for p in s["pattern"]]
    return {"architecture": "Vekolix", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "residual_mult": 0.8, "logit_scale": 0.5, "logit_softcap": 40.0, "max_positions": CONTEXT, "layers": layers}


def qwen3_config(s):
    n_layers = s["layers"] if "layers" in s else len(s["pattern"])
    return dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=s["width"],
                num_hidden_layers=n_layers, num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"],
                head_dim=s["dim"], intermediate_size=s["ff"], vocab_size=s["vocab"], rope_theta=1000000.0,
                rms_norm_eps=1e-6, max_position_embeddings=CONTEXT, tie_word_embeddings=True,
                **({"sliding_window": s["window"], "layer_types": ["sliding_attention"] * n_layers} if s["window"] else {}))


# kernel entry point -> class of kernels, for both designs
CLASSES = {
    "lumen_add_rmsnorm": "norm", "lumen_postnorm_add_rmsnorm": "norm", "lumen_canon_conv": "input conv",
    "lumen_qk_norm_rope_store": "q/k norm + cache write", "lumen_qkv_bias_norm_store": "q/k norm + cache write",
    "lumen_rope_table": "q/k norm + cache write", "lumen_silu_mul": "activation", "lumen_polynorm": "activation",
    "lumen_embed": "embedding", "lumen_embed_tiled": "embedding", "lumen_embed_pos": "embedding",
    "lumen_attn_decode": "attention", "lumen_attn_decode_qkv": "attention", "lumen_attn_prefill_tc": "attention",
    "lumen_attn_prefill": "attention", "lumen_attn_generic": "attention", "lumen_attn_talk": "attention",
    "lumen_attn_talk_prompt": "attention", "lumen_argmax": "sampling", "lumen_sample": "sampling",
    "lumen_gemm_tc_qkv": "qkv product + q/k norm + cache write",
    "lumen_conv_silu": "recurrence: convolution", "lumen_ssm_scan": "state-space: recurrence",
    "lumen_gated_part_norm": "state-space: gate + norm", "lumen_xielu": "activation",
    "lumen_moe_route": "experts: route + group", "lumen_moe_route_x": "experts: route + group",
    "lumen_moe_group": "experts: route + group",
    "lumen_qkv_head_norm_store": "q/k norm + cache write", "lumen_attn_generic_opt": "attention (general kernel)",
    "lumen_attn_prefill_tc_opt": "attention", "lumen_attn_decode_opt": "attention",
    "lumen_attn_latent": "attention (latent kernel)",
    "lumen_latent_store": "latent: norm + cache write", "lumen_latent_query": "latent: queries into the latent space",
    "lumen_head_product": "latent: values out of the latent space", "lumen_head_gemm": "latent: products of every head", "lumen_gelu_tanh": "activation",
    "lumen_token_gate": "token input", "lumen_add_cast": "token input", "lumen_cols_cast": "delta rule: low-rank inputs",
    "lumen_delta_rule": "delta rule: recurrence", "lumen_head_norm_gate": "recurrence: norm + gate",
    "lumen_add_scaled_dyt": "norm", "lumen_relu2": "activation", "lumen_clamped_glu": "activation",
    "lumen_cols_rmsnorm": "norm of some columns (+ gate)", "lumen_scale_softcap": "logits: scale + cap",
    "lumen_linear_attn": "linear attention: recurrence",
}


def _class_times(run):
    """Microseconds per class of kernels for one call of `run`, every launch bracketed by events."""
    import torch
    from .ops import native
    rec = []

    def probe(name, args):
        label = CLASSES.get(name)
        if label is None and name == "lumen_gemm_tc":
            label = f"product {int(args[4])}x{int(args[5])}"
        if label is None and name == "lumen_moe_product":
            label = "experts: gate/up product" if int(args[14]) else "experts: down product"
        rec.append([label or name, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)])
        return rec[-1]
    native.instrument(probe)
    try:
        run()
        torch.cuda.synchronize()
    finally:
        native.instrument(None)
    by = {}
    for label, e0, e1 in rec:
        by[label] = by.get(label, 0.0) + e0.elapsed_time(e1) * 1e3
    return {k: round(v, 1) for k, v in sorted(by.items(), key=lambda kv: -kv[1])}, len(rec)


def measure(config, batch, steps, warmup, seed=0):
    """Prompt tokens/s (one prompt of PROMPT_TOKENS tokens), decode tokens/s at `batch` (captured
    steps, tokens fed back on the device) and the classes' times of one step of each kind."""
    import torch
    from .engine import Engine, StepEntry
    from .sampling import SamplingConfig
    t_begin = time.perf_counter()
    eng = Engine.from_random(config, seed=seed, std=0.02, dtype="bfloat16",
                             max_tokens=batch * CONTEXT, max_slots=max(batch, 8), context_size=CONTEXT)
    eng.graphs.min_width = CONTEXT // 64
    g = torch.Generator().manual_seed(seed + 1)
    prompt = torch.randint(0, eng.vocab_size, (PROMPT_TOKENS,), generator=g).tolist()
    times = []
    for it in range(3 + 5):
        s = eng.alloc_slot()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([StepEntry(s, prompt, [PROMPT_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        eng.free_slot(s)
        if it >= 3:
            times.append(e0.elapsed_time(e1))
    prompt_ms = statistics.median(times)
    s = eng.alloc_slot()
    prompt_classes, prompt_launches = _class_times(lambda: eng.step([StepEntry(s, prompt, [PROMPT_TOKENS - 1])]))
    eng.free_slot(s)

    lens = torch.randint(DECODE_PROMPTS[0], DECODE_PROMPTS[1] + 1, (batch,), generator=g).tolist()
    slots = [eng.alloc_slot() for _ in range(batch)]
    logits = eng.step([StepEntry(sl, torch.randint(0, eng.vocab_size, (n,), generator=g).tolist(), [n - 1])
                       for sl, n in zip(slots, lens)])
    cfgs, us = [SamplingConfig()] * batch, [0.0] * batch
    tok = eng.sampler.pick(logits, cfgs, us)
    entries = [(sl, [0]) for sl in slots]
    for _ in range(warmup):
        tok = eng.run_device(entries, cfgs, us, tokens_on_device=tok)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        tok = eng.run_device(entries, cfgs, us, tokens_on_device=tok)
    e1.record()
    torch.cuda.synchronize()
    window = (t_begin, time.perf_counter())       # the clocks' samples of the whole measurement
    eng.check_kernels()
    decode_ms = e0.elapsed_time(e1) / steps
    per_replay = getattr(getattr(eng.graphs, "last", None), "kernels_per_replay", 0)
    was = eng.use_graphs
    eng.use_graphs = False
    try:
        for _ in range(2):
            eng.run_device([(sl, [1]) for sl in slots], cfgs, us)
        decode_classes, _ = _class_times(lambda: eng.run_device([(sl, [1]) for sl in slots], cfgs, us))
    finally:
        eng.use_graphs = was
    for sl in slots:
        eng.free_slot(sl)
    return {"prompt_tokens_per_s": round(PROMPT_TOKENS / (prompt_ms * 1e-3), 1), "prompt_ms": round(prompt_ms, 3),
            "decode_tokens_per_s": round(batch * 1000.0 / decode_ms, 1), "decode_ms_per_step": round(decode_ms, 4),
            "decode_kernels_per_step": per_replay, "prompt_kernels": prompt_launches,
            "prompt_us_by_class": prompt_classes, "decode_us_by_class": decode_classes, "window": window}


DESIGNS = {"dabevik": (SIZES, dabevik_config), "rasezen": (RASEZEN_SIZES, rasezen_config),
           "lebelix": (LEBELIX_SIZES, lebelix_config), "vekolix": (VEKOLIX_SIZES, vekolix_config)}


def sizes_of(design):
    if design not in DESIGNS:
        raise ValueError(f"no comparison is written for design {design!r}")
    return DESIGNS[design][0]


def run(design, sizes, batch, steps, warmup):
    table, make = DESIGNS[design] if design in DESIGNS else (sizes_of(design), None)
    import gc
    import torch
    out = {}
    for name in sizes:
        s = table[name]
        row = {"sizes": s}
        for label, cfg in ((design, make(s)), ("qwen3", qwen3_config(s))):
            row[label] = measure(cfg, batch, steps, warmup)
            gc.collect()
            torch.cuda.empty_cache()
        out[name] = row
    return out


def steps_main(argv=None) -> int:
    """`python -m lumenllm_b200.compare --design dabevik|qwen3 --kind prompt|decode [--size 2k]
    [--layers 2] [--batch 8]`: a few steps of one kind launched kernel by kernel, for a profiler's
    launch list (nothing is timed here)."""
    import argparse
    import torch
    from .engine import Engine, StepEntry
    from .sampling import SamplingConfig
    ap = argparse.ArgumentParser(prog="lumenllm_b200.compare")
    ap.add_argument("--design", default="dabevik", choices=sorted(DESIGNS) + ["qwen3"])
    ap.add_argument("--sizes-of", default=None, choices=sorted(DESIGNS),
                    help="with --design qwen3: whose table of sizes the twin takes (default dabevik)")
    ap.add_argument("--kind", default="decode", choices=["prompt", "decode"])
    ap.add_argument("--size", default="2k", choices=sorted(SIZES))
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--batch", type=int, default=8)
    a = ap.parse_args(argv)
    table, make = DESIGNS[a.design if a.design in DESIGNS else (a.sizes_of or "dabevik")]
    s = dict(table[a.size])
    if "pattern" in s:
        s["pattern"] = s["pattern"][:a.layers]
    else:
        s["layers"] = a.layers
    cfg = make(s) if a.design in DESIGNS else qwen3_config(s)
    eng = Engine.from_random(cfg, seed=0, std=0.02, dtype="bfloat16", max_tokens=a.batch * CONTEXT,
                             max_slots=max(a.batch, 8), context_size=CONTEXT, use_graphs=False)
    g = torch.Generator().manual_seed(1)
    rand = lambda n: torch.randint(0, eng.vocab_size, (n,), generator=g).tolist()
    if a.kind == "prompt":
        for _ in range(2):
            slot = eng.alloc_slot()
            eng.step([StepEntry(slot, rand(PROMPT_TOKENS), [PROMPT_TOKENS - 1])])
            eng.free_slot(slot)
    else:
        slots = [eng.alloc_slot() for _ in range(a.batch)]
        eng.step([StepEntry(sl, rand(1500), []) for sl in slots])
        for _ in range(3):
            eng.run_device([(sl, [1]) for sl in slots], [SamplingConfig()] * a.batch, [0.0] * a.batch)
    torch.cuda.synchronize()
    eng.check_kernels()
    print("ok")
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(steps_main())

"""Small Lebelix configurations and seeded weights for the tests. The sizes differ from one another
in everything that can differ: heads against kv heads (ratio 1, 2, 3, 4), key size against value
size, rotation over a part of a head, over all of it and none, chunks and windows shorter and longer
than a cache page (64), capped and uncapped scores; latent attention with rotation over part of the
rotated values, layers that read an earlier layer's latent cache through a narrower and a wider
window; delta-rule layers with one query/key head for several value heads, key sizes that one, two
and four threads hold, one to four taps, low ranks of 1 to 12; layers without feed-forward; models
with and without the per-layer token input.
"""
import json
from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, scale, size=None, rot=None, base=10000.0, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
    if softcap is not None:
        m["softcap"] = softcap
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, size=None, rot=None, base=10000.0, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def delta(heads, kv_heads, dim, vdim, conv, decay_rank=4, gate_rank=4):
    """The two ranks are not keys of the design's config.json (tensor shapes give them); they ride
    along here for make_weights and are dropped by write_model."""
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
            "decay_rank": decay_rank, "gate_rank": gate_rank}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(mixer, mlp):
    kind = "latent_attention" if "kv_rank" in mixer else ("channel_delta" if "conv" in mixer else "attention")
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(vocab, width, eps, layers, scale=1.0, side=None):
    c = {"architecture": "Lebelix", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "embedding": {"scale": scale}, "layers": layers}
    if side is not None:
        c["token_side"] = {"dim": side}
    return c


SMALL = {
    # chunks shorter than a page, rotation over half a head, values wider than keys; a latent cache
    # read by a later layer through a wider window; a delta rule with one query/key head for two
    # value heads; a layer without feed-forward
    "X": config(97, 64, 1e-6, [
        layer(attention(4, 2, 16, 24, 0.3, size=9, rot=8, softcap=5.0), dense(80)),
        layer(latent(2, 8, 16, 24, 40, 0.2, size=11, rot=8), dense(48)),
        layer(delta(2, 1, 24, 16, 3, 5, 3), None),
        layer(latent(3, 16, 16, 8, 40, 0.25, size=70, rot=8, kv_from=1), dense(72)),
        layer(attention(3, 3, 32, 8, 0.25, size=70, rot=32, base=500.0, softcap=30.0), dense(40))],
        scale=0.7, side=8),
    # no token input, scale 1, uncapped scores, no rotation in one layer, no mask in one layer; one
    # tap (no convolution state); a latent layer alone; a feed-forward wider than the model
    "Y": config(160, 96, 1e-5, [
        layer(delta(3, 3, 8, 40, 1, 1, 12), dense(200)),
        layer(attention(6, 2, 32, 32, 0.11), dense(64)),
        layer(latent(4, 24, 8, 16, 64, 0.15, rot=8, base=1e6), None),
        layer(attention(3, 1, 16, 48, 0.2, size=150, rot=4, softcap=8.0), dense(100))]),
    # key and value sizes that the tensor-core attention kernels take (64, 128) with chunks of several
    # pages and of less than one; a key size spread over four threads of the recurrence; two layers
    # that read one latent cache, one through a narrower window
    "Z": config(211, 128, 3e-6, [
        layer(latent(2, 32, 32, 32, 96, 0.1, size=100, rot=32), dense(96)),
        layer(attention(4, 2, 64, 64, 0.12, size=150, rot=32, softcap=20.0), dense(160)),
        layer(latent(4, 16, 32, 64, 96, 0.12, size=33, rot=32, kv_from=0), dense(64)),
        layer(delta(4, 2, 64, 32, 4, 12, 8), dense(96)),
        layer(attention(2, 1, 128, 128, 0.09, size=33, rot=128, base=1e5, softcap=50.0), dense(160)),
        layer(latent(2, 32, 32, 16, 96, 0.1, size=130, rot=32, kv_from=0), None)],
        scale=1.5, side=16),
}


def make_weights(cfg, seed):
    """Seeded bfloat16 tensors by the design's names, of a size that keeps activations of order one."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *shape, std=1.0: torch.randn(shape, generator=g) * std
    D, t = cfg["width"], {}
    t["embed"] = rn(cfg["vocab"], D)
    t["final.norm"] = rn(D, std=0.1)
    side = cfg.get("token_side", {}).get("dim", 0)
    if side:
        t["side.embed"] = rn(cfg["vocab"], side * len(cfg["layers"]))
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        t[p + "norm1"] = rn(D, std=0.1)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                t[p + "mix." + name] = rn(rows, D, std=D ** -0.5)
                t[p + "mix." + name + ".b"] = rn(rows, std=0.2)
            t[p + "mix.q.norm"], t[p + "mix.k.norm"] = 1 + rn(d, std=0.1), 1 + rn(d, std=0.1)
            t[p + "mix.g"] = rn(H * dv, D, std=D ** -0.5)
            t[p + "mix.o"] = rn(D, H * dv, std=(H * dv) ** -0.5)
        elif L["type"] == "latent_attention":
            H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            t[p + "mix.q"] = rn(H * (d + r), D, std=D ** -0.5)
            if m.get("kv_from") is None:
                t[p + "mix.dkv"] = rn(R + r, D, std=D ** -0.5)
                t[p + "mix.dkv.norm"] = 1 + rn(R, std=0.1)
            t[p + "mix.uk"], t[p + "mix.uv"] = rn(H * d, R, std=R ** -0.5), rn(H * dv, R, std=R ** -0.5)
            t[p + "mix.o"] = rn(D, H * dv, std=(H * dv) ** -0.5)
        else:
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = m["decay_rank"], m["gate_rank"]
            for name, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                t[p + "mix." + name] = rn(rows, D, std=D ** -0.5)
                t[p + "mix." + name + ".conv"] = rn(rows, taps, std=0.6)
            t[p + "mix.b"] = rn(H, D, std=D ** -0.5)
            t[p + "mix.A_log"], t[p + "mix.dt_bias"] = rn(H, std=0.5) - 1.0, rn(H * d, std=0.5)
            t[p + "mix.a1"], t[p + "mix.a2"] = rn(ra, D, std=D ** -0.5), rn(H * d, ra, std=ra ** -0.5)
            t[p + "mix.g1"], t[p + "mix.g2"] = rn(rg, D, std=D ** -0.5), rn(H * dv, rg, std=rg ** -0.5)
            t[p + "mix.norm"] = 1 + rn(dv, std=0.1)
            t[p + "mix.o"] = rn(D, H * dv, std=(H * dv) ** -0.5)
        if L["mlp"] is not None:
            F = L["mlp"]["ff"]
            t[p + "norm2"] = rn(D, std=0.1)
            t[p + "mlp.up"], t[p + "mlp.down"] = rn(F, D, std=D ** -0.5), rn(D, F, std=F ** -0.5)
        if side:
            t[p + "side.gate"], t[p + "side.proj"] = rn(side, D, std=D ** -0.5), rn(D, side, std=side ** -0.5)
            t[p + "side.norm"] = 0.5 + rn(D, std=0.1)
    return {k: v.to(torch.bfloat16) for k, v in t.items()}


def stored_config(cfg):
    """config.json as the design writes it: without the delta rule's ranks (its tensors' shapes say)."""
    c = json.loads(json.dumps(cfg))
    for L in c["layers"]:
        L["mixer"].pop("decay_rank", None)
        L["mixer"].pop("gate_rank", None)
    return c


def write_model(cfg, folder, seed):
    from lumenllm_b200.weights.safetensors_io import write_file
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(stored_config(cfg)))
    write_file(folder / "model.safetensors", make_weights(cfg, seed))
    return folder

"""Small Vekolix configurations and seeded weights for the tests. The sizes differ from one another
in everything that can differ: heads against kv heads (ratio 1, 2, 3, 4), key size against value
size, rotation over a part of a head, over all of it and none, stretched frequencies and plain
ones; linear attention with one to five heads, key sizes that fill one thread's share and that do
not, values that do not fill a block's columns; latent attention with rotation over part of the
rotated values and over all of them, query latents narrower and wider than the key latent; dense
layers, experts with one to three choices, with and without a shared expert, layers without
feed-forward; widths that are multiples of 16, of 8, of 4 and of 2 only; multipliers that are 1 and
that are not.
"""
import json
from pathlib import Path

import torch


def softmax_side(heads, kv_heads, dim, vdim, scale, rot=None, base=10000.0, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def linear_side(heads, dim, vdim, decay):
    assert len(decay) == heads
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def parallel(left, right, left_scale=1.0, right_scale=1.0):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot=None, base=10000.0):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(mixer, mlp):
    return {"type": "latent_attention" if "kv_rank" in mixer else "parallel", "mixer": mixer, "mlp": mlp}


def config(vocab, width, eps, layers, mult=1.0, logit_scale=1.0, softcap=None):
    c = {"architecture": "Vekolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
         "logit_scale": logit_scale, "layers": layers}
    if softcap is not None:
        c["logit_softcap"] = softcap
    return c


SMALL = {
    # values wider than keys, rotation over half a head with stretched frequencies, kv ratio 2; two
    # choices among five experts with a shared one; a latent layer whose rotation covers half of the
    # rotated values; a layer without feed-forward
    "X": config(97, 64, 1e-6, [
        layer(parallel(softmax_side(4, 2, 16, 24, 0.3, rot=8, base=5000.0, scaling=(4.0, 64, 8.0, 1.0)),
                       linear_side(2, 16, 24, (0.7, 0.98)), 0.8, 1.3), moe(5, 2, 24, 1.5, shared=(40, 0.8))),
        layer(latent(2, 8, 16, 24, 40, 24, 0.2, rot=8), dense(80)),
        layer(parallel(softmax_side(3, 3, 32, 8, 0.25, rot=32, base=500.0), linear_side(3, 8, 40, (0.5, 0.9, 0.999)),
                       1.2, 0.5), None),
        layer(latent(3, 16, 16, 8, 40, 56, 0.25, rot=16, base=3e5), moe(3, 1, 16, 0.7))],
        mult=0.6, logit_scale=0.5, softcap=12.0),
    # multipliers of 1, no cap on the logits, no rotation in the softmax side of one layer, plain
    # frequencies in the other; three choices among seven experts without a shared one; one linear
    # head; a feed-forward wider than the model
    "Y": config(160, 96, 1e-5, [
        layer(latent(4, 24, 8, 16, 64, 32, 0.15, rot=8, base=1e6), moe(7, 3, 40, 2.5)),
        layer(parallel(softmax_side(6, 2, 32, 32, 0.11), linear_side(1, 40, 24, (0.95,))), dense(200)),
        layer(parallel(softmax_side(3, 1, 16, 48, 0.2, rot=4), linear_side(5, 24, 16, (0.3, 0.8, 0.9, 0.99, 1.0)),
                       1.0, 2.0), moe(4, 4, 8, 1.0, shared=(8, 3.0)))]),
    # key and value sizes that the tensor-core attention kernels take (64, 128), latents that the
    # tensor-core latent kernel takes, linear keys of 64 and 128, a key size of 72 that leaves a part's
    # share part empty
    "Z": config(211, 128, 3e-6, [
        layer(parallel(softmax_side(4, 2, 64, 64, 0.12, rot=32, base=2e5, scaling=(16.0, 128, 16.0, 2.0)),
                       linear_side(2, 64, 64, (0.9, 0.995)), 0.5, 0.9), dense(160)),
        layer(latent(4, 32, 32, 32, 96, 64, 0.1, rot=32), moe(6, 2, 32, 1.2, shared=(64, 1.8))),
        layer(parallel(softmax_side(2, 1, 128, 128, 0.09, rot=128, base=1e5), linear_side(2, 128, 32, (0.97, 0.6)),
                       1.5, 0.7), dense(96)),
        layer(parallel(softmax_side(8, 2, 64, 64, 0.1, rot=16), linear_side(1, 72, 96, (0.99,)), 0.7, 1.1),
              moe(9, 1, 48, 0.9)),
        layer(latent(2, 64, 16, 64, 128, 128, 0.1, rot=16), None)],
        mult=1.4, logit_scale=0.3, softcap=25.0),
}


def make_weights(cfg, seed):
    """Seeded bfloat16 tensors by the design's names, of a size that keeps activations of order one."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *shape, std=1.0: torch.randn(shape, generator=g) * std
    D, t = cfg["width"], {}

    def norm(name):
        t[name], t[name + ".b"], t[name + ".alpha"] = 1 + rn(D, std=0.1), rn(D, std=0.1), 0.6 + rn(std=0.1)

    t["embed"] = rn(cfg["vocab"], D)
    norm("final.norm")
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        norm(p + "norm1")
        if L["type"] == "parallel":
            a, b = m["left"], m["right"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                t[p + "mix.left." + name] = rn(rows, D, std=D ** -0.5)
            t[p + "mix.left.o"] = rn(D, H * dv, std=(H * dv) ** -0.5)
            H, d, dv = b["heads"], b["dim"], b["vdim"]
            for name, rows in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                t[p + "mix.right." + name] = rn(rows, D, std=D ** -0.5)
            t[p + "mix.right.norm"] = 1 + rn(H * dv, std=0.1)
            t[p + "mix.right.o"] = rn(D, H * dv, std=(H * dv) ** -0.5)
        else:
            H, d, r, dv, R, Rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"] = rn(Rq, D, std=D ** -0.5), 1 + rn(Rq, std=0.1)
            t[p + "mix.uq"] = rn(H * (d + r), Rq, std=Rq ** -0.5)
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = rn(R + r, D, std=D ** -0.5), 1 + rn(R, std=0.1)
            t[p + "mix.uk"], t[p + "mix.uv"] = rn(H * d, R, std=R ** -0.5), rn(H * dv, R, std=R ** -0.5)
            t[p + "mix.g"] = rn(H, D, std=D ** -0.5)
            t[p + "mix.o"] = rn(D, H * dv, std=(H * dv) ** -0.5)
        f = L["mlp"]
        if f is None:
            continue
        norm(p + "norm2")
        if f["kind"] == "dense":
            F = f["ff"]
            t[p + "mlp.up"], t[p + "mlp.down"] = rn(F, D, std=D ** -0.5), rn(D, F, std=F ** -0.5)
            continue

        def expert(pre, F):
            t[pre + ".gate"], t[pre + ".up"] = rn(F, D, std=1.5 * D ** -0.5), rn(F, D, std=1.5 * D ** -0.5)
            t[pre + ".down"] = rn(D, F, std=F ** -0.5)

        t[p + "mlp.router"] = rn(f["router"]["experts"], D, std=2.0 * D ** -0.5)
        for e in range(f["router"]["experts"]):
            expert(f"{p}mlp.e{e}", f["expert"]["ff"])
        if f.get("shared"):
            expert(p + "mlp.shared", f["shared"]["ff"])
            t[p + "mlp.shared.sg"] = rn(1, D, std=D ** -0.5)
    return {k: v.to(torch.bfloat16) for k, v in t.items()}


def write_model(cfg, folder, seed):
    from lumenllm_b200.weights.safetensors_io import write_file
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_file(folder / "model.safetensors", make_weights(cfg, seed))
    return folder

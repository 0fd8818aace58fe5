"""A plain, slow implementation of the Vekolix decoder on the CPU, written from the design's
equations, one function per mechanism. It shares no code with the library: whole sequences only,
no cache, no batching, a Python loop over time for the recurrence. The tests compare the engine
with it.

Notation: a sequence of T tokens, width D. rms(x) = sqrt(mean(x^2) + eps) over the last axis.
Softmax attention: H query heads, G key/value heads, key size d, value size dv. Linear attention:
H heads, key size d, value size dv, state S [d, dv] a head. Latent attention: H heads, d plain and r
rotated key coordinates a head, latent width R, query latent width Rq.
"""
import json
import math
import struct
from pathlib import Path

import torch

F = torch.float32


def read_safetensors(path):
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    head = json.loads(raw[8:8 + n])
    data = memoryview(raw)[8 + n:]
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}
    out = {}
    for name, info in head.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
    return out


def load_model(folder, dtype=F):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: v.to(dtype) for k, v in read_safetensors(folder / "model.safetensors").items()}
    return cfg, w


# ------------------------------------------------------------------ small pieces

def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def dynamic_tanh(x, w, b, alpha):
    """The model's norm: no mean, no variance; one learned slope for all coordinates."""
    return torch.tanh(alpha * x) * w + b


def silu(z):
    return z * torch.sigmoid(z)


def relu_squared(z):
    return torch.relu(z) ** 2


def frequencies(base, dims, scaling=None):
    """f_i = base^(-2i/dims) for i < dims/2 and the factor both cos and sin are multiplied by. With
    `scaling` (factor, original, fast, slow) slow frequencies are divided by the factor, fast ones
    stay, and a linear ramp over the pair index lies between."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if scaling is None:
        return f.to(F), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    where = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f.to(F), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, base, dims, scaling=None, interleaved=False):
    """x [T, heads, n]; the first `dims` coordinates of each head are rotated in pairs, (i, i + dims/2)
    or, interleaved, (2i, 2i + 1), by the angle position * f_i; the rest pass."""
    if not dims:
        return x
    half = dims // 2
    freq, mag = frequencies(base, dims, scaling)
    a = positions.to(F)[:, None] * freq[None, :]
    c, s = (torch.cos(a) * mag)[:, None, :].to(x.dtype), (torch.sin(a) * mag)[:, None, :].to(x.dtype)
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        r = torch.stack([u * c - v * s, v * c + u * s], dim=-1).flatten(-2)
        return torch.cat([r, x[..., dims:]], dim=-1)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def causal_softmax(scores):
    """scores [H, T, T] (query, key): every key after the query is hidden."""
    T = scores.shape[-1]
    hidden = torch.ones(T, T, dtype=torch.bool).triu(1)
    return torch.softmax(scores.float().masked_fill(hidden, float("-inf")), dim=-1)


# ------------------------------------------------------------------ mixers

def softmax_attention(h, w, pre, m, positions):
    """Grouped-query causal attention without biases; rotation of the first rot.dims of each head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + ".q"].T).view(T, H, d)
    k = (h @ w[pre + ".k"].T).view(T, G, d)
    v = (h @ w[pre + ".v"].T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate(q, positions, rot["base"], rot["dims"], rot.get("scaling"))
        k = rotate(k, positions, rot["base"], rot["dims"], rot.get("scaling"))
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("thd,shd->hts", q.float(), k.float()) * m["scale"]
    p = causal_softmax(scores)
    out = torch.einsum("hts,shd->thd", p, v.float()).to(h.dtype)
    return out.reshape(T, H * dv) @ w[pre + ".o"].T


def linear_attention(h, w, pre, m, eps):
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v through SiLU; all heads together
    RMS-normed, gated by sigmoid(Wg h), projected."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[pre + ".q"].T).view(T, H, d).float()
    k = silu(h @ w[pre + ".k"].T).view(T, H, d).float()
    v = silu(h @ w[pre + ".v"].T).view(T, H, dv).float()
    decay = torch.tensor(m["decay"], dtype=F)
    S = torch.zeros(H, d, dv, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    o = norm_plain(out.reshape(T, H * dv), w[pre + ".norm"].float(), eps)
    o = o * torch.sigmoid((h @ w[pre + ".g"].T).float())
    return o.to(h.dtype) @ w[pre + ".o"].T


def side_by_side(h, w, pre, m, eps, positions):
    left = softmax_attention(h, w, pre + ".left", m["left"], positions)
    right = linear_attention(h, w, pre + ".right", m["right"], eps)
    return m["left_scale"] * left.float() + m["right_scale"] * right.float()


def latent_attention(h, w, pre, m, eps, positions):
    """Queries through a normed latent; keys and values of all heads from one normed latent a token
    plus one rotated key part that all heads share; a sigmoid gate a head on the output."""
    T = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = norm_plain((h @ w[pre + ".dq"].T).float(), w[pre + ".dq.norm"].float(), eps).to(h.dtype)
    q = (cq @ w[pre + ".uq"].T).view(T, H, d + r)
    z = h @ w[pre + ".dkv"].T
    c = norm_plain(z[:, :R].float(), w[pre + ".dkv.norm"].float(), eps).to(h.dtype)
    kr = z[:, R:].view(T, 1, r)
    rot = m.get("rot")
    q_rot = q[..., d:]
    if rot:
        q_rot = rotate(q_rot, positions, rot["base"], rot["dims"], rot.get("scaling"), interleaved=True)
        kr = rotate(kr, positions, rot["base"], rot["dims"], rot.get("scaling"), interleaved=True)
    k = (c @ w[pre + ".uk"].T).view(T, H, d)
    v = (c @ w[pre + ".uv"].T).view(T, H, dv)
    scores = (torch.einsum("thd,shd->hts", q[..., :d].float(), k.float())
              + torch.einsum("thr,sr->hts", q_rot.float(), kr[:, 0].float())) * m["scale"]
    p = causal_softmax(scores)
    out = torch.einsum("hts,shd->thd", p, v.float())
    gate = torch.sigmoid((h @ w[pre + ".g"].T).float())           # [T, H]
    out = (out * gate[:, :, None]).to(h.dtype)
    return out.reshape(T, H * dv) @ w[pre + ".o"].T


# ------------------------------------------------------------------ feed-forwards

def dense_ff(h, w, pre):
    return relu_squared(h @ w[pre + ".up"].T) @ w[pre + ".down"].T


def clamped_expert(x, w, pre, limit):
    g = torch.clamp(x @ w[pre + ".gate"].T, max=limit)
    u = torch.clamp(x @ w[pre + ".up"].T, min=-limit, max=limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return y @ w[pre + ".down"].T


def expert_ff(h, w, pre, mlp):
    """Sigmoid router; the `top` largest scores; a score multiplies its expert's INPUT."""
    T = h.shape[0]
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.sigmoid(h.float() @ w[pre + ".router"].float().T)          # [T, E]
    best = torch.topk(s, top, dim=-1)
    out = torch.zeros(T, h.shape[1], dtype=F)
    for t in range(T):
        for j in range(top):
            e = int(best.indices[t, j])
            x = (best.values[t, j] * h[t].float()).to(h.dtype)
            out[t] += clamped_expert(x[None], w, f"{pre}.e{e}", mlp["expert"]["limit"])[0].float()
    if mlp.get("shared"):
        sg = torch.sigmoid((h @ w[pre + ".shared.sg"].T).float())          # [T, 1]
        out = out + sg * clamped_expert(h, w, pre + ".shared", mlp["shared"]["limit"]).float()
    return out


# ------------------------------------------------------------------ the model

def forward(cfg, w, tokens, layers_out=None):
    """Logits float32 [T, vocab] of one whole sequence. `layers_out`, a list, receives the stream
    after every layer."""
    eps = cfg["norm"]["eps"]
    m = cfg["residual_mult"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    x = w["embed"][tokens].float()
    dt = w["embed"].dtype

    def norm(name, x):
        return dynamic_tanh(x, w[name].float(), w[name + ".b"].float(), w[name + ".alpha"].float()).to(dt)

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        h = norm(p + ".norm1", x)
        if layer["type"] == "parallel":
            a = side_by_side(h, w, p + ".mix", layer["mixer"], eps, positions)
        elif layer["type"] == "latent_attention":
            a = latent_attention(h, w, p + ".mix", layer["mixer"], eps, positions)
        else:
            raise ValueError(layer["type"])
        x = x + m * a.float()
        mlp = layer.get("mlp")
        if mlp is not None:
            h = norm(p + ".norm2", x)
            f = dense_ff(h, w, p + ".mlp") if mlp["kind"] == "dense" else expert_ff(h, w, p + ".mlp", mlp)
            x = x + m * f.float()
        if layers_out is not None:
            layers_out.append(x.clone())
    y = norm("final.norm", x)
    logits = (y @ w["embed"].T).float() * cfg["logit_scale"]
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def greedy(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]

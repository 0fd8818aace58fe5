"""A plain, slow implementation of the Lebelix decoder on the CPU, written from the design's
equations, one function per mechanism. It shares no code with the library: whole sequences only,
no cache, no batching, a Python loop over time for the recurrence. The tests compare the engine
with it.

Notation: a sequence of T tokens, width D. rms(x) = sqrt(mean(x^2) + eps) over the last axis.
Attention: H query heads, G key/value heads, key size d, value size dv. Latent attention: H heads,
d plain and r rotated key coordinates a head, latent width R. Delta rule: H value heads of dv
channels, G query/key heads of d channels, state S [d, dv] a head.
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


def norm_one_plus(x, w, eps):
    """The model's norm: the stored weight lies around zero and counts as 1 + w."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate(x, positions, base, dims):
    """x [T, heads, n]; the first `dims` coordinates of each head are rotated in pairs
    (i, i + dims/2) by the angle position * base^(-2i/dims); the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.tensor(float(base), dtype=x.dtype) ** (-2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def window_mask(T, size):
    """[query, key]: key j is seen from i when 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def chunk_mask(T, size):
    """[query, key]: key j <= i is seen when both lie in the same run of `size` positions counted
    from the sequence's first token."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def causal_conv_silu(x, taps_w):
    """x [T, C]; taps_w [C, taps], the last column the current token's; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + pad[j:j + T] * taps_w[:, j][None, :]
    return silu(y)


# ------------------------------------------------------------------ mixers

def attention(h, w, pre, m, eps, sink=1.0):
    """Biased projections, an RMS norm of every query and key head (one weight of d values for all
    heads), partial rotation, capped scores, sight within the query's own chunk, a softmax whose
    denominator has one more term exp(0) with no value behind it, and a sigmoid gate on the heads'
    outputs. (`sink` 0.0 gives the ordinary softmax; the tests use it to show that a case tells the
    two apart.)"""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, d)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G, d)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, dv)
    q = norm_plain(q, w[pre + "q.norm"], eps)
    k = norm_plain(k, w[pre + "k.norm"], eps)
    pos = torch.arange(T)
    if m.get("rot"):
        q = rotate(q, pos, m["rot"]["base"], m["rot"]["dims"])
        k = rotate(k, pos, m["rot"]["base"], m["rot"]["dims"])
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    seen = chunk_mask(T, m["mask"]["size"]) if m.get("mask") else window_mask(T, T)
    s = s.masked_fill(~seen[None], float("-inf"))
    big = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - big)
    p = e / (sink * torch.exp(-big) + e.sum(dim=-1, keepdim=True))
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def latent_of(h, w, pre, m, eps):
    """What a latent-attention layer leaves for keys and values: the normed latent c [T, R] and the
    rotated key part [T, r] that all heads share."""
    R, r = m["kv_rank"], m["rot_dim"]
    T = h.shape[0]
    z = h @ w[pre + "dkv"].T
    c = norm_plain(z[:, :R], w[pre + "dkv.norm"], eps)
    kr = z[:, R:]
    if m.get("rot"):
        kr = rotate(kr.reshape(T, 1, r), torch.arange(T), m["rot"]["base"], m["rot"]["dims"]).view(T, r)
    return c, kr


def latent_attention(h, w, pre, m, eps, latent):
    """latent = (c, kr) of this layer or of the layer it borrows from. Keys and values of a head
    are products of c; the rotated part is one for all heads; sliding window; ordinary softmax."""
    T = h.shape[0]
    H, d, r, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = latent
    q = (h @ w[pre + "q"].T).view(T, H, d + r)
    q_plain = q[..., :d]
    q_rot = q[..., d:]
    if m.get("rot"):
        q_rot = rotate(q_rot, torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[pre + "uk"].T).view(T, H, d)
    v = (c @ w[pre + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, kr)) * m["scale"]
    seen = window_mask(T, m["mask"]["size"]) if m.get("mask") else window_mask(T, T)
    s = s.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    return o @ w[pre + "o"].T


def channel_delta(h, w, pre, m, eps):
    """The gated delta rule with a decay of its own for every key channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ w[pre + "q"].T, w[pre + "q.conv"]).view(T, G, d)
    k = causal_conv_silu(h @ w[pre + "k"].T, w[pre + "k.conv"]).view(T, G, d)
    v = causal_conv_silu(h @ w[pre + "v"].T, w[pre + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    q = q.repeat_interleave(H // G, dim=1)
    k = k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ w[pre + "b"].T)                                     # [T, H]
    a = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "dt_bias"]             # [T, H d]
    decay = torch.exp(-torch.exp(w[pre + "A_log"])[None, :, None] * softplus(a).view(T, H, d))
    gate = torch.sigmoid((h @ w[pre + "g1"].T) @ w[pre + "g2"].T).view(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = decay[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hde,hd->he", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    out = rms_unit(out, eps) * w[pre + "norm"] * gate
    return out.reshape(T, H * dv) @ w[pre + "o"].T


# ------------------------------------------------------------------ the model

def dense_ff(y, w, pre):
    return gelu_tanh(y @ w[pre + "up"].T) @ w[pre + "down"].T


def token_side(x, tokens, w, i, dim, eps):
    """A layer's own small table of token vectors, gated by the stream and added back normed."""
    e = w["side.embed"][tokens][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ w[f"l{i}.side.gate"].T) * e
    y = g @ w[f"l{i}.side.proj"].T
    return rms_unit(y, eps) * w[f"l{i}.side.norm"]


def forward(cfg, w, tokens, streams=None):
    """Logits [T, vocab] of one whole sequence. With `streams` (a list) the residual stream after
    every layer is appended to it."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = w["embed"][tokens] * cfg["embedding"]["scale"]
    side = cfg.get("token_side")
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.mix.", layer["mixer"]
        h = norm_one_plus(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            a = attention(h, w, pre, m, eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(h, w, pre, m, eps)
                src = i
            a = latent_attention(h, w, pre, m, eps, latents[src])
        elif layer["type"] == "channel_delta":
            a = channel_delta(h, w, pre, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + a
        if layer.get("mlp") is not None:
            x = x + dense_ff(norm_one_plus(x, w[f"l{i}.norm2"], eps), w, f"l{i}.mlp.")
        if side:
            x = x + token_side(x, tokens, w, i, side["dim"], eps)
        if streams is not None:
            streams.append(x.clone())
    y = norm_one_plus(x, w["final.norm"], eps)
    return y @ w["embed"].T


def generate_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]

"""Latent attention: the keys and values of all heads are products of ONE vector a token.

For H heads with d plain and r rotated query/key values a head, value size dv and latent size R:
q = y Wq^T, laid out head by head as [d plain | r rotated]; z = y Wdkv^T has R + r values, of which
the first R, RMS-normed with the weight `.dkv.norm`, are the latent c, and the last r are a key part
that all heads share; the position part rotates the first `rotary_dim` of the r values of every
query head and of the shared key part. Head h's plain key is Uk_h c and its value Uv_h c
(`.uk` [H d, R], `.uv` [H dv, R]); score = softmax_scale * (q_plain . k_plain + q_rot . k_rot);
a query at position p sees key j if 0 <= p - j < window (window 0: every earlier key); ordinary
softmax; o = ctx Wo^T.

The cache keeps [c | rotated key part] per token and nothing per head (CacheNeed.values_in_keys:
one kv head whose rows are R + r wide and whose values are the rows' first R numbers). A query
head is carried into the latent space, q_plain Uk_h (kernels.latent_query), scores and weighted
sums are taken over the cached rows (kernels.attn_latent on the tensor cores in bfloat16, where a
block's rows are (token, head) pairs that share every cached row; the general attention kernel in
float32 and for widths the other does not take), and the sums come back through Uv_h
(kernels.head_product); nothing of a key or value is ever expanded. With `shares_cache` the
part has no Wdkv and reads the cache of the entry the schedule names, with its own Uk, Uv, queries
and window; `cache_window` is what the cache must keep in sight (the widest window of its readers).

Options. `query_rank` Rq > 0: the queries go through a latent of their own, cq = RMSnorm(y Wdq^T)
with the weight `.dq.norm`, q = cq Wuq^T (`.dq` [Rq, D], `.uq` [H (d + r), Rq] instead of `.q`).
`head_gate`: head h's output is multiplied by sigmoid(y Wg^T)_h, one number a head (`.g` [H, D]);
the factor is applied where the sums leave the latent space, before they are rounded.
`interleaved_rotation`: the rotation pairs coordinate 2i with 2i + 1 instead of i with i +
rotary_dim/2. A score is a dot product, so the same reordering of the rotated coordinates of
queries and keys leaves it as it is: the rows of the two projections that make them are put in
the other pairing's order once, at load, and the kernels rotate as they always do.
"""
from __future__ import annotations

import torch

from ..cache.kv import LAYOUT_LINEAR, CacheNeed
from ..ops import kernels as K
from .base import build_part, need, part_tensors, register_part
from .linear import Linear


@register_part("mixer", "latent_attention")
class LatentAttention:
    graph_safe = True

    @staticmethod
    def _sizes(p):
        return tuple(int(need(p, k, "latent_attention")) for k in
                     ("hidden_size", "num_heads", "head_dim", "rot_width", "value_dim", "latent_size"))

    @classmethod
    def tensors(cls, spec):
        p = spec.params
        D, H, d, r, dv, R = cls._sizes(p)
        pre = spec.prefix
        t = {f"{pre}.uk": ((H * d, R), "matrix"), f"{pre}.uv": ((H * dv, R), "matrix"),
             f"{pre}.o": ((D, H * dv), "matrix")}
        Rq = int(p.get("query_rank", 0) or 0)
        if Rq:
            t.update({f"{pre}.dq": ((Rq, D), "matrix"), f"{pre}.dq.norm": ((Rq,), "norm"),
                      f"{pre}.uq": ((H * (d + r), Rq), "matrix")})
        else:
            t[f"{pre}.q"] = ((H * (d + r), D), "matrix")
        if p.get("head_gate", False):
            t[f"{pre}.g"] = ((H, D), "matrix")
        if not p.get("shares_cache", False):
            t[f"{pre}.dkv"] = ((R + r, D), "matrix")
            t[f"{pre}.dkv.norm"] = ((R,), "norm")
        t.update(part_tensors("position", p["position"]))
        return t

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        _, self.H, self.d, self.r, self.dv, self.R = self._sizes(p)
        if self.R + self.r > 1024 or self.R > 512:
            raise ValueError(f"a latent of {self.R} + {self.r}: the attention kernel takes rows up to 1024 wide "
                             "and latents up to 512")
        self.window = int(p.get("window", 0) or 0)
        self.cache_window = int(p.get("cache_window", self.window) or 0)
        self.scale = float(need(p, "softmax_scale", "latent_attention"))
        self.eps = float(need(p, "norm_eps", "latent_attention"))
        self.shares_cache = bool(p.get("shares_cache", False))
        self.position = build_part("position", p["position"], weights, runtime)
        if self.position.rotary_dim > self.r:
            raise ValueError(f"a rotation over {self.position.rotary_dim} of {self.r} rotated values")
        pre = spec.prefix
        rot = self.position.rotary_dim
        pairs = None
        if p.get("interleaved_rotation", False) and rot:
            # coordinate 2i goes to place i, coordinate 2i + 1 to place i + rot/2
            pairs = torch.cat([torch.arange(0, rot, 2), torch.arange(1, rot, 2), torch.arange(rot, self.r)])

        def q_rows(w):          # the rotated coordinates of every query head in the kernels' pairing
            if pairs is None:
                return w
            w = w.view(self.H, self.d + self.r, -1)
            return torch.cat([w[:, :self.d], w[:, self.d:][:, pairs.to(w.device)]], dim=1).reshape(self.H * (self.d + self.r), -1)

        self.Rq = int(p.get("query_rank", 0) or 0)
        self.head_gate = bool(p.get("head_gate", False))
        f32 = lambda n: weights[n].to(device=runtime.device, dtype=torch.float32).contiguous()
        mats = [weights[f"{pre}.dq"]] if self.Rq else [q_rows(weights[f"{pre}.q"])]
        self.q_width = mats[0].shape[0]
        self.c_norm = self.q_norm = self.uq = None
        if self.Rq:
            self.q_norm = f32(f"{pre}.dq.norm")
            self.uq = Linear(q_rows(weights[f"{pre}.uq"]).contiguous(), runtime)
        if not self.shares_cache:
            dkv = weights[f"{pre}.dkv"]
            if pairs is not None:
                dkv = torch.cat([dkv[:self.R], dkv[self.R:][pairs.to(dkv.device)]], dim=0)
            mats.append(dkv)          # reads the same rows: one product for both
            self.c_norm = f32(f"{pre}.dkv.norm")
        self.c_col = self.q_width
        self.g_col = sum(m.shape[0] for m in mats)
        if self.head_gate:
            mats.append(weights[f"{pre}.g"])
        self.proj = Linear.stacked(mats, runtime)
        keep = torch.float32 if runtime.is_f32 else None
        self.uk = weights[f"{pre}.uk"].to(device=runtime.device, dtype=keep).contiguous()
        self.uv = weights[f"{pre}.uv"].to(device=runtime.device, dtype=keep).contiguous()
        self.o = Linear(weights[f"{pre}.o"], runtime)

    def cache_need(self):
        return CacheNeed(1, self.R + self.r, self.cache_window, v_dim=self.R, layout=LAYOUT_LINEAR,
                         values_in_keys=True)

    def state_shape(self):
        return None

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, entry, residual=None):
        kc, _, table = entry.cache()
        u = self.proj(y, split_ok=True)            # float32 [q (or its latent) | c and key part | gate], possibly partial sums
        rot = self.position.rotary_dim
        cs = self.position.angles(ctx) if rot else None
        if entry.writes_cache and not self.shares_cache:
            K.latent_store(u, self.c_col, self.R, self.r, self.c_norm, self.eps, cs, rot,
                           ctx.cache_pos, ctx.tok_seq, table, kc)
        qp = u
        if self.Rq:               # the queries' own latent, normed, and up again
            qp = self.uq(K.cols_rmsnorm(u, 0, self.Rq, self.q_norm, self.eps, self.runtime.dtype), split_ok=True)
        if K.attn_latent_takes(self.R + self.r, self.R, kc.dtype):
            # bfloat16: queries rounded once they are in the latent space, scores and sums on the tensor cores
            q = K.latent_query(qp, self.uk, self.H, self.d, self.r, self.R, cs, rot, out_dtype=torch.bfloat16)
            # a captured step is replayed for other divisions of its tokens than the one it was captured with
            q_lens = None if ctx.extras.get("captured") else ctx.q_lens
            mixed = K.attn_latent(q, kc, table, ctx.cu_q, ctx.seq_start, q_lens, self.R, self.window, self.scale,
                                  n_seqs=ctx.B, n_split=K.ATTN_LATENT_DECODE_SPLIT if ctx.is_decode else 1)
        else:
            q = K.latent_query(qp, self.uk, self.H, self.d, self.r, self.R, cs, rot)
            mixed = K.attn_generic_opt(q, kc, None, table, ctx.tok_seq, ctx.cache_pos, self.window, self.scale,
                                       layout=LAYOUT_LINEAR, values_in_keys=True, value_dim=self.R)
        out = K.head_product(mixed, self.uv, self.runtime.dtype, gate=u if self.head_gate else None, gate_col=self.g_col)
        return self.o(out, split_ok=True, add_to=residual)

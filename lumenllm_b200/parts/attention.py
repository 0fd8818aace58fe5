"""The attention mixers: grouped-query causal attention over the cache.

"gqa_attention" (GQAttention) norms each head, "wide_norm_attention" (WideNormAttention)
norms a whole projection at once, has biases, a value norm and values of their own width,
"head_norm_attention" (HeadNormAttention, at the end of this file) norms each head, has biases,
values of their own width, capped scores, chunks, a sink in the softmax and an output gate; all
hand their queries to `causal_attention`, which picks the kernel.

In order (crates/aegisllm-cuda/src/executor/attention.rs:139-202,241-250,341-352,
413-425; prompt twin executor/prefill/layer.rs:472-636,810-823,967-1047):
q, k, v = y Wq^T, y Wk^T, y Wv^T; optional per-head RMSNorm of q and k with a
weight of head_dim values; rotation of q and k; k, v appended to the cache at the
token's position; for query head h the kv head is h // (heads / kv_heads)
(attention_decode_common.cuh:112-115), scores scaled by `softmax_scale`, a query
at position p sees keys j <= p (and p - j < window if a window is set); o = ctx Wo^T.
Softmax, norms and angles are float32.
"""
from __future__ import annotations

import torch

from ..cache.kv import CacheNeed
from ..ops import kernels as K
from .base import build_part, need, part_tensors, register_part
from .linear import Linear


# Batches of a decode step for which the attention kernel does the rotary kernel's work itself
# (ops.kernels.attn_decode_qkv; the same bits either way). It saves a kernel and its wait on the
# step's path, and costs every block of a sequence's segments the making of its query heads:
# at the 8B shape 2,455 against 2,424 tokens/s at batch 8 and 4,428 against 4,372 at 16, but
# 6,985 against 7,083 at 32 and 10,290 against 10,600 at 64; at batch 1 338 against 340.
FUSED_DECODE_ROWS = (4, 16)


@register_part("mixer", "gqa_attention")
class GQAttention:
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        p = spec.params
        H, nq, nkv, d = (int(need(p, k, "gqa_attention")) for k in
                         ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        t = {f"{spec.prefix}.q_proj.weight": ((nq * d, H), "matrix"),
             f"{spec.prefix}.o_proj.weight": ((H, nq * d), "matrix")}
        if not p.get("shares_cache", False):
            t[f"{spec.prefix}.k_proj.weight"] = ((nkv * d, H), "matrix")
            t[f"{spec.prefix}.v_proj.weight"] = ((nkv * d, H), "matrix")
        if p.get("qk_norm", False):
            t[f"{spec.prefix}.q_norm.weight"] = ((d,), "norm")
            if not p.get("shares_cache", False):
                t[f"{spec.prefix}.k_norm.weight"] = ((d,), "norm")
        t.update(part_tensors("position", p["position"]))
        return t

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        self.H = int(p["hidden_size"])
        self.nq, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} heads are not a multiple of {self.nkv} kv heads")
        if self.d % 16 or self.d > 256:
            raise ValueError(f"head_dim {self.d}: the attention kernels take multiples of 16 up to 256")
        self.window = int(p.get("window", 0) or 0)
        self.scale = float(need(p, "softmax_scale", "gqa_attention"))
        self.shares_cache = bool(p.get("shares_cache", False))
        self.position = build_part("position", p["position"], weights, runtime)
        pre = spec.prefix
        mats = [weights[f"{pre}.q_proj.weight"]]
        if not self.shares_cache:
            mats += [weights[f"{pre}.k_proj.weight"], weights[f"{pre}.v_proj.weight"]]
        self.qkv = Linear.stacked(mats, runtime)
        # a run that reads another run's cache projects queries only
        self.q_only = self.qkv if self.shares_cache else self.qkv.first_rows(self.nq * self.d)
        self.o = Linear(weights[f"{pre}.o_proj.weight"], runtime)
        self.q_norm = self.k_norm = None
        self.qk_eps = float(p.get("qk_norm_eps", 0.0))
        if p.get("qk_norm", False):
            off = float(p.get("qk_norm_weight_offset", 0.0))
            f32 = lambda n: (weights[n].to(device=runtime.device, dtype=torch.float32) + off).contiguous()
            self.q_norm = f32(f"{pre}.q_norm.weight")
            if not self.shares_cache:
                self.k_norm = f32(f"{pre}.k_norm.weight")

    def cache_need(self):
        return CacheNeed(self.nkv, self.d, self.window)

    def state_shape(self):
        return None

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, entry, residual=None):
        kc, vc, table = entry.cache()
        writes = entry.writes_cache and not self.shares_cache
        if (writes and not self.qkv.f32 and entry.layout == K.LAYOUT_SW128 and y.is_contiguous()
                and K.gemm_tc_qkv_takes(y.shape[0], self.qkv.out_features, self.qkv.in_features, self.nq,
                                        self.nkv, self.d, self.position.rotary_dim)):
            # a prompt with heads of 128: norm, rotation and cache write in the product's epilogue
            q = K.gemm_tc_qkv(y, self.qkv.weight, self.q_norm, self.k_norm, self.qk_eps,
                              self.position.angles(ctx), self.position.rotary_dim, ctx.cache_pos,
                              ctx.tok_seq, table, kc, vc, self.nq, self.nkv)
            out = self.attend(q, kc, vc, table, ctx, entry.layout)
            return self.o(out.view(-1, self.nq * self.d), split_ok=True, add_to=residual)
        # float32 [N, (nq + 2 nkv) d], possibly as S partial sums
        qkv = self.qkv(y, split_ok=True) if writes else self.q_only(y, split_ok=True)
        if (writes and ctx.is_decode and FUSED_DECODE_ROWS[0] <= ctx.B <= FUSED_DECODE_ROWS[1]
                and entry.layout == K.LAYOUT_SW128 and self.d == 128
                and self.nq // self.nkv <= 16 and self.position.rotary_dim in (0, 128)
                and kc.dtype == torch.bfloat16):
            # one token a sequence, heads of 128: the attention blocks make their query heads and
            # the new key and value themselves, from the projection's partial sums
            out = K.attn_decode_qkv(qkv, self.q_norm, self.k_norm, self.qk_eps, self.position.angles(ctx),
                                    self.position.rotary_dim, kc, vc, table, ctx.cache_pos, self.window,
                                    self.scale, self.nq, self.nkv)
            return self.o(out.view(-1, self.nq * self.d), split_ok=True, add_to=residual)
        nkv_new = self.nkv if writes else 0
        q = K.qk_norm_rope_store(qkv, self.q_norm, self.k_norm, self.qk_eps,
                                 self.position.angles(ctx), self.position.rotary_dim,
                                 ctx.cache_pos, ctx.tok_seq, table,
                                 kc if nkv_new else None, vc if nkv_new else None,
                                 self.nq, nkv_new, self.d, self.runtime.dtype, layout=entry.layout)
        out = self.attend(q, kc, vc, table, ctx, entry.layout)
        return self.o(out.view(-1, self.nq * self.d), split_ok=True, add_to=residual)

    def attend(self, q, kc, vc, table, ctx, layout):
        return causal_attention(q, kc, vc, table, ctx, layout, layout, self.window, self.scale)


def causal_attention(q, kc, vc, table, ctx, k_layout, v_layout, window, scale, chunk=0, softcap=0.0,
                     sink=False, gate=None, gate_col=0):
    """Chooses the kernel by the step's shape: the split-KV kernel when every sequence
    brings one token, the flash kernel for prompts, and the general kernel for the
    32-bit path and for head sizes the fast kernels do not take (keys and values of
    different widths among them). All agree within rounding. q [N, nq, d].
    `chunk`, `softcap`, `sink` and `gate` are the options of ops.kernels.attn_generic_opt."""
    nq, d = q.shape[1], q.shape[2]
    nkv, dv = kc.shape[1], vc.shape[3]
    opts = dict(chunk=chunk, softcap=softcap, sink=sink, gate=gate, gate_col=gate_col)
    fast = (k_layout == K.LAYOUT_SW128 and v_layout == K.LAYOUT_SW128 and q.dtype == torch.bfloat16
            and d == dv and d in (64, 128) and nq // nkv <= 16)
    if fast and ctx.is_decode:
        return K.attn_decode(q, kc, vc, table, ctx.cache_pos, window, scale, **opts)
    if fast:
        # a captured step is replayed for other divisions of its tokens than the one it was
        # captured with: the kernel then takes the division from the device alone
        q_lens = None if ctx.extras.get("captured") else ctx.q_lens
        return K.attn_prefill(q, kc, vc, table, ctx.cu_q, ctx.seq_start, q_lens, window, scale, n_seqs=ctx.B, **opts)
    if chunk or softcap or sink or gate is not None:
        return K.attn_generic_opt(q, kc, vc, table, ctx.tok_seq, ctx.cache_pos, window, scale, layout=k_layout,
                                  v_layout=v_layout, **opts)
    return K.attn_generic(q, kc, vc, table, ctx.tok_seq, ctx.cache_pos, window, scale, layout=k_layout,
                          v_layout=v_layout)


@register_part("mixer", "wide_norm_attention")
class WideNormAttention:
    """q, k, v = y Wq^T + bq, y Wk^T + bk, y Wv^T + bv; ONE RMS norm over the whole query
    projection (all heads at once, a weight of heads x dim values) and one over the whole key
    projection; then the position part's rotation of the first `rotary_dim` values of every
    query and key head; every value head divided by its own root mean square (no weight) and
    cached so; a query at position p sees key j if 0 <= p - j < window (window 0: every earlier
    key); ordinary softmax of scale * q . k; query head h reads kv head h // (heads / kv_heads);
    o = ctx Wo^T, without a bias. Keys are `head_dim` wide, values `value_dim`. Norms, angles,
    scores and weights are float32. Parameters: hidden_size, num_heads, num_kv_heads, head_dim,
    value_dim, softmax_scale, window, norm_eps, value_norm (bool), position (a PartSpec)."""
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        p = spec.params
        D, H, G, d, dv = (int(need(p, k, "wide_norm_attention")) for k in
                          ("hidden_size", "num_heads", "num_kv_heads", "head_dim", "value_dim"))
        pre = spec.prefix
        t = {f"{pre}.q": ((H * d, D), "matrix"), f"{pre}.q.b": ((H * d,), "matrix"),
             f"{pre}.k": ((G * d, D), "matrix"), f"{pre}.k.b": ((G * d,), "matrix"),
             f"{pre}.v": ((G * dv, D), "matrix"), f"{pre}.v.b": ((G * dv,), "matrix"),
             f"{pre}.q.norm": ((H * d,), "norm"), f"{pre}.k.norm": ((G * d,), "norm"),
             f"{pre}.o": ((D, H * dv), "matrix")}
        t.update(part_tensors("position", p["position"]))
        return t

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        self.H, self.G = int(p["num_heads"]), int(p["num_kv_heads"])
        self.d, self.dv = int(p["head_dim"]), int(p["value_dim"])
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} kv heads")
        if self.d > 256 or self.dv > 256:
            raise ValueError(f"key size {self.d}, value size {self.dv}: the attention kernels take up to 256")
        self.window = int(p.get("window", 0) or 0)
        self.scale = float(need(p, "softmax_scale", "wide_norm_attention"))
        self.eps = float(need(p, "norm_eps", "wide_norm_attention"))
        self.value_norm = bool(p.get("value_norm", False))
        self.position = build_part("position", p["position"], weights, runtime)
        pre = spec.prefix
        f32 = lambda n: weights[n].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.qkv = Linear.stacked([weights[f"{pre}.q"], weights[f"{pre}.k"], weights[f"{pre}.v"]], runtime)
        self.qkv_bias = torch.cat([f32(f"{pre}.q.b"), f32(f"{pre}.k.b"), f32(f"{pre}.v.b")]).contiguous()
        self.q_norm, self.k_norm = f32(f"{pre}.q.norm"), f32(f"{pre}.k.norm")
        self.o = Linear(weights[f"{pre}.o"], runtime)

    def cache_need(self):
        return CacheNeed(self.G, self.d, self.window, v_dim=0 if self.dv == self.d else self.dv)

    def state_shape(self):
        return None

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, entry, residual=None):
        kc, vc, table = entry.cache()
        qkv = self.qkv(y, split_ok=True)
        rot = self.position.rotary_dim
        q = K.qkv_bias_norm_store(qkv, self.qkv_bias, self.q_norm, self.k_norm, self.eps, ctx.cache_pos,
                                  ctx.tok_seq, table, kc, vc, self.H, self.G, self.d, self.dv, self.runtime.dtype,
                                  k_layout=entry.layout, v_layout=entry.v_layout,
                                  cs=self.position.angles(ctx) if rot else None, rotary_dim=rot,
                                  value_unit_eps=self.eps if self.value_norm else None)
        out = causal_attention(q, kc, vc, table, ctx, entry.layout, entry.v_layout, self.window, self.scale)
        return self.o(out.view(-1, self.H * self.dv), split_ok=True, add_to=residual)


@register_part("mixer", "head_norm_attention")
class HeadNormAttention:
    """q, k, v = y Wq^T (+ bq), y Wk^T (+ bk), y Wv^T (+ bv); every query head and every key head
    RMS-normed over its `head_dim` values with ONE weight of that size for all heads (plain weight);
    then the position part's rotation of the first `rotary_dim` values of every query and key head;
    score = softmax_scale * q . k, and with `softcap` c > 0 then c * tanh(score / c); a query at
    position p sees key j <= p, with `chunk` n > 0 only where p // n == j // n, with `window` w > 0
    only where p - j < w; weights exp(s_j) / (sink + sum exp(s_j)) with sink = 1 when `sink` is set
    (a key of score 0 without a value) and 0 otherwise; query head h reads kv head
    h // (heads / kv_heads); with `output_gate` the heads' outputs are multiplied by
    sigmoid(y Wg^T) element by element; o = ctx Wo^T without a bias. Keys are `head_dim` wide,
    values `value_dim`. Norms, angles, scores and weights are float32. Tensors: `<prefix>.q`, `.k`,
    `.v` (each with `.b` when `bias`), `.q.norm`, `.k.norm` (when `qk_norm`, the default), `.g`
    (when `output_gate`), `.o`."""
    graph_safe = True

    @staticmethod
    def _sizes(p):
        return tuple(int(need(p, k, "head_norm_attention")) for k in
                     ("hidden_size", "num_heads", "num_kv_heads", "head_dim", "value_dim"))

    @classmethod
    def tensors(cls, spec):
        p = spec.params
        D, H, G, d, dv = cls._sizes(p)
        pre = spec.prefix
        t = {f"{pre}.q": ((H * d, D), "matrix"), f"{pre}.k": ((G * d, D), "matrix"),
             f"{pre}.v": ((G * dv, D), "matrix"), f"{pre}.o": ((D, H * dv), "matrix")}
        if p.get("bias", False):
            t.update({f"{pre}.q.b": ((H * d,), "matrix"), f"{pre}.k.b": ((G * d,), "matrix"),
                      f"{pre}.v.b": ((G * dv,), "matrix")})
        if p.get("qk_norm", True):
            t.update({f"{pre}.q.norm": ((d,), "norm"), f"{pre}.k.norm": ((d,), "norm")})
        if p.get("output_gate", False):
            t[f"{pre}.g"] = ((H * dv, D), "matrix")
        t.update(part_tensors("position", p["position"]))
        return t

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        _, self.H, self.G, self.d, self.dv = self._sizes(p)
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} kv heads")
        if self.d > 512 or self.dv > 512:
            raise ValueError(f"key size {self.d}, value size {self.dv}: the attention kernels take up to 512")
        self.window = int(p.get("window", 0) or 0)
        self.chunk = int(p.get("chunk", 0) or 0)
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        self.sink = bool(p.get("sink", False))
        self.scale = float(need(p, "softmax_scale", "head_norm_attention"))
        self.eps = float(need(p, "norm_eps", "head_norm_attention"))
        self.position = build_part("position", p["position"], weights, runtime)
        pre = spec.prefix
        f32 = lambda n: weights[n].to(device=runtime.device, dtype=torch.float32).contiguous()
        mats = [weights[f"{pre}.q"], weights[f"{pre}.k"], weights[f"{pre}.v"]]
        self.gated = bool(p.get("output_gate", False))
        if self.gated:
            mats.append(weights[f"{pre}.g"])       # the gate reads the same rows: one product for all four
        # `external_projection`: whoever runs this part makes the product (stacked with others that read
        # the same rows) and hands its result to forward; these are the matrices, in the order of the columns
        self.input_mats = mats if p.get("external_projection", False) else None
        self.proj = None if self.input_mats is not None else Linear.stacked(mats, runtime)
        self.bias = (torch.cat([f32(f"{pre}.q.b"), f32(f"{pre}.k.b"), f32(f"{pre}.v.b")]).contiguous()
                     if p.get("bias", False) else None)
        self.q_norm = self.k_norm = None
        if p.get("qk_norm", True):
            self.q_norm, self.k_norm = f32(f"{pre}.q.norm"), f32(f"{pre}.k.norm")
        self.gate_col = self.H * self.d + self.G * (self.d + self.dv)
        self.o = Linear(weights[f"{pre}.o"], runtime)

    def cache_need(self):
        return CacheNeed(self.G, self.d, self.window, v_dim=0 if self.dv == self.d else self.dv, chunk=self.chunk)

    def state_shape(self):
        return None

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    projects_input = True         # may be built with `external_projection` and fed `projected`
    needs_first_columns = True    # its kernels read q, k, v (and the gate) from column 0 of the projection's rows

    def forward(self, y, ctx, entry, residual=None, projected=None, col0=0):
        kc, vc, table = entry.cache()
        if projected is not None and col0 != 0:
            raise ValueError("head_norm_attention reads its columns from the start of the projection's rows")
        # float32 [q | k | v | gate | ...], possibly partial sums
        u = projected if projected is not None else self.proj(y, split_ok=True)
        rot = self.position.rotary_dim
        q = K.qkv_head_norm_store(u, self.bias, self.q_norm, self.k_norm, self.eps,
                                  self.position.angles(ctx) if rot else None, rot, ctx.cache_pos, ctx.tok_seq, table,
                                  kc, vc, self.H, self.G, self.d, self.dv, self.runtime.dtype,
                                  k_layout=entry.layout, v_layout=entry.v_layout)
        out = causal_attention(q, kc, vc, table, ctx, entry.layout, entry.v_layout, self.window, self.scale,
                               chunk=self.chunk, softcap=self.softcap, sink=self.sink,
                               gate=u if self.gated else None, gate_col=self.gate_col)
        return self.o(out.view(-1, self.H * self.dv), split_ok=True, add_to=residual)

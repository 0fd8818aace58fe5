"""The gated delta rule with a decay for every key channel ("channel_delta"): a linear recurrence
over time with a matrix state per head, in place of attention.

In order, for H value heads of dv channels and G query/key heads of d channels (head h reads
query/key head h // (H / G)): q = y Wq^T, k = y Wk^T (G d wide), v = y Wv^T (H dv wide); each goes
through a causal convolution over time on every channel of its own (`taps` taps, no bias, the last
tap the current token's, zeros before a sequence's start) and SiLU; q and k become unit vectors per
head (x / sqrt(sum x^2 + 1e-6)), q also times d^-1/2; beta = sigmoid(y Wb^T), one a head;
g = exp(-exp(A_log_h) softplus((y Wa1^T) Wa2^T + dt_bias)), one a (head, key channel); per head
S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q (S is d x dv, and o sees the
token's own write); every head's o is divided by its root mean square over dv, times the weight
`.norm` (dv values, one for all heads), times sigmoid((y Wg1^T) Wg2^T); out = that Wo^T.

A sequence's state is S of every head (float32, kept [H, dv, d]) and the convolution's last
taps - 1 inputs; both start at zero and are carried from step to step, so a sequence may be fed in
any portions. Everything that enters the recurrence is float32; the projections run in the run's
type. The six projections that read y are one product.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import need, register_part
from .linear import Linear


@register_part("mixer", "channel_delta")
class ChannelDeltaMixer:
    graph_safe = True

    @staticmethod
    def _sizes(p):
        return tuple(int(need(p, k, "channel_delta")) for k in
                     ("hidden_size", "num_heads", "num_kv_heads", "head_dim", "value_dim", "taps", "decay_rank",
                      "gate_rank"))

    @classmethod
    def tensors(cls, spec):
        D, H, G, d, dv, taps, ra, rg = cls._sizes(spec.params)
        pre = spec.prefix
        return {f"{pre}.q": ((G * d, D), "matrix"), f"{pre}.q.conv": ((G * d, taps), "matrix"),
                f"{pre}.k": ((G * d, D), "matrix"), f"{pre}.k.conv": ((G * d, taps), "matrix"),
                f"{pre}.v": ((H * dv, D), "matrix"), f"{pre}.v.conv": ((H * dv, taps), "matrix"),
                f"{pre}.b": ((H, D), "matrix"), f"{pre}.A_log": ((H,), "matrix"),
                f"{pre}.a1": ((ra, D), "matrix"), f"{pre}.a2": ((H * d, ra), "matrix"),
                f"{pre}.dt_bias": ((H * d,), "matrix"),
                f"{pre}.g1": ((rg, D), "matrix"), f"{pre}.g2": ((H * dv, rg), "matrix"),
                f"{pre}.norm": ((dv,), "norm"), f"{pre}.o": ((D, H * dv), "matrix")}

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        self.D, self.H, self.G, self.d, self.dv, self.taps, self.ra, self.rg = self._sizes(p)
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} query/key heads")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"a convolution of {self.taps} taps: this kernel takes 1 to 16")
        if self.d > 512:
            raise ValueError(f"key size {self.d}: the recurrence takes up to 512")
        self.eps = float(need(p, "norm_eps", "channel_delta"))
        pre = spec.prefix
        f32 = lambda n: weights[n].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.C = 2 * self.G * self.d + self.H * self.dv           # convolved columns: q, k, v
        self.proj = Linear.stacked([weights[f"{pre}.{n}"] for n in ("q", "k", "v", "b", "a1", "g1")], runtime)
        self.a2 = Linear(weights[f"{pre}.a2"], runtime)
        self.g2 = Linear(weights[f"{pre}.g2"], runtime)
        self.o = Linear(weights[f"{pre}.o"], runtime)
        # [taps, channels]: a tap's weights lie together
        self.conv_w = torch.cat([f32(f"{pre}.q.conv"), f32(f"{pre}.k.conv"), f32(f"{pre}.v.conv")]).t().contiguous()
        self.dt_bias, self.a_log, self.norm_w = f32(f"{pre}.dt_bias"), f32(f"{pre}.A_log"), f32(f"{pre}.norm")
        self.n_state = self.H * self.dv * self.d
        self.n_conv = (self.taps - 1) * self.C

    def cache_need(self):
        return None

    def state_shape(self):
        """One float32 row a sequence: the heads' states [H, dv, d], then the convolution's last
        inputs [taps - 1, C]."""
        return ((self.n_state + self.n_conv,), torch.float32)

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, entry, residual=None):
        store = entry.state()
        S = store[:, :self.n_state].unflatten(1, (self.H, self.dv, self.d))
        conv_state = store[:, self.n_state:].unflatten(1, (self.taps - 1, self.C)) if self.taps > 1 else None
        u = self.proj(y, split_ok=True)                     # float32 [q | k | v | b | a1 | g1], possibly partial sums
        x = K.conv_silu(u, 0, self.C, self.conv_w, None, conv_state, ctx.tok_seq, ctx.cu_q, ctx.seq_slot, ctx.B,
                        ctx.is_decode)
        dt = self.runtime.dtype
        a = self.a2(K.cols_cast(u, self.C + self.H, self.ra, dt), split_ok=True)
        g = self.g2(K.cols_cast(u, self.C + self.H + self.ra, self.rg, dt), split_ok=True)
        o = K.delta_rule(x, 0, self.G * self.d, 2 * self.G * self.d, u, self.C, a, self.dt_bias, self.a_log, S,
                         ctx.cu_q, ctx.seq_slot, ctx.B, self.H, self.G, self.d, self.dv)
        v = K.head_norm_gate(o, self.norm_w, self.eps, g, 0, self.H, dt)
        return self.o(v, split_ok=True, add_to=residual)

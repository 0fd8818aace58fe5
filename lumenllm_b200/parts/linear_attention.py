"""Linear attention with a fixed decay a head ("decay_linear_attention"): a recurrence over time
with a matrix state per head, in place of a softmax over cached keys.

In order, for H heads with keys of d and values of dv channels: q = act(y Wq^T), k = act(y Wk^T)
(H d wide), v = act(y Wv^T) (H dv wide), act = SiLU (`activation` "silu") or nothing ("none"); per
head S <- decay_h S + k v^T, o = S^T q (S is d x dv; o sees the token's own write; no other
scale); the heads' o side by side are divided by their root mean square over all H dv channels,
times the weight `.norm` (H dv values), times sigmoid(y Wg^T) when `output_gate`; out = that Wo^T.
`decay` is one number a head, from the configuration.

A sequence's state is S of every head (float32, kept [H, d, dv]); it starts at zero and is carried
from step to step, so a sequence may be fed in any portions. Activations, state, sums, norm and
gate are float32; the projections run in the run's type, and the ones that read y are one product.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import need, register_part
from .linear import Linear


@register_part("mixer", "decay_linear_attention")
class DecayLinearAttention:
    graph_safe = True

    @staticmethod
    def _sizes(p):
        return tuple(int(need(p, k, "decay_linear_attention")) for k in ("hidden_size", "num_heads", "head_dim", "value_dim"))

    @classmethod
    def tensors(cls, spec):
        D, H, d, dv = cls._sizes(spec.params)
        pre = spec.prefix
        t = {f"{pre}.q": ((H * d, D), "matrix"), f"{pre}.k": ((H * d, D), "matrix"), f"{pre}.v": ((H * dv, D), "matrix"),
             f"{pre}.norm": ((H * dv,), "norm"), f"{pre}.o": ((D, H * dv), "matrix")}
        if spec.params.get("output_gate", True):
            t[f"{pre}.g"] = ((H * dv, D), "matrix")
        return t

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        self.D, self.H, self.d, self.dv = self._sizes(p)
        if self.d > K.linear_attn_max_dim():
            raise ValueError(f"key size {self.d}: the recurrence takes up to {K.linear_attn_max_dim()}")
        decay = [float(x) for x in need(p, "decay", "decay_linear_attention")]
        if len(decay) != self.H:
            raise ValueError(f"{len(decay)} decays for {self.H} heads")
        act = p.get("activation", "silu")
        if act not in ("silu", "none"):
            raise ValueError(f"decay_linear_attention: activation {act!r} (known: 'silu', 'none')")
        self.silu = act == "silu"
        self.eps = float(need(p, "norm_eps", "decay_linear_attention"))
        self.gated = bool(p.get("output_gate", True))
        pre = spec.prefix
        f32 = lambda n: weights[n].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.decay = torch.tensor(decay, dtype=torch.float32, device=runtime.device)
        mats = [weights[f"{pre}.{n}"] for n in ("q", "k", "v") + (("g",) if self.gated else ())]
        # `external_projection`: whoever runs this part makes the product (stacked with others that read
        # the same rows) and hands its result, and the column where this part's begin, to forward
        self.input_mats = mats if p.get("external_projection", False) else None
        self.proj = None if self.input_mats is not None else Linear.stacked(mats, runtime)
        self.norm_w = f32(f"{pre}.norm")
        self.o = Linear(weights[f"{pre}.o"], runtime)
        self.k_col, self.v_col = self.H * self.d, 2 * self.H * self.d
        self.g_col = self.v_col + self.H * self.dv

    def cache_need(self):
        return None

    def state_shape(self):
        """The heads' states [H, d, dv], float32."""
        return ((self.H, self.d, self.dv), torch.float32)

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    projects_input = True         # may be built with `external_projection` and fed `projected`

    def forward(self, y, ctx, entry, residual=None, projected=None, col0=0):
        S = entry.state()
        # float32 [... | q | k | v | g | ...] from column col0, possibly partial sums
        u = projected if projected is not None else self.proj(y, split_ok=True)
        o = K.linear_attn(u, col0, col0 + self.k_col, col0 + self.v_col, self.silu, self.decay, S, ctx.cu_q, ctx.seq_slot,
                          ctx.B, self.H, self.d, self.dv)
        dt = self.runtime.dtype
        v = K.cols_rmsnorm(o, 0, self.H * self.dv, self.norm_w, self.eps, dt, gate=u if self.gated else None,
                           gate_col=col0 + self.g_col)
        return self.o(v, split_ok=True, add_to=residual)

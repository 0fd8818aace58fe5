"""Position encodings that a mixer applies to its queries and keys.

"rotary": half-split pairs (i, i + rot/2) rotated by angle = pos * inv_freq_i with
inv_freq_i = 1 / theta^(2i/rot), computed in float32
(norm_rope_kv.cu:437-447,465-492; crates/aegisllm-cpu/src/cpu/rope.rs:34-84).
`rotary_dim` < head_dim rotates only the first dims. A position part offers `rotary_dim` and `angles(ctx)`, the (cos, sin) of every
token of the step as float32 [N, rotary_dim/2, 2]; an encoding with other
frequencies or other positions is another way to fill that table; "none"
rotates nothing.

With `scaling` = {factor, original, fast, slow} the frequencies are stretched for contexts longer
than `original` positions: pair i would make original * f_i / (2 pi) turns over the original
context; pairs that make more than `fast` turns keep f_i, pairs that make fewer than `slow` get
f_i / factor, and between them a ramp that is linear in the pair's index mixes the two:
where(t) = dims * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(where(fast)), 0),
hi = min(ceil(where(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
f_i' = f_i / factor * ramp_i + f_i * (1 - ramp_i); cos and sin are both multiplied by
0.1 ln(factor) + 1 (so that scores grow by its square). Taken in 64-bit, rounded once.
"""
from __future__ import annotations

import math

import torch

from .base import need, register_part


@register_part("position", "rotary")
class Rotary:
    @classmethod
    def tensors(cls, spec):
        return {}

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.head_dim = int(need(p, "head_dim", "rotary"))
        self.rotary_dim = int(p.get("rotary_dim", self.head_dim))
        self.theta = float(need(p, "theta", "rotary"))
        # `wide_frequencies`: theta^(-2i/rot) taken in 64-bit and rounded once to float32,
        # instead of the float32 power and reciprocal above
        self.wide = bool(p.get("wide_frequencies", False))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim")
        sc = p.get("scaling")
        self.scaling = None if not sc else tuple(float(need(sc, k, "rotary scaling"))
                                                 for k in ("factor", "original", "fast", "slow"))
        self.magnitude = 1.0 if self.scaling is None else 0.1 * math.log(self.scaling[0]) + 1.0
        self.inv_freq = self.frequencies().to(runtime.device).contiguous()

    def angles(self, ctx):
        """(cos, sin) for every token of the step, float32 [N, rot/2, 2]; made once per step
        and shared by all layers whose encoding has the same frequencies."""
        shared = ctx.extras.setdefault("per_step", {})   # emptied when the step's forward begins
        key = ("rope", self.rotary_dim, self.theta, self.wide, self.scaling)
        cs = shared.get(key)
        if cs is None:
            from ..ops import kernels as K
            cs = shared[key] = K.rope_table(ctx.rope_pos, self.inv_freq, self.magnitude)
        return cs

    def frequencies(self) -> torch.Tensor:
        if self.scaling is not None:
            factor, original, fast, slow = self.scaling
            dims = self.rotary_dim
            i = torch.arange(dims // 2, dtype=torch.float64)
            f = torch.tensor(self.theta, dtype=torch.float64) ** (-2.0 * i / dims)
            where = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
            lo, hi = max(math.floor(where(fast)), 0), min(math.ceil(where(slow)), dims - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            return (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32)
        if self.wide:
            i2 = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
            return (torch.tensor(self.theta, dtype=torch.float64) ** (-i2 / self.rotary_dim)).to(torch.float32)
        i2 = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        return 1.0 / (torch.tensor(self.theta, dtype=torch.float32) ** (i2 / self.rotary_dim))


@register_part("position", "none")
class NoPosition:
    @classmethod
    def tensors(cls, spec):
        return {}

    def __init__(self, spec, weights, runtime):
        self.rotary_dim = 0
        self.inv_freq = None

    def angles(self, ctx):
        return None

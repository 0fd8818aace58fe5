"""RMSNorm, with the residual add that precedes it fused in.

y_i = x_i * 1/sqrt(mean(x^2) + eps) * w_i, everything in float32
(crates/aegisllm-cuda/src/cuda/kernels/blackwell/norm_rope_kv.cu:36-62;
crates/aegisllm-cpu/src/cpu/math.rs:4-8). `weight_offset` 1 gives the (1 + w)
form that the reference folds in for other families (executor/loader.rs:189-194);
it is a parameter, 0 for Qwen3 dense. With `scalar` the stored weight is ONE number
(a tensor without dimensions) that multiplies every coordinate.

"dynamic_tanh": y_i = tanh(alpha * x_i) * w_i + b_i with one learned slope `alpha` for all
coordinates (`<name>.alpha`, a tensor without dimensions) and a bias `<name>.b` beside the weight
`<name>`: no mean and no variance are taken, so a row needs no reduction. Float32.

A pending update may come as a ScaledUpdate: groups of partial sums, each with a factor of its own
(a residual multiplier, two mixers side by side with different weights). The Dynamic Tanh kernel
adds them while it reads the stream; the RMS norm has them added by a kernel before its own.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import need, register_part, tensor_name


class NormedUpdate:
    """An update of the residual stream that is RMS-normed BEFORE it is added (a norm at a
    sublayer's output): h += rmsnorm(sum of `delta`'s partial sums + `bias`) * `weight`. A block
    hands it on as `pending` like a plain stack of partial sums, and the norm that follows does
    the whole chain, norm of the update, add, its own norm, in one kernel."""
    __slots__ = ("delta", "weight", "eps", "bias")

    def __init__(self, delta, weight, eps, bias=None):
        self.delta, self.weight, self.eps, self.bias = delta, weight, float(eps), bias


class ScaledUpdate:
    """An update of the residual stream in groups, h += sum_g scale_g * (sum of the partial sums of
    delta_g): `groups` is a list of (delta float32 [N, H] or [S, N, H], scale)."""
    __slots__ = ("groups",)

    def __init__(self, groups):
        self.groups = [(d, float(s)) for d, s in groups]

    @classmethod
    def of(cls, update, scale: float):
        """`update` (None, a tensor of partial sums, a list of such tensors, or a ScaledUpdate) times `scale`."""
        if update is None:
            return None
        if isinstance(update, ScaledUpdate):
            return cls([(d, s * scale) for d, s in update.groups])
        if isinstance(update, (list, tuple)):
            return cls([(d, scale) for d in update if d is not None])
        if isinstance(update, NormedUpdate):
            raise TypeError("an update that is normed before it is added cannot also be scaled")
        return cls([(update, scale)])


def add_pending(h, delta):
    """Adds a ScaledUpdate into the stream in place and returns what is left to add (None); any other
    kind of pending update is handed back untouched."""
    if isinstance(delta, ScaledUpdate):
        K.add_scaled_dyt(h, delta.groups, None, None, None, torch.float32)
        return None
    return delta


@register_part("norm", "dynamic_tanh")
class DynamicTanh:
    @classmethod
    def tensors(cls, spec):
        size = need(spec.params, "size", "dynamic_tanh")
        name = tensor_name(spec)
        return {name: ((size,), "norm"), f"{name}.b": ((size,), "matrix"), f"{name}.alpha": ((), "norm")}

    def __init__(self, spec, weights, runtime):
        self.size = int(need(spec.params, "size", "dynamic_tanh"))
        name = tensor_name(spec)
        f32 = lambda n: weights[n].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.weight, self.bias = f32(name), f32(f"{name}.b")
        self.alpha = f32(f"{name}.alpha").reshape(1)

    def forward(self, h, delta, out_dtype, rows=None, write_h=True):
        if isinstance(delta, NormedUpdate):
            raise TypeError("dynamic_tanh: an update that is normed before it is added is not taken here")
        groups = delta.groups if isinstance(delta, ScaledUpdate) else ([] if delta is None else [(delta, 1.0)])
        return K.add_scaled_dyt(h, groups, self.weight, self.bias, self.alpha, out_dtype, rows=rows, write_h=write_h)


@register_part("norm", "rmsnorm")
class RMSNorm:
    @classmethod
    def tensors(cls, spec):
        size = need(spec.params, "size", "rmsnorm")
        return {tensor_name(spec): (() if spec.params.get("scalar") else (size,), "norm")}

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.size = int(need(p, "size", "rmsnorm"))
        self.eps = float(need(p, "eps", "rmsnorm"))
        w = weights[tensor_name(spec)].to(device=runtime.device, dtype=torch.float32)
        if p.get("scalar"):
            w = w.reshape(1).expand(self.size)        # the kernels read one weight a coordinate
        off = float(p.get("weight_offset", 0.0))
        self.weight = (w + off).contiguous() if off else w.contiguous()

    def forward(self, h, delta, out_dtype, rows=None, write_h=True):
        delta = add_pending(h, delta)
        if isinstance(delta, NormedUpdate):
            return K.postnorm_add_rmsnorm(h, delta.delta, delta.bias, delta.weight, delta.eps, self.weight,
                                          self.eps, out_dtype, rows=rows, write_h=write_h)
        return K.add_rmsnorm(h, delta, self.weight, self.eps, out_dtype, rows=rows, write_h=write_h)

    def forward_conv(self, h, delta, conv, state, ctx, out_dtype):
        """The norm and, behind it, an input convolution (parts/conv.py) of the normed rows. A
        step of one token a sequence whose pending update is a NormedUpdate (or nothing) is one
        kernel; everything else is the norm, in float32, and then the convolution."""
        if ctx.is_decode and (delta is None or isinstance(delta, NormedUpdate)):
            d = delta
            return K.postnorm_add_rmsnorm(h, None if d is None else d.delta, None if d is None else d.bias,
                                          None if d is None else d.weight, 0.0 if d is None else d.eps,
                                          self.weight, self.eps, out_dtype,
                                          conv=(conv.weight, state, ctx.seq_slot))
        return conv.forward(self.forward(h, delta, torch.float32), state, ctx, out_dtype)

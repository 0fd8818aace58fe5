"""Arrangements of a mixer and a feed-forward around the residual stream.

"pre_norm": r = h + mixer(norm_mixer(h)); h' = r + ffn(norm_ffn(r))
(crates/aegisllm-cuda/src/executor/prefill/layer.rs:476-482,1090,1381-1439).
The adds are not done here: a block hands its last update on as `pending`, and
the next norm (the next block's, or the model's final one) adds it while it
reads the stream anyway. A layer may lack the feed-forward (and its norm); with
`extras["token_input"]` a part of that category (parts/token_input.py) runs after the
sublayers and adds an input that comes from the tokens themselves. With the layer's parameter
`residual_scale` m != 1 every update counts m times, r = h + m mixer(..), h' = r + m ffn(..): the
updates then go on as a ScaledUpdate (parts/norm.py), whose factors the next norm applies while it
adds, and no part adds into the stream by itself.

"parallel": h' = h + (mixer(norm(h)) + ffn(norm(h))): ONE norm, whose output both sublayers
read; a layer may lack the feed-forward. The two updates go on side by side as one stack of
partial sums.

"sandwich_conv": r = h + norm_b(mixer(conv(norm_a(h)))); h' = r + norm_d(ffn(conv(norm_c(r)))):
a norm before and after each sublayer, and a short causal convolution over time of what each
sublayer reads (parts/conv.py), whose last inputs are the block's per-sequence state. The second
half is left out for a layer without a feed-forward. A sublayer's update is handed on as a
NormedUpdate, so that its norm, the add and the next sublayer's norm are one kernel.
"""
from __future__ import annotations

import torch

from .base import build_part, part_tensors, register_part
from .norm import NormedUpdate, ScaledUpdate


@register_part("block", "pre_norm")
class PreNormBlock:
    @classmethod
    def tensors(cls, layer_spec):
        t = {}
        t.update(part_tensors("norm", layer_spec.norms["mixer"]))
        t.update(part_tensors("mixer", layer_spec.mixer))
        if layer_spec.ffn is not None:
            t.update(part_tensors("norm", layer_spec.norms["ffn"]))
            t.update(part_tensors("ffn", layer_spec.ffn))
        if "token_input" in layer_spec.extras:
            t.update(part_tensors("token_input", layer_spec.extras["token_input"]))
        return t

    def __init__(self, layer_spec, weights, runtime):
        self.runtime = runtime
        self.norm_mixer = build_part("norm", layer_spec.norms["mixer"], weights, runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, weights, runtime)
        self.norm_ffn = self.ffn = self.token_input = None
        if layer_spec.ffn is not None:
            self.norm_ffn = build_part("norm", layer_spec.norms["ffn"], weights, runtime)
            self.ffn = build_part("ffn", layer_spec.ffn, weights, runtime)
        if "token_input" in layer_spec.extras:
            self.token_input = build_part("token_input", layer_spec.extras["token_input"], weights, runtime)
        self.residual_scale = float(layer_spec.params.get("residual_scale", 1.0))

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in (self.mixer, self.ffn, self.token_input) if p is not None)

    def forward(self, h, pending, ctx, entry):
        # A part that says `adds_residual` is offered the stream itself: it may add its update
        # there (a prompt-sized product does so in its epilogue) and return None, or return the
        # update as any part does. Either way the next norm sees the stream plus what is pending.
        y = self.norm_mixer.forward(h, pending, self.runtime.dtype)
        scaled = self.residual_scale != 1.0
        if getattr(self.mixer, "adds_residual", False) and not scaled:
            a = self.mixer.forward(y, ctx, entry, residual=h)
        else:
            a = self.mixer.forward(y, ctx, entry)
        if scaled or isinstance(a, (list, tuple)):
            a = ScaledUpdate.of(a, self.residual_scale)
        m = a
        if self.ffn is not None:
            y2 = self.norm_ffn.forward(h, a, self.runtime.dtype)
            if getattr(self.ffn, "adds_residual", False) and not scaled:
                m = self.ffn.forward(y2, ctx, residual=h)
            else:
                m = self.ffn.forward(y2, ctx)
            if scaled or isinstance(m, (list, tuple)):
                m = ScaledUpdate.of(m, self.residual_scale)
        if self.token_input is not None:
            return self.token_input.forward(h, m, ctx)
        return h, m


@register_part("block", "sandwich_conv")
class SandwichConvBlock:
    @classmethod
    def tensors(cls, layer_spec):
        t = {}
        for name in ("mixer", "mixer_out") + (("ffn", "ffn_out") if layer_spec.ffn is not None else ()):
            t.update(part_tensors("norm", layer_spec.norms[name]))
        t.update(part_tensors("input_conv", layer_spec.extras["mixer_conv"]))
        t.update(part_tensors("mixer", layer_spec.mixer))
        if layer_spec.ffn is not None:
            t.update(part_tensors("input_conv", layer_spec.extras["ffn_conv"]))
            t.update(part_tensors("ffn", layer_spec.ffn))
        return t

    def __init__(self, layer_spec, weights, runtime):
        self.runtime = runtime
        norm = lambda name: build_part("norm", layer_spec.norms[name], weights, runtime)
        self.norm_mixer, self.norm_mixer_out = norm("mixer"), norm("mixer_out")
        self.conv_mixer = build_part("input_conv", layer_spec.extras["mixer_conv"], weights, runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, weights, runtime)
        self.ffn = None
        if layer_spec.ffn is not None:
            self.norm_ffn, self.norm_ffn_out = norm("ffn"), norm("ffn_out")
            self.conv_ffn = build_part("input_conv", layer_spec.extras["ffn_conv"], weights, runtime)
            self.ffn = build_part("ffn", layer_spec.ffn, weights, runtime)
        self.convs = [self.conv_mixer] + ([self.conv_ffn] if self.ffn is not None else [])
        self.width = self.norm_mixer.size

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in [self.mixer] + ([self.ffn] if self.ffn else []))

    def state_shape(self):
        """The convolutions' last inputs: one [taps - 1, width] piece a sublayer, float32."""
        rows = sum(c.state_rows() for c in self.convs)
        return ((rows, self.width), torch.float32) if rows else None

    def forward(self, h, pending, ctx, entry):
        state = entry.state("block")
        r1 = self.conv_mixer.state_rows()
        x = self.norm_mixer.forward_conv(h, pending, self.conv_mixer, None if state is None or not r1 else state[:, :r1],
                                         ctx, self.runtime.dtype)
        a = self.mixer.forward(x, ctx, entry, bias_downstream=True)
        update = NormedUpdate(a, self.norm_mixer_out.weight, self.norm_mixer_out.eps,
                              getattr(self.mixer, "update_bias", None))
        if self.ffn is None:
            return h, update
        x = self.norm_ffn.forward_conv(h, update, self.conv_ffn,
                                       None if state is None or not self.conv_ffn.state_rows() else state[:, r1:],
                                       ctx, self.runtime.dtype)
        m = self.ffn.forward(x, ctx)
        return h, NormedUpdate(m, self.norm_ffn_out.weight, self.norm_ffn_out.eps)


@register_part("block", "parallel")
class ParallelBlock:
    @classmethod
    def tensors(cls, layer_spec):
        t = {}
        t.update(part_tensors("norm", layer_spec.norms["input"]))
        t.update(part_tensors("mixer", layer_spec.mixer))
        if layer_spec.ffn is not None:
            t.update(part_tensors("ffn", layer_spec.ffn))
        return t

    def __init__(self, layer_spec, weights, runtime):
        self.runtime = runtime
        self.norm = build_part("norm", layer_spec.norms["input"], weights, runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, weights, runtime)
        self.ffn = build_part("ffn", layer_spec.ffn, weights, runtime) if layer_spec.ffn is not None else None

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in [self.mixer] + ([self.ffn] if self.ffn else []))

    def forward(self, h, pending, ctx, entry):
        # Both sublayers read y, which is made before either of them touches the stream: a part that
        # says `adds_residual` is offered the stream and may add its update there in place (a
        # prompt-sized product does so in its epilogue) and return None.
        y = self.norm.forward(h, pending, self.runtime.dtype)
        if getattr(self.mixer, "adds_residual", False):
            a = self.mixer.forward(y, ctx, entry, residual=h)
        else:
            a = self.mixer.forward(y, ctx, entry)
        m = None
        if self.ffn is not None:
            if getattr(self.ffn, "adds_residual", False):
                m = self.ffn.forward(y, ctx, residual=h)
            else:
                m = self.ffn.forward(y, ctx)
        left = [d if d.dim() == 3 else d.unsqueeze(0) for d in (a, m) if d is not None]
        if not left:
            return h, None
        return h, left[0] if len(left) == 1 else torch.cat(left, dim=0)

"""Several mixers side by side ("side_by_side"): all read the same normed rows, and the layer's
update is the weighted sum of theirs, sum_i scale_i * mixer_i(y).

Parameters: `parts`, a list of {"mixer": PartSpec, "scale": number}. Each child is a mixer part like
any other, with tensors under its own prefix. At most one child may keep a key/value cache and at
most one a per-sequence state: the layer's run has one cache entry and one state row, and the
child that declared the need is the one that finds it in the EntryView. The children's updates are
not added up here: they go on as the groups of a ScaledUpdate, each with its factor, for the next
norm to add while it reads the stream.
"""
from __future__ import annotations

from .base import build_part, need, part_tensors, register_part
from .norm import ScaledUpdate


@register_part("mixer", "side_by_side")
class SideBySide:
    @classmethod
    def tensors(cls, spec):
        t = {}
        for child in need(spec.params, "parts", "side_by_side"):
            t.update(part_tensors("mixer", child["mixer"]))
        return t

    def __init__(self, spec, weights, runtime):
        children = need(spec.params, "parts", "side_by_side")
        if not children:
            raise ValueError("side_by_side: at least one mixer")
        self.mixers = [build_part("mixer", c["mixer"], weights, runtime) for c in children]
        self.scales = [float(c.get("scale", 1.0)) for c in children]
        if sum(m.cache_need() is not None for m in self.mixers) > 1:
            raise ValueError("side_by_side: at most one of the mixers may keep a key/value cache")
        if sum(m.state_shape() is not None for m in self.mixers) > 1:
            raise ValueError("side_by_side: at most one of the mixers may keep a per-sequence state")

    @property
    def graph_safe(self):
        return all(getattr(m, "graph_safe", False) for m in self.mixers)

    def cache_need(self):
        return next((n for n in (m.cache_need() for m in self.mixers) if n is not None), None)

    def state_shape(self):
        return next((s for s in (m.state_shape() for m in self.mixers) if s is not None), None)

    def forward(self, y, ctx, entry):
        return ScaledUpdate([(m.forward(y, ctx, entry), s) for m, s in zip(self.mixers, self.scales)])

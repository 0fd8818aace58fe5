"""Several mixers side by side ("side_by_side"): all read the same normed rows, and the layer's
update is the weighted sum of theirs, sum_i scale_i * mixer_i(y).

Parameters: `parts`, a list of {"mixer": PartSpec, "scale": number}. Each child is a mixer part like
any other, with tensors under its own prefix. At most one child may keep a key/value cache and at
most one a per-sequence state: the layer's run has one cache entry and one state row, and the
child that declared the need is the one that finds it in the EntryView. The children's updates are
not added up here: they go on as the groups of a ScaledUpdate, each with its factor, for the next
norm to add while it reads the stream.

Where every child says `projects_input` (its first step is a product of the rows with matrices of
its own) the children are built with `external_projection`, their matrices are stacked row-wise,
and ONE product serves them all; a child is handed the product and the column where its own
columns begin. A child whose kernels read from column 0 (`needs_first_columns`) comes first in the
stack; two such children are not fused.
"""
from __future__ import annotations

from ..config.spec import PartSpec
from .base import build_part, need, part_class, part_tensors, register_part
from .linear import Linear
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
        kinds = [part_class("mixer", c["mixer"].kind) for c in children]
        fused = (len(children) > 1 and all(getattr(k, "projects_input", False) for k in kinds)
                 and sum(bool(getattr(k, "needs_first_columns", False)) for k in kinds) <= 1)
        specs = [c["mixer"] if not fused else PartSpec(c["mixer"].kind, dict(c["mixer"].params, external_projection=True),
                                                        c["mixer"].prefix) for c in children]
        self.mixers = [build_part("mixer", sp, weights, runtime) for sp in specs]
        self.scales = [float(c.get("scale", 1.0)) for c in children]
        self.proj, self.col0 = None, [0] * len(children)
        if fused:
            order = sorted(range(len(children)), key=lambda i: not getattr(kinds[i], "needs_first_columns", False))
            mats, at = [], 0
            for i in order:
                self.col0[i] = at
                mats += self.mixers[i].input_mats
                at += sum(m.shape[0] for m in self.mixers[i].input_mats)
                self.mixers[i].input_mats = True        # the stack holds them now
            self.proj = Linear.stacked(mats, runtime)
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
        if self.proj is None:
            return ScaledUpdate([(m.forward(y, ctx, entry), s) for m, s in zip(self.mixers, self.scales)])
        u = self.proj(y, split_ok=True)            # the children's columns side by side, possibly partial sums
        return ScaledUpdate([(m.forward(y, ctx, entry, projected=u, col0=c), s)
                             for m, c, s in zip(self.mixers, self.col0, self.scales)])

"""A per-layer input from the token itself ("gated_token_table"), added to the stream after a
layer's sublayers: e = table[token][column : column + dim] (a table of small vectors, one run of
`dim` columns a layer); g = gelu_tanh(x Wgate^T) * e with x the residual stream itself (not
normed); z = g Wproj^T; x <- x + z / sqrt(mean(z^2) + eps) * w. Tensors: the shared table
(`table`, [vocab, table_width]), `<prefix>.gate` [dim, hidden], `<prefix>.proj` [hidden, dim],
`<prefix>.norm` [hidden] (a plain weight).

`forward(h, pending, ctx)` adds what is pending into the stream (the gate reads the stream as it
stands after the sublayers) and hands on a NormedUpdate, so that the norm of z, the add and the
next layer's input norm are one kernel.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import need, register_part
from .linear import Linear
from .norm import NormedUpdate


@register_part("token_input", "gated_token_table")
class GatedTokenTable:
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        p = spec.params
        D, V, dim, W = (int(need(p, k, "gated_token_table")) for k in ("hidden_size", "vocab_size", "dim", "table_width"))
        return {need(p, "table", "gated_token_table"): ((V, W), "matrix"),
                f"{spec.prefix}.gate": ((dim, D), "matrix"), f"{spec.prefix}.proj": ((D, dim), "matrix"),
                f"{spec.prefix}.norm": ((D,), "norm")}

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        self.dim, self.column = int(p["dim"]), int(need(p, "column", "gated_token_table"))
        self.eps = float(need(p, "norm_eps", "gated_token_table"))
        table = weights[p["table"]]
        if runtime.is_f32 and table.dtype != torch.float32:
            # one widened copy for all layers (the loader's dictionary is shared)
            table = weights[p["table"]] = table.to(torch.float32)
        self.table = table.contiguous()
        if self.column + self.dim > self.table.shape[1]:
            raise ValueError(f"columns {self.column}..{self.column + self.dim} are beyond the table's {self.table.shape[1]}")
        self.gate = Linear(weights[f"{spec.prefix}.gate"], runtime)
        self.proj = Linear(weights[f"{spec.prefix}.proj"], runtime)
        self.weight = weights[f"{spec.prefix}.norm"].to(device=runtime.device, dtype=torch.float32).contiguous()

    def forward(self, h, pending, ctx):
        if isinstance(pending, NormedUpdate):
            raise ValueError("gated_token_table: the update before it must be a plain one")
        x = K.add_cast(h, pending, self.runtime.dtype)          # the stream after the sublayers, and its copy
        g = K.token_gate(self.gate(x, split_ok=True), ctx.tokens, self.table, self.column, self.runtime.dtype)
        return h, NormedUpdate(self.proj(g, split_ok=True), self.weight, self.eps)

"""Token embedding and output head.

Embedding: h[t] = float32(E[token[t]]) (norm_rope_kv.cu:19-34), optionally times a
scale (none for Qwen: crates/aegisllm-base/src/model/mod.rs:128-130).
Head: logits = y W^T in float32, with W the embedding table when the head is tied
(crates/aegisllm-cuda/src/executor/full.rs:171-181; executor/forward.rs:288-297).
"""
from __future__ import annotations

from ..ops import kernels as K
from .base import need, register_part, tensor_name
from .linear import Linear, tiled_form


@register_part("embedding", "token_embedding")
class TokenEmbedding:
    """`scale` multiplies the token's vector; `position_tensor` names a learned table
    [max_positions, hidden] whose row at the token's position is added (not scaled)."""

    @classmethod
    def tensors(cls, spec):
        H = int(need(spec.params, "hidden_size", "embedding"))
        t = {tensor_name(spec): ((int(need(spec.params, "vocab_size", "embedding")), H), "matrix")}
        if spec.params.get("position_tensor"):
            t[spec.params["position_tensor"]] = ((int(need(spec.params, "max_positions", "embedding")), H), "matrix")
        return t

    def __init__(self, spec, weights, runtime):
        self.table = weights[tensor_name(spec)].contiguous()
        pos = spec.params.get("position_tensor")
        self.positions = weights[pos].contiguous() if pos else None
        self.vocab_size = self.table.shape[0]
        # in a bfloat16 run the table is kept in the form an output head would read it in, so
        # that a head tied to it shares the one copy
        if not runtime.is_f32 and K.can_tile(self.table):
            self.table = tiled_form(self.table)
        self.scale = spec.params.get("scale")

    def forward(self, tokens, ctx=None):
        if self.positions is not None:
            if ctx is None:
                raise ValueError("an embedding with learned positions needs the step's positions")
            return K.embed_pos(tokens, self.table, 1.0 if self.scale is None else float(self.scale),
                               ctx.rope_pos, self.positions)
        if self.scale is not None:
            return K.embed_pos(tokens, self.table, float(self.scale), None, None)
        return K.embed(tokens, self.table)


@register_part("head", "linear_head")
class LinearHead:
    """`tied_to` names the embedding table when config.json ties the head to it. Which matrix
    is used follows the reference, by presence (executor/full.rs:171-181): the head's own
    tensor when the file stores one, else the table named by `tied_to` or `falls_back_to`.
    So a tied checkpoint that also stores a head, and an untied one that stores none, both
    load; the loader reports the second case in its `stood_in`. With `logit_scale` s the logits
    are multiplied by s, and with `softcap` c > 0 then bent to c tanh(logit / c), in float32."""

    @classmethod
    def tensors(cls, spec):
        if not spec.params.get("own_tensor", True):        # the head IS the tied table: no tensor of its own
            return {}
        shape = (int(need(spec.params, "vocab_size", "head")), int(need(spec.params, "hidden_size", "head")))
        return {tensor_name(spec): (shape, "optional" if spec.params.get("tied_to") else "matrix")}

    @classmethod
    def fallbacks(cls, spec):
        other = spec.params.get("falls_back_to")
        return {tensor_name(spec): other} if other and not spec.params.get("tied_to") else {}

    def __init__(self, spec, weights, runtime):
        own = tensor_name(spec)
        name = own if spec.params.get("own_tensor", True) and own in weights else spec.params.get("tied_to")
        if name is None or name not in weights:
            raise KeyError(f"the output head needs '{own}'")
        self.proj = Linear(weights[name], runtime)
        self.logit_scale = float(spec.params.get("logit_scale", 1.0))
        self.softcap = float(spec.params.get("softcap", 0.0) or 0.0)

    def forward(self, y):
        logits = self.proj(y)
        if self.logit_scale != 1.0 or self.softcap > 0.0:
            logits = K.scale_softcap(logits.contiguous(), self.logit_scale, self.softcap)
        return logits

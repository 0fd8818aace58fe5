"""Feed-forward parts.

"swiglu": g = y Wg^T, u = y Wu^T, z = g / (1 + exp(-g)) * u, out = z Wd^T
(crates/aegisllm-cuda/src/executor/mlp.rs:271-356; norm_rope_kv.cu:314-325).
Gate and up weights are stacked so that both cost one product. For bfloat16 their rows
are interleaved (gate_0, up_0, gate_1, up_1, ...): then a tile of the product holds both
halves of each pair, and the tensor-core kernel applies SiLU(gate) * up in its epilogue
and writes bfloat16 directly. With few rows the product returns float32 (partial sums)
and a small kernel adds them and applies the activation.

"polynorm_mlp": u = y Wu^T, z = a N(u) + b N(u^2) + c N(u^3) + e, out = z Wd^T, where powers are
taken element by element, N divides a token's vector by its root mean square
(sqrt(mean(v^2) + eps)), and (a, b, c, e) are the four values of the tensor `<prefix>.act`.
The activation is one float32 kernel over the product's partial sums.

"xielu_mlp": u = y Wu^T, out = xIELU(u) Wd^T with xIELU(z) = softplus(p) z^2 + z/2 for z > 0 and
(1/2 + softplus(q)) (e^z - 1 - z) + z/2 for z <= 0, (p, q) the two values of `<prefix>.act`.

"gelu_mlp": u = y Wu^T, out = gelu_tanh(u) Wd^T with gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi)
(z + 0.044715 z^3))); tensors `<prefix>.up`, `<prefix>.down`.

"relu2_mlp": u = y Wu^T, out = max(u, 0)^2 Wd^T; tensors `<prefix>.up`, `<prefix>.down`.

"clamped_glu": g = min(y Wg^T, limit), v = clamp(y Wu^T, -limit, limit), z = g sigmoid(alpha g) (v + 1),
out = z Wd^T; tensors `<prefix>.gate`, `.up`, `.down`. With `token_gate` the output is multiplied by
sigmoid(y Wsg^T), one number a token (`<prefix>.sg` [1, D]); the factor is applied to z, in float32,
before z is rounded for the down product (the product is linear in z).

"routed_experts": many small SwiGLU experts (`<prefix>.e<i>.gate/up/down`, no biases) of which
each token uses `top`. The router's logits y Wr^T are float32; s = softmax over ALL router
outputs; the `top` outputs with the largest s + correction are chosen, and each counts with its
s (without the correction) times `scale`, not renormalised. The last `identity` router outputs
are experts without tensors that hand their input on. A shared expert (`<prefix>.shared`), when
the model has one, runs for every token and is added. The update goes on as partial sums: one
for each of a token's choices, then the shared expert's. Options: `router` "sigmoid" scores every
router output by itself, s = sigmoid(logit), instead of the softmax; `correction` False: no
`.correction` tensor; `weight_on` "input": a choice's weight multiplies the expert's input, out =
sum expert(w y), which the gated product does by multiplying its two sums by w before the
activation; `expert` {"kind": "clamped_glu", "limit", "alpha"}: the experts are clamped gated
units as above instead of SwiGLU; `shared` {"size", "kind", "limit", "alpha", "token_gate"}: the
shared expert's own form; `update_in_pieces`: the routed experts' and the shared expert's updates are
handed on as a list of two stacks instead of being copied into one (for arrangements that add a
list's pieces, parts/block.py "pre_norm").
"""
from __future__ import annotations

import torch

from ..ops import gemm as G
from ..ops import kernels as K
from .base import build_part, need, part_class, register_part
from .linear import Linear


@register_part("ffn", "swiglu")
class SwiGLU:
    graph_safe = True

    @staticmethod
    def names(spec):
        """The three tensors' names; `tensor_names` = {"gate": suffix, "up": ..., "down": ...}
        replaces the usual `.gate_proj.weight` and so on."""
        sfx = spec.params.get("tensor_names") or {"gate": ".gate_proj.weight", "up": ".up_proj.weight",
                                                  "down": ".down_proj.weight"}
        return tuple(spec.prefix + sfx[k] for k in ("gate", "up", "down"))

    @classmethod
    def tensors(cls, spec):
        H = int(need(spec.params, "hidden_size", "swiglu"))
        I = int(need(spec.params, "intermediate_size", "swiglu"))
        gate, up, down = cls.names(spec)
        return {gate: ((I, H), "matrix"), up: ((I, H), "matrix"), down: ((H, I), "matrix")}

    def __init__(self, spec, weights, runtime):
        self.runtime = runtime
        gate, up, down = self.names(spec)
        g, u = weights[gate], weights[up]
        self.down = Linear(weights[down], runtime)
        self.interleaved = (not runtime.is_f32 and g.dtype == torch.bfloat16
                            and u.dtype == torch.bfloat16)
        if self.interleaved:
            I, H = g.shape
            self.gate_up = Linear(torch.stack([g, u], dim=1).reshape(2 * I, H), runtime)
        else:
            self.gate_up = Linear.stacked([g, u], runtime)

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, residual=None):
        if self.interleaved and not self.down.f32:
            z = G.gemm_gate_up_silu(y, self.gate_up.weight)         # many rows: one kernel
            if z is not None:
                return self.down(z, split_ok=True, add_to=residual)
        gu = self.gate_up(y, split_ok=True)        # float32 [N, 2I], possibly S partials
        z = K.silu_mul(gu, self.runtime.dtype, interleaved=self.interleaved)
        return self.down(z, split_ok=True)


@register_part("ffn", "polynorm_mlp")
class PolyNormMLP:
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        H = int(need(spec.params, "hidden_size", "polynorm_mlp"))
        I = int(need(spec.params, "intermediate_size", "polynorm_mlp"))
        return {f"{spec.prefix}.up": ((I, H), "matrix"), f"{spec.prefix}.down": ((H, I), "matrix"),
                f"{spec.prefix}.act": ((4,), "norm")}

    def __init__(self, spec, weights, runtime):
        self.runtime = runtime
        self.eps = float(need(spec.params, "eps", "polynorm_mlp"))
        self.up = Linear(weights[f"{spec.prefix}.up"], runtime)
        self.down = Linear(weights[f"{spec.prefix}.down"], runtime)
        self.act = weights[f"{spec.prefix}.act"].to(device=runtime.device, dtype=torch.float32).contiguous()

    def forward(self, y, ctx):
        u = self.up(y, split_ok=True)                       # float32 [N, I], possibly S partials
        z = K.polynorm(u, self.act, self.eps, self.runtime.dtype)
        return self.down(z, split_ok=True)


@register_part("ffn", "gelu_mlp")
class GeluMLP:
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        H = int(need(spec.params, "hidden_size", "gelu_mlp"))
        I = int(need(spec.params, "intermediate_size", "gelu_mlp"))
        return {f"{spec.prefix}.up": ((I, H), "matrix"), f"{spec.prefix}.down": ((H, I), "matrix")}

    def __init__(self, spec, weights, runtime):
        self.runtime = runtime
        self.up = Linear(weights[f"{spec.prefix}.up"], runtime)
        self.down = Linear(weights[f"{spec.prefix}.down"], runtime)

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, residual=None):
        z = K.gelu_tanh(self.up(y, split_ok=True), self.runtime.dtype)      # adds the partial sums, float32
        return self.down(z, split_ok=True, add_to=residual)


@register_part("ffn", "relu2_mlp")
class SquaredReluMLP:
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        H = int(need(spec.params, "hidden_size", "relu2_mlp"))
        I = int(need(spec.params, "intermediate_size", "relu2_mlp"))
        return {f"{spec.prefix}.up": ((I, H), "matrix"), f"{spec.prefix}.down": ((H, I), "matrix")}

    def __init__(self, spec, weights, runtime):
        self.runtime = runtime
        self.up = Linear(weights[f"{spec.prefix}.up"], runtime)
        self.down = Linear(weights[f"{spec.prefix}.down"], runtime)

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, residual=None):
        z = K.relu2(self.up(y, split_ok=True), self.runtime.dtype)      # adds the partial sums, float32
        return self.down(z, split_ok=True, add_to=residual)


@register_part("ffn", "clamped_glu")
class ClampedGLU:
    """Parameters: hidden_size, intermediate_size, limit, alpha (1.702 unless given), token_gate."""
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        H = int(need(spec.params, "hidden_size", "clamped_glu"))
        I = int(need(spec.params, "intermediate_size", "clamped_glu"))
        pre = spec.prefix
        t = {f"{pre}.gate": ((I, H), "matrix"), f"{pre}.up": ((I, H), "matrix"), f"{pre}.down": ((H, I), "matrix")}
        if spec.params.get("token_gate", False):
            t[f"{pre}.sg"] = ((1, H), "matrix")
        return t

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        self.I = int(p["intermediate_size"])
        self.limit = float(need(p, "limit", "clamped_glu"))
        self.alpha = float(p.get("alpha", 1.702))
        pre = spec.prefix
        mats = [weights[f"{pre}.gate"], weights[f"{pre}.up"]]
        self.token_gate = bool(p.get("token_gate", False))
        if self.token_gate:
            mats.append(weights[f"{pre}.sg"])          # reads the same rows: one product for all three
        self.gate_up = Linear.stacked(mats, runtime)
        self.down = Linear(weights[f"{pre}.down"], runtime)

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, residual=None):
        u = self.gate_up(y, split_ok=True)          # float32 [gate | up | token gate], possibly partial sums
        z = K.clamped_glu(u, self.I, self.limit, self.alpha, self.runtime.dtype,
                          token_gate_col=2 * self.I if self.token_gate else -1)
        return self.down(z, split_ok=True, add_to=residual)


@register_part("ffn", "xielu_mlp")
class XieluMLP:
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        H = int(need(spec.params, "hidden_size", "xielu_mlp"))
        I = int(need(spec.params, "intermediate_size", "xielu_mlp"))
        return {f"{spec.prefix}.up": ((I, H), "matrix"), f"{spec.prefix}.down": ((H, I), "matrix"),
                f"{spec.prefix}.act": ((2,), "matrix")}

    def __init__(self, spec, weights, runtime):
        self.runtime = runtime
        self.up = Linear(weights[f"{spec.prefix}.up"], runtime)
        self.down = Linear(weights[f"{spec.prefix}.down"], runtime)
        self.act = weights[f"{spec.prefix}.act"].to(device=runtime.device, dtype=torch.float32).contiguous()

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, residual=None):
        u = self.up(y, split_ok=True)                       # float32 [N, I], possibly S partials
        return self.down(K.xielu(u, self.act, self.runtime.dtype), split_ok=True, add_to=residual)


@register_part("ffn", "routed_experts")
class RoutedExperts:
    """Parameters: hidden_size, expert_size, num_experts (with tensors), identity_experts,
    top, scale, shared_size (0 or absent: no shared expert)."""
    graph_safe = True

    @staticmethod
    def _sizes(p):
        D, F, E, top = (int(need(p, k, "routed_experts")) for k in ("hidden_size", "expert_size", "num_experts", "top"))
        shared = p.get("shared") or {}
        return D, F, E, int(p.get("identity_experts", 0)), top, int(shared.get("size", 0) or p.get("shared_size", 0) or 0)

    @classmethod
    def _shared_spec(cls, spec):
        from ..config.spec import PartSpec
        D, _, _, _, _, Fs = cls._sizes(spec.params)
        shared = spec.params.get("shared") or {}
        if shared.get("kind", "swiglu") == "clamped_glu":
            return PartSpec("clamped_glu", {"hidden_size": D, "intermediate_size": Fs,
                                            "limit": need(shared, "limit", "routed_experts.shared"),
                                            "alpha": shared.get("alpha", 1.702),
                                            "token_gate": bool(shared.get("token_gate", False))},
                            prefix=f"{spec.prefix}.shared")
        return PartSpec("swiglu", {"hidden_size": D, "intermediate_size": Fs,
                                   "tensor_names": {"gate": ".gate", "up": ".up", "down": ".down"}},
                        prefix=f"{spec.prefix}.shared")

    @classmethod
    def tensors(cls, spec):
        D, F, E, ident, _, Fs = cls._sizes(spec.params)
        pre = spec.prefix
        t = {f"{pre}.router": ((E + ident, D), "matrix")}
        if spec.params.get("correction", True):
            t[f"{pre}.correction"] = ((E + ident,), "matrix")
        for e in range(E):
            t.update({f"{pre}.e{e}.gate": ((F, D), "matrix"), f"{pre}.e{e}.up": ((F, D), "matrix"),
                      f"{pre}.e{e}.down": ((D, F), "matrix")})
        if Fs:
            sh = cls._shared_spec(spec)
            t.update(part_class("ffn", sh.kind).tensors(sh))
        return t

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.runtime = runtime
        self.D, self.F, self.E, self.ident, self.top, Fs = self._sizes(p)
        if not 1 <= self.top <= self.E + self.ident:
            raise ValueError(f"{self.top} choices among {self.E + self.ident} experts")
        self.scale = float(p.get("scale", 1.0))
        self.mode = p.get("router", "softmax")
        if self.mode not in K.ROUTER_MODES:
            raise ValueError(f"routed_experts: router {self.mode!r} (known: {sorted(K.ROUTER_MODES)})")
        self.weight_on_input = {"output": False, "input": True}[p.get("weight_on", "output")]
        if self.weight_on_input and self.ident:
            raise ValueError("routed_experts: identity experts with weights on the experts' input are not built")
        ex = p.get("expert") or {}
        if ex.get("kind", "swiglu") not in ("swiglu", "clamped_glu"):
            raise ValueError(f"routed_experts: expert kind {ex.get('kind')!r} (known: 'swiglu', 'clamped_glu')")
        self.clamp = ((float(need(ex, "limit", "routed_experts.expert")), float(ex.get("alpha", 1.702)))
                      if ex.get("kind") == "clamped_glu" else None)
        pre = spec.prefix
        dev = runtime.device
        # the router is multiplied in true 32-bit whatever the run's type
        self.router = weights[f"{pre}.router"].to(device=dev, dtype=torch.float32).contiguous()
        self.correction = (weights[f"{pre}.correction"].to(device=dev, dtype=torch.float32).contiguous()
                           if p.get("correction", True) else None)
        # the grouped products take the experts' weights in the run's type
        stack = lambda names: torch.stack([weights[n].to(runtime.dtype) for n in names]).contiguous()
        gate = stack([f"{pre}.e{e}.gate" for e in range(self.E)])
        up = stack([f"{pre}.e{e}.up" for e in range(self.E)])
        self.w_gate_up = torch.cat([gate, up], dim=1).contiguous()          # [E, 2 F, D]: gate rows, then up rows
        self.w_down = stack([f"{pre}.e{e}.down" for e in range(self.E)])    # [E, D, F]
        self.shared = build_part("ffn", self._shared_spec(spec), weights, runtime) if Fs else None
        self.update_in_pieces = bool(p.get("update_in_pieces", False))

    adds_residual = True      # forward takes `residual`; the shared expert may add its update there in place

    def forward(self, y, ctx, residual=None):
        N = y.shape[0]
        # one slice of the update for each of a token's choices; the routing kernel fills in the
        # identity experts' slices, the down product the others
        out = torch.empty((self.top, N, self.D), dtype=torch.float32, device=y.device)
        idx, wt = K.moe_route_x(y, self.router, self.correction, self.top, self.scale,
                                identity_out=out if self.ident else None, n_experts=self.E, mode=self.mode)
        # bfloat16 operands with rows of whole 16 bytes go to the tensor cores, in both products
        tc = K.moe_takes_tensor_cores(y.dtype, self.w_gate_up) and K.moe_takes_tensor_cores(y.dtype, self.w_down)
        group = K.moe_group(idx, self.E, tensor_cores=tc)
        z = K.moe_product(y, self.w_gate_up, group, wt if self.weight_on_input else None, self.top, N, gated=True,
                          clamp=self.clamp)
        K.moe_product(z, self.w_down, group, None if self.weight_on_input else wt, self.top, N, gated=False, out=out)
        if self.shared is None:
            return out
        s = self.shared.forward(y, ctx, residual=residual)
        if s is None:
            return out
        if self.update_in_pieces:
            return [out, s]       # the arrangement adds the pieces as they are (no copy into one stack)
        return torch.cat([out, s if s.dim() == 3 else s.unsqueeze(0)], dim=0)

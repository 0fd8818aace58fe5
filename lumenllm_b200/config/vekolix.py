"""Typed configuration of Vekolix (config.json key "architecture": "Vekolix").

A small decoder of pre-norm layers whose updates count `residual_mult` = m times,
x <- x + m mixer(norm1(x)), x <- x + m ff(norm2(x)), with Dynamic Tanh in place of a norm
(tanh(alpha x) w + b; tensors `<name>`, `<name>.b`, `<name>.alpha`). The head is the embedding
table itself; logits are multiplied by `logit_scale` and bent by `logit_softcap` c to
c tanh(logit / c). config.json lists the layers one by one; a layer's mixer is one of

- "parallel": two mixers side by side on the same input, `left_scale` * left + `right_scale` * right.
  Left (`.left`): grouped-query causal softmax attention without biases, keys of `dim` and values
  of `vdim`, rotation of the first rot.dims of a head in the half-split pairing, optionally with
  stretched frequencies (rot.scaling: factor, original, fast, slow). Right (`.right`): linear
  attention with a fixed decay a head over SiLU'd q, k, v, the heads together RMS-normed, gated by
  a sigmoid and projected;
- "latent_attention": queries through a normed latent of `q_rank`; keys and values of all heads are
  products of ONE normed latent vector a token (`kv_rank`), plus a short rotated key part
  (`rot_dim`) that all heads share, rotated in the interleaved pairing; a sigmoid gate a head on
  the output.

Its feed-forward is dense (the square of ReLU between two matrices), a mixture of experts (sigmoid
router, the `top` largest scores, a score multiplies its expert's input, clamped gated experts, an
optional shared expert with a sigmoid gate a token), or absent. config.json gives every size and
constant.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .dabevik import _int, _num, _obj
from .rasezen import UNBOUNDED_POSITIONS
from .registry import eos_ids_of, register_architecture
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

GLU_ALPHA = 1.702        # the slope inside the experts' sigmoid: fixed by the design


def _rot(m, where, limit):
    """(dims, base, scaling or None); dims 0 without a rotation."""
    rot = m.get("rot")
    if rot is None:
        return 0, 1.0, None
    if not isinstance(rot, dict):
        raise ConfigError(f"config.json: {where}rot must be an object")
    dims, base = _int(rot, "dims", where + "rot.", 0), _num(rot, "base", where + "rot.")
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most {limit}")
    sc = rot.get("scaling")
    if sc is not None:
        w = where + "rot.scaling."
        if not isinstance(sc, dict):
            raise ConfigError(f"config.json: {where}rot.scaling must be an object")
        sc = (_num(sc, "factor", w), _num(sc, "original", w), _num(sc, "fast", w), _num(sc, "slow", w))
        if sc[0] <= 0 or sc[1] <= 0 or sc[2] <= 0 or sc[3] <= 0 or base <= 1:
            raise ConfigError(f"config.json: {w}factor, original, fast and slow must be positive (and rot.base above 1)")
    return dims, base, sc


def _rot_dict(dims, base, scaling):
    d = {"base": base, "dims": dims}
    if scaling is not None:
        d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return d


@dataclass(frozen=True)
class VekolixSoftmaxSide:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[Tuple[float, float, float, float]]

    @classmethod
    def from_dict(cls, m, where):
        dim = _int(m, "dim", where)
        dims, base, sc = _rot(m, where, dim)
        a = cls(heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where), dim=dim, vdim=_int(m, "vdim", where),
                scale=_num(m, "scale", where), rot_dims=dims, rot_base=base, rot_scaling=sc)
        if a.heads % a.kv_heads:
            raise ConfigError(f"config.json: {where}{a.heads} heads are not a multiple of {a.kv_heads} kv_heads")
        return a

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_dims:
            d["rot"] = _rot_dict(self.rot_dims, self.rot_base, self.rot_scaling)
        return d


@dataclass(frozen=True)
class VekolixLinearSide:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @classmethod
    def from_dict(cls, m, where):
        decay = m.get("decay")
        heads = _int(m, "heads", where)
        if not isinstance(decay, list) or len(decay) != heads or any(isinstance(x, bool) or not isinstance(x, (int, float))
                                                                      for x in decay):
            raise ConfigError(f"config.json: {where}decay must list one number for each of the {heads} heads")
        return cls(heads=heads, dim=_int(m, "dim", where), vdim=_int(m, "vdim", where), decay=tuple(float(x) for x in decay))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class VekolixParallel:
    left: VekolixSoftmaxSide
    right: VekolixLinearSide
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, m, where):
        return cls(left=VekolixSoftmaxSide.from_dict(_obj(m, "left", where), where + "left."),
                   right=VekolixLinearSide.from_dict(_obj(m, "right", where), where + "right."),
                   left_scale=_num(m, "left_scale", where) if "left_scale" in m else 1.0,
                   right_scale=_num(m, "right_scale", where) if "right_scale" in m else 1.0)

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class VekolixLatent:
    heads: int
    dim: int             # unrotated query/key values a head
    rot_dim: int         # rotated values a head (the key's are shared by all heads)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[Tuple[float, float, float, float]]

    @classmethod
    def from_dict(cls, m, where):
        rot_dim = _int(m, "rot_dim", where, 0)
        dims, base, sc = _rot(m, where, rot_dim)
        return cls(heads=_int(m, "heads", where), dim=_int(m, "dim", where), rot_dim=rot_dim, vdim=_int(m, "vdim", where),
                   kv_rank=_int(m, "kv_rank", where), q_rank=_int(m, "q_rank", where), scale=_num(m, "scale", where),
                   rot_dims=dims, rot_base=base, rot_scaling=sc)

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "q_rank": self.q_rank, "scale": self.scale}
        if self.rot_dims:
            d["rot"] = _rot_dict(self.rot_dims, self.rot_base, self.rot_scaling)
        return d


@dataclass(frozen=True)
class VekolixMlp:
    kind: str                 # "dense" or "moe"
    ff: int = 0               # dense: the inner width; moe: an expert's
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    shared_ff: int = 0        # 0: no shared expert
    shared_limit: float = 0.0

    @classmethod
    def from_dict(cls, m, where):
        kind = m.get("kind")
        if kind == "dense":
            return cls("dense", ff=_int(m, "ff", where))
        if kind != "moe":
            raise ConfigError(f"config.json: {where}kind {kind!r} is not a feed-forward of this design "
                              "(known: 'dense', 'moe')")
        ex, ro = _obj(m, "expert", where), _obj(m, "router", where)
        sh = m.get("shared")
        if sh is not None and not isinstance(sh, dict):
            raise ConfigError(f"config.json: {where}shared must be null or an object")
        c = cls("moe", ff=_int(ex, "ff", where + "expert."), limit=_num(ex, "limit", where + "expert."),
                experts=_int(ro, "experts", where + "router."), top=_int(ro, "top", where + "router."),
                shared_ff=_int(sh, "ff", where + "shared.") if sh else 0,
                shared_limit=_num(sh, "limit", where + "shared.") if sh else 0.0)
        if c.top > c.experts:
            raise ConfigError(f"config.json: {where}router.top {c.top} is more than the {c.experts} experts")
        return c

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
             "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return d


@dataclass(frozen=True)
class VekolixLayer:
    type: str
    mixer: Any
    mlp: Optional[VekolixMlp]


@register_architecture("Vekolix")
@dataclass(frozen=True)
class VekolixConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_scale: float
    logit_softcap: float                         # 0: the logits are not bent
    layers: Tuple[VekolixLayer, ...]
    max_positions: int = UNBOUNDED_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    MIXERS = {"parallel": VekolixParallel, "latent_attention": VekolixLatent}

    @classmethod
    def from_dict(cls, d: dict) -> "VekolixConfig":
        for k in ("vocab", "width", "norm", "layers"):
            if k not in d:
                raise ConfigError(f"config.json: missing key '{k}'")
        entries = d["layers"]
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = e.get("type")
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is not a mixer of this design "
                                  f"(known: {sorted(cls.MIXERS)})")
            mixer = cls.MIXERS[kind].from_dict(_obj(e, "mixer", where), where + "mixer.")
            mlp = e.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: {where}mlp must be null or an object, got {mlp!r}")
            layers.append(VekolixLayer(kind, mixer, None if mlp is None else VekolixMlp.from_dict(mlp, where + "mlp.")))
        known = ("architecture", "vocab", "width", "norm", "layers", "residual_mult", "logit_scale", "logit_softcap",
                 "max_positions", "eos_token_id", "torch_dtype")
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                  norm_eps=_num(_obj(d, "norm", ""), "eps", "norm."),
                  residual_mult=_num(d, "residual_mult", "") if "residual_mult" in d else 1.0,
                  logit_scale=_num(d, "logit_scale", "") if "logit_scale" in d else 1.0,
                  logit_softcap=_num(d, "logit_softcap", "") if d.get("logit_softcap") is not None else 0.0,
                  layers=tuple(layers),
                  max_positions=_int(d, "max_positions", "") if "max_positions" in d else UNBOUNDED_POSITIONS,
                  eos_token_ids=eos_ids_of(d.get("eos_token_id"), "config.json"),
                  extra={k: v for k, v in d.items() if k not in known})
        if cfg.norm_eps < 0 or cfg.logit_softcap < 0:
            raise ConfigError("config.json: norm.eps and logit_softcap must not be negative")
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": "Vekolix", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "residual_mult": self.residual_mult, "logit_scale": self.logit_scale,
             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                        for l in self.layers]}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.max_positions != UNBOUNDED_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ------------------------------------------------------------ meaning
    def model_spec(self) -> ModelSpec:
        D, eps = self.width, self.norm_eps

        def norm(name):
            return PartSpec("dynamic_tanh", {"size": D, "tensor": name})

        def rotary(head_dim, dims, base, scaling):
            if not dims:
                return PartSpec("none", {})
            p = {"head_dim": head_dim, "rotary_dim": dims, "theta": base, "wide_frequencies": True}
            if scaling is not None:
                p["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
            return PartSpec("rotary", p)

        specs, schedule = [], []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}", l.mixer
            if l.type == "parallel":
                a, b = m.left, m.right
                left = PartSpec("head_norm_attention", {
                    "hidden_size": D, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
                    "value_dim": a.vdim, "softmax_scale": a.scale, "qk_norm": False, "bias": False, "norm_eps": eps,
                    "position": rotary(a.dim, a.rot_dims, a.rot_base, a.rot_scaling)}, prefix=f"{p}.mix.left")
                right = PartSpec("decay_linear_attention", {
                    "hidden_size": D, "num_heads": b.heads, "head_dim": b.dim, "value_dim": b.vdim,
                    "decay": list(b.decay), "activation": "silu", "output_gate": True, "norm_eps": eps},
                    prefix=f"{p}.mix.right")
                mixer = PartSpec("side_by_side", {"parts": [{"mixer": left, "scale": m.left_scale},
                                                            {"mixer": right, "scale": m.right_scale}]}, prefix=f"{p}.mix")
            else:
                mixer = PartSpec("latent_attention", {
                    "hidden_size": D, "num_heads": m.heads, "head_dim": m.dim, "rot_width": m.rot_dim,
                    "value_dim": m.vdim, "latent_size": m.kv_rank, "query_rank": m.q_rank, "softmax_scale": m.scale,
                    "window": 0, "norm_eps": eps, "head_gate": True, "interleaved_rotation": True,
                    "position": rotary(m.rot_dim, m.rot_dims, m.rot_base, m.rot_scaling)}, prefix=f"{p}.mix")
            ffn, norms = None, {"mixer": norm(f"{p}.norm1")}
            if l.mlp is not None:
                f = l.mlp
                if f.kind == "dense":
                    ffn = PartSpec("relu2_mlp", {"hidden_size": D, "intermediate_size": f.ff}, prefix=f"{p}.mlp")
                else:
                    params = {"hidden_size": D, "expert_size": f.ff, "num_experts": f.experts, "top": f.top,
                              "scale": 1.0, "router": "sigmoid", "correction": False, "weight_on": "input",
                              "update_in_pieces": True,
                              "expert": {"kind": "clamped_glu", "limit": f.limit, "alpha": GLU_ALPHA}}
                    if f.shared_ff:
                        params["shared"] = {"size": f.shared_ff, "kind": "clamped_glu", "limit": f.shared_limit,
                                            "alpha": GLU_ALPHA, "token_gate": True}
                    ffn = PartSpec("routed_experts", params, prefix=f"{p}.mlp")
                norms["ffn"] = norm(f"{p}.norm2")
            specs.append(LayerSpec("pre_norm", mixer, ffn, norms, prefix=p,
                                   params={"residual_scale": self.residual_mult}))
            schedule.append(ScheduleEntry(i))
        head = {"vocab_size": self.vocab, "hidden_size": D, "own_tensor": False, "tied_to": "embed",
                "logit_scale": self.logit_scale, "softcap": self.logit_softcap}
        spec = ModelSpec(
            architecture="Vekolix", vocab_size=self.vocab, hidden_size=D, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D, "tensor": "embed"}),
            layers=tuple(specs), schedule=tuple(schedule), final_norm=norm("final.norm"),
            head=PartSpec("linear_head", head), eos_token_ids=self.eos_token_ids)
        spec.validate()
        return spec

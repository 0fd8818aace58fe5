"""Typed configuration of Lebelix (config.json key "architecture": "Lebelix").

A small decoder of pre-norm layers, x <- x + mixer(norm1(x)), x <- x + ff(norm2(x)), with RMS norms
whose stored weight w counts as 1 + w. Token vectors are scaled; the head is the embedding table
itself. After a layer's feed-forward a small per-layer table of token vectors, gated by a
projection of the stream, is projected back, RMS-normed and added ("token_side"). config.json
lists the layers one by one; a layer's mixer is one of

- "attention": biased q/k/v projections, an RMS norm of every query and key head, rotation of part
  of a head, scores capped by a tanh, sight limited to the query's own chunk of positions, a
  softmax with one more term exp(0) in its denominator, a sigmoid gate on the heads' outputs;
- "latent_attention": keys and values of all heads are products of ONE normed latent vector a
  token, plus a short rotated key part that all heads share; sliding window; a layer may read
  the latent cache of an earlier layer ("kv_from") instead of making its own;
- "channel_delta": the gated delta rule, a matrix state per head with a decay of its own for every
  key channel, short causal convolutions on q, k and v, low-rank projections for decay and gate.

Its feed-forward is dense with the tanh form of GELU, or absent. config.json gives every size and
constant but the two low ranks of "channel_delta", which are the shapes of its tensors `.a1` and
`.g1` (`sized_by` reads them from the checkpoint; a config.json may also name them as
`decay_rank` and `gate_rank`, as the random-weights mode writes it).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Dict, Optional, Tuple

from .dabevik import _int, _num, _obj
from .rasezen import UNBOUNDED_POSITIONS
from .registry import eos_ids_of, register_architecture
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mask(m, where) -> int:
    return _int(_obj(m, "mask", where), "size", where + "mask.") if m.get("mask") is not None else 0


def _rot(m, where, limit):
    rot = m.get("rot")
    if rot is None:
        return 0, 1.0
    dims, base = _int(rot, "dims", where + "rot.", 0), _num(rot, "base", where + "rot.")
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most {limit}")
    return dims, base


@dataclass(frozen=True)
class LebelixAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int           # positions a chunk; 0: every earlier key is seen
    softcap: float       # 0: scores are not capped
    rot_dims: int
    rot_base: float

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "LebelixAttention":
        dim = _int(m, "dim", where)
        rot_dims, rot_base = _rot(m, where, dim)
        a = cls(heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where), dim=dim, vdim=_int(m, "vdim", where),
                scale=_num(m, "scale", where), chunk=_mask(m, where),
                softcap=_num(m, "softcap", where) if m.get("softcap") is not None else 0.0,
                rot_dims=rot_dims, rot_base=rot_base)
        if a.heads % a.kv_heads:
            raise ConfigError(f"config.json: {where}{a.heads} heads are not a multiple of {a.kv_heads} kv_heads")
        if a.softcap < 0:
            raise ConfigError(f"config.json: {where}softcap must not be negative")
        return a

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.chunk:
            d["mask"] = {"size": self.chunk}
        if self.softcap:
            d["softcap"] = self.softcap
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class LebelixLatentAttention:
    heads: int
    dim: int             # unrotated query/key values a head
    rot_dim: int         # rotated values a head (the key's are shared by all heads)
    vdim: int
    kv_rank: int
    scale: float
    window: int          # 0: every earlier key is seen
    rot_dims: int
    rot_base: float
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "LebelixLatentAttention":
        rot_dim = _int(m, "rot_dim", where, 0)
        rot_dims, rot_base = _rot(m, where, rot_dim)
        src = m.get("kv_from")
        if src is not None and (isinstance(src, bool) or not isinstance(src, int) or src < 0):
            raise ConfigError(f"config.json: {where}kv_from must be a layer's index, got {src!r}")
        return cls(heads=_int(m, "heads", where), dim=_int(m, "dim", where), rot_dim=rot_dim, vdim=_int(m, "vdim", where),
                   kv_rank=_int(m, "kv_rank", where), scale=_num(m, "scale", where), window=_mask(m, where),
                   rot_dims=rot_dims, rot_base=rot_base, kv_from=src)

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class LebelixChannelDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int = 0      # 0: not known yet (the shape of `.a1` says)
    gate_rank: int = 0       # 0: not known yet (the shape of `.g1` says)

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "LebelixChannelDelta":
        c = cls(heads=_int(m, "heads", where), kv_heads=_int(m, "kv_heads", where), dim=_int(m, "dim", where),
                vdim=_int(m, "vdim", where), conv=_int(m, "conv", where),
                decay_rank=_int(m, "decay_rank", where) if "decay_rank" in m else 0,
                gate_rank=_int(m, "gate_rank", where) if "gate_rank" in m else 0)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}{c.heads} heads are not a multiple of {c.kv_heads} kv_heads")
        return c

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.decay_rank:
            d["decay_rank"] = self.decay_rank
        if self.gate_rank:
            d["gate_rank"] = self.gate_rank
        return d


@dataclass(frozen=True)
class LebelixLayer:
    type: str
    mixer: Any
    ff: int                 # width of the dense feed-forward; 0: the layer has none


@register_architecture("Lebelix")
@dataclass(frozen=True)
class LebelixConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    side_dim: int                                # 0: no per-layer token input
    layers: Tuple[LebelixLayer, ...]
    max_positions: int = UNBOUNDED_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    MIXERS = {"attention": LebelixAttention, "latent_attention": LebelixLatentAttention,
              "channel_delta": LebelixChannelDelta}

    @classmethod
    def from_dict(cls, d: dict) -> "LebelixConfig":
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
            if mlp is not None and mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind')!r} is not a feed-forward of this "
                                  "design (known: 'dense')")
            layers.append(LebelixLayer(kind, mixer, 0 if mlp is None else _int(mlp, "ff", where + "mlp.")))
        for i, l in enumerate(layers):
            if l.type != "latent_attention" or l.mixer.kv_from is None:
                continue
            j, m = l.mixer.kv_from, l.mixer
            where = f"config.json: layers[{i}].mixer.kv_from {j}: "
            if j >= i or layers[j].type != "latent_attention" or layers[j].mixer.kv_from is not None:
                raise ConfigError(where + "must name an earlier latent_attention layer that keeps a cache of its own")
            o = layers[j].mixer
            if (o.kv_rank, o.rot_dim, o.rot_dims, o.rot_base) != (m.kv_rank, m.rot_dim, m.rot_dims, m.rot_base):
                raise ConfigError(where + "latent width, rotated width and rotation must equal that layer's")
        emb, side = d.get("embedding"), d.get("token_side")
        known = ("architecture", "vocab", "width", "norm", "layers", "embedding", "token_side", "max_positions",
                 "eos_token_id", "torch_dtype")
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                  norm_eps=_num(_obj(d, "norm", ""), "eps", "norm."),
                  embedding_scale=_num(emb, "scale", "embedding.") if emb is not None else 1.0,
                  side_dim=_int(side, "dim", "token_side.") if side is not None else 0,
                  layers=tuple(layers),
                  max_positions=_int(d, "max_positions", "") if "max_positions" in d else UNBOUNDED_POSITIONS,
                  eos_token_ids=eos_ids_of(d.get("eos_token_id"), "config.json"),
                  extra={k: v for k, v in d.items() if k not in known})
        if cfg.norm_eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": "Lebelix", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale},
             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(),
                         "mlp": {"kind": "dense", "ff": l.ff} if l.ff else None} for l in self.layers]}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.max_positions != UNBOUNDED_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def sized_by(self, shape_of) -> "LebelixConfig":
        """The sizes that only tensors give: `shape_of(name)` is a stored tensor's shape or None."""
        layers = []
        for i, l in enumerate(self.layers):
            if l.type == "channel_delta" and not (l.mixer.decay_rank and l.mixer.gate_rank):
                a1, g1 = shape_of(f"l{i}.mix.a1"), shape_of(f"l{i}.mix.g1")
                l = replace(l, mixer=replace(l.mixer,
                                             decay_rank=l.mixer.decay_rank or (int(a1[0]) if a1 else 0),
                                             gate_rank=l.mixer.gate_rank or (int(g1[0]) if g1 else 0)))
            layers.append(l)
        return replace(self, layers=tuple(layers))

    # ------------------------------------------------------------ meaning
    def model_spec(self) -> ModelSpec:
        D, eps = self.width, self.norm_eps

        def norm(name):
            return PartSpec("rmsnorm", {"size": D, "eps": eps, "weight_offset": 1.0, "tensor": name})

        # a latent cache serves its own layer and every layer that reads it: it keeps what the
        # widest of their windows sees
        reach = {}
        for i, l in enumerate(self.layers):
            if l.type == "latent_attention":
                j = i if l.mixer.kv_from is None else l.mixer.kv_from
                w = l.mixer.window
                reach[j] = 0 if (w == 0 or reach.get(j, w) == 0) else max(reach.get(j, w), w)
        specs, schedule = [], []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}", l.mixer
            if l.type == "attention":
                position = (PartSpec("rotary", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                                "wide_frequencies": True}) if m.rot_dims else PartSpec("none", {}))
                mixer = PartSpec("head_norm_attention", {
                    "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "softmax_scale": m.scale, "chunk": m.chunk, "softcap": m.softcap,
                    "sink": True, "output_gate": True, "bias": True, "norm_eps": eps, "position": position},
                    prefix=f"{p}.mix")
            elif l.type == "latent_attention":
                position = (PartSpec("rotary", {"head_dim": m.rot_dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                                "wide_frequencies": True}) if m.rot_dims else PartSpec("none", {}))
                mixer = PartSpec("latent_attention", {
                    "hidden_size": D, "num_heads": m.heads, "head_dim": m.dim, "rot_width": m.rot_dim,
                    "value_dim": m.vdim, "latent_size": m.kv_rank, "softmax_scale": m.scale, "window": m.window,
                    "cache_window": reach[i if m.kv_from is None else m.kv_from], "norm_eps": eps,
                    "shares_cache": m.kv_from is not None, "position": position}, prefix=f"{p}.mix")
            else:
                if not (m.decay_rank and m.gate_rank):
                    raise ConfigError(f"config.json: layers[{i}].mixer: the ranks of the decay and gate projections "
                                      f"are the shapes of '{p}.mix.a1' and '{p}.mix.g1'; without a checkpoint name "
                                      "them as 'decay_rank' and 'gate_rank'")
                mixer = PartSpec("channel_delta", {
                    "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "taps": m.conv, "decay_rank": m.decay_rank, "gate_rank": m.gate_rank,
                    "norm_eps": eps}, prefix=f"{p}.mix")
            ffn, norms = None, {"mixer": norm(f"{p}.norm1")}
            if l.ff:
                ffn = PartSpec("gelu_mlp", {"hidden_size": D, "intermediate_size": l.ff}, prefix=f"{p}.mlp")
                norms["ffn"] = norm(f"{p}.norm2")
            extras = {}
            if self.side_dim:
                extras["token_input"] = PartSpec("gated_token_table", {
                    "hidden_size": D, "vocab_size": self.vocab, "dim": self.side_dim, "table": "side.embed",
                    "table_width": self.side_dim * len(self.layers), "column": i * self.side_dim, "norm_eps": eps},
                    prefix=f"{p}.side")
            specs.append(LayerSpec("pre_norm", mixer, ffn, norms, prefix=p, extras=extras))
            src = m.kv_from if l.type == "latent_attention" else None
            schedule.append(ScheduleEntry(i, cache_from=src))
        spec = ModelSpec(
            architecture="Lebelix", vocab_size=self.vocab, hidden_size=D, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D, "tensor": "embed",
                                                   "scale": self.embedding_scale}),
            layers=tuple(specs), schedule=tuple(schedule), final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D, "own_tensor": False,
                                          "tied_to": "embed"}),
            eos_token_ids=self.eos_token_ids)
        spec.validate()
        return spec

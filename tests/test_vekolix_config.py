"""Vekolix without a GPU: config.json to typed configuration and back, what is refused, the
model's parts as data (two mixers side by side, latent attention with its options, the three
feed-forwards, the multiplier on every update), the names and shapes of its tensors, stretched
rotation frequencies, and the plain implementation against itself (the recurrence written as a
decayed causal sum; the interleaved pairing as a reordering of the half-split one; a weight on an
expert's input)."""
import copy
import math

import pytest
import torch

import plain_vekolix as P
from vekolix_models import SMALL, make_weights, write_model


def test_round_trip_and_registry():
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.config.vekolix import VekolixConfig
    for name, d in SMALL.items():
        c = config_from_dict(d)
        assert isinstance(c, VekolixConfig)
        assert c.to_dict() == d, name
        assert config_from_dict(c.to_dict()) == c


def test_parts_of_the_model_as_data():
    from lumenllm_b200.config import config_from_dict
    spec = config_from_dict(SMALL["X"]).model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3] and all(e.cache_from is None for e in spec.schedule)
    assert [l.mixer.kind for l in spec.layers] == ["side_by_side", "latent_attention", "side_by_side", "latent_attention"]
    assert all(l.block == "pre_norm" and l.params["residual_scale"] == 0.6 for l in spec.layers)
    assert all(n.kind == "dynamic_tanh" for l in spec.layers for n in l.norms.values()) and spec.final_norm.kind == "dynamic_tanh"
    left, right = (c["mixer"] for c in spec.layers[0].mixer.params["parts"])
    assert [c["scale"] for c in spec.layers[0].mixer.params["parts"]] == [0.8, 1.3]
    a = left.params
    assert left.kind == "head_norm_attention" and not a["qk_norm"] and not a["bias"]
    assert (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["value_dim"], a["softmax_scale"]) == (4, 2, 16, 24, 0.3)
    assert a["position"].params["rotary_dim"] == 8 and a["position"].params["scaling"]["factor"] == 4.0
    b = right.params
    assert right.kind == "decay_linear_attention" and b["decay"] == [0.7, 0.98] and b["activation"] == "silu"
    assert left.prefix == "l0.mix.left" and right.prefix == "l0.mix.right"
    lat = spec.layers[1].mixer.params
    assert (lat["query_rank"], lat["latent_size"], lat["rot_width"], lat["head_gate"], lat["interleaved_rotation"]) == \
        (24, 40, 16, True, True)
    assert lat["position"].params["rotary_dim"] == 8 and lat["window"] == 0
    f = spec.layers[0].ffn
    assert f.kind == "routed_experts" and f.params["router"] == "sigmoid" and f.params["weight_on"] == "input"
    assert f.params["expert"] == {"kind": "clamped_glu", "limit": 1.5, "alpha": 1.702} and not f.params["correction"]
    assert f.params["shared"] == {"size": 40, "kind": "clamped_glu", "limit": 0.8, "alpha": 1.702, "token_gate": True}
    assert spec.layers[1].ffn.kind == "relu2_mlp" and spec.layers[2].ffn is None and "shared" not in spec.layers[3].ffn.params
    assert spec.head.params["logit_scale"] == 0.5 and spec.head.params["softcap"] == 12.0 and spec.head.params["tied_to"] == "embed"
    # no rotation on one side, no cap, multipliers of 1
    spec = config_from_dict(SMALL["Y"]).model_spec()
    assert spec.layers[1].mixer.params["parts"][0]["mixer"].params["position"].kind == "none"
    assert spec.head.params["softcap"] == 0.0 and spec.layers[0].params["residual_scale"] == 1.0


def test_expected_tensors_are_the_designs_names():
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.engine.model import expected_tensors
    for name, d in SMALL.items():
        exp = expected_tensors(config_from_dict(d).model_spec())
        w = make_weights(d, 0)
        assert set(exp) == set(w), (name, set(exp) ^ set(w))
        for n, (shape, _) in exp.items():
            assert tuple(w[n].shape) == tuple(shape), n


def test_a_folder_is_read_by_its_architecture(tmp_path):
    from lumenllm_b200.config import load_config
    from lumenllm_b200.config.vekolix import VekolixConfig
    folder = write_model(SMALL["X"], tmp_path / "x", seed=1)
    c = load_config(folder)
    assert isinstance(c, VekolixConfig) and c.to_dict() == SMALL["X"]


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].__setitem__("type", "attention"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 18), "at most"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "feed-forward"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 6), "more than"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_what_is_refused(edit, word):
    from lumenllm_b200.config import ConfigError, config_from_dict
    c = copy.deepcopy(SMALL["X"])
    edit(c)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(c)


def test_stretched_frequencies():
    """Fast pairs keep their frequency, slow ones are divided by the factor, a ramp lies between;
    the library's rotary part makes the same numbers as the plain implementation."""
    from lumenllm_b200.config.spec import PartSpec
    from lumenllm_b200.parts import Runtime, build_part
    base, dims, sc = 10000.0, 32, {"factor": 8.0, "original": 256, "fast": 16.0, "slow": 2.0}
    f, mag = P.frequencies(base, dims, sc)
    f0, one = P.frequencies(base, dims)
    assert one == 1.0 and abs(mag - (0.1 * math.log(8.0) + 1.0)) < 1e-12
    turns = 256 * f0.double() / (2 * math.pi)
    assert torch.equal(f[turns > 16.0 * 1.5], f0[turns > 16.0 * 1.5])
    slow = turns < 2.0 / 1.5
    assert slow.any() and torch.allclose(f[slow], f0[slow] / 8.0, rtol=1e-6)
    ratio = (f0 / f)
    assert bool((ratio[1:] >= ratio[:-1] - 1e-6).all()) and 1.0 - 1e-6 <= float(ratio.min()) and float(ratio.max()) <= 8.0 + 1e-5
    part = build_part("position", PartSpec("rotary", {"head_dim": 48, "rotary_dim": dims, "theta": base,
                                                      "wide_frequencies": True, "scaling": sc}),
                      {}, Runtime(torch.device("cpu"), torch.float32))
    assert torch.equal(part.inv_freq, f) and abs(part.magnitude - mag) < 1e-12
    plain = build_part("position", PartSpec("rotary", {"head_dim": 48, "rotary_dim": dims, "theta": base,
                                                       "wide_frequencies": True}), {}, Runtime(torch.device("cpu"), torch.float32))
    assert torch.equal(plain.inv_freq, f0) and plain.magnitude == 1.0


def test_plain_recurrence_equals_a_decayed_causal_sum():
    """o_t = sum_{j <= t} decay^(t - j) (q_t . k_j) v_j: the recurrence written as attention without a
    softmax."""
    g = torch.Generator().manual_seed(3)
    T, D, m = 19, 24, {"heads": 3, "dim": 8, "vdim": 5, "decay": [0.5, 0.9, 1.0]}
    H, d, dv = 3, 8, 5
    w = {"p.q": torch.randn(H * d, D, generator=g) * 0.3, "p.k": torch.randn(H * d, D, generator=g) * 0.3,
         "p.v": torch.randn(H * dv, D, generator=g) * 0.3, "p.g": torch.randn(H * dv, D, generator=g) * 0.3,
         "p.norm": torch.ones(H * dv), "p.o": torch.eye(H * dv)}
    h = torch.randn(T, D, generator=g)
    got = P.linear_attention(h, w, "p", m, 1e-6)
    q, k, v = (P.silu(h @ w["p." + n].T).view(T, H, -1) for n in "qkv")
    t = torch.arange(T)
    power = (t[:, None] - t[None, :]).clamp(min=0).float()
    weight = torch.tensor(m["decay"])[:, None, None] ** power[None] * (t[:, None] >= t[None, :])
    o = torch.einsum("hts,thd,shd,she->the", weight, q, k, v).reshape(T, H * dv)
    ref = P.norm_plain(o, w["p.norm"], 1e-6) * torch.sigmoid(h @ w["p.g"].T)
    assert float((got - ref).abs().max()) < 1e-5


def test_interleaved_pairs_are_the_half_split_pairs_reordered():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(7, 2, 12, generator=g)
    pos = torch.tensor([0, 1, 5, 64, 100, 1000, 3])
    dims = 8
    order = torch.cat([torch.arange(0, dims, 2), torch.arange(1, dims, 2), torch.arange(dims, 12)])
    a = P.rotate(x, pos, 1000.0, dims, interleaved=True)[..., order]
    b = P.rotate(x[..., order], pos, 1000.0, dims)
    assert float((a - b).abs().max()) < 1e-6


def test_a_weight_on_the_input_is_not_a_weight_on_the_output():
    """The experts are not linear: expert(w x) differs from w expert(x), and the plain mixture uses the first."""
    cfg = SMALL["X"]
    w = {k: v.float() for k, v in make_weights(cfg, 5).items()}
    h = torch.randn(6, cfg["width"], generator=torch.Generator().manual_seed(6))
    mlp = cfg["layers"][0]["mlp"]
    got = P.expert_ff(h, w, "l0.mlp", dict(mlp, shared=None))
    s = torch.sigmoid(h @ w["l0.mlp.router"].T)
    best = torch.topk(s, mlp["router"]["top"], dim=-1)
    on_input, on_output = torch.zeros_like(h), torch.zeros_like(h)
    for t in range(6):
        for j in range(mlp["router"]["top"]):
            e, sc = int(best.indices[t, j]), best.values[t, j]
            on_input[t] += P.clamped_expert(sc * h[t:t + 1], w, f"l0.mlp.e{e}", mlp["expert"]["limit"])[0]
            on_output[t] += sc * P.clamped_expert(h[t:t + 1], w, f"l0.mlp.e{e}", mlp["expert"]["limit"])[0]
    assert float((got - on_input).abs().max()) < 1e-5
    assert float((got - on_output).abs().max()) > 1e-2


def test_plain_model_runs_and_decodes_greedily():
    for name, cfg in SMALL.items():
        w = {k: v.float() for k, v in make_weights(cfg, 7).items()}
        toks = torch.randint(0, cfg["vocab"], (9,), generator=torch.Generator().manual_seed(8)).tolist()
        out = []
        lg = P.forward(cfg, w, toks, out)
        assert lg.shape == (9, cfg["vocab"]) and torch.isfinite(lg).all() and len(out) == len(cfg["layers"])
        cap = cfg.get("logit_softcap")
        assert cap is None or float(lg.abs().max()) <= cap
        # causal: a prefix's logits do not depend on what follows
        assert float((P.forward(cfg, w, toks[:4]) - lg[:4]).abs().max()) < 1e-4
    assert len(P.greedy(cfg, w, toks[:3], 2)) == 2

"""Lebelix without a GPU: config.json to typed configuration and back, what is refused, the
model's parts as data (layers that read another layer's latent cache, layers without feed-forward,
the per-layer token input), the names and shapes of its tensors, sizes that only tensors give, the
cache's bookkeeping for chunks, and the plain implementation against itself (a sequence fed whole
equals the same recurrence written as one matrix a token)."""
import copy

import pytest
import torch

import plain_lebelix as P
from lebelix_models import SMALL, make_weights, stored_config, write_model


def test_round_trip_and_registry():
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.config.lebelix import LebelixConfig
    for name, d in SMALL.items():
        c = config_from_dict(d)
        assert isinstance(c, LebelixConfig)
        assert c.to_dict() == d, name
        assert config_from_dict(c.to_dict()) == c


def test_parts_of_the_model_as_data():
    from lumenllm_b200.config import config_from_dict
    spec = config_from_dict(SMALL["X"]).model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3, 4]
    assert [e.cache_from for e in spec.schedule] == [None, None, None, 1, None]
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["head_norm_attention", "latent_attention", "channel_delta", "latent_attention",
                     "head_norm_attention"]
    assert spec.layers[2].ffn is None and spec.layers[0].ffn.kind == "gelu_mlp"
    a = spec.layers[0].mixer.params
    assert (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["value_dim"], a["chunk"], a["softcap"]) == \
        (4, 2, 16, 24, 9, 5.0)
    assert a["sink"] and a["output_gate"] and a["bias"]
    assert a["position"].params["rotary_dim"] == 8
    # the cache of layer 1 serves layer 3 as well: it keeps what the wider window sees
    own, reader = spec.layers[1].mixer.params, spec.layers[3].mixer.params
    assert (own["window"], own["cache_window"], own["shares_cache"]) == (11, 70, False)
    assert (reader["window"], reader["cache_window"], reader["shares_cache"]) == (70, 70, True)
    side = [l.extras["token_input"].params for l in spec.layers]
    assert [s["column"] for s in side] == [0, 8, 16, 24, 32] and side[0]["table_width"] == 40
    assert spec.embedding.params["scale"] == 0.7 and spec.head.params["tied_to"] == "embed"
    # no token input, no mask, no rotation, no cap
    spec = config_from_dict(SMALL["Y"]).model_spec()
    assert all("token_input" not in l.extras for l in spec.layers)
    a = spec.layers[1].mixer.params
    assert a["chunk"] == 0 and a["softcap"] == 0.0 and a["position"].kind == "none"
    assert spec.layers[2].mixer.params["window"] == 0 and spec.layers[2].mixer.params["cache_window"] == 0
    # two readers of one cache, one through a narrower and one through a wider window
    spec = config_from_dict(SMALL["Z"]).model_spec()
    assert [e.cache_from for e in spec.schedule] == [None, None, 0, None, None, 0]
    assert [spec.layers[i].mixer.params["cache_window"] for i in (0, 2, 5)] == [130, 130, 130]


def test_expected_tensors_are_the_designs_names():
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.engine.model import expected_tensors
    for name, d in SMALL.items():
        want = {k: tuple(v.shape) for k, v in make_weights(d, 0).items()}
        got = {k: tuple(shape) for k, (shape, _) in expected_tensors(config_from_dict(d).model_spec()).items()}
        assert got == want, name


def test_low_ranks_come_from_the_tensors_shapes(tmp_path):
    from lumenllm_b200.config import ConfigError, config_from_dict, load_config
    stored = stored_config(SMALL["X"])
    assert "decay_rank" not in stored["layers"][2]["mixer"]
    with pytest.raises(ConfigError, match="decay_rank"):
        config_from_dict(stored).model_spec()
    folder = write_model(SMALL["X"], tmp_path / "m", seed=1)
    cfg = load_config(folder)
    assert (cfg.layers[2].mixer.decay_rank, cfg.layers[2].mixer.gate_rank) == (5, 3)
    assert cfg == config_from_dict(SMALL["X"])


@pytest.mark.parametrize("edit, word", [
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d["layers"][0].update(type="recurrent"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][2]["mixer"].update(kv_heads=4), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=18), "at most"),
    (lambda d: d["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "dense"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=4), "earlier"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=0), "earlier"),
    (lambda d: d["layers"][3]["mixer"].update(kv_rank=48), "equal"),
    (lambda d: d["layers"][0]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda d: d["embedding"].update(scale="big"), "scale"),
])
def test_what_is_refused(edit, word):
    from lumenllm_b200.config import ConfigError, config_from_dict
    d = copy.deepcopy(SMALL["X"])
    edit(d)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_pages_before_the_querys_chunk_are_given_back():
    from lumenllm_b200.cache import PAGE, CacheNeed, KVCache
    chunk = 2 * PAGE + 10
    cache = KVCache({0: CacheNeed(2, 16, v_dim=24, chunk=chunk), 1: CacheNeed(1, 40, window=PAGE + 5, v_dim=32,
                                                                               values_in_keys=True)},
                    16 * PAGE, 2, 16 * PAGE)
    chunked, latent = cache.groups[cache.group_of[0]], cache.groups[cache.group_of[1]]
    s = cache.alloc_slot()
    for step in range(9 * PAGE):
        cache.reserve(s, 1)
        cache.commit(s, 1)
        n = step + 1                                   # the next query sits at position n
        held = {i for i in range(chunked.table.shape[1]) if chunked.table[s, i] != 0}
        assert held == set(range(n // chunk * chunk // PAGE, -(-n // PAGE))), n
        held = {i for i in range(latent.table.shape[1]) if latent.table[s, i] != 0}
        assert held == set(range(max(0, n - (PAGE + 5) + 1) // PAGE, -(-n // PAGE))), n
    cache.check()
    cache.free_slot(s)
    cache.check()
    assert chunked.pool.free_count == latent.pool.free_count == 16


def test_plain_delta_rule_equals_its_matrix_form():
    """The recurrence of the plain implementation against the same written as one transition a
    token: S_t = (I - beta k k^T) diag(g) S_{t-1} + beta k v^T, o = S_t^T q."""
    cfg = SMALL["X"]
    w = {k: v.double() for k, v in make_weights(cfg, 3).items()}
    m, pre = cfg["layers"][2]["mixer"], "l2.mix."
    T, D = 12, cfg["width"]
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(4)).double()
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = P.causal_conv_silu(h @ w[pre + "q"].T, w[pre + "q.conv"]).view(T, G, d)
    k = P.causal_conv_silu(h @ w[pre + "k"].T, w[pre + "k.conv"]).view(T, G, d)
    v = P.causal_conv_silu(h @ w[pre + "v"].T, w[pre + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[pre + "b"].T)
    a = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "dt_bias"]
    g = torch.exp(-torch.exp(w[pre + "A_log"])[None, :, None] * torch.nn.functional.softplus(a).view(T, H, d))
    gate = torch.sigmoid((h @ w[pre + "g1"].T) @ w[pre + "g2"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=torch.float64)
        kk, qq = k[:, hd // (H // G)], q[:, hd // (H // G)]
        for t in range(T):
            A = (torch.eye(d, dtype=torch.float64) - beta[t, hd] * torch.outer(kk[t], kk[t])) @ torch.diag(g[t, hd])
            S = A @ S + beta[t, hd] * torch.outer(kk[t], v[t, hd])
            out[t, hd] = S.T @ qq[t]
    ref = (P.rms_unit(out, cfg["norm"]["eps"]) * w[pre + "norm"] * gate).reshape(T, H * dv) @ w[pre + "o"].T
    got = P.channel_delta(h, w, pre, m, cfg["norm"]["eps"])
    assert float((got - ref).abs().max()) < 1e-10


def test_plain_latent_attention_equals_expanded_keys_and_values():
    """Latent attention of the plain implementation against ordinary attention whose keys are
    [Uk c | shared rotated part] and whose values are Uv c, written out head by head."""
    cfg = SMALL["Z"]
    w = {k: v.double() for k, v in make_weights(cfg, 5).items()}
    m, pre, eps = cfg["layers"][0]["mixer"], "l0.mix.", cfg["norm"]["eps"]
    T = 120
    h = torch.randn(T, cfg["width"], generator=torch.Generator().manual_seed(6)).double()
    got = P.latent_attention(h, w, pre, m, eps, P.latent_of(h, w, pre, m, eps))
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    z = h @ w[pre + "dkv"].T
    c = z[:, :R] / torch.sqrt((z[:, :R] ** 2).mean(-1, keepdim=True) + eps) * w[pre + "dkv.norm"]
    pos = torch.arange(T)
    kr = P.rotate(z[:, None, R:], pos, m["rot"]["base"], m["rot"]["dims"])[:, 0]
    q = (h @ w[pre + "q"].T).view(T, H, d + r)
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for hd in range(H):
        qh = torch.cat([q[:, hd, :d], P.rotate(q[:, hd:hd + 1, d:], pos, m["rot"]["base"], m["rot"]["dims"])[:, 0]], -1)
        kh = torch.cat([c @ w[pre + "uk"][hd * d:(hd + 1) * d].T, kr], -1)
        vh = c @ w[pre + "uv"][hd * dv:(hd + 1) * dv].T
        for i in range(T):
            lo = max(0, i - m["mask"]["size"] + 1)
            p = torch.softmax(kh[lo:i + 1] @ qh[i] * m["scale"], 0)
            out[i, hd] = p @ vh[lo:i + 1]
    ref = out.reshape(T, H * dv) @ w[pre + "o"].T
    assert float((got - ref).abs().max()) < 1e-10

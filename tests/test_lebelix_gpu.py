"""Lebelix in the engine against the plain implementation (tests/plain_lebelix.py): every mechanism
alone, then whole prompts, prompts in portions, decoding token by token, batches of unequal
requests, slots, pages and state that are used again, and greedy generation through the library's
entry point."""
import json

import pytest
import torch

import plain_lebelix as P
from lebelix_models import SMALL, attention, config, delta, dense, latent, layer, make_weights, write_model

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
DTYPES = ["float32", "bfloat16"]


def tol(dtype):
    return 3e-5 if dtype in (F32, "float32") else 3e-2


def close(got, ref, dtype, what=""):
    got, ref = got.detach().float().cpu(), ref.float()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), what
    err, scale = float((got - ref).abs().max()), max(1.0, float(ref.abs().max()))
    assert err <= tol(dtype) * scale, f"{what}: {err:.3e} > {tol(dtype) * scale:.3e}"


def runtime(dtype):
    from lumenllm_b200.parts import Runtime
    return Runtime(torch.device("cuda", 0), dtype)


def tokens_of(cfg, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


def cut(y, sizes):
    out, at = [], 0
    for n in sizes:
        out.append(y[at:at + n])
        at += n
    assert at == y.shape[0]
    return out


def mixer_part(m, D, dtype, seed, edit=None, eps=1e-6):
    """A one-layer model's mixer, built as the engine builds it; its weights as the plain
    implementation reads them (what bfloat16 stores, widened)."""
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.parts import build_part
    cfg = config(8, D, eps, [layer(m, None)])
    w = make_weights(cfg, seed)
    if edit is not None:
        edit(w)
    spec = config_from_dict(cfg).model_spec().layers[0].mixer
    part = build_part("mixer", spec, {k: v.cuda() for k, v in w.items()}, runtime(dtype))
    return part, {k: v.float() for k, v in w.items()}


def run_mixer(mixer, rt, pieces_by_seq, twice=False):
    """Feeds sequences' rows piece by piece through a mixer alone. pieces_by_seq: for each sequence
    a list of row blocks (an empty block: the sequence pauses that step). With `twice` everything
    runs a second time on the slots, pages and state rows that the first run gave back. Returns
    each sequence's updates in order."""
    from lumenllm_b200.cache import KVCache
    from lumenllm_b200.engine.context import EntryView, StepEntry, build_context
    need, shape = mixer.cache_need(), mixer.state_shape()
    cache = KVCache({0: need} if need is not None else {}, 4096, 4, 4096, dtype=rt.dtype, device=rt.device,
                    state_shapes={0: shape} if shape is not None else None)
    for round_ in range(2 if twice else 1):
        slots = [cache.alloc_slot() for _ in pieces_by_seq]
        outs = [[] for _ in pieces_by_seq]
        for step in range(max(len(p) for p in pieces_by_seq)):
            live = [b for b, p in enumerate(pieces_by_seq) if step < len(p) and p[step].shape[0]]
            if not live:
                continue
            ctx, _ = build_context(cache, rt, [StepEntry(slots[b], [0] * pieces_by_seq[b][step].shape[0]) for b in live])
            y = torch.cat([pieces_by_seq[b][step] for b in live]).to(rt.dtype).cuda()
            out = mixer.forward(y, ctx, EntryView(ctx, 0, 0 if need is not None else None, True))
            out = (out.sum(0) if out.dim() == 3 else out).float().cpu()
            at = 0
            for b in live:
                n = pieces_by_seq[b][step].shape[0]
                outs[b].append(out[at:at + n])
                cache.commit(slots[b], n)
                at += n
        for s in slots:
            cache.free_slot(s)
        cache.check()
    return [torch.cat(o) for o in outs]


def rows(T, D, dtype, seed, std=1.0):
    return (torch.randn(T, D, generator=torch.Generator().manual_seed(seed)) * std).to(dtype).float()


# ------------------------------------------------------------------ mechanisms alone

@pytest.mark.parametrize("dtype", [F32, BF16])
def test_gelu_and_the_gated_token_vectors(dtype):
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(0)
    z = torch.randn(3, 9, 70, generator=g) * 2.5
    close(K.gelu_tanh(z.cuda(), dtype), P.gelu_tanh(z.sum(0)), dtype, "gelu")
    table = torch.randn(30, 44, generator=g).to(BF16)
    tok = torch.tensor([0, 29, 7, 7, 13, 2, 2, 1, 28], dtype=torch.int32)
    zz = torch.randn(2, 9, 12, generator=g)
    ref = P.gelu_tanh(zz.sum(0)) * table.float()[tok.long()][:, 20:32]
    for t in (table, table.float()):
        close(K.token_gate(zz.cuda(), tok.cuda(), t.cuda(), 20, dtype), ref, dtype, "token gate")


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("pending_parts", [0, 1, 3])
def test_per_layer_token_input(dtype, pending_parts):
    """The part after a layer's sublayers: it takes in what is pending, gates the layer's own token
    vectors by the stream, and hands on an update that is normed before it is added."""
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.engine.context import StepEntry, build_context
    from lumenllm_b200.cache import KVCache
    from lumenllm_b200.ops import kernels as K
    from lumenllm_b200.parts import build_part
    D, V, side, N = 56, 40, 12, 11
    cfg = config(V, D, 1e-5, [layer(attention(2, 1, 8, 8, 0.3), None) for _ in range(3)], side=side)
    w = make_weights(cfg, 21)
    rt = runtime(dtype)
    spec = config_from_dict(cfg).model_spec().layers[1].extras["token_input"]
    part = build_part("token_input", spec, {k: v.cuda() for k, v in w.items()}, rt)
    wf = {k: v.float() for k, v in w.items()}
    g = torch.Generator().manual_seed(22)
    h = torch.randn(N, D, generator=g)
    pend = torch.randn(pending_parts, N, D, generator=g) if pending_parts else None
    toks = torch.randint(0, V, (N,), generator=g)
    x = h + (pend.sum(0) if pend is not None else 0)
    if dtype == BF16:
        x_read = x.to(BF16).float()          # the gate's product reads the stream in the run's type
    else:
        x_read = x
    ref = x + P.token_side(x_read, toks, wf, 1, side, 1e-5)
    cache = KVCache({}, 256, 2, 256, dtype=rt.dtype, device=rt.device)
    ctx, _ = build_context(cache, rt, [StepEntry(cache.alloc_slot(), toks.tolist())])
    hc = h.clone().cuda()
    h2, upd = part.forward(hc, None if pend is None else pend.cuda(), ctx)
    close(h2, x, F32, "the stream after the sublayers")
    out = h2.clone()
    K.postnorm_add_rmsnorm(out, upd.delta, upd.bias, upd.weight, upd.eps, None, 0.0, F32)
    close(out, ref, dtype, "the stream with the token input")


ATTENTIONS = [attention(4, 2, 16, 24, 0.3, size=9, rot=8, softcap=5.0),
              attention(6, 6, 32, 32, 0.11, size=70),                       # no rotation, no cap
              attention(3, 1, 32, 16, 0.2, rot=32, base=500.0, softcap=2.0),   # no mask
              attention(2, 2, 64, 128, 0.15, size=64, rot=16, softcap=30.0),   # chunks of exactly a page
              attention(5, 5, 24, 8, 0.5, size=1, rot=24),                  # every query sees itself only
              attention(12, 1, 20, 10, 0.4, size=130, rot=4, softcap=50.0),
              attention(4, 2, 128, 128, 0.09, size=100, rot=64, softcap=20.0),
              # key and value sizes that the tensor-core kernels of a bfloat16 run take
              attention(4, 1, 64, 64, 0.125, size=96, rot=32, softcap=50.0),
              attention(2, 2, 64, 64, 0.2, size=200),                       # uncapped: sink and gate alone
              attention(16, 1, 128, 128, 0.09, rot=128, softcap=3.0),       # no mask, sixteen heads a kv head
              attention(3, 3, 128, 128, 0.1, size=64)]


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("m", ATTENTIONS)
def test_attention_part(m, dtype):
    """The mixer alone: a prompt, then the same sequence continued in portions and token by token."""
    D, T = 48, 210
    mixer, w = mixer_part(m, D, dtype, seed=5)
    y = rows(T, D, dtype, 6)
    ref = P.attention(y, w, "l0.mix.", m, 1e-6)
    got = run_mixer(mixer, runtime(dtype), [cut(y, [131, 2, 40] + [1] * 37)], twice=True)[0]
    close(got, ref, dtype)


@pytest.mark.parametrize("d", [32, 64])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_the_sink_takes_weight_and_the_cap_bounds_scores(dtype, d):
    """Keys that all point away from the queries: nearly all weight goes to the sink, and the output
    is small, where an ordinary softmax would give an average of the values. Then loud queries and
    keys with a low cap: the weights stay spread where uncapped scores would pick one key."""
    H, T = 2, 50
    D = H * d
    m = attention(H, H, d, d, 1.0, size=40, softcap=30.0)

    def away(w):
        for name in ("q", "k", "v", "g"):
            w["l0.mix." + name] = torch.eye(D).to(BF16)
        w["l0.mix.k"] = -torch.eye(D).to(BF16)
        for name in ("q", "k", "v"):
            w["l0.mix." + name + ".b"] = torch.zeros(D).to(BF16)
        w["l0.mix.q.norm"] = w["l0.mix.k.norm"] = torch.ones(d).to(BF16)
    mixer, w = mixer_part(m, D, dtype, seed=7, edit=away)
    u = torch.nn.functional.normalize(torch.randn(D, generator=torch.Generator().manual_seed(8)), dim=0)
    y = (rows(T, D, dtype, 9, 0.05) + 3 * u).to(dtype).float()      # every token points the same way
    ref = P.attention(y, w, "l0.mix.", m, 1e-6)
    plain_softmax = P.attention(y, w, "l0.mix.", m, 1e-6, sink=0.0)
    assert float((plain_softmax - ref).abs().max()) > 0.3 * float(plain_softmax.abs().max())
    for sizes in ([T], [30] + [1] * 20):
        close(run_mixer(mixer, runtime(dtype), [cut(y, sizes)])[0], ref, dtype, f"sink, cut as {sizes[:3]}")
    # the cap
    m2 = attention(H, H, d, d, 4.0, softcap=1.5)
    mixer, w = mixer_part(m2, D, dtype, seed=10)
    y = rows(T, D, dtype, 11, 2.0)
    ref = P.attention(y, w, "l0.mix.", m2, 1e-6)
    uncapped = P.attention(y, w, "l0.mix.", dict(m2, softcap=None), 1e-6)
    assert float((uncapped - ref).abs().max()) > 0.2 * float(ref.abs().max())
    close(run_mixer(mixer, runtime(dtype), [cut(y, [35] + [1] * 15)])[0], ref, dtype, "cap")


def loud_pair(w, D, shift):
    """Queries and values are the inputs themselves and keys the inputs rolled by `shift` channels."""
    for name in ("q", "k", "v"):
        w["l0.mix." + name] = torch.eye(D).to(BF16)
        w["l0.mix." + name + ".b"] = torch.zeros(D).to(BF16)
    w["l0.mix.k"] = torch.roll(torch.eye(D), shift, dims=0).to(BF16)


@pytest.mark.parametrize("d", [32, 64])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_one_loud_key_at_every_edge_of_a_chunk(dtype, decode, d):
    """One earlier token is made loud so that its KEY points where the last QUERY points: this single
    key takes nearly all of the query's weight where it is in sight and none where it is not: on both
    sides of the chunk's edge, at page borders inside the chunk, at the chunk's far end among
    hundreds of keys, and the token just before the query. Beside each edge case stands the chunk
    size that differs by one: the plain result under it must be far from the right one, else the
    case would show nothing. Chunks are counted from the sequence's first token also when the
    sequence came in portions."""
    H = 2
    D = H * d
    size = 150
    T = 2 * size + 140                   # the last query is the 140th token of the third chunk
    m = attention(H, H, d, d, 1.0, size=size)

    def edit(w):
        loud_pair(w, D, 7)
        w["l0.mix.q.norm"] = w["l0.mix.k.norm"] = torch.ones(d).to(BF16)
    mixer, w = mixer_part(m, D, dtype, seed=7, edit=edit)
    g = torch.Generator().manual_seed(8)
    u = torch.nn.functional.normalize(torch.randn(D, generator=g), dim=0)
    query, lo = T - 1, 2 * size
    # with chunks one longer the third chunk starts two tokens later, with chunks one shorter two earlier
    cases = [(0, None), (lo - 3, attention(H, H, d, d, 1.0, size=size - 2)), (lo - 1, attention(H, H, d, d, 1.0, size=size - 1)),
             (lo, attention(H, H, d, d, 1.0, size=size + 1)), (lo + 1, attention(H, H, d, d, 1.0, size=size + 1)),
             (319, None), (320, None), (383, None), (384, None), (query - 1, None)]
    for loud, off_by_one in cases:
        y = torch.randn(T, D, generator=g) * 0.3
        y[loud] += 12 * torch.roll(u, -7)
        y[query] += 12 * u
        y = y.to(dtype).float()
        ref = P.attention(y, w, "l0.mix.", m, 1e-6)
        if off_by_one is not None:
            wrong = P.attention(y, w, "l0.mix.", off_by_one, 1e-6)
            assert float((wrong[query] - ref[query]).abs().max()) > 10 * tol(BF16) * max(1.0, float(ref.abs().max())), loud
        pieces = cut(y, [T - 45, 3, 2] + [1] * 40) if decode else [y]
        got = run_mixer(mixer, runtime(dtype), [pieces])[0]
        close(got, ref, dtype, f"loud key {loud}")


LATENTS = [latent(2, 8, 16, 24, 40, 0.2, size=11, rot=8),
           latent(4, 24, 8, 16, 64, 0.15, rot=8, base=1e6),            # no window
           latent(3, 16, 32, 8, 96, 0.25, size=70, rot=32),
           latent(1, 64, 64, 128, 192, 0.1, size=64, rot=64),
           latent(5, 12, 4, 20, 36, 0.3, size=1, rot=4),
           latent(2, 32, 16, 48, 52, 0.2, size=300),                  # no rotation at all
           # widths the tensor-core kernel takes: an odd number of 16-value steps and heads that do not
           # divide a block's rows; a latent wider than 256; more heads than a block has rows
           latent(5, 16, 16, 32, 160, 0.2, size=45, rot=16),
           latent(3, 32, 32, 64, 320, 0.1, size=130, rot=32),
           latent(70, 8, 16, 8, 48, 0.2, size=33, rot=8)]


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("m", LATENTS)
def test_latent_attention_part(m, dtype):
    """The mixer alone over its latent cache: a prompt, then portions and single tokens."""
    D, T = 40, 210
    mixer, w = mixer_part(m, D, dtype, seed=15)
    y = rows(T, D, dtype, 16)
    ref = P.latent_attention(y, w, "l0.mix.", m, 1e-6, P.latent_of(y, w, "l0.mix.", m, 1e-6))
    got = run_mixer(mixer, runtime(dtype), [cut(y, [131, 2, 40] + [1] * 37)], twice=True)[0]
    close(got, ref, dtype)


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_one_loud_latent_at_every_edge_of_the_window(dtype, decode):
    """Latent attention whose up-projections are identities, so that a head's plain key is the
    normed latent itself: one earlier token's latent is made to point where the last query points.
    It takes the query's weight just inside the window and none just outside, and at page
    borders; the window that differs by one gives a far result."""
    H, d, r, R, D = 1, 48, 16, 48, 64
    size = 130
    T = 300
    m = latent(H, d, r, R, R, 1.0, size=size, rot=16)

    def edit(w):
        w["l0.mix.q"] = torch.eye(d + r, D).to(BF16)
        w["l0.mix.dkv"] = torch.roll(torch.eye(R + r, D), 5, dims=1).to(BF16)     # c_i = y_{i+5}
        w["l0.mix.dkv.norm"] = torch.ones(R).to(BF16)
        w["l0.mix.uk"] = torch.eye(d, R).to(BF16)
        w["l0.mix.uv"] = torch.eye(R).to(BF16)
    mixer, w = mixer_part(m, D, dtype, seed=17, edit=edit)
    g = torch.Generator().manual_seed(18)
    u = torch.zeros(D)
    u[:d] = torch.nn.functional.normalize(torch.randn(d, generator=g), dim=0)
    query = T - 1
    lo = query - size + 1
    cases = [(0, None), (63, None), (lo - 1, latent(H, d, r, R, R, 1.0, size=size + 1, rot=16)),
             (lo, latent(H, d, r, R, R, 1.0, size=size - 1, rot=16)), (191, None), (192, None), (255, None),
             (256, None), (query - 1, None)]
    for loud, off_by_one in cases:
        y = torch.randn(T, D, generator=g) * 0.3
        y[loud] += 12 * torch.roll(u, 5)
        y[query] += 3 * u
        y = y.to(dtype).float()
        lat = P.latent_of(y, w, "l0.mix.", m, 1e-6)
        ref = P.latent_attention(y, w, "l0.mix.", m, 1e-6, lat)
        if off_by_one is not None:
            wrong = P.latent_attention(y, w, "l0.mix.", off_by_one, 1e-6, lat)
            assert float((wrong[query] - ref[query]).abs().max()) > 10 * tol(BF16) * max(1.0, float(ref.abs().max())), loud
        pieces = cut(y, [T - 45, 3, 2] + [1] * 40) if decode else [y]
        close(run_mixer(mixer, runtime(dtype), [pieces])[0], ref, dtype, f"loud latent {loud}")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_a_reader_of_another_layers_latents_looks_through_its_own_window(dtype):
    """Two readers of one latent cache, one through a narrower and one through a wider window than
    the layer that writes it: each sees what its own window says, in a prompt and decoded."""
    from lumenllm_b200.engine import Engine, StepEntry
    import tempfile
    cfg = config(40, 48, 1e-6, [layer(latent(2, 16, 8, 8, 32, 0.2, size=20, rot=8), None),
                                layer(latent(3, 8, 8, 16, 32, 0.3, size=5, rot=8, kv_from=0), None),
                                layer(latent(1, 24, 8, 8, 32, 0.2, size=90, rot=8, kv_from=0), None)])
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_model(cfg, tmp, seed=19)
        _, w = P.load_model(folder)
        toks = tokens_of(cfg, (160,), seed=20)[0]
        ref = P.forward(cfg, w, toks)
        eng = Engine.from_folder(folder, dtype={F32: "float32", BF16: "bfloat16"}[dtype], max_tokens=1024, max_slots=2)
        slot = eng.alloc_slot()
        got = [eng.step([StepEntry(slot, toks[:100], list(range(100)))])]
        got += [eng.step([StepEntry(slot, [t], [0])]) for t in toks[100:]]
        close(torch.cat(got), ref, dtype)
        eng.check_kernels()


DELTAS = [delta(2, 1, 24, 16, 3, 5, 3),
          delta(3, 3, 8, 40, 1, 1, 12),            # one tap: no convolution state
          delta(4, 2, 64, 32, 4, 12, 8),
          delta(1, 1, 128, 128, 2, 4, 4),
          delta(6, 2, 16, 8, 4, 2, 1),
          delta(2, 2, 40, 24, 3, 7, 9),
          delta(2, 1, 6, 9, 2, 3, 2),              # a column of the state in one thread
          delta(1, 1, 272, 12, 2, 4, 4)]           # key channels beyond 256: sixteen rows a thread


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("m", DELTAS)
def test_delta_rule_part_in_any_portions(m, dtype):
    """Two sequences fed in unequal portions (down to one token, one of them pausing) give what the
    whole sequences give: the convolution's last inputs and the heads' states are carried across
    every cut; the slots' next users start from zeros."""
    D = 40
    mixer, w = mixer_part(m, D, dtype, seed=11)
    g = torch.Generator().manual_seed(12)
    ys = [torch.randn(n, D, generator=g).to(dtype).float() for n in (61, 23)]
    refs = [P.channel_delta(y, w, "l0.mix.", m, 1e-6) for y in ys]
    pieces = [cut(ys[0], [1, 1, 2, 37, 0, 20]), cut(ys[1], [3, 0, 1, 1, 17, 1])]
    for got, ref in zip(run_mixer(mixer, runtime(dtype), pieces, twice=True), refs):
        close(got, ref, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_the_state_remembers_far_back_and_forgets_by_channel(dtype):
    """Decays close to one and one loud early token: what the state holds of that token decides the
    outputs hundreds of tokens later, whole, in portions and decoded one by one (the plain result
    without the early token is far from the right one, so a lost or restarted state shows). Then
    half of the key channels are made to forget fast: the plain result with one decay a head
    (the channels' mean) is far from the right one, so a decay that is not per channel shows."""
    d = 64
    m = delta(2, 1, d, 24, 2, 3, 3)
    D, T = 32, 420

    def slow(w):
        w["l0.mix.A_log"] = torch.full((2,), -7.0).to(BF16)
        w["l0.mix.dt_bias"] = torch.full((2 * d,), -1.0).to(BF16)
        w["l0.mix.a2"] = torch.zeros(2 * d, 3).to(BF16)
    mixer, w = mixer_part(m, D, dtype, seed=13, edit=slow)
    g = torch.Generator().manual_seed(14)
    y = torch.randn(T, D, generator=g) * 0.2
    y[3] *= 40
    y = y.to(dtype).float()
    ref = P.channel_delta(y, w, "l0.mix.", m, 1e-6)
    quiet = y.clone()
    quiet[3] /= 40
    assert float((P.channel_delta(quiet, w, "l0.mix.", m, 1e-6)[-1] - ref[-1]).abs().max()) > 0.2 * float(ref[-1].abs().max())
    for sizes in ([T], [200, 2, 2, 150, 66], [380] + [1] * 40):
        close(run_mixer(mixer, runtime(dtype), [cut(y, sizes)])[0], ref, dtype, f"cut as {sizes[:4]}")

    def by_channel(w):
        slow(w)
        b = torch.full((2, d), -1.0)
        b[:, ::2] = 6.0
        w["l0.mix.A_log"] = torch.full((2,), -2.0).to(BF16)
        w["l0.mix.dt_bias"] = b.reshape(-1).to(BF16)
    mixer, w = mixer_part(m, D, dtype, seed=13, edit=by_channel)
    y = rows(90, D, dtype, 15)
    ref = P.channel_delta(y, w, "l0.mix.", m, 1e-6)
    mean = dict(w)
    mean["l0.mix.dt_bias"] = torch.full((2 * d,), float(w["l0.mix.dt_bias"].mean()))
    assert float((P.channel_delta(y, mean, "l0.mix.", m, 1e-6) - ref).abs().max()) > 0.1 * float(ref.abs().max())
    close(run_mixer(mixer, runtime(dtype), [cut(y, [50, 2] + [1] * 38)])[0], ref, dtype, "decay by channel")


# ------------------------------------------------------------------ the engine

@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {name: write_model(cfg, tmp_path_factory.mktemp(f"lebelix{name}"), seed=60 + i)
            for i, (name, cfg) in enumerate(SMALL.items())}


@pytest.fixture(scope="module")
def plain(models):
    """name -> (config, float32 weights, plain logits by token tuple)."""
    return {name: (*P.load_model(folder), {}) for name, folder in models.items()}


def plain_logits(plain, name, tokens):
    cfg, w, memo = plain[name]
    key = tuple(tokens)
    if key not in memo:
        memo[key] = P.forward(cfg, w, list(tokens))
    return memo[key]


def engine_of(models, name, dtype, **kw):
    from lumenllm_b200.engine import Engine
    kw.setdefault("max_tokens", 4096)
    return Engine.from_folder(models[name], dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_whole_prompts(name, dtype, models, plain):
    from lumenllm_b200.engine import StepEntry
    eng = engine_of(models, name, dtype)
    for toks in tokens_of(SMALL[name], (1, 2, 37, 201) + ((640,) if name == "Z" else ()), seed=1):
        slot = eng.alloc_slot()
        got = eng.step([StepEntry(slot, toks, list(range(len(toks))))])
        eng.free_slot(slot)
        close(got, plain_logits(plain, name, toks), dtype, f"{name} {len(toks)} tokens")
    eng.check_kernels()
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_residual_stream_after_every_layer(name, dtype, models, plain):
    """Layer by layer: the stream with everything a layer adds, against the plain one. What a
    layer hands on is either a stack of partial sums or an update that is normed before it is
    added."""
    from lumenllm_b200.engine import StepEntry
    from lumenllm_b200.engine.context import EntryView
    from lumenllm_b200.parts.norm import NormedUpdate
    cfg, w, _ = plain[name]
    toks = tokens_of(cfg, (45,), seed=2)[0]
    streams = []
    P.forward(cfg, w, toks, streams)
    eng = engine_of(models, name, dtype)
    slot = eng.alloc_slot()
    ctx = eng.build_context([StepEntry(slot, toks)])
    h, pending = eng.model.embedding.forward(ctx.tokens, ctx), None
    for i, e in enumerate(eng.model.schedule):
        group = i if e.cache_from is None else e.cache_from
        view = EntryView(ctx, i, group if group in ctx.cache.group_of else None, e.cache_from is None)
        h, pending = eng.model.blocks[e.layer].forward(h, pending, ctx, view)
        x = h.float().cpu()
        if isinstance(pending, NormedUpdate):
            z = pending.delta.float()
            z = (z.sum(0) if z.dim() == 3 else z).cpu()
            x = x + P.rms_unit(z, pending.eps) * pending.weight.float().cpu()
        elif pending is not None:
            x = x + (pending.sum(0) if pending.dim() == 3 else pending).float().cpu()
        close(x, streams[i], dtype, f"{name} after layer {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_prompt_in_portions_and_decoded_token_by_token(name, dtype, models, plain):
    from lumenllm_b200.engine import StepEntry
    toks = tokens_of(SMALL[name], (230,), seed=3)[0]
    ref = plain_logits(plain, name, toks)
    eng = engine_of(models, name, dtype)
    for cuts in ([2, 2, 3, 60, 1, 64, 5, 93], [127, 1, 1, 101], [100] + [1] * 130, [1] * 40):
        slot = eng.alloc_slot()
        got, at = [], 0
        for n in cuts:
            got.append(eng.step([StepEntry(slot, toks[at:at + n], list(range(n)))]))
            at += n
        eng.free_slot(slot)
        close(torch.cat(got), ref[:at], dtype, f"{name} cut as {cuts[:4]}...")
    eng.check_kernels()
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_a_batch_of_unequal_requests_equals_each_alone(name, dtype, models, plain):
    """Prompts of unequal lengths in one step, then decoded together while the shorter requests
    leave; their slots, pages and state rows go to a second batch at once."""
    from lumenllm_b200.engine import StepEntry
    eng = engine_of(models, name, dtype, max_tokens=1024, max_slots=4)
    lens, tail = (1, 66, 140, 17), (3, 30, 12, 20)
    for round_ in range(2):
        seqs = tokens_of(SMALL[name], [n + t for n, t in zip(lens, tail)], seed=10 + round_)
        refs = [plain_logits(plain, name, s) for s in seqs]
        slots = [eng.alloc_slot() for _ in seqs]
        got = eng.step([StepEntry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, lens)])
        close(got, torch.cat([r[:n] for r, n in zip(refs, lens)]), dtype, f"{name} prompts")
        live = list(range(len(seqs)))
        rows_, want = [], []
        for t in range(max(tail)):
            live = [b for b in live if t < tail[b]]
            rows_.append(eng.step([StepEntry(slots[b], [seqs[b][lens[b] + t]], [0]) for b in live]))
            want.append(torch.stack([refs[b][lens[b] + t] for b in live]))
            for b in [b for b in live if t + 1 == tail[b]]:
                eng.free_slot(slots[b])
        close(torch.cat(rows_), torch.cat(want), dtype, f"{name} decoded together")
        eng.cache.check()
        assert not eng.cache.slots.held
    eng.check_kernels()


@pytest.mark.parametrize("name", ["X", "Z"])
def test_decoded_logits_do_not_depend_on_the_batch(name, models):
    """The same request decoded alone and among others: the same bits, in both precisions."""
    from lumenllm_b200.engine import StepEntry
    for dtype in DTYPES:
        eng = engine_of(models, name, dtype)
        seqs = tokens_of(SMALL[name], (90, 150, 31), seed=20)

        def run(members):
            slots = {b: eng.alloc_slot() for b in members}
            eng.step([StepEntry(slots[b], seqs[b][:-8]) for b in members])
            out_rows = []
            for t in range(8):
                out = eng.step([StepEntry(slots[b], [seqs[b][len(seqs[b]) - 8 + t]], [0]) for b in members])
                out_rows.append(out[members.index(0)].clone())
            for s in slots.values():
                eng.free_slot(s)
            return torch.stack(out_rows)
        assert torch.equal(run([0]), run([1, 0, 2])), (name, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_while_chunks_and_windows_pass(dtype, models, plain):
    """A request decoded one token at a time over several pages: chunks of 9 and 70 positions and
    windows of 11 and 70 keys pass over decoded tokens and page borders, the layers whose sight is
    bounded hold few pages at a time, and the delta rule carries its state all the way."""
    from lumenllm_b200.cache import PAGE
    from lumenllm_b200.engine import StepEntry
    name = "X"
    toks = tokens_of(SMALL[name], (3 * PAGE + 20,), seed=30)[0]
    ref = plain_logits(plain, name, toks)
    eng = engine_of(models, name, dtype, max_tokens=6 * PAGE, max_slots=2)
    slot = eng.alloc_slot()
    got = [eng.step([StepEntry(slot, toks[:5], list(range(5)))])]
    for t in range(5, len(toks)):
        got.append(eng.step([StepEntry(slot, [toks[t]], [0])]))
        assert all(g.n_held[slot] <= 3 for g in eng.cache.groups)
    close(torch.cat(got), ref, dtype)
    other = eng.alloc_slot()                      # the pages given back serve another request meanwhile
    got = eng.step([StepEntry(other, toks[:2 * PAGE], [2 * PAGE - 1])])
    close(got, ref[2 * PAGE - 1:2 * PAGE], dtype)
    eng.free_slot(slot)
    eng.free_slot(other)
    eng.cache.check()
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_model_whose_rows_are_no_multiples_of_16_bytes(dtype, tmp_path):
    """Width 44, heads of 6 keys and 10 values, a latent of 18 + 6, a recurrence of 7 key channels,
    a token input of 3: no row of any matrix is a multiple of 16 bytes, so the products go the
    ways that need no alignment."""
    from lumenllm_b200.engine import Engine, StepEntry
    cfg = config(61, 44, 1e-5, [layer(attention(3, 1, 6, 10, 0.4, size=20, rot=4, softcap=9.0), dense(30)),
                                layer(latent(3, 10, 6, 5, 18, 0.3, size=13, rot=2), dense(9)),
                                layer(delta(2, 1, 7, 5, 2, 3, 1), None),
                                layer(latent(1, 6, 6, 7, 18, 0.3, size=40, rot=2, kv_from=1), None)], scale=2.0, side=3)
    folder = write_model(cfg, tmp_path / "m", seed=90)
    _, w = P.load_model(folder)
    toks = tokens_of(cfg, (90,), seed=91)[0]
    ref = P.forward(cfg, w, toks)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=2)
    slot = eng.alloc_slot()
    got = [eng.step([StepEntry(slot, toks[:70], list(range(70)))])]
    got += [eng.step([StepEntry(slot, [toks[t]], [0])]) for t in range(70, 90)]
    close(torch.cat(got), ref, dtype)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_model_of_delta_rule_layers_only(dtype, tmp_path):
    """No cache group at all: the sequences' state is everything that is kept; a prompt, portions,
    single tokens, and two requests in a batch."""
    from lumenllm_b200.engine import Engine, StepEntry
    cfg = config(50, 48, 1e-5, [layer(delta(3, 1, 16, 12, 3, 2, 2), dense(40)),
                                layer(delta(2, 2, 8, 36, 2, 3, 5), None)])
    folder = write_model(cfg, tmp_path / "m", seed=80)
    _, w = P.load_model(folder)
    a, b = tokens_of(cfg, (150, 40), seed=81)
    ra, rb = P.forward(cfg, w, a), P.forward(cfg, w, b)
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=2)
    assert not eng.cache.groups
    sa, sb = eng.alloc_slot(), eng.alloc_slot()
    got = eng.step([StepEntry(sa, a[:100], list(range(100))), StepEntry(sb, b[:7], list(range(7)))])
    close(got, torch.cat([ra[:100], rb[:7]]), dtype)
    got = eng.step([StepEntry(sa, a[100:103], [0, 1, 2]), StepEntry(sb, b[7:39], list(range(32)))])
    close(got, torch.cat([ra[100:103], rb[7:39]]), dtype)
    out = [eng.step([StepEntry(sa, [a[t]], [0])] + ([StepEntry(sb, [b[39]], [0])] if t == 103 else []))
           for t in range(103, 150)]
    close(torch.cat([r[:1] for r in out]), ra[103:], dtype)
    close(out[0][1:], rb[39:], dtype)
    eng.check_kernels()


def test_a_long_prompt_whose_products_add_into_the_stream(tmp_path):
    """A prompt long and wide enough for the output products to add their result to the residual
    stream in their epilogue (no update is handed on then), with every kind of mixer."""
    from lumenllm_b200.engine import Engine, StepEntry
    from lumenllm_b200.ops import kernels as K
    cfg = config(64, 1024, 1e-6, [
        layer(attention(4, 2, 64, 64, 0.125, size=300, rot=64, softcap=30.0), dense(512)),
        layer(latent(4, 64, 32, 64, 256, 0.1, size=500, rot=32), dense(256)),
        layer(delta(4, 2, 64, 64, 4, 16, 16), dense(512)),
        layer(latent(2, 32, 32, 128, 256, 0.1, size=100, rot=32, kv_from=1), None)], side=32)
    T = 4900
    assert K.gemm_tc_adds(T, 1024)
    folder = write_model(cfg, tmp_path / "wide", seed=70)
    toks = tokens_of(cfg, (T,), seed=71)[0]
    want = [0, 1, 299, 300, 301, 2047, T - 2, T - 1]
    _, w = P.load_model(folder)
    ref = P.forward(cfg, w, toks)[want]
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=8192)
    slot = eng.alloc_slot()
    got = eng.step([StepEntry(slot, toks, want)])
    close(got, ref, "bfloat16")
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype, models, plain):
    """build(EngineConfig).generate: batches, the scheduler's run-ahead and captured steps."""
    from lumenllm_b200 import EngineConfig, GenerateRequest, build
    name = "Z"
    cfg, w, _ = plain[name]
    built = build(EngineConfig(model_path=str(models[name]), dtype=dtype, context_size=512, max_batch=3))
    assert built.engine.model.graph_safe
    prompts = tokens_of(cfg, (70, 3, 29, 130), seed=40)
    outs = built.generate([GenerateRequest(p, 10) for p in prompts], eos_token_ids=[])
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "length" and len(o.tokens) == 10
        lg = P.forward(cfg, w, list(p) + o.tokens)
        for k, tok in enumerate(o.tokens):
            row = lg[len(p) - 1 + k]
            gap = float(row.max() - row[tok])     # 0 where the plain choice was made
            assert gap <= (1e-4 if dtype == "float32" else 0.05 * max(1.0, float(row.abs().max()))), (k, gap)
        if dtype == "float32":
            assert o.tokens == P.generate_greedy(cfg, w, p, 10)
    built.engine.check_kernels()


def test_command_line_generates(models, capsys):
    from lumenllm_b200.cli import main
    rc = main(["generate", "--model", str(models["X"]), "--prompt-tokens", "5,6,7", "--prompt-tokens", "1",
               "--max-tokens", "4", "--ctx-size", "128", "--format", "json", "--dtype", "float32"])
    assert rc == 0
    outs = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    cfg, w = P.load_model(models["X"])
    assert [o["tokens"] for o in outs] == [P.generate_greedy(cfg, w, p, 4) for p in ([5, 6, 7], [1])]


def test_trace_replay_writes_the_wanted_logits(models, plain, tmp_path):
    """bin/trace_run as a user starts it: a batch of two prompts, decoded together, one request
    ending early; the files hold the plain logits at the wanted places."""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    name = "Y"
    cfg = SMALL[name]
    a, b = tokens_of(cfg, (40, 9), seed=50)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]},
                                     {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[30]], "want": []},
                                     {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]}]
    steps += [{"step": 2 + t, "entries": [{"id": "a", "tokens": [a[31 + t]], "want": [0]}],
               "end": ["a"] if t == 8 else []} for t in range(9)]
    runner = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, str(runner), "--model", str(models[name]), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "128"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [l for l in done.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    ra, rb = plain_logits(plain, name, a), plain_logits(plain, name, b)
    read = lambda s: torch.from_numpy(np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy())
    close(read(0), torch.stack([ra[0], ra[29], rb[7]]), F32, "prompts")
    close(read(1), rb[8:9], F32, "the short request's last token")
    for t in range(9):
        close(read(2 + t), ra[31 + t:32 + t], F32, f"decoded {t}")


# ------------------------------------------------------------------ the tensor-core kernels of latent attention alone
def _latent_case(lens, starts, H, W, seed, n_pages=24):
    """A latent cache [pages, 1, 64, W] that holds starts[b] + lens[b] rows a sequence on pages that
    are not in order, and queries [sum lens, H, W] for every sequence's last lens[b] positions."""
    g = torch.Generator().manual_seed(seed)
    totals = [s + n for s, n in zip(starts, lens)]
    table = torch.zeros(len(lens), max((t + 63) // 64 for t in totals), dtype=torch.int32)
    free = list(range(n_pages - 1, 0, -1))
    cache = torch.zeros(n_pages, 1, 64, W)
    rows = []
    for b, t in enumerate(totals):
        r = torch.randn(t, W, generator=g).to(BF16).float()
        rows.append(r)
        for p in range((t + 63) // 64):
            pg = free.pop(2 if len(free) > 2 else 0)
            table[b, p] = pg
            n = min(64, t - 64 * p)
            cache[pg, 0, :n] = r[64 * p:64 * p + n]
    q = [(0.3 * torch.randn(n, H, W, generator=g)).to(BF16).float() for n in lens]
    return table, cache, rows, q


@pytest.mark.parametrize("H,W,dv,window", [(3, 64, 48, 0), (16, 176, 160, 45), (70, 64, 40, 33), (4, 352, 320, 100),
                                           (2, 96, 96, 1), (1, 32, 8, 64)])
def test_latent_attention_kernel_against_plain_sums(H, W, dv, window):
    """Prompts, a prompt's later portion and single tokens in one launch: (token, head) rows that
    straddle tokens, more heads than a block has rows, windows that end inside a tile of keys, value
    widths that fill one, two and four warps' columns."""
    from lumenllm_b200.ops import kernels as K
    lens, starts = [70, 1, 1, 130], [0, 299, 63, 5]
    table, cache, rows, q = _latent_case(lens, starts, H, W, seed=31)
    assert K.attn_latent_takes(W, dv, BF16)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    scale = 0.2
    # None: a captured step, the division of the tokens is read on the device; 8 and 3: a row's keys shared
    # out among blocks (more of them than some rows have tiles of keys)
    for q_lens, n_split in ((lens, 1), (None, 1), (lens, 8), (None, 3)):
        got = K.attn_latent(torch.cat(q).to(BF16).cuda(), cache.to(BF16).cuda(), table.cuda(), cu.cuda(),
                            torch.tensor(starts, dtype=torch.int32).cuda(), q_lens, dv, window, scale,
                            n_seqs=len(lens), n_split=n_split).cpu()
        ref = []
        for b, (n, s) in enumerate(zip(lens, starts)):
            pos = torch.arange(s, s + n)[:, None]
            j = torch.arange(s + n)[None, :]
            seen = (j <= pos) & ((pos - j < window) if window else torch.ones_like(j, dtype=torch.bool))
            sc = torch.einsum("nhw,tw->nht", q[b], rows[b]) * scale
            sc = sc.masked_fill(~seen[:, None, :], float("-inf"))
            ref.append(torch.einsum("nht,tv->nhv", torch.softmax(sc, dim=-1), rows[b][:, :dv]))
        ref = torch.cat(ref)
        assert got.shape == ref.shape and torch.isfinite(got).all()
        assert float((got - ref).abs().max()) < 2e-2


@pytest.mark.parametrize("N", [1, 9, 150])
def test_products_of_every_head_on_the_tensor_cores(N):
    """Both per-head products of latent attention against float32 sums: the query into the latent
    space from partial sums (outputs that do not fill a block's 128 columns), and the weighted sums
    back through the values' up-projection."""
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(41)
    H, d, r, R, dv = 3, 64, 16, 200, 40
    qf = torch.randn(N, H * (d + r), generator=g)
    uk = (0.2 * torch.randn(H * d, R, generator=g)).to(BF16)
    parts = torch.stack([0.5 * qf, 0.125 * qf, 0.375 * qf]).cuda()
    got = K.latent_query(parts, uk.cuda(), H, d, r, R, None, 0, out_dtype=BF16).float().cpu()
    qh = qf.view(N, H, d + r)
    ref = torch.cat([torch.einsum("nhj,hjr->nhr", qh[:, :, :d].to(BF16).float(), uk.float().view(H, d, R)), qh[:, :, d:]], dim=-1)
    assert float((got - ref).abs().max()) < 3e-2 * max(1.0, float(ref.abs().max()))
    x = torch.randn(N, H, R + 24, generator=g)         # J = 224
    uv = (0.2 * torch.randn(H * dv, R + 24, generator=g)).to(BF16)
    got = K.head_product(x.cuda(), uv.cuda(), BF16).float().cpu()
    ref = torch.einsum("nhj,hej->nhe", x.to(BF16).float(), uv.float().view(H, dv, R + 24)).reshape(N, H * dv)
    assert float((got - ref).abs().max()) < 3e-2 * max(1.0, float(ref.abs().max()))

"""Vekolix in the engine against the plain implementation (tests/plain_vekolix.py): every mechanism
alone, then whole prompts, prompts in portions, decoding token by token, batches of unequal
requests, slots, pages and state that are used again, and greedy generation through the library's
entry point."""
import json
import math

import pytest
import torch

import plain_vekolix as P
from vekolix_models import (SMALL, config, dense, latent, layer, linear_side, make_weights, moe, parallel, softmax_side,
                            write_model)

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


def rows(T, D, dtype, seed, std=1.0):
    return (torch.randn(T, D, generator=torch.Generator().manual_seed(seed)) * std).to(dtype).float()


def pieces(y, sizes):
    out, at = [], 0
    for n in sizes:
        out.append(y[at:at + n])
        at += n
    assert at == y.shape[0]
    return out


def total(update):
    """An update of the stream, however it is handed on, as one float32 tensor on the host."""
    from lumenllm_b200.parts.norm import ScaledUpdate
    if isinstance(update, ScaledUpdate):
        return sum(s * total(d) for d, s in update.groups)
    if isinstance(update, (list, tuple)):
        return sum(total(d) for d in update)
    return (update.sum(0) if update.dim() == 3 else update).float().cpu()


def mixer_part(m, D, dtype, seed, child=None, edit=None, eps=1e-6):
    """A one-layer model's mixer, built as the engine builds it (`child` 0 or 1: one side of two
    mixers side by side, alone); its weights as the plain implementation reads them."""
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.parts import build_part
    cfg = config(8, D, eps, [layer(m, None)])
    w = make_weights(cfg, seed)
    if edit is not None:
        edit(w)
    spec = config_from_dict(cfg).model_spec().layers[0].mixer
    if child is not None:
        spec = spec.params["parts"][child]["mixer"]
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
    for _ in range(2 if twice else 1):
        slots = [cache.alloc_slot() for _ in pieces_by_seq]
        outs = [[] for _ in pieces_by_seq]
        for step in range(max(len(p) for p in pieces_by_seq)):
            live = [b for b, p in enumerate(pieces_by_seq) if step < len(p) and p[step].shape[0]]
            if not live:
                continue
            ctx, _ = build_context(cache, rt, [StepEntry(slots[b], [0] * pieces_by_seq[b][step].shape[0]) for b in live])
            y = torch.cat([pieces_by_seq[b][step] for b in live]).to(rt.dtype).cuda()
            out = total(mixer.forward(y, ctx, EntryView(ctx, 0, 0 if need is not None else None, True)))
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


PORTIONS = {150: [(150,), (64, 64, 22), (2, 2, 61, 1, 84), (1,) * 150], 70: [(70,), (3, 67), (69, 1), (2,) * 35]}


def in_any_portions(part, rt, plain_of, D, dtype, seed, std=1.0):
    """Two sequences of 150 and 70 rows, fed whole, in portions down to two rows and row by row, side
    by side in one batch, twice on the same slots: always the plain implementation's update."""
    ya, yb = rows(150, D, dtype, seed, std), rows(70, D, dtype, seed + 1, std)
    ra, rb = plain_of(ya), plain_of(yb)
    for pa, pb in zip(PORTIONS[150], PORTIONS[70]):
        ga, gb = run_mixer(part, rt, [pieces(ya, pa), pieces(yb, pb)], twice=True)
        close(ga, ra, dtype, f"{pa[:3]}")
        close(gb, rb, dtype, f"{pb[:3]}")


# ------------------------------------------------------------------ kernels alone

@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("width", [64, 50, 1032])
def test_dynamic_tanh_with_scaled_updates(dtype, width):
    """The stream plus groups of partial sums, each group with its factor; the norm of the sum; rows
    gathered; the stream left alone on request; more groups than one launch takes; adding only."""
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(width)
    N = 37
    h = torch.randn(N, width, generator=g)
    w, b, alpha = 1 + 0.1 * torch.randn(width, generator=g), 0.1 * torch.randn(width, generator=g), torch.tensor([0.7])
    groups = [(torch.randn(3, N, width, generator=g), 0.6), (torch.randn(N, width, generator=g), -1.25),
              (torch.randn(2, N, width, generator=g), 0.5)]
    x = h + sum(s * (d.sum(0) if d.dim() == 3 else d) for d, s in groups)
    dev = [(d.cuda(), s) for d, s in groups]
    hd = h.clone().cuda()
    y = K.add_scaled_dyt(hd, dev, w.cuda(), b.cuda(), alpha.cuda(), dtype)
    close(y, P.dynamic_tanh(x, w, b, alpha), dtype, "norm")
    close(hd, x, F32, "stream")
    want = torch.tensor([5, 0, 36, 5], dtype=torch.int32)
    hd = h.clone().cuda()
    y = K.add_scaled_dyt(hd, dev, w.cuda(), b.cuda(), alpha.cuda(), dtype, rows=want.cuda(), write_h=False)
    close(y, P.dynamic_tanh(x, w, b, alpha)[want.long()], dtype, "gathered rows")
    assert torch.equal(hd.cpu(), h)
    hd = h.clone().cuda()
    assert K.add_scaled_dyt(hd, dev * 2, None, None, None, dtype) is None          # six groups, two launches
    close(hd, 2 * x - h, F32, "adding only")
    close(K.add_scaled_dyt(h.clone().cuda(), [], w.cuda(), b.cuda(), alpha.cuda(), dtype), P.dynamic_tanh(h, w, b, alpha),
          dtype, "nothing pending")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_elementwise_pieces(dtype):
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(0)
    z = torch.randn(3, 9, 70, generator=g) * 2.5
    close(K.relu2(z.cuda(), dtype), P.relu_squared(z.sum(0)), dtype, "squared relu")
    F = 13
    u = torch.randn(2, 9, 2 * F + 3, generator=g) * 2.0
    s = u.sum(0)
    for limit in (0.8, 3.0):
        gate, up = torch.clamp(s[:, :F], max=limit), torch.clamp(s[:, F:2 * F], -limit, limit)
        ref = gate * torch.sigmoid(1.702 * gate) * (up + 1)
        close(K.clamped_glu(u.cuda(), F, limit, 1.702, dtype), ref, dtype, "clamped unit")
        close(K.clamped_glu(u.cuda(), F, limit, 1.702, dtype, token_gate_col=2 * F + 1),
              ref * torch.sigmoid(s[:, 2 * F + 1:2 * F + 2]), dtype, "clamped unit with a gate a token")
    for C, c0 in ((24, 5), (1100, 3)):
        u = torch.randn(2, 7, c0 + C + 2, generator=g)
        w = 1 + 0.1 * torch.randn(C, generator=g)
        close(K.cols_rmsnorm(u.cuda(), c0, C, w.cuda(), 1e-5, dtype), P.norm_plain(u.sum(0)[:, c0:c0 + C], w, 1e-5), dtype,
              "norm of some columns")
    lg = torch.randn(5, 33, generator=g) * 40
    close(K.scale_softcap(lg.clone().cuda(), 0.5, 7.0), 7.0 * torch.tanh(lg * 0.5 / 7.0), F32, "capped logits")
    close(K.scale_softcap(lg.clone().cuda(), 0.25, 0.0), lg * 0.25, F32, "scaled logits")


def test_rotation_table_with_stretched_frequencies():
    from lumenllm_b200.ops import kernels as K
    sc = {"factor": 8.0, "original": 256, "fast": 16.0, "slow": 2.0}
    f, mag = P.frequencies(10000.0, 32, sc)
    pos = torch.tensor([0, 1, 7, 255, 256, 4000], dtype=torch.int32)
    cs = K.rope_table(pos.cuda(), f.cuda(), mag).cpu()
    a = pos.float()[:, None] * f[None, :]
    assert float((cs[..., 0] - torch.cos(a) * mag).abs().max()) < 2e-6
    assert float((cs[..., 1] - torch.sin(a) * mag).abs().max()) < 2e-6


@pytest.mark.parametrize("H,d,dv", [(2, 8, 40), (1, 72, 96), (3, 128, 32), (2, 200, 24), (5, 16, 24), (1, 256, 8),
                                    (2, 300, 16)])
def test_linear_attention_kernel(H, d, dv):
    """Three sequences in one launch (150 tokens, one token, 33 tokens), then each again with more
    tokens from the state the first launch left; partial sums; a slot that is not the sequence's index."""
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(d + dv)
    decay = torch.rand(H, generator=g) * 0.5 + 0.5
    decay[0] = 1.0
    W = 2 * H * d + H * dv + 5
    lens1, lens2 = [150, 1, 33], [1, 40, 2]
    u = [[torch.randn(2, n, W, generator=g) * 0.6 for n in lens] for lens in (lens1, lens2)]
    state = torch.zeros(5, H, d, dv).cuda()
    slots = torch.tensor([3, 0, 4], dtype=torch.int32).cuda()
    got = []
    for step, lens in enumerate((lens1, lens2)):
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).cuda()
        out = K.linear_attn(torch.cat(u[step], dim=1).cuda(), 3, 3 + H * d, 3 + 2 * H * d, True, decay.cuda(), state, cu,
                            slots, 3, H, d, dv).cpu()
        got.append(pieces(out, lens))
    assert float(state[1].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0
    for b in range(3):
        x = torch.cat([u[0][b].sum(0), u[1][b].sum(0)])
        T = x.shape[0]
        q, k = (P.silu(x[:, 3 + i * H * d:3 + (i + 1) * H * d]).view(T, H, d) for i in (0, 1))
        v = P.silu(x[:, 3 + 2 * H * d:3 + 2 * H * d + H * dv]).view(T, H, dv)
        S, ref = torch.zeros(H, d, dv), []
        for t in range(T):
            S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
            ref.append(torch.einsum("hde,hd->he", S, q[t]).reshape(H * dv))
        close(torch.cat([got[0][b], got[1][b]]), torch.stack(ref), F32, f"sequence {b}")
        close(state[int(slots[b])], S, F32, f"state {b}")


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("J,E", [(64, 16), (40, 6)])
def test_a_gate_a_head_where_sums_leave_the_latent_space(dtype, J, E):
    from lumenllm_b200.ops import kernels as K
    g = torch.Generator().manual_seed(J)
    N, H = 70, 3
    x = torch.randn(N, H, J, generator=g)
    w = (0.2 * torch.randn(H * E, J, generator=g)).to(dtype)
    gate = torch.randn(2, N, 9, generator=g)
    got = K.head_product(x.cuda(), w.cuda(), dtype, gate=gate.cuda(), gate_col=4)
    xr = x.to(dtype).float() if dtype == BF16 else x
    ref = torch.einsum("nhj,hej->nhe", xr, w.float().view(H, E, J)) * torch.sigmoid(gate.sum(0)[:, 4:4 + H])[:, :, None]
    close(got, ref.reshape(N, H * E), dtype)


# ------------------------------------------------------------------ mixers alone

SOFTMAX = [softmax_side(4, 2, 16, 24, 0.3, rot=8, base=5000.0, scaling=(4.0, 64, 8.0, 1.0)),
           softmax_side(3, 3, 32, 8, 0.25, rot=32, base=500.0),
           softmax_side(6, 2, 64, 64, 0.12),
           softmax_side(4, 1, 128, 128, 0.09, rot=64, base=1e5, scaling=(16.0, 128, 16.0, 2.0))]
LINEAR = [linear_side(2, 16, 24, (0.7, 0.98)), linear_side(1, 72, 96, (0.99,)), linear_side(3, 128, 32, (1.0, 0.9, 0.5)),
          linear_side(5, 8, 40, (0.3, 0.8, 0.9, 0.99, 0.999))]
LATENT = [latent(2, 8, 16, 24, 40, 24, 0.2, rot=8), latent(3, 16, 16, 8, 40, 56, 0.25, rot=16, base=3e5),
          latent(4, 32, 32, 32, 96, 64, 0.1, rot=32), latent(1, 24, 8, 16, 64, 32, 0.15)]
ANY_LEFT, ANY_RIGHT = SOFTMAX[1], LINEAR[0]


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("m", SOFTMAX)
def test_softmax_side_in_any_portions(m, dtype):
    D = 64
    part, w = mixer_part(parallel(m, ANY_RIGHT), D, dtype, seed=11, child=0)
    in_any_portions(part, runtime(dtype), lambda y: P.softmax_attention(y, w, "l0.mix.left", m, torch.arange(y.shape[0])),
                    D, dtype, seed=12)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("m", LINEAR)
def test_linear_side_in_any_portions(m, dtype):
    D = 48
    part, w = mixer_part(parallel(ANY_LEFT, m), D, dtype, seed=13, child=1)
    assert part.cache_need() is None and part.state_shape()[0] == (m["heads"], m["dim"], m["vdim"])
    in_any_portions(part, runtime(dtype), lambda y: P.linear_attention(y, w, "l0.mix.right", m, 1e-6), D, dtype, seed=14)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_two_mixers_side_by_side(dtype):
    """One cache entry (the softmax side's) and one state row (the linear side's) a run of the layer,
    and the weighted sum of both updates."""
    D = 64
    m = parallel(SOFTMAX[0], LINEAR[3], 0.8, -1.3)
    part, w = mixer_part(m, D, dtype, seed=15)
    assert part.cache_need().n_kv == 2 and part.state_shape()[0] == (5, 8, 40)
    # both sides start with a product of the same rows: ONE product, the linear side's columns behind the other's
    assert part.proj is not None and part.col0 == [0, 4 * 16 + 2 * (16 + 24)] and part.mixers[0].proj is None
    assert part.proj.out_features == part.col0[1] + 2 * 5 * 8 + 2 * 5 * 40
    in_any_portions(part, runtime(dtype), lambda y: P.side_by_side(y, w, "l0.mix", m, 1e-6, torch.arange(y.shape[0])),
                    D, dtype, seed=16)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("m", LATENT)
def test_latent_attention_in_any_portions(m, dtype):
    D = 64
    part, w = mixer_part(m, D, dtype, seed=17)
    need = part.cache_need()
    assert need.n_kv == 1 and need.head_dim == m["kv_rank"] + m["rot_dim"] and need.values_in_keys
    in_any_portions(part, runtime(dtype), lambda y: P.latent_attention(y, w, "l0.mix", m, 1e-6, torch.arange(y.shape[0])),
                    D, dtype, seed=18)


FAR = (0, 1, 63, 64, 65, 127, 128, 191, 192, 298)


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_one_loud_key_far_back_and_at_page_borders_softmax(dtype, decode):
    """Key heads made of the query heads' weights with their columns moved on by one, and one earlier
    row equal to the last row moved the same way: that key equals the last query, and its score
    stands out among 300, wherever it lies, first tokens and both sides of every page border
    included, for a prompt's last row and for a row decoded alone."""
    D, T = 64, 300
    m = softmax_side(4, 2, 32, 16, 1.0, rot=8, base=1e4)

    def edit(w):
        q = w["l0.mix.left.q"].view(4, 32, D).clone()
        q[1], q[3] = q[0], q[2]                     # the query heads of a group alike, so that every head hears the key
        w["l0.mix.left.q"] = q.reshape(128, D)
        w["l0.mix.left.k"] = torch.roll(torch.stack([q[0], q[2]]), -1, dims=2).reshape(64, D).clone()

    part, w = mixer_part(parallel(m, ANY_RIGHT), D, dtype, seed=21, child=0, edit=edit)
    rt = runtime(dtype)
    for j0 in FAR:
        y = rows(T, D, dtype, seed=22 + j0, std=0.3)
        y[T - 1] = (y[T - 1] * 6).to(dtype).float()
        y[j0] = torch.roll(y[T - 1], -1)
        ref = P.softmax_attention(y, w, "l0.mix.left", m, torch.arange(T))
        quiet = y.clone()
        quiet[j0] = 0.0
        assert float((P.softmax_attention(quiet, w, "l0.mix.left", m, torch.arange(T))[-1] - ref[-1]).abs().max()) > 0.1
        (got,) = run_mixer(part, rt, [pieces(y, (T - 1, 1) if decode else (T,))])
        close(got[-1:], ref[-1:], dtype, f"key {j0}")


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_one_loud_latent_far_back_and_at_page_borders(dtype, decode):
    """The queries' latent made of the keys' with its columns moved on by one, the queries'
    up-projection a multiple of the keys', and one earlier row equal to the last row moved the same
    way: that row's latent equals the last query's, and its score stands out among 300."""
    D, T = 64, 300
    m = latent(2, 16, 8, 24, 32, 32, 1.0, rot=8)

    def edit(w):
        w["l0.mix.dq"] = torch.roll(w["l0.mix.dkv"][:32], -1, dims=1).clone()
        w["l0.mix.dq.norm"] = w["l0.mix.dkv.norm"].clone()
        uq = w["l0.mix.uq"].view(2, 24, 32).clone()
        uq[:, :16] = 1.5 * w["l0.mix.uk"].view(2, 16, 32)
        w["l0.mix.uq"] = uq.reshape(48, 32)

    part, w = mixer_part(m, D, dtype, seed=23, edit=edit)
    rt = runtime(dtype)
    for j0 in FAR:
        y = rows(T, D, dtype, seed=24 + j0)
        y[j0] = torch.roll(y[T - 1], 1)
        ref = P.latent_attention(y, w, "l0.mix", m, 1e-6, torch.arange(T))
        quiet = y.clone()
        quiet[j0] = -quiet[j0]
        assert float((P.latent_attention(quiet, w, "l0.mix", m, 1e-6, torch.arange(T))[-1] - ref[-1]).abs().max()) > 0.1
        (got,) = run_mixer(part, rt, [pieces(y, (T - 1, 1) if decode else (T,))])
        close(got[-1:], ref[-1:], dtype, f"key {j0}")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_the_state_remembers_far_back_and_forgets_by_head(dtype):
    """A loud first token, then 400 quiet ones fed in portions: the head without decay still carries
    it at the end, the head that halves its state a token has long lost it."""
    D, T = 48, 401
    m = linear_side(2, 16, 8, (1.0, 0.5))
    part, w = mixer_part(parallel(ANY_LEFT, m), D, dtype, seed=25, child=1)
    y = rows(T, D, dtype, seed=26, std=0.5)
    y[0] = (y[0] * 8).to(dtype).float()
    ref = P.linear_attention(y, w, "l0.mix.right", m, 1e-6)
    quiet = y.clone()
    quiet[0] = 0.0
    assert float((P.linear_attention(quiet, w, "l0.mix.right", m, 1e-6)[-1] - ref[-1]).abs().max()) > 0.05
    (got,) = run_mixer(part, runtime(dtype), [pieces(y, (1, 199, 2, 198, 1))])
    close(got, ref, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("mlp", [moe(5, 2, 24, 1.5, shared=(40, 0.8)), moe(3, 1, 16, 0.7), moe(7, 3, 40, 2.5),
                                 moe(4, 4, 8, 1.0, shared=(8, 3.0)), dense(80)])
@pytest.mark.parametrize("N", [1, 9, 150])
def test_feed_forwards(mlp, dtype, N):
    """The dense layer and the mixture (sigmoid scores, the largest chosen, a score on its expert's
    input, clamped units, a gated shared expert) for one row, a few and many."""
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.parts import build_part
    D = 64
    cfg = config(8, D, 1e-6, [layer(LATENT[0], mlp)])
    w = make_weights(cfg, seed=27)
    spec = config_from_dict(cfg).model_spec().layers[0].ffn
    part = build_part("ffn", spec, {k: v.cuda() for k, v in w.items()}, runtime(dtype))
    y = rows(N, D, dtype, seed=28)
    wf = {k: v.float() for k, v in w.items()}
    ref = P.dense_ff(y, wf, "l0.mlp") if mlp["kind"] == "dense" else P.expert_ff(y, wf, "l0.mlp", mlp)
    out = part.forward(y.to(dtype).cuda(), None)
    close(total(out), ref, dtype)


# ------------------------------------------------------------------ the model in the engine

def calm(cfg):
    """The same model with every mixture using ALL its experts. A choice among experts is not continuous:
    a token whose best scores differ in the last bits goes elsewhere in a bfloat16 run than in the plain
    32-bit one, and its row then differs by far more than rounding. So whole models are compared in
    32-bit as they are (choices and all, strictly), and in bfloat16 in this form, where the scores still
    weigh every expert's input; the choice itself is compared in bfloat16 on equal inputs
    (test_feed_forwards)."""
    c = json.loads(json.dumps(cfg))
    for L in c["layers"]:
        if L["mlp"] is not None and L["mlp"]["kind"] == "moe":
            L["mlp"]["router"]["top"] = L["mlp"]["router"]["experts"]
    return c


def pick(name, dtype):
    return name if dtype in (F32, "float32") else name + "~"


MODELS = dict(SMALL, **{name + "~": calm(cfg) for name, cfg in SMALL.items()})


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("vekolix")
    return {name: write_model(cfg, root / name, seed=3 + i % len(SMALL)) for i, (name, cfg) in enumerate(MODELS.items())}


@pytest.fixture(scope="module")
def plain(models):
    return {name: P.load_model(folder) + ({},) for name, folder in models.items()}


def plain_logits(plain, name, tokens):
    cfg, w, memo = plain[name]
    key = tuple(tokens)
    if key not in memo:
        memo[key] = P.forward(cfg, w, tokens)
    return memo[key]


def engine_of(models, name, dtype, **kw):
    from lumenllm_b200.engine import Engine
    kw.setdefault("max_tokens", 2048)
    return Engine.from_folder(models[name], dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_whole_prompts(name, dtype, models, plain):
    name = pick(name, dtype)
    from lumenllm_b200.engine import StepEntry
    eng = engine_of(models, name, dtype)
    for toks in tokens_of(MODELS[name], (1, 2, 65, 200), seed=30):
        slot = eng.alloc_slot()
        close(eng.step([StepEntry(slot, toks, list(range(len(toks))))]), plain_logits(plain, name, toks), dtype, f"{len(toks)} tokens")
        eng.free_slot(slot)
    eng.cache.check()
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_residual_stream_after_every_layer(name, dtype, models, plain):
    name = pick(name, dtype)
    from lumenllm_b200.engine import StepEntry
    from lumenllm_b200.engine.context import EntryView
    from lumenllm_b200.ops import kernels as K
    from lumenllm_b200.parts.norm import ScaledUpdate
    cfg, w, _ = plain[name]
    toks = tokens_of(cfg, (40,), seed=31)[0]
    ref = []
    P.forward(cfg, w, toks, ref)
    eng = engine_of(models, name, dtype)
    ctx = eng.build_context([StepEntry(eng.alloc_slot(), toks, [])])
    m = eng.model
    h, pending = m.embedding.forward(ctx.tokens, ctx), None
    for i, e in enumerate(m.schedule):
        h, pending = m.blocks[e.layer].forward(h, pending, ctx, EntryView(ctx, i, i if i in ctx.cache.group_of else None, True))
        x = h.clone()
        if isinstance(pending, ScaledUpdate):
            K.add_scaled_dyt(x, pending.groups, None, None, None, F32)
        elif pending is not None:
            x += pending if pending.dim() == 2 else pending.sum(0)
        close(x, ref[i], dtype, f"after layer {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_prompt_in_portions_and_decoded_token_by_token(name, dtype, models, plain):
    name = pick(name, dtype)
    from lumenllm_b200.engine import StepEntry
    toks = tokens_of(MODELS[name], (171,), seed=32)[0]
    ref = plain_logits(plain, name, toks)
    eng = engine_of(models, name, dtype, max_slots=2)
    for cuts in ((64, 2, 62, 3), (1, 127), (130,)):
        slot = eng.alloc_slot()
        got, at = [], 0
        for n in cuts:
            got.append(eng.step([StepEntry(slot, toks[at:at + n], list(range(n)))]))
            at += n
        got += [eng.step([StepEntry(slot, [toks[t]], [0])]) for t in range(at, len(toks))]
        close(torch.cat(got), ref, dtype, f"{cuts}")
        eng.free_slot(slot)
    eng.cache.check()
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(SMALL))
def test_a_batch_of_unequal_requests_equals_each_alone(name, dtype, models, plain):
    """Prompts of 1, 2, 64, 65 and 131 tokens in one batch, decoded together while the shorter ones
    end; then the slots, pages and state rows they gave back serve the same requests in another order."""
    name = pick(name, dtype)
    from lumenllm_b200.engine import StepEntry
    lens = (65, 1, 131, 2, 64)
    prompts = tokens_of(MODELS[name], [n + k for k, n in enumerate(lens)], seed=33)      # request k decodes k tokens
    refs = [plain_logits(plain, name, p) for p in prompts]
    eng = engine_of(models, name, dtype, max_slots=5)
    for order in ((0, 1, 2, 3, 4), (4, 2, 0, 3, 1)):
        slots = {k: eng.alloc_slot() for k in order}
        got = eng.step([StepEntry(slots[k], prompts[k][:lens[k]], list(range(lens[k]))) for k in order])
        close(got, torch.cat([refs[k][:lens[k]] for k in order]), dtype, "prompts")
        for t in range(4):
            live = [k for k in order if k > t]
            got = eng.step([StepEntry(slots[k], [prompts[k][lens[k] + t]], [0]) for k in live])
            close(got, torch.stack([refs[k][lens[k] + t] for k in live]), dtype, f"decoded {t}")
            for k in order:
                if k == t + 1:
                    eng.free_slot(slots[k])
        eng.free_slot(slots[0])
        eng.cache.check()
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_page_borders(dtype, models, plain):
    from lumenllm_b200.cache import PAGE
    from lumenllm_b200.engine import StepEntry
    name = pick("X", dtype)
    toks = tokens_of(MODELS[name], (3 * PAGE + 20,), seed=34)[0]
    ref = plain_logits(plain, name, toks)
    eng = engine_of(models, name, dtype, max_tokens=6 * PAGE, max_slots=2)
    slot = eng.alloc_slot()
    got = [eng.step([StepEntry(slot, toks[:5], list(range(5)))])]
    got += [eng.step([StepEntry(slot, [toks[t]], [0])]) for t in range(5, len(toks))]
    close(torch.cat(got), ref, dtype)
    eng.free_slot(slot)
    eng.cache.check()
    eng.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [44, 50])
def test_a_model_whose_rows_are_no_multiples_of_16_bytes(dtype, width, tmp_path):
    """Widths 44 and 50, heads of 6 keys and 10 values, latents of 18 + 6 and 9, a recurrence of 7 key
    channels, experts of 5: no row of any matrix is a multiple of 16 bytes (with 50 not even of 8), so
    the products and the row kernels go the ways that need no alignment."""
    from lumenllm_b200.engine import Engine, StepEntry
    cfg = config(61, width, 1e-5, [
        layer(parallel(softmax_side(3, 1, 6, 10, 0.4, rot=4, scaling=(2.0, 32, 4.0, 1.0)), linear_side(2, 7, 5, (0.9, 0.6)),
                       0.9, 1.1), moe(3, 2, 5, 1.1, shared=(7, 0.9))),
        layer(latent(3, 10, 6, 5, 18, 9, 0.3, rot=2), dense(9))], mult=0.8, logit_scale=0.7, softcap=9.0)
    cfg = cfg if dtype == "float32" else calm(cfg)
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


def test_a_long_wide_prompt(tmp_path):
    """A prompt long and wide enough for the tensor-core kernels of every product, of the softmax
    side (keys and values of 128) and of the latent layer, with updates that count once (the
    output products may then add into the stream by themselves) and with a multiplier."""
    from lumenllm_b200.engine import Engine, StepEntry
    for mult in (1.0, 0.5):
        cfg = config(64, 1024, 1e-6, [
            layer(parallel(softmax_side(4, 2, 128, 128, 0.09, rot=64, scaling=(6.0, 512, 24.0, 1.5)),
                           linear_side(4, 64, 64, (0.9, 0.99, 0.995, 0.5)), 0.65, 1.15), dense(512)),
            layer(latent(4, 64, 32, 64, 256, 192, 0.1, rot=32), moe(8, 2, 128, 1.0, shared=(128, 2.0)))],
            mult=mult, logit_scale=0.35, softcap=20.0)
        cfg = calm(cfg)
        T = 2300
        folder = write_model(cfg, tmp_path / f"wide{mult}", seed=70)
        toks = tokens_of(cfg, (T,), seed=71)[0]
        want = [0, 1, 63, 64, 1023, 1024, T - 2, T - 1]
        _, w = P.load_model(folder)
        ref = P.forward(cfg, w, toks)[want]
        eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=4096)
        slot = eng.alloc_slot()
        close(eng.step([StepEntry(slot, toks, want)]), ref, "bfloat16", f"multiplier {mult}")
        eng.check_kernels()
        del eng


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(dtype, models, plain):
    """build(EngineConfig).generate: batches, the scheduler's run-ahead and captured steps."""
    from lumenllm_b200 import EngineConfig, GenerateRequest, build
    name = pick("Z", dtype)
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
            assert o.tokens == P.greedy(cfg, w, p, 10)
    built.engine.check_kernels()


def test_command_line_generates(models, capsys):
    from lumenllm_b200.cli import main
    rc = main(["generate", "--model", str(models["X"]), "--prompt-tokens", "5,6,7", "--prompt-tokens", "1",
               "--max-tokens", "4", "--ctx-size", "128", "--format", "json", "--dtype", "float32"])
    assert rc == 0
    outs = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    cfg, w = P.load_model(models["X"])
    assert [o["tokens"] for o in outs] == [P.greedy(cfg, w, p, 4) for p in ([5, 6, 7], [1])]


def test_random_weights_mode_builds_and_steps():
    """A configuration alone is enough for an engine with random weights (the throughput runs use it)."""
    from lumenllm_b200.engine import Engine, StepEntry
    eng = Engine.from_random(SMALL["Z"], seed=1, std=0.05, max_tokens=512)
    slot = eng.alloc_slot()
    lg = eng.step([StepEntry(slot, list(range(40)), [39])])
    assert lg.shape == (1, SMALL["Z"]["vocab"]) and torch.isfinite(lg).all()
    eng.check_kernels()


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

"""Python faces of the hand-written kernels. Each function checks dtypes and
shapes, launches on the current CUDA stream and returns its output tensor.
Float32 tensors select the 32-bit variants, bfloat16 tensors the serving ones.

A tensor that a split matrix product made may come as S partial results stacked
in front, [S, rows, width]; the consumers below add the partials while reading.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..csrc.build import page_size as _page_size
from .native import KernelError, check, fn, int_fn, library, ptr, require, stream_ptr

P = c_void_p
F32 = torch.float32
BF16 = torch.bfloat16
I32 = torch.int32

PAGE = _page_size()   # tokens per cache page: LUMEN_PAGE of csrc/common.cuh
LAYOUT_LINEAR, LAYOUT_SW128 = 0, 1   # tile layouts of the cache, as in csrc/common.cuh


def _is_bf16(t) -> int:
    if t.dtype == BF16:
        return 1
    if t.dtype == F32:
        return 0
    raise KernelError(f"expected float32 or bfloat16, got {t.dtype}")


def _partials(t, name):
    """[rows, width] or [S, rows, width] -> (tensor as [S, rows, width], S)."""
    require(t, F32, name)
    if t.dim() == 2:
        t = t.unsqueeze(0)
    if t.dim() != 3:
        raise KernelError(f"{name}: expected [rows, width] or [S, rows, width]")
    return t, t.shape[0]


def embed(tokens, table, out=None):
    """h[t] = float32(table[tokens[t]]). tokens int32 [N]; table [V, H] float32|bfloat16, or
    a TiledWeight (the table an output head shares)."""
    require(tokens, I32, "embed.tokens")
    N = tokens.numel()
    V, H = table.shape
    if isinstance(table, TiledWeight):
        if out is None:
            out = torch.empty((N, H), dtype=F32, device=table.device)
        f = fn("core", "lumen_embed_tiled", [P, P, P, c_int, c_int, c_int, c_int, P])
        check(f(ptr(tokens), ptr(table.data), ptr(out), N, H, V, table.padded_rows, stream_ptr()), "embed")
        return out
    if not table.is_contiguous() or not table.is_cuda:
        raise KernelError("embed.table must be a contiguous CUDA tensor")
    if out is None:
        out = torch.empty((N, H), dtype=F32, device=table.device)
    f = fn("core", "lumen_embed", [P, P, c_int, P, c_int, c_int, c_int, P])
    check(f(ptr(tokens), ptr(table), _is_bf16(table), ptr(out), N, H, V, stream_ptr()), "embed")
    return out


def embed_pos(tokens, table, scale, positions, pos_table, out=None):
    """h[t] = float32(table[tokens[t]]) * scale + float32(pos_table[positions[t]]) (no position
    term with pos_table None). table [V, H] float32|bfloat16 or a TiledWeight; pos_table [P, H]
    float32|bfloat16; tokens, positions int32 [N]."""
    require(tokens, I32, "embed_pos.tokens")
    N = tokens.numel()
    V, H = table.shape
    tiled = isinstance(table, TiledWeight)
    data = table.data if tiled else table
    if not tiled and (not table.is_contiguous() or not table.is_cuda):
        raise KernelError("embed_pos.table must be a contiguous CUDA tensor")
    P_rows = 0
    if pos_table is not None:
        require(positions, I32, "embed_pos.positions")
        if pos_table.dim() != 2 or pos_table.shape[1] != H or not pos_table.is_contiguous() or positions.numel() < N:
            raise KernelError(f"embed_pos: the position table must be [P, {H}], one position a token")
        P_rows = pos_table.shape[0]
    if out is None:
        out = torch.empty((N, H), dtype=F32, device=data.device)
    f = fn("layer_ops", "lumen_embed_pos", [P, P, c_int, c_int, c_float, P, P, c_int, c_int, P, c_int, c_int, c_int, P])
    check(f(ptr(tokens), ptr(data), 1 if tiled else _is_bf16(table), table.padded_rows if tiled else 0, float(scale),
            ptr(positions) if pos_table is not None else 0, ptr(pos_table),
            _is_bf16(pos_table) if pos_table is not None else 0, P_rows, ptr(out), N, H, V, stream_ptr()), "embed_pos")
    return out


def postnorm_add_rmsnorm(h, delta, bias, w_update, eps_update, w_next, eps_next, out_dtype, rows=None,
                         write_h=True, conv=None):
    """u = sum(delta[s]) (+ bias); x = h + rmsnorm(u) * w_update (stored back to h when write_h);
    y = rmsnorm(x) * w_next in out_dtype (None with w_next None). h float32 [N, H]; delta float32
    [N, H] or [S, N, H], or None (nothing to add: x = h); rows int32 [W] gathers the rows to
    work on. With conv = (weight float32 [taps, H], state float32 [slots, taps - 1, H] or None,
    seq_slot int32 [N]) row b is the one new token of sequence b, and what goes out is the
    convolution of canon_conv applied to y, the state moved on by one."""
    require(h, F32, "postnorm_add_rmsnorm.h")
    N, H = h.shape
    S = 0
    if delta is not None:
        require(w_update, F32, "postnorm_add_rmsnorm.w_update")
        delta, S = _partials(delta, "postnorm_add_rmsnorm.delta")
        if tuple(delta.shape[1:]) != (N, H) or w_update.numel() != H:
            raise KernelError(f"postnorm_add_rmsnorm: delta {tuple(delta.shape)} / weight do not match h {(N, H)}")
    for t, nm in ((bias, "bias"), (w_next, "w_next")):
        if t is not None:
            require(t, F32, f"postnorm_add_rmsnorm.{nm}")
            if t.numel() != H:
                raise KernelError(f"postnorm_add_rmsnorm: {nm} has {t.numel()} values, rows have {H}")
    n_rows = N
    if rows is not None:
        require(rows, I32, "postnorm_add_rmsnorm.rows")
        n_rows = rows.numel()
    cw = state = slots = None
    taps, stride = 0, 0
    if conv is not None:
        cw, state, slots = conv
        require(cw, F32, "postnorm_add_rmsnorm.conv weight")
        require(slots, I32, "postnorm_add_rmsnorm.seq_slot")
        taps = cw.shape[0]
        if rows is not None or w_next is None or cw.shape[1] != H or not 1 <= taps <= CANON_MAX_TAPS or slots.numel() < N:
            raise KernelError("postnorm_add_rmsnorm: the convolution takes whole steps of one token a sequence")
        if taps > 1:
            if state is None or state.dtype != F32 or tuple(state.shape[1:]) != (taps - 1, H) \
                    or state.stride(2) != 1 or state.stride(1) != H:
                raise KernelError(f"postnorm_add_rmsnorm: state must be float32 [slots, {taps - 1}, {H}] with dense rows")
            stride = state.stride(0)
    y = torch.empty((n_rows, H), dtype=out_dtype, device=h.device) if w_next is not None else None
    f = fn("layer_ops", "lumen_postnorm_add_rmsnorm",
           [P, P, c_int, c_longlong, P, P, c_float, P, c_float, P, c_int, P, c_int, c_int, c_int, P, c_int, P,
            c_longlong, P, P])
    check(f(ptr(h), ptr(delta), S, N * H, ptr(bias), ptr(w_update), float(eps_update), ptr(w_next), float(eps_next),
            ptr(y), _is_bf16(y) if y is not None else 0, ptr(rows), n_rows, H, 1 if write_h else 0, ptr(cw), taps,
            ptr(state) if taps > 1 else 0, stride, ptr(slots), stream_ptr()), "postnorm_add_rmsnorm")
    return y


CANON_MAX_TAPS = 16


def canon_conv(y, weight, state, tok_seq, cu_q, seq_slot, n_seqs, out_dtype):
    """out_t = y_t + sum_j weight[j] * y_(t - taps + 1 + j) per channel within each sequence of the
    step; inputs before the step's first token come from `state` (float32 [slots, taps - 1, H],
    possibly a view with a larger slot stride), which is moved on to the step's end.
    y float32 [N, H]; weight float32 [taps, H]."""
    require(y, F32, "canon_conv.y")
    require(weight, F32, "canon_conv.weight")
    N, H = y.shape
    taps = weight.shape[0]
    if weight.shape[1] != H or not 1 <= taps <= CANON_MAX_TAPS:
        raise KernelError(f"canon_conv: weight {tuple(weight.shape)} does not fit rows of {H} (1 to {CANON_MAX_TAPS} taps)")
    stride = 0
    if taps > 1:
        if state is None or state.dtype != F32 or not state.is_cuda or tuple(state.shape[1:]) != (taps - 1, H) \
                or state.stride(2) != 1 or state.stride(1) != H:
            raise KernelError(f"canon_conv: state must be float32 [slots, {taps - 1}, {H}] with dense rows")
        stride = state.stride(0)
    for t, nm in ((tok_seq, "tok_seq"), (cu_q, "cu_q"), (seq_slot, "seq_slot")):
        require(t, I32, f"canon_conv.{nm}")
    out = torch.empty((N, H), dtype=out_dtype, device=y.device)
    f = fn("layer_ops", "lumen_canon_conv", [P, P, c_int, P, c_longlong, P, P, P, c_int, c_int, P, c_int, c_int, P])
    check(f(ptr(y), ptr(weight), taps, ptr(state) if taps > 1 else 0, stride, ptr(tok_seq), ptr(cu_q), ptr(seq_slot),
            N, int(n_seqs), ptr(out), _is_bf16(out), H, stream_ptr()), "canon_conv")
    return out


def polynorm(z, act, eps, out_dtype):
    """a N(z) + b N(z^2) + c N(z^3) + e with N(v) = v / sqrt(mean(v^2) + eps) over a row and
    act = (a, b, c, e) float32 on the device; z float32 [N, F] or [S, N, F] partials."""
    z, S = _partials(z, "polynorm.z")
    require(act, F32, "polynorm.act")
    if act.numel() != 4:
        raise KernelError("polynorm: act holds four values")
    _, N, Fw = z.shape
    out = torch.empty((N, Fw), dtype=out_dtype, device=z.device)
    f = fn("layer_ops", "lumen_polynorm", [P, c_int, c_longlong, P, c_float, P, c_int, c_int, c_int, P])
    check(f(ptr(z), S, N * Fw, ptr(act), float(eps), ptr(out), _is_bf16(out), N, Fw, stream_ptr()), "polynorm")
    return out


def qkv_bias_norm_store(qkv, bias, q_norm_w, k_norm_w, eps, cache_pos, tok_seq, block_table, kcache, vcache,
                        nq, nkv, d, dv, out_dtype, k_layout=LAYOUT_LINEAR, v_layout=LAYOUT_LINEAR,
                        cs=None, rotary_dim=0, value_unit_eps=None):
    """Bias, one RMS norm over the WHOLE query projection (weight [nq * d]) and one over the whole
    key projection (weight [nkv * d]), q out as [N, nq, d], k and v written to the paged cache
    (keys [pages, nkv, PAGE, d], values [pages, nkv, PAGE, dv]). With rotary_dim > 0 the first
    rotary_dim values of every query and key head are rotated after the norm by the angles of
    `cs` (rope_table: float32 [N, rotary_dim/2, 2]); with value_unit_eps every value head is
    divided by its root mean square (that eps inside the root).
    qkv float32 [N, nq*d + nkv*d + nkv*dv] or [S, N, ...] partials; bias float32 of that width or None."""
    qkv, S = _partials(qkv, "qkv_bias_norm_store.qkv")
    N = qkv.shape[1]
    width = nq * d + nkv * d + nkv * dv
    if qkv.shape[2] != width:
        raise KernelError(f"qkv_bias_norm_store: row width {qkv.shape[2]} != {width}")
    for t, nm, n in ((bias, "bias", width), (q_norm_w, "q_norm", nq * d), (k_norm_w, "k_norm", nkv * d)):
        if t is not None:
            require(t, F32, f"qkv_bias_norm_store.{nm}")
            if t.numel() != n:
                raise KernelError(f"qkv_bias_norm_store: {nm} must have {n} values")
    for t, nm in ((cache_pos, "cache_pos"), (tok_seq, "tok_seq")):
        require(t, I32, nm)
        if t.numel() < N:
            raise KernelError(f"{nm} shorter than the token count")
    require(block_table, I32, "block_table")
    require(kcache, out_dtype, "kcache")
    require(vcache, out_dtype, "vcache")
    if tuple(kcache.shape[1:]) != (nkv, PAGE, d) or tuple(vcache.shape[1:]) != (nkv, PAGE, dv):
        raise KernelError(f"qkv_bias_norm_store: caches {tuple(kcache.shape)}, {tuple(vcache.shape)} do not fit "
                          f"{nkv} kv heads of {d} and {dv}")
    if rotary_dim:
        require(cs, F32, "qkv_bias_norm_store.cs")
        if rotary_dim % 2 or rotary_dim > d or tuple(cs.shape) != (N, rotary_dim // 2, 2):
            raise KernelError(f"qkv_bias_norm_store: angles {tuple(cs.shape)} do not fit {N} tokens and a rotation "
                              f"over {rotary_dim} of {d} values")
    q_out = torch.empty((N, nq, d), dtype=out_dtype, device=qkv.device)
    f = fn("layer_ops", "lumen_qkv_bias_norm_store",
           [P, c_int, c_longlong, P, P, P, c_float, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int,
            c_int, c_int, P, c_int, c_int, c_float, P])
    check(f(ptr(qkv), S, N * width, ptr(bias), ptr(q_norm_w), ptr(k_norm_w), float(eps), ptr(cache_pos), ptr(tok_seq),
            ptr(block_table), block_table.stride(0), ptr(q_out), ptr(kcache), ptr(vcache), _is_bf16(q_out), N, nq * d,
            nkv, d, dv, int(k_layout), int(v_layout), ptr(cs) if rotary_dim else 0, int(rotary_dim),
            0 if value_unit_eps is None else 1, float(value_unit_eps or 0.0), stream_ptr()), "qkv_bias_norm_store")
    return q_out


ATTN_TALK_SCRATCH_BYTES = 256 << 20     # weights matrix of one pass over a step's tokens
ATTN_TALK_PART = 128                    # columns a block of the values kernel walks (TV_PART)


# Scratch of a prompt step's weights matrix; a step that needs more is worked on in passes over its
# rows. (Passes small enough for the matrix to stay in the L2 between the three kernels were measured
# and lost: 9.3 against 5.9 ms for eight layers at 2,048 tokens, since a pass then has fewer blocks
# than the device holds and each block's walk over its pages takes as long as before.)
ATTN_TALK_PROMPT_SCRATCH_BYTES = 1 << 30


def attn_talk_prompt_takes(q, nkv, dv, k_layout, v_layout) -> bool:
    """Whether the tensor-core kernels take this step (bfloat16, plain tiles, sizes in 16s)."""
    return (q.dtype == BF16 and k_layout == LAYOUT_LINEAR and v_layout == LAYOUT_LINEAR and
            bool(int_fn("attn_talk", "lumen_attn_talk_prompt_ok", [c_int] * 4)(
                int(q.shape[1]), int(nkv), int(q.shape[2]), int(dv))))


def attn_talk(q, kcache, vcache, block_table, tok_seq, tok_pos, talk, window, keep_first, scale, dv,
              k_layout=LAYOUT_LINEAR, v_layout=LAYOUT_LINEAR, cu_q=None, seq_start=None, n_seqs=0):
    """Attention with softmax weights mixed across heads (talk float32 [nq, nq]) before they meet
    the values, over the paged cache; a query at position p sees key j <= p if p - j < window
    (window 0: every key) or j < keep_first. q [N, nq, d]; keys [pages, nkv, PAGE, d]; values
    [pages, nkv, PAGE, dv]; returns [N, nq, dv] in q's type. With cu_q int32 [B + 1], seq_start
    int32 [B] and n_seqs = B (a step of prompts) the scores and the value products run on the
    tensor cores where attn_talk_prompt_takes says so."""
    N, nq, d = q.shape
    nkv = kcache.shape[1]
    require(q, q.dtype, "attn_talk.q")
    require(kcache, q.dtype, "attn_talk.kcache")
    require(vcache, q.dtype, "attn_talk.vcache")
    require(block_table, I32, "attn_talk.block_table")
    require(tok_seq, I32, "attn_talk.tok_seq")
    require(tok_pos, I32, "attn_talk.tok_pos")
    require(talk, F32, "attn_talk.talk")
    if tuple(talk.shape) != (nq, nq) or kcache.shape[3] != d or tuple(vcache.shape[1:]) != (nkv, PAGE, dv):
        raise KernelError(f"attn_talk: talk {tuple(talk.shape)}, keys {tuple(kcache.shape)}, values "
                          f"{tuple(vcache.shape)} do not fit {nq} heads of {d} / {dv}")
    bound = block_table.shape[1] * PAGE           # no sequence of the step is longer than its page table
    row_stride = max(1, min(int(window) + int(keep_first), bound) if window > 0 else bound)
    out = torch.empty((N, nq, dv), dtype=q.dtype, device=q.device)
    if cu_q is not None and n_seqs > 0 and attn_talk_prompt_takes(q, nkv, dv, k_layout, v_layout):
        require(cu_q, I32, "attn_talk.cu_q")
        require(seq_start, I32, "attn_talk.seq_start")
        if cu_q.numel() < n_seqs + 1 or seq_start.numel() < n_seqs:
            raise KernelError("attn_talk: metadata shorter than the batch")
        row_stride = (row_stride + 3) // 4 * 4
        rows_per_pass = min(N, max(64, ATTN_TALK_PROMPT_SCRATCH_BYTES // (nq * row_stride * 4) // 64 * 64))
        W = torch.empty((rows_per_pass, nq, row_stride), dtype=F32, device=q.device)
        f = fn("attn_talk", "lumen_attn_talk_prompt",
               [P, P, P, P, c_int, P, P, c_int, c_int, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                c_int, c_int, c_float, P])
        check(f(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), block_table.stride(0), ptr(cu_q), ptr(seq_start),
                int(n_seqs), N // 64 + int(n_seqs), ptr(tok_pos), ptr(talk), ptr(out), ptr(W), N, rows_per_pass,
                row_stride, nq, nkv, d, dv, int(window), int(keep_first), float(scale), stream_ptr()),
              "attn_talk_prompt")
        return out
    rows_per_pass = max(1, min(N, ATTN_TALK_SCRATCH_BYTES // (nq * row_stride * 4)))
    W = torch.empty((rows_per_pass, nq, row_stride), dtype=F32, device=q.device)      # the scores
    chunks = -(-row_stride // 64)             # per 64 columns the scores kernel leaves (maximum, sum)
    stats = torch.empty((rows_per_pass, nq, chunks, 2), dtype=F32, device=q.device)
    Z = -(-row_stride // ATTN_TALK_PART)
    parts = torch.empty((Z, rows_per_pass, nq, dv), dtype=F32, device=q.device) if Z > 1 else None
    f = fn("attn_talk", "lumen_attn_talk",
           [P, P, P, P, c_int, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
            c_int, c_float, c_int, c_int, P])
    check(f(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), block_table.stride(0), ptr(tok_seq), ptr(tok_pos),
            ptr(talk), ptr(out), ptr(W), ptr(stats), ptr(parts), _is_bf16(q), N, rows_per_pass, row_stride, nq, nkv, d, dv,
            int(window), int(keep_first), float(scale), int(k_layout), int(v_layout), stream_ptr()), "attn_talk")
    return out


def conv_silu(u, c0, C, weight, bias, state, ctx_tok_seq, cu_q, seq_slot, n_seqs, decode):
    """silu(bias + causal convolution over time) of columns c0 .. c0 + C - 1 of a projection that
    arrives as partial sums u float32 [S, N, W] (or [N, W]); weight float32 [taps, C], the last
    row the current token's; bias float32 [C] or None; state float32 [slots, taps - 1, C], the
    sequences' last inputs (row seq_slot[b] is sequence b's), moved on to the step's end.
    `decode`: every sequence brings exactly one token and row b is sequence b's. float32 [N, C]."""
    u, S = _partials(u, "conv_silu.u")
    _, N, W = u.shape
    require(weight, F32, "conv_silu.weight")
    taps = weight.shape[0]
    if weight.shape[1] != C or c0 < 0 or c0 + C > W or not 1 <= taps <= 16:
        raise KernelError(f"conv_silu: weight {tuple(weight.shape)} does not fit {C} of {W} columns (1 to 16 taps)")
    stride = 0
    if taps > 1:
        if state is None or state.dtype != F32 or tuple(state.shape[1:]) != (taps - 1, C) or state.stride(2) != 1 \
                or state.stride(1) != C:
            raise KernelError(f"conv_silu: state must be float32 [slots, {taps - 1}, {C}] with dense rows")
        stride = state.stride(0)
    if bias is not None:
        require(bias, F32, "conv_silu.bias")
    for t, nm in ((ctx_tok_seq, "tok_seq"), (cu_q, "cu_q"), (seq_slot, "seq_slot")):
        require(t, I32, f"conv_silu.{nm}")
    out = torch.empty((N, C), dtype=F32, device=u.device)
    f = fn("ssm", "lumen_conv_silu", [P, c_int, c_longlong, c_int, c_int, c_int, P, P, c_int, P, c_longlong, P, P, P,
                                      c_int, c_int, P, c_int, P])
    check(f(ptr(u), S, N * W, W, int(c0), int(C), ptr(weight), ptr(bias), taps, ptr(state) if taps > 1 else 0, stride,
            ptr(ctx_tok_seq), ptr(cu_q), ptr(seq_slot), int(n_seqs), 1 if decode else 0, ptr(out), N, stream_ptr()),
          "conv_silu")
    return out


def ssm_scan(xbc, heads, head_dim, state_size, groups, u, dt_col, dt_bias, a_log, d_skip, state, cu_q, seq_slot, n_seqs):
    """The recurrence of a state-space mixer, per head h (group g = h // (heads / groups)):
    S <- exp(-exp(a_log[h]) dt) S + dt B x^T, y = S^T C + d_skip[h] x, with dt = softplus(the
    projection's column dt_col + h, summed over its partials, + dt_bias[h]). xbc float32
    [N, heads * head_dim + 2 * groups * state_size] = (x, B, C); u float32 [S, N, W] or [N, W];
    state float32 [slots, heads, state_size, head_dim], row seq_slot[b] sequence b's, updated in
    place. Returns y float32 [N, heads * head_dim]."""
    require(xbc, F32, "ssm_scan.xbc")
    u, S = _partials(u, "ssm_scan.u")
    _, N, W = u.shape
    inner = heads * head_dim
    if tuple(xbc.shape) != (N, inner + 2 * groups * state_size) or heads % groups:
        raise KernelError(f"ssm_scan: xbc {tuple(xbc.shape)} does not fit {heads} heads of {head_dim}, "
                          f"{groups} groups of {state_size}")
    for t, nm in ((dt_bias, "dt_bias"), (a_log, "a_log"), (d_skip, "d_skip")):
        require(t, F32, f"ssm_scan.{nm}")
        if t.numel() != heads:
            raise KernelError(f"ssm_scan: {nm} must have {heads} values")
    require(state, F32, "ssm_scan.state", contiguous=False)
    if tuple(state.shape[1:]) != (heads, state_size, head_dim) or not state[0].is_contiguous():
        raise KernelError(f"ssm_scan: state must be float32 [slots, {heads}, {state_size}, {head_dim}]")
    require(cu_q, I32, "ssm_scan.cu_q")
    require(seq_slot, I32, "ssm_scan.seq_slot")
    y = torch.empty((N, inner), dtype=F32, device=xbc.device)
    f = fn("ssm", "lumen_ssm_scan", [P, c_int, c_int, c_int, c_int, P, c_int, c_longlong, c_int, c_int, P, P, P, P,
                                     c_longlong, P, P, c_int, P, c_int, P])
    check(f(ptr(xbc), heads, head_dim, state_size, groups, ptr(u), S, N * W, W, int(dt_col), ptr(dt_bias), ptr(a_log),
            ptr(d_skip), ptr(state), state.stride(0), ptr(cu_q), ptr(seq_slot), int(n_seqs), ptr(y), N, stream_ptr()),
          "ssm_scan")
    return y


def gated_part_norm(y, u, z_col, weight, eps, parts, out_dtype):
    """v = y * silu(z) with z the columns z_col .. of the projection's partial sums u, then an RMS
    norm of each of `parts` equal pieces of the row by its own root mean square, times weight.
    y float32 [N, W]; weight float32 [W]; returns [N, W] in out_dtype."""
    require(y, F32, "gated_part_norm.y")
    require(weight, F32, "gated_part_norm.weight")
    u, S = _partials(u, "gated_part_norm.u")
    N, W = y.shape
    if u.shape[1] != N or weight.numel() != W or parts < 1 or W % parts or z_col < 0 or z_col + W > u.shape[2]:
        raise KernelError(f"gated_part_norm: rows of {W} in {parts} parts do not fit {tuple(u.shape)}")
    out = torch.empty((N, W), dtype=out_dtype, device=y.device)
    f = fn("ssm", "lumen_gated_part_norm", [P, P, c_int, c_longlong, c_int, c_int, P, c_float, c_int, c_int, P, c_int,
                                            c_int, P])
    check(f(ptr(y), ptr(u), S, N * u.shape[2], u.shape[2], int(z_col), ptr(weight), float(eps), W, int(parts), ptr(out),
            _is_bf16(out), N, stream_ptr()), "gated_part_norm")
    return out


def xielu(z, act, out_dtype):
    """x > 0: softplus(p) x^2 + x/2; x <= 0: (1/2 + softplus(q)) (e^x - 1 - x) + x/2, with
    (p, q) = act float32 [2] on the device; z float32 [N, F] or [S, N, F] partials."""
    z, S = _partials(z, "xielu.z")
    require(act, F32, "xielu.act")
    if act.numel() != 2:
        raise KernelError("xielu: act holds two values")
    _, N, Fw = z.shape
    out = torch.empty((N, Fw), dtype=out_dtype, device=z.device)
    f = fn("ssm", "lumen_xielu", [P, c_int, c_longlong, P, P, c_int, c_longlong, P])
    check(f(ptr(z), S, N * Fw, ptr(act), ptr(out), _is_bf16(out), N * Fw, stream_ptr()), "xielu")
    return out


_moe_tile_rows = {}


def moe_tile_rows(tensor_cores: int) -> int:
    """Entries a row tile of the grouped products: 0 the 32-bit kernel's, 1 the tensor-core
    kernel's tall tiles, 2 its short ones (steps with few entries an expert)."""
    tensor_cores = int(tensor_cores)
    if tensor_cores not in _moe_tile_rows:
        _moe_tile_rows[tensor_cores] = int(int_fn("moe", "lumen_moe_tile_rows", [c_int])(tensor_cores))
    return _moe_tile_rows[tensor_cores]


def moe_takes_tensor_cores(a_dtype, w) -> bool:
    """bfloat16 activations and weights whose rows are multiples of 16 bytes go to the tensor
    cores; everything else (a 32-bit run, odd widths) to the 32-bit grouped product."""
    return (a_dtype == BF16 and w.dtype == BF16 and w.shape[2] % 8 == 0 and w.data_ptr() % 16 == 0)


ROUTER_MODES = {"softmax": 0, "sigmoid": 1}


def moe_route(logits, correction, top, scale, mode="softmax"):
    """Softmax over a token's router logits (float32 [N, E]) or, mode "sigmoid", a sigmoid of every
    logit by itself; the `top` experts with the largest score + correction (equal ones: the lower
    index), and their scores (without the correction) times `scale` as weights. Returns (idx int32
    [N, top], weights float32 [N, top])."""
    require(logits, F32, "moe_route.logits")
    N, E = logits.shape
    if correction is not None:
        require(correction, F32, "moe_route.correction")
        if correction.numel() != E:
            raise KernelError(f"moe_route: the correction must have {E} values")
    idx = torch.empty((N, top), dtype=I32, device=logits.device)
    wt = torch.empty((N, top), dtype=F32, device=logits.device)
    f = fn("moe", "lumen_moe_route", [P, P, c_int, c_int, c_float, P, P, c_int, c_int, P])
    check(f(ptr(logits), ptr(correction), E, int(top), float(scale), ptr(idx), ptr(wt), N, ROUTER_MODES[mode],
            stream_ptr()), "moe_route")
    return idx, wt


def moe_route_x(x, router, correction, top, scale, identity_out=None, n_experts=0, mode="softmax"):
    """moe_route with the router's product in the same kernel: x [N, K] in the run's type, router
    float32 [E, K]; the logits are float32 sums over float32(x) * router. With identity_out
    (float32 [top, N, K]) the choices whose index is >= n_experts are filled in there at once:
    weight * float32(x[token]) at [choice][token]."""
    require(router, F32, "moe_route_x.router")
    N, Kw = x.shape
    E = router.shape[0]
    if router.shape[1] != Kw or not x.is_contiguous() or not x.is_cuda:
        raise KernelError(f"moe_route_x: rows {tuple(x.shape)} do not fit the router {tuple(router.shape)}")
    if correction is not None:
        require(correction, F32, "moe_route_x.correction")
        if correction.numel() != E:
            raise KernelError(f"moe_route_x: the correction must have {E} values")
    if identity_out is not None:
        require(identity_out, F32, "moe_route_x.identity_out")
        if tuple(identity_out.shape) != (top, N, Kw):
            raise KernelError(f"moe_route_x: identity_out {tuple(identity_out.shape)} is not [{top}, {N}, {Kw}]")
    idx = torch.empty((N, top), dtype=I32, device=x.device)
    wt = torch.empty((N, top), dtype=F32, device=x.device)
    f = fn("moe", "lumen_moe_route_x", [P, c_int, P, c_int, P, c_int, c_int, c_float, P, P, P, c_int, c_int, c_int, P])
    check(f(ptr(x), _is_bf16(x), ptr(router), Kw, ptr(correction), E, int(top), float(scale), ptr(idx), ptr(wt),
            ptr(identity_out), int(n_experts), N, ROUTER_MODES[mode], stream_ptr()), "moe_route_x")
    return idx, wt


def moe_group(idx, n_experts, tensor_cores=False):
    """The step's (token, choice) entries in order of their expert, and the row tiles the grouped
    products walk (as tall as the kernel that will walk them takes: `tensor_cores`); entries
    whose index is >= n_experts are left out. Returns (sorted int32 [entries], tiles int32
    [max_tiles, 3], n_tiles int32 [1], max_tiles, which tiles: 0, 1 tall or 2 short)."""
    require(idx, I32, "moe_group.idx")
    entries = idx.numel()
    # few entries an expert (decode steps): short tiles, else the tensor cores spend the step on
    # empty rows. A row's sums do not depend on its tile's height, so both give the same bits.
    tensor_cores = (2 if entries <= 32 * int(n_experts) else 1) if tensor_cores else 0
    rows = moe_tile_rows(tensor_cores)
    max_tiles = entries // rows + min(int(n_experts), entries)
    sorted_ = torch.empty((entries,), dtype=I32, device=idx.device)
    tiles = torch.empty((max(max_tiles, 1), 3), dtype=I32, device=idx.device)
    n_tiles = torch.empty((1,), dtype=I32, device=idx.device)
    f = fn("moe", "lumen_moe_group", [P, c_int, c_int, c_int, P, P, P, P])
    check(f(ptr(idx), entries, int(n_experts), rows, ptr(sorted_), ptr(tiles), ptr(n_tiles), stream_ptr()), "moe_group")
    return sorted_, tiles, n_tiles, max_tiles, tensor_cores


def moe_product(a, w, group, weights, top, n_tokens, gated, out=None, clamp=None):
    """A grouped product over the tiles of moe_group. gated: a [tokens, K] in the run's type, w
    [E, 2 F, K] (gate rows, then up rows) -> silu(gate) * up as [entries, F] in a's type; with
    `weights` both sums are multiplied by the entry's weight first (the weight on the expert's
    input), with clamp = (limit, alpha) the activation is g sigmoid(alpha g) (v + 1), g = min(gate,
    limit), v = clamp(up, -limit, limit). Not gated: a [entries, K], w [E, D, K] -> float32 [top,
    tokens, D] with every entry's product times its weight (1 without `weights`) at [choice][token]
    (into `out` when given); rows of entries that are left out (identity experts) are not
    written."""
    sorted_, tiles, n_tiles, max_tiles, tensor_cores = group
    E, rows, K = w.shape
    if tensor_cores and not (moe_takes_tensor_cores(a.dtype, w) and a.data_ptr() % 16 == 0):
        raise KernelError("moe_product: tiles made for the tensor cores, operands that they do not take")
    if a.shape[1] != K or not a.is_contiguous() or not w.is_contiguous():
        raise KernelError(f"moe_product: activations {tuple(a.shape)} do not fit weights {tuple(w.shape)}")
    if gated:
        if rows % 2:
            raise KernelError("moe_product: gate and up rows come in equal numbers")
        n_out = rows // 2
        out = torch.empty((n_tokens * top, n_out), dtype=a.dtype, device=a.device)
    else:
        n_out = rows
        if out is None:
            out = torch.empty((top, n_tokens, n_out), dtype=F32, device=a.device)
        elif out.dtype != F32 or tuple(out.shape) != (top, n_tokens, n_out) or not out.is_contiguous():
            raise KernelError(f"moe_product: out {tuple(out.shape)} is not float32 [{top}, {n_tokens}, {n_out}]")
    if weights is not None:
        require(weights, F32, "moe_product.weights")
        if weights.numel() != n_tokens * top:
            raise KernelError(f"moe_product: {weights.numel()} weights for {n_tokens * top} entries")
    limit, alpha = (0.0, 1.0) if clamp is None else clamp
    f = fn("moe", "lumen_moe_product", [P, c_int, P, c_int, P, P, P, c_int, P, P, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_float, c_float, P])
    check(f(ptr(a), _is_bf16(a), ptr(w), _is_bf16(w), ptr(sorted_), ptr(tiles), ptr(n_tiles), int(max_tiles),
            ptr(weights), ptr(out), K, n_out, int(top), int(n_tokens), 1 if gated else 0, int(tensor_cores),
            0 if clamp is None else 1, float(limit), float(alpha), stream_ptr()), "moe_product")
    return out


def add_rmsnorm(h, delta, weight, eps, out_dtype, rows=None, write_h=True):
    """x = h + sum(delta[s]) ; y = rmsnorm(x) * weight. h float32 [N, H] (updated in
    place when write_h); delta None or float32 [S, N, H]; rows int32 [W] gathers."""
    require(h, F32, "add_rmsnorm.h")
    require(weight, F32, "add_rmsnorm.weight")
    N, H = h.shape
    if weight.numel() != H:
        raise KernelError(f"add_rmsnorm: weight has {weight.numel()} values, rows have {H}")
    S, stride = 0, 0
    if delta is not None:
        delta, S = _partials(delta, "add_rmsnorm.delta")
        if tuple(delta.shape[1:]) != (N, H):
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} does not match h {(N, H)}")
        stride = N * H
    n_rows = N
    if rows is not None:
        require(rows, I32, "add_rmsnorm.rows")
        n_rows = rows.numel()
    y = torch.empty((n_rows, H), dtype=out_dtype, device=h.device)
    f = fn("core", "lumen_add_rmsnorm",
           [P, P, c_int, c_longlong, P, c_float, P, c_int, P, c_int, c_int, c_int, P])
    check(f(ptr(h), ptr(delta), S, stride, ptr(weight), float(eps), ptr(y), _is_bf16(y), ptr(rows),
            n_rows, H, 1 if write_h else 0, stream_ptr()), "add_rmsnorm")
    return y


def silu_mul(gu, out_dtype, interleaved=False):
    """z = silu(gate) * up with gate = gu[..., :I], up = gu[..., I:] (or, interleaved,
    gate_i = gu[..., 2i], up_i = gu[..., 2i+1]); gu float32 [N, 2I] or [S, N, 2I] partials."""
    gu, S = _partials(gu, "silu_mul.gu")
    _, N, I2 = gu.shape
    if I2 % 2:
        raise KernelError("silu_mul: width must be even")
    z = torch.empty((N, I2 // 2), dtype=out_dtype, device=gu.device)
    f = fn("core", "lumen_silu_mul", [P, c_int, P, c_int, c_int, c_int, c_int, P])
    check(f(ptr(gu), S, ptr(z), _is_bf16(z), N, I2 // 2, 1 if interleaved else 0, stream_ptr()),
          "silu_mul")
    return z


def rope_table(positions, inv_freq, magnitude=1.0):
    """magnitude * (cos, sin) of float32(pos) * inv_freq: float32 [N, rot/2, 2]."""
    require(positions, I32, "rope_table.positions")
    require(inv_freq, F32, "rope_table.inv_freq")
    N, half = positions.numel(), inv_freq.numel()
    cs = torch.empty((N, half, 2), dtype=F32, device=positions.device)
    f = fn("core", "lumen_rope_table", [P, P, P, c_int, c_int, c_float, P])
    check(f(ptr(positions), ptr(inv_freq), ptr(cs), N, half, float(magnitude), stream_ptr()), "rope_table")
    return cs


def qk_norm_rope_store(qkv, q_norm_w, k_norm_w, eps, cs, rotary_dim, cache_pos, tok_seq,
                       block_table, kcache, vcache, nq, nkv, d, out_dtype, layout=LAYOUT_LINEAR):
    """Per-head RMSNorm of q and k, rotation by the angles of `cs` (from rope_table; None
    with rotary_dim 0), q out and k/v written to the paged cache.
    qkv float32 [N, (nq + 2 nkv) d] or [S, N, ...] partials; caches [pages, nkv, PAGE, d] of
    out_dtype (None with nkv == 0: a layer that reads another layer's cache)."""
    qkv, S = _partials(qkv, "qk_norm_rope_store.qkv")
    N = qkv.shape[1]
    if qkv.shape[2] != (nq + 2 * nkv) * d:
        raise KernelError(f"qk_norm_rope_store: row width {qkv.shape[2]} != (nq+2nkv)*d")
    for t, nm in ((q_norm_w, "q_norm"), (k_norm_w, "k_norm")):
        if t is not None:
            require(t, F32, nm)
            if t.numel() != d:
                raise KernelError(f"{nm} weight must have head_dim={d} values")
    if rotary_dim:
        require(cs, F32, "rope angles")
        if tuple(cs.shape) != (N, rotary_dim // 2, 2):
            raise KernelError(f"rope angles must be [N, rotary_dim/2, 2], got {tuple(cs.shape)}")
    for t, nm in ((cache_pos, "cache_pos"), (tok_seq, "tok_seq")):
        require(t, I32, nm)
        if t.numel() < N:
            raise KernelError(f"{nm} shorter than the token count")
    require(block_table, I32, "block_table")
    q_out = torch.empty((N, nq, d), dtype=out_dtype, device=qkv.device)
    if nkv:
        require(kcache, out_dtype, "kcache")
        require(vcache, out_dtype, "vcache")
    f = fn("core", "lumen_qk_norm_rope_store",
           [P, c_int, P, P, c_float, P, c_int, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int,
            c_int, c_int, P])
    check(f(ptr(qkv), S, ptr(q_norm_w), ptr(k_norm_w), float(eps), ptr(cs), int(rotary_dim),
            ptr(cache_pos), ptr(tok_seq), ptr(block_table), block_table.stride(0),
            ptr(q_out), ptr(kcache), ptr(vcache), _is_bf16(q_out), N, nq, nkv, d, int(layout),
            stream_ptr()),
          "qk_norm_rope_store")
    return q_out


def gemm_tc_qkv_takes(M, N, K, nq, nkv, d, rotary_dim) -> bool:
    """Whether gemm_tc_qkv takes this shape (a prompt-sized product, heads of 128, rotation
    over the whole head or none)."""
    return bool(int_fn("gemm_tc", "lumen_gemm_tc_qkv_ok", [c_int] * 7)(
        int(M), int(N), int(K), int(nq), int(nkv), int(d), int(rotary_dim)))


def gemm_tc_qkv(x, w, q_norm_w, k_norm_w, eps, cs, rotary_dim, cache_pos, tok_seq, block_table,
                kcache, vcache, nq, nkv):
    """The QKV product of a prompt with qk_norm_rope_store folded into its epilogue: x bfloat16
    [M, K], w a TiledWeight [(nq + 2 nkv) * 128, K] (q heads, k heads, v heads); returns q bfloat16
    [M, nq, 128], normed and rotated, and writes k and v to their places in the swizzled
    bfloat16 cache. Only where gemm_tc_qkv_takes says so."""
    require(x, BF16, "gemm_tc_qkv.x")
    if not isinstance(w, TiledWeight):
        raise KernelError("gemm_tc_qkv takes its weight in tiled form (tile_weight)")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not gemm_tc_qkv_takes(M, N, K, nq, nkv, 128, rotary_dim):
        raise KernelError(f"gemm_tc_qkv does not take [{M}, {K}] x [{N}, {w.shape[1]}] with {nq}+2x{nkv} heads")
    for t, nm in ((q_norm_w, "q_norm"), (k_norm_w, "k_norm")):
        if t is not None:
            require(t, F32, nm)
            if t.numel() != 128:
                raise KernelError(f"{nm} weight must have 128 values")
    if rotary_dim:
        require(cs, F32, "rope angles")
        if tuple(cs.shape) != (M, 64, 2):
            raise KernelError(f"rope angles must be [M, 64, 2], got {tuple(cs.shape)}")
    for t, nm in ((cache_pos, "cache_pos"), (tok_seq, "tok_seq")):
        require(t, I32, nm)
        if t.numel() < M:
            raise KernelError(f"{nm} shorter than the token count")
    require(block_table, I32, "block_table")
    require(kcache, BF16, "kcache")
    require(vcache, BF16, "vcache")
    if kcache.shape[1:] != (nkv, PAGE, 128) or vcache.shape != kcache.shape:
        raise KernelError(f"gemm_tc_qkv: caches must be [pages, nkv, {PAGE}, 128]")
    q_out = torch.empty((M, nq, 128), dtype=BF16, device=x.device)
    f = fn("gemm_tc", "lumen_gemm_tc_qkv",
           [P, P, c_int, c_int, c_int, c_int, P, P, P, P, P, c_float, P, c_int, P, P, P, c_int, c_int, c_int, P, P])
    check(f(ptr(x), ptr(w.data), M, N, K, w.padded_rows, ptr(q_out), ptr(kcache), ptr(vcache), ptr(q_norm_w), ptr(k_norm_w),
            float(eps), ptr(cs), int(rotary_dim), ptr(cache_pos), ptr(tok_seq), ptr(block_table),
            block_table.stride(0), nq, nkv, ptr(error_flag(x.device)), stream_ptr()), "gemm_tc_qkv")
    return q_out


def attn_generic(q, kcache, vcache, block_table, tok_seq, tok_pos, window, scale,
                 layout=LAYOUT_LINEAR, v_layout=None):
    """Causal attention of N query tokens over the paged cache. q [N, nq, d]; keys
    [pages, nkv, PAGE, d]; values [pages, nkv, PAGE, dv] (dv may differ from d); returns
    [N, nq, dv]. Scores and weights are float32 in either type."""
    N, nq, d = q.shape
    nkv = kcache.shape[1]
    dv = vcache.shape[3]
    v_layout = layout if v_layout is None else v_layout
    require(q, q.dtype, "attn.q")
    require(kcache, q.dtype, "attn.kcache")
    require(vcache, q.dtype, "attn.vcache")
    require(block_table, I32, "attn.block_table")
    require(tok_seq, I32, "attn.tok_seq")
    require(tok_pos, I32, "attn.tok_pos")
    if d > 1024 or dv > 512 or kcache.shape[3] != d or tuple(vcache.shape[1:3]) != tuple(kcache.shape[1:3]):
        raise KernelError(f"attention takes key sizes up to 1024, value sizes up to 512 and caches that fit them, not "
                          f"{d} / {dv} with {tuple(kcache.shape)} / {tuple(vcache.shape)}")
    out = torch.empty((N, nq, dv), dtype=q.dtype, device=q.device)
    f = fn("attn_generic", "lumen_attn_generic",
           [P, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, P])
    check(f(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), block_table.stride(0), ptr(tok_seq),
            ptr(tok_pos), ptr(out), _is_bf16(q), N, nq, nkv, d, dv, int(window), float(scale), int(layout),
            int(v_layout), stream_ptr()), "attn_generic")
    return out


def attn_generic_opt(q, kcache, vcache, block_table, tok_seq, tok_pos, window, scale, layout=LAYOUT_LINEAR,
                     v_layout=None, chunk=0, softcap=0.0, sink=False, values_in_keys=False, value_dim=None,
                     gate=None, gate_col=0):
    """attn_generic with options. `chunk` > 0: a query sees only keys of its own run of `chunk`
    positions (counted from the sequence's start); `softcap` > 0: scores become softcap *
    tanh(score / softcap); `sink`: the softmax's denominator has one more term exp(0);
    `values_in_keys`: a key's value is the first `value_dim` numbers of the key's row (vcache is
    not read); `gate` (float32 [N, W] or [S, N, W] partial sums): the output is multiplied by
    sigmoid of its columns gate_col + head * dv + e. q may be float32 over a bfloat16 cache; the
    output has q's type."""
    N, nq, d = q.shape
    nkv = kcache.shape[1]
    dv = int(value_dim) if values_in_keys else vcache.shape[3]
    v_layout = layout if (v_layout is None or values_in_keys) else v_layout
    require(q, q.dtype, "attn.q")
    require(kcache, kcache.dtype, "attn.kcache")
    if not values_in_keys:
        require(vcache, kcache.dtype, "attn.vcache")
    if q.dtype not in (F32, kcache.dtype):
        raise KernelError(f"attention: queries are float32 or of the cache's type, not {q.dtype} over {kcache.dtype}")
    for t, nm in ((block_table, "block_table"), (tok_seq, "tok_seq"), (tok_pos, "tok_pos")):
        require(t, I32, f"attn.{nm}")
    if d > 1024 or dv > 512 or kcache.shape[3] != d or (values_in_keys and dv > d):
        raise KernelError(f"attention takes key sizes up to 1024 and value sizes up to 512, not {d} / {dv}")
    gS = gstride = gW = 0
    if gate is not None:
        gate, gS = _partials(gate, "attn.gate")
        gW, gstride = gate.shape[2], gate.shape[1] * gate.shape[2]
        if gate.shape[1] != N:
            raise KernelError("attention: the gate has one row a token")
    out = torch.empty((N, nq, dv), dtype=q.dtype, device=q.device)
    f = fn("attn_generic", "lumen_attn_generic_opt",
           [P, c_int, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
            c_int, c_float, c_int, c_int, P, c_int, c_longlong, c_int, c_int, P])
    check(f(ptr(q), 1 if q.dtype == F32 else 0, ptr(kcache), ptr(kcache if values_in_keys else vcache), ptr(block_table),
            block_table.stride(0), ptr(tok_seq), ptr(tok_pos), ptr(out), _is_bf16(kcache), N, nq, nkv, d, dv,
            int(window), float(scale), int(layout), int(v_layout), int(chunk), float(softcap or 0.0), 1 if sink else 0,
            1 if values_in_keys else 0, ptr(gate), gS, gstride, gW, int(gate_col), stream_ptr()), "attn_generic_opt")
    return out


def qkv_head_norm_store(qkv, bias, q_norm_w, k_norm_w, eps, cs, rotary_dim, cache_pos, tok_seq, block_table, kcache,
                        vcache, nq, nkv, d, dv, out_dtype, k_layout=LAYOUT_LINEAR, v_layout=LAYOUT_LINEAR,
                        store_kv=True):
    """Biases, an RMS norm of every query and key head (weights of d values, or None), rotation of
    the first rotary_dim values of every query and key head by the angles of `cs`, q out as
    [N, nq, d], keys [pages, nkv, PAGE, d] and values [pages, nkv, PAGE, dv] into the paged cache.
    qkv float32 [N, W] or [S, N, W] partial sums whose rows begin with nq heads of d, nkv of d and
    nkv of dv (further columns are not read); bias float32 over those columns or None. With
    store_kv False only the queries are made."""
    qkv, S = _partials(qkv, "qkv_head_norm_store.qkv")
    N, W = qkv.shape[1], qkv.shape[2]
    used = nq * d + (nkv * (d + dv) if store_kv else 0)
    if W < used:
        raise KernelError(f"qkv_head_norm_store: rows of {W} are narrower than the {used} columns of q, k and v")
    for t, nm, n in ((bias, "bias", used), (q_norm_w, "q_norm", d), (k_norm_w, "k_norm", d)):
        if t is not None:
            require(t, F32, f"qkv_head_norm_store.{nm}")
            if t.numel() < n:
                raise KernelError(f"qkv_head_norm_store: {nm} must have {n} values")
    if rotary_dim:
        require(cs, F32, "qkv_head_norm_store.cs")
        if tuple(cs.shape) != (N, rotary_dim // 2, 2):
            raise KernelError(f"qkv_head_norm_store: angles {tuple(cs.shape)} do not fit {N} tokens and {rotary_dim}")
    for t, nm in ((cache_pos, "cache_pos"), (tok_seq, "tok_seq")):
        require(t, I32, nm)
        if t.numel() < N:
            raise KernelError(f"{nm} shorter than the token count")
    require(block_table, I32, "block_table")
    if store_kv:
        require(kcache, out_dtype, "kcache")
        require(vcache, out_dtype, "vcache")
        if tuple(kcache.shape[1:]) != (nkv, PAGE, d) or tuple(vcache.shape[1:]) != (nkv, PAGE, dv):
            raise KernelError(f"qkv_head_norm_store: caches {tuple(kcache.shape)}, {tuple(vcache.shape)} do not fit "
                              f"{nkv} kv heads of {d} and {dv}")
    q_out = torch.empty((N, nq, d), dtype=out_dtype, device=qkv.device)
    f = fn("head_ops", "lumen_qkv_head_norm_store",
           [P, c_int, c_longlong, c_int, P, P, P, c_float, P, c_int, P, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int,
            c_int, c_int, c_int, c_int, c_int, P])
    check(f(ptr(qkv), S, N * W, W, ptr(bias), ptr(q_norm_w), ptr(k_norm_w), float(eps), ptr(cs) if rotary_dim else 0,
            int(rotary_dim), ptr(cache_pos), ptr(tok_seq), ptr(block_table), block_table.stride(0), ptr(q_out),
            ptr(kcache) if store_kv else 0, ptr(vcache) if store_kv else 0, _is_bf16(q_out), N, nq, nkv, d, dv,
            int(k_layout), int(v_layout), 1 if store_kv else 0, stream_ptr()), "qkv_head_norm_store")
    return q_out


def latent_store(u, col, rank, rot_width, norm_w, eps, cs, rotary_dim, cache_pos, tok_seq, block_table, cache):
    """What latent attention keeps of a token: columns col .. col + rank of the projection u (float32
    [N, W] or partial sums), RMS-normed with norm_w, and behind them the next rot_width columns with
    their first rotary_dim values rotated by `cs`; written as one row [rank + rot_width] of the paged
    cache [pages, 1, PAGE, rank + rot_width] (plain tiles)."""
    u, S = _partials(u, "latent_store.u")
    N, W = u.shape[1], u.shape[2]
    require(norm_w, F32, "latent_store.norm_w")
    if norm_w.numel() != rank or tuple(cache.shape[1:]) != (1, PAGE, rank + rot_width):
        raise KernelError(f"latent_store: weight of {norm_w.numel()}, cache {tuple(cache.shape)} do not fit a latent "
                          f"of {rank} + {rot_width}")
    if rotary_dim:
        require(cs, F32, "latent_store.cs")
        if tuple(cs.shape) != (N, rotary_dim // 2, 2):
            raise KernelError(f"latent_store: angles {tuple(cs.shape)} do not fit {N} tokens and {rotary_dim}")
    for t, nm in ((cache_pos, "cache_pos"), (tok_seq, "tok_seq"), (block_table, "block_table")):
        require(t, I32, f"latent_store.{nm}")
    f = fn("head_ops", "lumen_latent_store",
           [P, c_int, c_longlong, c_int, c_int, c_int, c_int, P, c_float, P, c_int, P, P, P, c_int, P, c_int, c_int, P])
    check(f(ptr(u), S, N * W, W, int(col), int(rank), int(rot_width), ptr(norm_w), float(eps),
            ptr(cs) if rotary_dim else 0, int(rotary_dim), ptr(cache_pos), ptr(tok_seq), ptr(block_table),
            block_table.stride(0), ptr(cache), _is_bf16(cache), N, stream_ptr()), "latent_store")


def latent_query(q, up_k, heads, d, rot_width, rank, cs, rotary_dim, out_dtype=F32):
    """Queries carried into the latent space: q float32 [N, W] or partial sums, rows of `heads` heads
    of [d | rot_width]; up_k [heads * d, rank] (the keys' up-projection). Returns [N, heads,
    rank + rot_width] in out_dtype (float32 or bfloat16): sum_j q[h, j] up_k[h d + j, :], then the
    rot_width values with the first rotary_dim rotated by `cs`."""
    q, S = _partials(q, "latent_query.q")
    N, W = q.shape[1], q.shape[2]
    if tuple(up_k.shape) != (heads * d, rank) or not up_k.is_contiguous() or W < heads * (d + rot_width):
        raise KernelError(f"latent_query: up-projection {tuple(up_k.shape)} and rows of {W} do not fit {heads} heads "
                          f"of {d} + {rot_width} over a latent of {rank}")
    if rotary_dim:
        require(cs, F32, "latent_query.cs")
        if tuple(cs.shape) != (N, rotary_dim // 2, 2):
            raise KernelError(f"latent_query: angles {tuple(cs.shape)} do not fit {N} tokens and {rotary_dim}")
    out = torch.empty((N, heads, rank + rot_width), dtype=out_dtype, device=q.device)
    Wo = rank + rot_width
    product = 1
    if out_dtype == BF16 and up_k.dtype == BF16 and _head_gemm_takes(W, d + rot_width, N * W, rank, d * rank,
                                                                   heads * Wo, Wo, d, rank):
        # the products on the tensor cores; the kernel below then only moves and rotates the rest
        g = fn("head_ops", "lumen_head_gemm", _HEAD_GEMM_ARGS)
        check(g(ptr(q), S, N * W, W, d + rot_width, ptr(up_k), 1, rank, d * rank, ptr(out), heads * Wo, Wo, N,
                int(heads), int(d), int(rank), *_NO_HEAD_GATE, stream_ptr()), "head_gemm")
        product = 0
    f = fn("head_ops", "lumen_latent_query",
           [P, c_int, c_longlong, c_int, P, c_int, c_int, c_int, c_int, c_int, P, c_int, P, c_int, c_int, c_int, P])
    check(f(ptr(q), S, N * W, W, ptr(up_k), _is_bf16(up_k), int(heads), int(d), int(rot_width), int(rank),
            ptr(cs) if rotary_dim else 0, int(rotary_dim), ptr(out), _is_bf16(out), product, N, stream_ptr()),
          "latent_query")
    return out


_HEAD_GEMM_ARGS = [P, c_int, c_longlong, c_longlong, c_int, P, c_int, c_int, c_longlong, P, c_longlong, c_int, c_int,
                   c_int, c_int, c_int, P, c_int, c_longlong, c_int, c_int, P]
_NO_HEAD_GATE = (0, 0, 0, 0, 0)


def _head_gemm_takes(xrs, xhs, split_stride, ldw, w_head_stride, ors, ohs, J, E) -> bool:
    f = int_fn("head_ops", "lumen_head_gemm_takes",
               [c_longlong, c_int, c_longlong, c_int, c_longlong, c_longlong, c_int, c_int, c_int])
    return bool(f(int(xrs), int(xhs), int(split_stride), int(ldw), int(w_head_stride), int(ors), int(ohs), int(J), int(E)))


ATTN_LATENT_ROWS = 64      # (token, head) rows a block of attn_latent takes


def attn_latent_takes(width, value_dim, dtype) -> bool:
    """Whether attn_latent runs a bfloat16 latent cache with rows of `width` values, the first
    `value_dim` of them the value: widths that are multiples of 16 and fit a block's shared memory
    with the queries and two key tiles, values that are multiples of 8 up to 512."""
    if dtype != BF16:
        return False
    f = int_fn("attn_latent", "lumen_attn_latent_takes", [c_int, c_int])
    return bool(f(int(width), int(value_dim)))


ATTN_LATENT_DECODE_SPLIT = 8   # blocks that share a row's keys in steps of one token a sequence


def attn_latent(q, cache, block_table, cu_q, seq_start, q_lens, value_dim, window, scale, n_seqs=None, n_split=1):
    """Causal attention over a latent cache on the tensor cores (mma.sync): q bfloat16 [N, H, W],
    already in the cache's space; cache bfloat16 [pages, 1, PAGE, W] (plain tiles), a row the key of
    every head and its first value_dim numbers the value of every head; a query at position p sees
    key j if 0 <= p - j < window (window 0: every earlier key). Returns float32 [N, H, value_dim].
    Prompts and decoded tokens alike; q_lens (host list) or, with q_lens None, n_seqs = B as in
    attn_prefill. n_split > 1 shares a row's keys out among that many blocks (a second kernel merges
    them): for steps with few rows."""
    N, H, W = q.shape
    B = len(q_lens) if q_lens is not None else int(n_seqs)
    require(q, BF16, "attn_latent.q")
    require(cache, BF16, "attn_latent.cache")
    for t, nm in ((block_table, "block_table"), (cu_q, "cu_q"), (seq_start, "seq_start")):
        require(t, I32, f"attn_latent.{nm}")
    if tuple(cache.shape[1:]) != (1, PAGE, W):
        raise KernelError(f"attn_latent: cache {tuple(cache.shape)} does not fit rows of {W}")
    if cu_q.numel() < B + 1 or seq_start.numel() < B or block_table.shape[0] < B or \
            (q_lens is not None and sum(q_lens) != N):
        raise KernelError("attn_latent: metadata does not match the batch")
    rows = ATTN_LATENT_ROWS
    # sum of ceil(q_b H / rows) over any division of N tokens into B sequences is at most N H // rows + B
    n_tiles = sum((n * H + rows - 1) // rows for n in q_lens) if q_lens is not None else N * H // rows + B
    out = torch.empty((N, H, int(value_dim)), dtype=F32, device=q.device)
    n_split = int(n_split)
    part = torch.empty((n_split, N * H, int(value_dim) + 2), dtype=F32, device=q.device) if n_split > 1 else None
    f = fn("attn_latent", "lumen_attn_latent",
           [P, P, P, c_int, P, P, c_int, c_int, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_float, P, P])
    check(f(ptr(q), ptr(cache), ptr(block_table), block_table.stride(0), ptr(cu_q), ptr(seq_start), B, n_tiles,
            ptr(out), ptr(part), n_split, N, H, W, int(value_dim), int(window), float(scale),
            ptr(error_flag(q.device)), stream_ptr()), "attn_latent")
    return out


def head_product(x, w, out_dtype, gate=None, gate_col=0):
    """out[n, h, :] = w_h x[n, h, :] with w [heads * E, J] cut into `heads` matrices [E, J]; x float32
    [N, heads, J]; returns [N, heads * E] in out_dtype. In bfloat16, with J a multiple of 32 and E of
    8, on the tensor cores (x rounded to bfloat16 as it is staged). With `gate` (float32 [N, W] or
    partial sums) head h's output is multiplied by sigmoid(gate[n, gate_col + h]) before it is
    rounded."""
    require(x, F32, "head_product.x")
    N, H, J = x.shape
    hg = _NO_HEAD_GATE
    if gate is not None:
        gate, gS = _partials(gate, "head_product.gate")
        if gate.shape[1] != N or gate_col + H > gate.shape[2]:
            raise KernelError(f"head_product: gate {tuple(gate.shape)} has no {H} columns from {gate_col} for {N} tokens")
        hg = (ptr(gate), gS, N * gate.shape[2], gate.shape[2], int(gate_col))
    if w.dim() != 2 or w.shape[1] != J or w.shape[0] % H or not w.is_contiguous():
        raise KernelError(f"head_product: weight {tuple(w.shape)} does not fit {H} heads of {J}")
    E = w.shape[0] // H
    out = torch.empty((N, H * E), dtype=out_dtype, device=x.device)
    if out_dtype == BF16 and w.dtype == BF16 and _head_gemm_takes(H * J, J, 0, J, E * J, H * E, E, J, E):
        g = fn("head_ops", "lumen_head_gemm", _HEAD_GEMM_ARGS)
        check(g(ptr(x), 1, 0, H * J, J, ptr(w), 0, J, E * J, ptr(out), H * E, E, N, H, J, E, *hg, stream_ptr()),
              "head_gemm")
        return out
    f = fn("head_ops", "lumen_head_product", [P, P, c_int, P, c_int, c_int, c_int, c_int, c_int, P, c_int, c_longlong,
                                              c_int, c_int, P])
    check(f(ptr(x), ptr(w), _is_bf16(w), ptr(out), _is_bf16(out), N, H, J, E, *hg, stream_ptr()), "head_product")
    return out


def gelu_tanh(z, out_dtype):
    """0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); z float32 [N, F] or [S, N, F] partial sums."""
    z, S = _partials(z, "gelu_tanh.z")
    _, N, Fw = z.shape
    out = torch.empty((N, Fw), dtype=out_dtype, device=z.device)
    f = fn("head_ops", "lumen_gelu_tanh", [P, c_int, c_longlong, P, c_int, c_longlong, P])
    check(f(ptr(z), S, N * Fw, ptr(out), _is_bf16(out), N * Fw, stream_ptr()), "gelu_tanh")
    return out


def relu2(z, out_dtype):
    """max(z, 0)^2; z float32 [N, F] or [S, N, F] partial sums."""
    z, S = _partials(z, "relu2.z")
    _, N, Fw = z.shape
    out = torch.empty((N, Fw), dtype=out_dtype, device=z.device)
    f = fn("head_ops", "lumen_relu2", [P, c_int, c_longlong, P, c_int, c_longlong, P])
    check(f(ptr(z), S, N * Fw, ptr(out), _is_bf16(out), N * Fw, stream_ptr()), "relu2")
    return out


def clamped_glu(u, width, limit, alpha, out_dtype, token_gate_col=-1):
    """A gated unit with clamped halves: u float32 [N, W] or partial sums, a row `width` gate values,
    then `width` up values; g = min(gate, limit), v = clamp(up, -limit, limit); returns
    g sigmoid(alpha g) (v + 1) as [N, width] in out_dtype, times sigmoid(u[n, token_gate_col]) where
    that column is given (one gate a token)."""
    u, S = _partials(u, "clamped_glu.u")
    _, N, W = u.shape
    if 2 * width > W or token_gate_col >= W:
        raise KernelError(f"clamped_glu: rows of {W} do not hold two halves of {width} (and the gate's column)")
    out = torch.empty((N, int(width)), dtype=out_dtype, device=u.device)
    f = fn("head_ops", "lumen_clamped_glu", [P, c_int, c_longlong, c_int, c_int, c_float, c_float, c_int, P, c_int, c_int, P])
    check(f(ptr(u), S, N * W, W, int(width), float(limit), float(alpha), int(token_gate_col), ptr(out), _is_bf16(out), N,
            stream_ptr()), "clamped_glu")
    return out


def cols_rmsnorm(u, col, width, weight, eps, out_dtype, gate=None, gate_col=0):
    """Columns col .. col + width of u (float32 [N, W] or partial sums, added) divided by their root
    mean square (sqrt(mean(x^2) + eps)) times weight [width], in out_dtype; with `gate` (float32 [N, Wg]
    or partial sums) also times sigmoid(gate[n, gate_col + c]), element by element."""
    u, S = _partials(u, "cols_rmsnorm.u")
    _, N, W = u.shape
    hg = (0, 0, 0, 0, 0)
    if gate is not None:
        gate, gS = _partials(gate, "cols_rmsnorm.gate")
        if gate.shape[1] != N or gate_col < 0 or gate_col + width > gate.shape[2]:
            raise KernelError(f"cols_rmsnorm: gate {tuple(gate.shape)} has no {width} columns from {gate_col} for {N} rows")
        hg = (ptr(gate), gS, N * gate.shape[2], gate.shape[2], int(gate_col))
    require(weight, F32, "cols_rmsnorm.weight")
    if weight.numel() != width or col < 0 or col + width > W:
        raise KernelError(f"cols_rmsnorm: {width} columns from {col} of rows of {W}, a weight of {weight.numel()}")
    out = torch.empty((N, int(width)), dtype=out_dtype, device=u.device)
    f = fn("head_ops", "lumen_cols_rmsnorm", [P, c_int, c_longlong, c_int, c_int, c_int, P, c_float, P, c_int, c_int,
                                              P, c_int, c_longlong, c_int, c_int, P])
    check(f(ptr(u), S, N * W, W, int(col), int(width), ptr(weight), float(eps), ptr(out), _is_bf16(out), N, *hg,
            stream_ptr()), "cols_rmsnorm")
    return out


def scale_softcap(logits, scale, cap):
    """In place: logits * scale, then, with cap > 0, cap * tanh(that / cap). float32, contiguous."""
    require(logits, F32, "scale_softcap.logits")
    f = fn("head_ops", "lumen_scale_softcap", [P, c_float, c_float, c_longlong, P])
    check(f(ptr(logits), float(scale), float(cap or 0.0), logits.numel(), stream_ptr()), "scale_softcap")
    return logits


SCALED_GROUPS = 4      # groups of partial sums one launch of add_scaled_dyt takes


def add_scaled_dyt(h, groups, weight, bias, alpha, out_dtype, rows=None, write_h=True):
    """x = h + sum over (delta, scale) in `groups`, over delta's partial sums, of scale * delta[s]
    (h float32 [N, H], updated in place when write_h; a delta float32 [N, H] or [S, N, H]); then
    y = tanh(alpha * x) * weight + bias in out_dtype, alpha a float32 tensor of one value on the
    device. With weight None nothing is normed and None is returned (the stream has its update);
    rows int32 [W] gathers the rows to work on."""
    require(h, F32, "add_scaled_dyt.h")
    N, H = h.shape
    groups = list(groups or ())
    while len(groups) > SCALED_GROUPS:          # more groups than a launch takes: the first ones in launches of their own
        add_scaled_dyt(h, groups[:SCALED_GROUPS], None, None, None, out_dtype)
        groups = groups[SCALED_GROUPS:]
    n = len(groups)
    ptrs, strides, counts, scales = (c_void_p * max(n, 1))(), (c_longlong * max(n, 1))(), (c_int * max(n, 1))(), \
        (c_float * max(n, 1))()
    for g, (delta, scale) in enumerate(groups):
        delta, S = _partials(delta, "add_scaled_dyt.delta")
        if tuple(delta.shape[1:]) != (N, H):
            raise KernelError(f"add_scaled_dyt: update {tuple(delta.shape)} does not fit the stream {(N, H)}")
        ptrs[g], strides[g], counts[g], scales[g] = ptr(delta), N * H, S, float(scale)
    n_rows, y = N, None
    if rows is not None:
        require(rows, I32, "add_scaled_dyt.rows")
        n_rows = rows.numel()
    if weight is not None:
        for t, nm, k in ((weight, "weight", H), (bias, "bias", H), (alpha, "alpha", 1)):
            require(t, F32, f"add_scaled_dyt.{nm}")
            if t.numel() != k:
                raise KernelError(f"add_scaled_dyt: {nm} has {t.numel()} values, not {k}")
        y = torch.empty((n_rows, H), dtype=out_dtype, device=h.device)
    elif n == 0:
        return None
    f = fn("layer_ops", "lumen_add_scaled_dyt", [P, P, P, P, P, c_int, P, P, P, P, c_int, P, c_int, c_int, c_int, P])
    check(f(ptr(h), ptrs, strides, counts, scales, n, ptr(weight), ptr(bias), ptr(alpha), ptr(y),
            _is_bf16(y) if y is not None else 0, ptr(rows), n_rows, H, 1 if write_h else 0, stream_ptr()),
          "add_scaled_dyt")
    return y


def linear_attn_max_dim() -> int:
    return int(int_fn("linear_attn", "lumen_linear_attn_max_dim", [])())


def linear_attn(u, q_col, k_col, v_col, silu, decay, state, cu_q, seq_slot, n_seqs, heads, d, dv):
    """Linear attention with a fixed decay a head (csrc/linear_attn.cu): S <- decay_h S + k v^T,
    o = S^T q for every token in order. u: float32 [N, W] or partial sums with q and k (heads of d)
    from q_col and k_col and v (heads of dv) from v_col, each through SiLU when `silu`; decay float32
    [heads]; state float32 [slots, heads, d, dv] (row seq_slot[b] sequence b's, updated in place).
    Returns float32 [N, heads * dv]."""
    u, S = _partials(u, "linear_attn.u")
    N, W = u.shape[1], u.shape[2]
    require(decay, F32, "linear_attn.decay")
    require(state, F32, "linear_attn.state", contiguous=False)
    if decay.numel() != heads or tuple(state.shape[1:]) != (heads, d, dv) or not state[0].is_contiguous():
        raise KernelError(f"linear_attn: decay of {decay.numel()}, state {tuple(state.shape)} do not fit {heads} heads of "
                          f"{d} x {dv}")
    require(cu_q, I32, "linear_attn.cu_q")
    require(seq_slot, I32, "linear_attn.seq_slot")
    if cu_q.numel() < n_seqs + 1 or seq_slot.numel() < n_seqs:
        raise KernelError("linear_attn: metadata does not match the batch")
    out = torch.empty((N, heads * dv), dtype=F32, device=u.device)
    # prompts: the activated q, k and v once for all blocks, in a dense buffer that the walk copies from
    dense = None
    if int_fn("linear_attn", "lumen_linear_attn_wants_dense", [c_int, c_int, c_int, c_int])(N, int(n_seqs), int(d), int(dv)):
        dense = torch.empty((N, 2 * heads * d + heads * dv), dtype=F32, device=u.device)
    f = fn("linear_attn", "lumen_linear_attn",
           [P, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, P, P, c_longlong, P, P, c_int, P, c_int, c_int,
            c_int, P, c_int, P])
    check(f(ptr(u), S, N * W, W, int(q_col), int(k_col), int(v_col), 1 if silu else 0, ptr(decay), ptr(state),
            state.stride(0), ptr(cu_q), ptr(seq_slot), int(n_seqs), ptr(out), int(heads), int(d), int(dv), ptr(dense), N,
            stream_ptr()), "linear_attn")
    return out


def token_gate(z, tokens, table, col, out_dtype):
    """gelu_tanh(z[n, c]) * table[tokens[n], col + c]; z float32 [N, C] or partial sums; table [V, W]."""
    z, S = _partials(z, "token_gate.z")
    _, N, C = z.shape
    require(tokens, I32, "token_gate.tokens")
    if table.dim() != 2 or not table.is_contiguous() or not table.is_cuda or tokens.numel() < N:
        raise KernelError("token_gate: the table must be a contiguous CUDA matrix, one token a row of z")
    out = torch.empty((N, C), dtype=out_dtype, device=z.device)
    f = fn("head_ops", "lumen_token_gate", [P, c_int, c_longlong, P, P, c_int, c_int, c_int, c_int, P, c_int, c_int, P])
    check(f(ptr(z), S, N * C, ptr(tokens), ptr(table), _is_bf16(table), table.shape[1], int(col), C, ptr(out),
            _is_bf16(out), N, stream_ptr()), "token_gate")
    return out


def add_cast(h, delta, out_dtype):
    """h += the partial sums of delta (float32 [N, H] or [S, N, H]; None: nothing to add), in place;
    returns h in out_dtype."""
    require(h, F32, "add_cast.h")
    S = 0
    if delta is not None:
        delta, S = _partials(delta, "add_cast.delta")
        if tuple(delta.shape[1:]) != tuple(h.shape):
            raise KernelError(f"add_cast: update {tuple(delta.shape)} does not fit the stream {tuple(h.shape)}")
    out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
    f = fn("head_ops", "lumen_add_cast", [P, P, c_int, c_longlong, P, c_int, c_longlong, P])
    check(f(ptr(h), ptr(delta), S, h.numel(), ptr(out), _is_bf16(out), h.numel(), stream_ptr()), "add_cast")
    return out


def cols_cast(u, col, width, out_dtype):
    """Columns col .. col + width of u (float32 [N, W] or partial sums, added) in out_dtype."""
    u, S = _partials(u, "cols_cast.u")
    _, N, W = u.shape
    out = torch.empty((N, width), dtype=out_dtype, device=u.device)
    f = fn("head_ops", "lumen_cols_cast", [P, c_int, c_longlong, c_int, c_int, c_int, P, c_int, c_int, P])
    check(f(ptr(u), S, N * W, W, int(col), int(width), ptr(out), _is_bf16(out), N, stream_ptr()), "cols_cast")
    return out


def head_norm_gate(y, weight, eps, gate, gate_col, heads, out_dtype):
    """Every head of y (float32 [N, heads * E]) divided by its root mean square, times weight [E],
    times sigmoid of the gate's columns gate_col + h E + e (float32 [N, W] or partial sums)."""
    require(y, F32, "head_norm_gate.y")
    require(weight, F32, "head_norm_gate.weight")
    gate, S = _partials(gate, "head_norm_gate.gate")
    N = y.shape[0]
    E = y.shape[1] // heads
    if weight.numel() != E or gate.shape[1] != N or heads * E != y.shape[1]:
        raise KernelError(f"head_norm_gate: weight of {weight.numel()}, gate {tuple(gate.shape)} do not fit {heads} "
                          f"heads of {E}")
    out = torch.empty((N, heads * E), dtype=out_dtype, device=y.device)
    f = fn("head_ops", "lumen_head_norm_gate",
           [P, P, c_float, P, c_int, c_longlong, c_int, c_int, P, c_int, c_int, c_int, c_int, P])
    check(f(ptr(y), ptr(weight), float(eps), ptr(gate), S, N * gate.shape[2], gate.shape[2], int(gate_col), ptr(out),
            _is_bf16(out), N, int(heads), E, stream_ptr()), "head_norm_gate")
    return out


def delta_rule(x, q_col, k_col, v_col, u, beta_col, a, dt_bias, a_log, state, cu_q, seq_slot, n_seqs, heads, kv_heads,
               d, dv):
    """The gated delta rule with a decay a key channel (csrc/delta_rule.cu). x float32 [N, C]: q
    (kv_heads heads of d from q_col), k (k_col), v (heads of dv from v_col), convolved and activated;
    u: projection partial sums with the heads' beta logits from beta_col; a: partial sums [.., N,
    heads * d] of the decay logits; state float32 [slots, heads, dv, d] (row seq_slot[b] sequence
    b's, updated in place). Returns float32 [N, heads * dv]."""
    require(x, F32, "delta_rule.x")
    u, uS = _partials(u, "delta_rule.u")
    a, aS = _partials(a, "delta_rule.a")
    N, C = x.shape
    if u.shape[1] != N or tuple(a.shape[1:]) != (N, heads * d):
        raise KernelError(f"delta_rule: projections {tuple(u.shape)}, {tuple(a.shape)} do not fit {N} tokens and "
                          f"{heads} heads of {d}")
    for t, nm, n in ((dt_bias, "dt_bias", heads * d), (a_log, "a_log", heads)):
        require(t, F32, f"delta_rule.{nm}")
        if t.numel() != n:
            raise KernelError(f"delta_rule: {nm} must have {n} values")
    require(state, F32, "delta_rule.state", contiguous=False)
    if tuple(state.shape[1:]) != (heads, dv, d) or not state[0].is_contiguous():
        raise KernelError(f"delta_rule: state must be float32 [slots, {heads}, {dv}, {d}]")
    require(cu_q, I32, "delta_rule.cu_q")
    require(seq_slot, I32, "delta_rule.seq_slot")
    y = torch.empty((N, heads * dv), dtype=F32, device=x.device)
    # what does not depend on the state, a row a (token, head), made by the kernel's first launch
    row = int_fn("delta_rule", "lumen_delta_rule_scratch_row", [c_int])(int(d))
    prep = torch.empty((N, int(heads), row), dtype=F32, device=x.device)
    f = fn("delta_rule", "lumen_delta_rule",
           [P, c_int, c_int, c_int, c_int, P, c_int, c_longlong, c_int, c_int, P, c_int, c_longlong, P, P, P, c_longlong,
            P, P, c_int, P, P, c_int, c_int, c_int, c_int, c_int, P])
    check(f(ptr(x), C, int(q_col), int(k_col), int(v_col), ptr(u), uS, N * u.shape[2], u.shape[2], int(beta_col), ptr(a),
            aS, N * heads * d, ptr(dt_bias), ptr(a_log), ptr(state), state.stride(0), ptr(cu_q), ptr(seq_slot),
            int(n_seqs), ptr(y), ptr(prep), N, int(heads), int(kv_heads), int(d), int(dv), stream_ptr()), "delta_rule")
    return y


def gemm_f32(a, w, out=None):
    """C = a @ w.T in true float32 (FFMA). a float32 [M, K]; w [N, K] float32|bfloat16."""
    require(a, F32, "gemm_f32.a")
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm_f32: inner sizes differ ({K} vs {K2})")
    if not (w.is_cuda and w.is_contiguous()):
        raise KernelError("gemm_f32.w must be a contiguous CUDA tensor")
    if out is None:
        out = torch.empty((M, N), dtype=F32, device=a.device)
    f = fn("gemm_f32", "lumen_gemm_f32", [P, P, c_int, P, c_int, c_int, c_int, P])
    check(f(ptr(a), ptr(w), _is_bf16(w), ptr(out), M, N, K, stream_ptr()), "gemm_f32")
    return out


class TiledWeight:
    """A bfloat16 weight [rows, cols] in the form the tensor-core products read: the image its
    tiles have in shared memory, k block after k block, rows padded to `padded_rows` (see the
    head of csrc/gemm_tc.cu). `first_rows(n)` is the weight's first n rows on the same memory."""
    __slots__ = ("data", "rows", "cols", "padded_rows")

    def __init__(self, data, rows, cols, padded_rows):
        self.data, self.rows, self.cols, self.padded_rows = data, int(rows), int(cols), int(padded_rows)

    @property
    def shape(self):
        return (self.rows, self.cols)

    @property
    def dtype(self):
        return self.data.dtype

    @property
    def device(self):
        return self.data.device

    def data_ptr(self):
        return self.data.data_ptr()

    def first_rows(self, n: int) -> "TiledWeight":
        if not 0 < n <= self.rows:
            raise KernelError(f"a tiled weight of {self.rows} rows has no first {n} rows")
        return TiledWeight(self.data, n, self.cols, self.padded_rows)

    def row_major(self) -> torch.Tensor:
        """The weight as an ordinary [rows, cols] tensor again (a copy; tests and debugging)."""
        kb = (self.cols + 63) // 64
        t = self.data.view(kb, self.padded_rows, 8, 8)                 # [k block, row, piece, 8 values]
        r = torch.arange(self.padded_rows, device=t.device) % 8
        j = torch.arange(8, device=t.device)
        src = (j[None, :] ^ r[:, None])                                # piece c of row r sits at place c ^ (r & 7)
        t = torch.gather(t, 2, src[None, :, :, None].expand(kb, -1, -1, 8))
        return t.permute(1, 0, 2, 3).reshape(self.padded_rows, kb * 64)[: self.rows, : self.cols].contiguous()


def can_tile(w) -> bool:
    return (isinstance(w, torch.Tensor) and w.dtype == BF16 and w.is_cuda and w.dim() == 2
            and w.shape[1] % 8 == 0 and w.shape[0] > 0)


def tile_weight(w) -> TiledWeight:
    """The tiled form of a bfloat16 weight [N, K], K a multiple of 8."""
    require(w, BF16, "tile_weight.w")
    if not can_tile(w):
        raise KernelError(f"tile_weight takes bfloat16 [N, K] with K a multiple of 8, not {tuple(w.shape)}")
    N, K = w.shape
    padded = int(int_fn("gemm_tc", "lumen_tiled_weight_rows", [c_int])(int(N)))
    out = torch.empty(((K + 63) // 64) * padded * 64, dtype=BF16, device=w.device)
    f = fn("gemm_tc", "lumen_tile_weight", [P, P, c_int, c_int, P])
    check(f(ptr(w), ptr(out), N, K, stream_ptr()), "tile_weight")
    return TiledWeight(out, N, K, padded)


def gemm_tc_splits(M, N, K, silu=False) -> int:
    return int(int_fn("gemm_tc", "lumen_gemm_tc_splits", [c_int, c_int, c_int, c_int])(
        int(M), int(N), int(K), 1 if silu else 0))


def gemm_tc_adds(M, N) -> bool:
    """Whether gemm_tc can add a product of this shape to a float32 matrix in place."""
    return bool(int_fn("gemm_tc", "lumen_gemm_tc_adds", [c_int, c_int])(int(M), int(N)))


def gemm_tc(x, w, silu_interleaved=False, add_to=None):
    """x @ w.T on the tcgen05 tensor cores. x bfloat16 [M, K], w a TiledWeight [N, K], K a
    multiple of 8. Returns float32 partials [S, M, N] (S = 1 unless M <= 256); or, with
    silu_interleaved (rows of w alternate gate_i, up_i), bfloat16 [M, N/2] = silu(gate)*up;
    or, with add_to (float32 [M, N], only where gemm_tc_adds(M, N)), adds the product to it
    in place (one float32 add an element, by the copy engine) and returns None."""
    require(x, BF16, "gemm_tc.x")
    if not isinstance(w, TiledWeight):
        raise KernelError("gemm_tc takes its weight in tiled form (tile_weight)")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2 or K % 8:
        raise KernelError(f"gemm_tc: inner sizes {K} and {K2} must agree and be a multiple of 8")
    epi = 0
    if add_to is not None:
        require(add_to, F32, "gemm_tc.add_to")
        if silu_interleaved or tuple(add_to.shape) != (M, N) or not gemm_tc_adds(M, N):
            raise KernelError(f"gemm_tc: a product [{M}, {N}] cannot be added in place")
        out, epi = add_to, 2
    elif silu_interleaved:
        if N % 2:
            raise KernelError("gemm_tc: gate/up rows must come in pairs")
        out, epi = torch.empty((M, N // 2), dtype=BF16, device=x.device), 1
    else:
        out = torch.empty((gemm_tc_splits(M, N, K), M, N), dtype=F32, device=x.device)
    f = fn("gemm_tc", "lumen_gemm_tc", [P, P, P, c_int, c_int, c_int, c_int, c_int, P, P])
    check(f(ptr(x), ptr(w.data), ptr(out), M, N, K, w.padded_rows, epi, ptr(error_flag(x.device)), stream_ptr()),
          "gemm_tc")
    return None if add_to is not None else out


def argmax(logits, out=None):
    """Row-wise argmax of float32 [B, V]; equal maxima give the lowest index."""
    require(logits, F32, "argmax.logits", contiguous=False)
    B, V = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("argmax: rows must be contiguous")
    if out is None:
        out = torch.empty((B,), dtype=I32, device=logits.device)
    scratch = torch.empty((2 * 64 * B,), dtype=I32, device=logits.device) if V >= 16384 else None
    f = fn("sample", "lumen_argmax", [P, c_longlong, c_int, c_int, P, P, P])
    check(f(ptr(logits), logits.stride(0), B, V, ptr(out), ptr(scratch), stream_ptr()), "argmax")
    return out


def sample(logits, opts, top_k, out=None):
    """Row-wise sampling. opts float32 [B, 4] = (temperature, top_p, min_p, u); top_k int32 [B]."""
    require(logits, F32, "sample.logits", contiguous=False)
    require(opts, F32, "sample.opts")
    require(top_k, I32, "sample.top_k")
    B, V = logits.shape
    if logits.stride(1) != 1 or opts.shape != (B, 4) or top_k.numel() != B:
        raise KernelError("sample: bad shapes")
    if out is None:
        out = torch.empty((B,), dtype=I32, device=logits.device)
    f = fn("sample", "lumen_sample", [P, c_longlong, c_int, c_int, P, P, P, P])
    check(f(ptr(logits), logits.stride(0), B, V, ptr(opts), ptr(top_k), ptr(out), stream_ptr()),
          "sample")
    return out


_err_flags = {}


def error_flag(device) -> torch.Tensor:
    """A device int that kernels with bounded waits set when a wait ran out."""
    key = torch.device(device).index
    t = _err_flags.get(key)
    if t is None:
        t = _err_flags[key] = torch.zeros((1,), dtype=I32, device=device)
    return t


def check_error_flags() -> None:
    """Raises if any kernel gave up on a wait since the last check (synchronises)."""
    for dev, t in _err_flags.items():
        if int(t.item()) != 0:
            recover(dev)
            raise KernelError(f"a kernel on cuda:{dev} gave up waiting for its own copies")


def recover(device) -> None:
    """After a kernel gave up: the flag back to zero, and the counters that the decode
    attention's blocks leave at zero only when all of them arrive."""
    key = torch.device("cuda", device).index if isinstance(device, int) else torch.device(device).index
    for table in (_err_flags, _counters):
        t = table.get(key)
        if t is not None:
            t.zero_()


_COUNTERS = 1 << 16
_counters = {}


def _decode_counters(device) -> torch.Tensor:
    """Zeroed ints that the decode-attention blocks count themselves in with; every call
    leaves them zero again, and calls on a device run in stream order."""
    key = torch.device(device).index
    t = _counters.get(key)
    if t is None:
        t = _counters[key] = torch.zeros((_COUNTERS,), dtype=I32, device=device)
    return t


DECODE_MAX_SEGS = 32
# Pages a decode-attention block walks (unless the sequence is longer than 32 segments of them).
# One number for every batch: how a sequence's keys are cut, and so the order in which its
# partial results are merged, depends on the sequence alone, never on who else is in the batch
# or on the page table's width.
DECODE_SEG_PAGES = 4


def _gate_args(gate, rows, what):
    """(tensor, splits, split stride, width) of a gate that arrives as float32 partial sums [N, W] or
    [S, N, W]; zeros without one."""
    if gate is None:
        return None, 0, 0, 0
    gate, gS = _partials(gate, what)
    if gate.shape[1] != rows:
        raise KernelError(f"{what}: the gate has one row a token")
    return gate, gS, gate.shape[1] * gate.shape[2], gate.shape[2]


def attn_decode(q, kcache, vcache, block_table, seq_pos, window, scale, chunk=0, softcap=0.0, sink=False,
                gate=None, gate_col=0):
    """Split-KV decode attention, bfloat16, swizzled cache, head size 64 or 128, at most
    16 query heads per kv head. q [B, nq, d]; seq_pos int32 [B]: each query's position.
    `chunk`, `softcap`, `sink`, `gate` and `gate_col` as in attn_generic_opt."""
    B, nq, d = q.shape
    nkv = kcache.shape[1]
    require(q, BF16, "attn_decode.q")
    require(kcache, BF16, "attn_decode.kcache")
    require(vcache, BF16, "attn_decode.vcache")
    require(block_table, I32, "attn_decode.block_table")
    require(seq_pos, I32, "attn_decode.seq_pos")
    if seq_pos.numel() < B or block_table.shape[0] < B:
        raise KernelError("attn_decode: metadata shorter than the batch")
    width = block_table.shape[1]
    seg_pages = DECODE_SEG_PAGES
    max_segs = min(-(-width // seg_pages), DECODE_MAX_SEGS)
    out = torch.empty_like(q)
    part_o = torch.empty((B, nq, max_segs, d), dtype=F32, device=q.device)
    part_ml = torch.empty((B, nq, max_segs, 2), dtype=F32, device=q.device)
    counters = _decode_counters(q.device) if B * nkv <= _COUNTERS else None
    if chunk or softcap or sink or gate is not None:
        gate, gS, gstride, gW = _gate_args(gate, B, "attn_decode.gate")
        f = fn("attn_decode", "lumen_attn_decode_opt",
               [P, P, P, P, c_int, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_float,
                c_int, P, c_int, c_longlong, c_int, c_int, P, P, P])
        check(f(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), block_table.stride(0), ptr(seq_pos),
                ptr(out), ptr(part_o), ptr(part_ml), B, nq, nkv, d, int(window), float(scale), max_segs, seg_pages,
                int(chunk), float(softcap or 0.0), 1 if sink else 0, ptr(gate), gS, gstride, gW, int(gate_col),
                ptr(error_flag(q.device)), ptr(counters), stream_ptr()), "attn_decode_opt")
        return out
    f = fn("attn_decode", "lumen_attn_decode",
           [P, P, P, P, c_int, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, P, P, P])
    check(f(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), block_table.stride(0), ptr(seq_pos),
            ptr(out), ptr(part_o), ptr(part_ml), B, nq, nkv, d, int(window), float(scale), max_segs,
            seg_pages,
            ptr(error_flag(q.device)), ptr(counters), stream_ptr()), "attn_decode")
    return out


def attn_decode_qkv(qkv, q_norm_w, k_norm_w, eps, cs, rotary_dim, kcache, vcache, block_table, seq_pos,
                    window, scale, nq, nkv, store_kv=True):
    """Decode attention that does the rotary kernel's work itself: qkv is the projection as
    the product left it, float32 [B, (nq + 2 nkv) * 128] or [S, B, ...] partial sums; every
    block makes its query heads (sum of the parts, head norm with q_norm_w / k_norm_w [128] or
    None, rotation over the whole head when rotary_dim == 128, by cs [B, 64, 2]), and with
    store_kv the new token's key and value are made and written to the cache. The same bits as
    qk_norm_rope_store followed by attn_decode. Head size 128, swizzled bfloat16 cache."""
    qkv, S = _partials(qkv, "attn_decode_qkv.qkv")
    B = qkv.shape[1]
    d = 128
    if qkv.shape[2] != (nq + 2 * nkv) * d or kcache.shape[1:] != (nkv, PAGE, d) or rotary_dim not in (0, d):
        raise KernelError(f"attn_decode_qkv: projection {tuple(qkv.shape)} and cache {tuple(kcache.shape)} do not "
                          f"fit {nq}+2x{nkv} heads of {d} (rotation over {rotary_dim})")
    require(kcache, BF16, "attn_decode_qkv.kcache")
    require(vcache, BF16, "attn_decode_qkv.vcache")
    require(block_table, I32, "attn_decode_qkv.block_table")
    require(seq_pos, I32, "attn_decode_qkv.seq_pos")
    for t, nm in ((q_norm_w, "q_norm"), (k_norm_w, "k_norm")):
        if t is not None:
            require(t, F32, nm)
            if t.numel() != d:
                raise KernelError(f"{nm} weight must have {d} values")
    if rotary_dim:
        require(cs, F32, "rope angles")
        if cs.numel() < B * 64 * 2:
            raise KernelError("rope angles shorter than the batch")
    if seq_pos.numel() < B or block_table.shape[0] < B:
        raise KernelError("attn_decode_qkv: metadata shorter than the batch")
    width = block_table.shape[1]
    seg_pages = DECODE_SEG_PAGES
    max_segs = min(-(-width // seg_pages), DECODE_MAX_SEGS)
    out = torch.empty((B, nq, d), dtype=BF16, device=qkv.device)
    part_o = torch.empty((B, nq, max_segs, d), dtype=F32, device=qkv.device)
    part_ml = torch.empty((B, nq, max_segs, 2), dtype=F32, device=qkv.device)
    counters = _decode_counters(qkv.device) if B * nkv <= _COUNTERS else None
    f = fn("attn_decode", "lumen_attn_decode_qkv",
           [P, c_int, c_longlong, P, P, c_float, P, c_int, c_int, P, P, P, c_int, P, P, P, P, c_int, c_int, c_int,
            c_int, c_int, c_float, c_int, c_int, P, P, P])
    check(f(ptr(qkv), S, qkv.stride(0) if S > 1 else 0, ptr(q_norm_w), ptr(k_norm_w), float(eps), ptr(cs),
            1 if rotary_dim else 0, 1 if store_kv else 0, ptr(kcache), ptr(vcache), ptr(block_table),
            block_table.stride(0), ptr(seq_pos), ptr(out), ptr(part_o), ptr(part_ml), B, nq, nkv, d, int(window),
            float(scale), max_segs, seg_pages, ptr(error_flag(qkv.device)), ptr(counters), stream_ptr()),
          "attn_decode_qkv")
    return out


def attn_prefill(q, kcache, vcache, block_table, cu_q, seq_start, q_lens, window, scale,
                 tensor_memory=True, n_seqs=None, chunk=0, softcap=0.0, sink=False, gate=None, gate_col=0):
    """Causal flash attention for sequences that bring q_lens[b] tokens each (host list),
    bfloat16, swizzled cache, head size 64 or 128, at most 16 query heads per kv head.
    q [N, nq, d]; cu_q int32 [B+1]; seq_start int32 [B]. With tensor_memory the tcgen05
    kernel (128 rows a block, S and O in tensor memory), else the mma.sync kernel (64 rows).
    With q_lens None and n_seqs = B the host need not know how the N tokens are divided (a
    captured step does not): enough blocks are launched for any division, every block finds
    its sequence and tile from cu_q on the device, and the blocks left over return at once.
    `chunk`, `softcap`, `sink`, `gate` and `gate_col` as in attn_generic_opt (tensor-memory kernel
    only)."""
    N, nq, d = q.shape
    nkv = kcache.shape[1]
    B = len(q_lens) if q_lens is not None else int(n_seqs)
    require(q, BF16, "attn_prefill.q")
    require(kcache, BF16, "attn_prefill.kcache")
    require(vcache, BF16, "attn_prefill.vcache")
    require(block_table, I32, "attn_prefill.block_table")
    require(cu_q, I32, "attn_prefill.cu_q")
    require(seq_start, I32, "attn_prefill.seq_start")
    if nq % nkv or nq // nkv > 16:
        raise KernelError("attn_prefill: at most 16 query heads per kv head")
    if cu_q.numel() < B + 1 or seq_start.numel() < B or block_table.shape[0] < B or \
            (q_lens is not None and sum(q_lens) != N):
        raise KernelError("attn_prefill: metadata does not match the batch")
    tq = (128 if tensor_memory else 64) // (nq // nkv)
    # sum of ceil(q_b / tq) over any division of N tokens into B sequences is at most N // tq + B
    n_tiles = sum((n + tq - 1) // tq for n in q_lens) if q_lens is not None else N // tq + B
    out = torch.empty_like(q)
    if chunk or softcap or sink or gate is not None:
        if not tensor_memory:
            raise KernelError("attn_prefill: the options are the tensor-memory kernel's")
        gate, gS, gstride, gW = _gate_args(gate, N, "attn_prefill.gate")
        f = fn("attn_prefill_tc", "lumen_attn_prefill_tc_opt",
               [P, P, P, P, c_int, P, P, c_int, c_int, P, c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_int,
                P, c_int, c_longlong, c_int, c_int, P, P])
        check(f(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), block_table.stride(0), ptr(cu_q),
                ptr(seq_start), B, n_tiles, ptr(out), nq, nkv, d, int(window), float(scale), int(chunk),
                float(softcap or 0.0), 1 if sink else 0, ptr(gate), gS, gstride, gW, int(gate_col),
                ptr(error_flag(q.device)), stream_ptr()), "attn_prefill_opt")
        return out
    f = fn("attn_prefill_tc" if tensor_memory else "attn_prefill",
           "lumen_attn_prefill_tc" if tensor_memory else "lumen_attn_prefill",
           [P, P, P, P, c_int, P, P, c_int, c_int, P, c_int, c_int, c_int, c_int, c_float, P, P])
    check(f(ptr(q), ptr(kcache), ptr(vcache), ptr(block_table), block_table.stride(0), ptr(cu_q),
            ptr(seq_start), B, n_tiles, ptr(out), nq, nkv, d, int(window), float(scale),
            ptr(error_flag(q.device)), stream_ptr()), "attn_prefill")
    return out

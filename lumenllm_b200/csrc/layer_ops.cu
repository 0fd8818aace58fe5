// Row kernels of layers that are arranged otherwise than the plain pre-norm decoder:
//   - token embedding times a scale plus a learned position vector,
//   - an update that is RMS-normed BEFORE it joins the residual stream, fused with the norm
//     of the next sublayer (post-norm + add + pre-norm in one pass over the row),
//   - a short causal convolution over time on each channel of a sublayer's input, with the
//     last inputs of every sequence kept as state,
//   - PolyNorm, an activation made of three unit-RMS powers,
//   - bias + one RMS norm over the WHOLE query (and key) projection + cache write.
// All arithmetic is float32; T / TOut is float (32-bit path) or __nv_bfloat16. Inputs that come
// from a split matrix product arrive as S partial results [S, rows, width] and are added in
// rising order of S while they are read.
#include "common.cuh"

__device__ __forceinline__ float ld_f32(const float* p) { return *p; }
__device__ __forceinline__ float ld_f32(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// V consecutive values at a time: 4 where a row's width is a multiple of 4 (16-byte moves), else 1.
template <int V> struct Vals { float v[V]; };
template <int V> __device__ __forceinline__ Vals<V> ldv(const float* p) {
    Vals<V> r;
    if (V == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        r.v[0] = t.x; r.v[1 % V] = t.y; r.v[2 % V] = t.z; r.v[3 % V] = t.w;
    } else {
        r.v[0] = *p;
    }
    return r;
}
template <int V> __device__ __forceinline__ void stv(float* p, const Vals<V>& x) {
    if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(x.v[0], x.v[1 % V], x.v[2 % V], x.v[3 % V]);
    else *p = x.v[0];
}
template <int V> __device__ __forceinline__ void stv(__nv_bfloat16* p, const Vals<V>& x) {
    if (V == 4) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(x.v[0], x.v[1 % V]), hi = __floats2bfloat162_rn(x.v[2 % V], x.v[3 % V]);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo);
        u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = u;
    } else {
        *p = __float2bfloat16_rn(x.v[0]);
    }
}

// ---------------------------------------------------------------- embedding + position
// h[t, :] = float(E[token[t], :]) * scale + float(P[pos[t], :]). A token or a position outside
// its table contributes zeros (the host has refused it before; this is the second guard).
template <typename TW, typename TP>
__global__ void embed_pos_kernel(const int* __restrict__ tokens, const TW* __restrict__ table, float scale,
                                 const int* __restrict__ positions, const TP* __restrict__ pos_table, int P,
                                 float* __restrict__ h, int H, int V) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < V;
    const TW* row = table + (size_t)(ok ? tok : 0) * H;
    const int pos = pos_table ? positions[t] : -1;
    const bool pok = pos >= 0 && pos < P;
    const TP* prow = pos_table + (size_t)(pok ? pos : 0) * H;
    float* out = h + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = ok ? __fmul_rn(ld_f32(row + i), scale) : 0.0f;
        if (pok) v = __fadd_rn(v, ld_f32(prow + i));
        out[i] = v;
    }
}

// The same from a token table kept in the tiled form of the tensor-core products (piece c, 8
// values, of row r lies in k block c / 8 at row kb * w_rows + r, place (c & 7) ^ (r & 7)).
template <typename TP>
__global__ void embed_pos_tiled_kernel(const int* __restrict__ tokens, const uint4* __restrict__ table, float scale,
                                       const int* __restrict__ positions, const TP* __restrict__ pos_table, int P,
                                       float* __restrict__ h, int H, int V, int w_rows) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < V;
    const int pos = pos_table ? positions[t] : -1;
    const bool pok = pos >= 0 && pos < P;
    const TP* prow = pos_table + (size_t)(pok ? pos : 0) * H;
    float* out = h + (size_t)t * H;
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = 0.0f;
        if (ok) {
            const uint4 raw = table[((size_t)(c >> 3) * w_rows + tok) * 8 + ((c & 7) ^ (tok & 7))];
            const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __fmul_rn(__bfloat162float(b[k]), scale);
        }
        if (pok) {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __fadd_rn(v[k], ld_f32(prow + 8 * c + k));
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) out[8 * c + k] = v[k];
    }
}

LUMEN_API int lumen_embed_pos(const int* tokens, const void* table, int table_is_bf16, int tiled_rows, float scale,
                              const int* positions, const void* pos_table, int pos_is_bf16, int P, float* h,
                              int N, int H, int V, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || V <= 0 || (pos_table && (!positions || P <= 0))) return LUMEN_ERR_BAD_ARGUMENT;
    if (tiled_rows > 0) {
        if ((H & 7) || tiled_rows < V || (tiled_rows & 7) || ((uintptr_t)table & 15)) return LUMEN_ERR_BAD_ARGUMENT;
        if (pos_is_bf16)
            lumen_launch(embed_pos_tiled_kernel<__nv_bfloat16>, dim3(N), dim3(128), 0, stream, tokens, (const uint4*)table,
                         scale, positions, (const __nv_bfloat16*)pos_table, P, h, H, V, tiled_rows);
        else
            lumen_launch(embed_pos_tiled_kernel<float>, dim3(N), dim3(128), 0, stream, tokens, (const uint4*)table, scale,
                         positions, (const float*)pos_table, P, h, H, V, tiled_rows);
    } else if (table_is_bf16 && pos_is_bf16) {
        lumen_launch(embed_pos_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(N), dim3(256), 0, stream, tokens,
                     (const __nv_bfloat16*)table, scale, positions, (const __nv_bfloat16*)pos_table, P, h, H, V);
    } else if (table_is_bf16) {
        lumen_launch(embed_pos_kernel<__nv_bfloat16, float>, dim3(N), dim3(256), 0, stream, tokens,
                     (const __nv_bfloat16*)table, scale, positions, (const float*)pos_table, P, h, H, V);
    } else if (pos_is_bf16) {
        lumen_launch(embed_pos_kernel<float, __nv_bfloat16>, dim3(N), dim3(256), 0, stream, tokens, (const float*)table,
                     scale, positions, (const __nv_bfloat16*)pos_table, P, h, H, V);
    } else {
        lumen_launch(embed_pos_kernel<float, float>, dim3(N), dim3(256), 0, stream, tokens, (const float*)table, scale,
                     positions, (const float*)pos_table, P, h, H, V);
    }
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- post-norm + add + norm
// u = delta[0][r] + ... + delta[S-1][r] (+ bias);  x = h[r] + u / sqrt(mean(u^2) + eps_u) * wu;
// if write_h, h[r] = x;  if wn, y[b] = x / sqrt(mean(x^2) + eps_n) * wn.
// With `rows`, block b reads row rows[b] and writes y row b; without, row b.
// With `cw` (a step in which row b is the ONE new token of sequence b): what goes out is the
// convolution of the sublayer's input, y + sum_j cw[j] * (the sequence's last inputs, then y),
// and the sequence's state (row seq_slot[b] of `state`) moves on by y; see canon_conv_kernel.
#define CANON_MAX_TAPS 16
template <typename TOut, int V>
__global__ void __launch_bounds__(1024)
postnorm_add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int S, size_t delta_stride,
                            const float* __restrict__ bias, const float* __restrict__ wu, float eps_u,
                            const float* __restrict__ wn, float eps_n, TOut* __restrict__ y,
                            const int* __restrict__ rows, int H, int write_h, const float* __restrict__ cw, int taps,
                            float* __restrict__ state, size_t slot_stride, const int* __restrict__ seq_slot) {
    extern __shared__ __align__(16) float xs[];  // H floats
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    const int r = rows ? rows[b] : b;
    float* hr = h + (size_t)r * H;
    // Few rows (wide blocks, one group of V values a thread): the stream's values and the norms'
    // weights are asked for at once with the update's, not one round trip after the other.
    const bool one = (int)blockDim.x * V >= H;
    const int i1 = threadIdx.x * V;
    Vals<V> h1, gu1, gn1;
#pragma unroll
    for (int k = 0; k < V; ++k) h1.v[k] = gu1.v[k] = gn1.v[k] = 0.0f;
    if (one && i1 < H) {
        h1 = ldv<V>(hr + i1);
        if (delta) gu1 = ldv<V>(wu + i1);
        if (wn) gn1 = ldv<V>(wn + i1);
    }
    float ss = 0.0f;
    if (delta) {
        const float* dr = delta + (size_t)r * H;
        for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
            Vals<V> u = ldv<V>(dr + i);
            for (int s = 1; s < S; ++s) {
                const Vals<V> d = ldv<V>(dr + (size_t)s * delta_stride + i);
#pragma unroll
                for (int k = 0; k < V; ++k) u.v[k] += d.v[k];
            }
            if (bias) {
                const Vals<V> d = ldv<V>(bias + i);
#pragma unroll
                for (int k = 0; k < V; ++k) u.v[k] += d.v[k];
            }
            stv<V>(xs + i, u);
#pragma unroll
            for (int k = 0; k < V; ++k) ss += u.v[k] * u.v[k];
        }
        ss = block_sum(ss, red);
    }
    const float su = 1.0f / sqrtf(ss / (float)H + eps_u);
    float ss2 = 0.0f;
    for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
        Vals<V> x = one ? h1 : ldv<V>(hr + i);
        if (delta) {
            const Vals<V> u = ldv<V>(xs + i), g = one ? gu1 : ldv<V>(wu + i);
#pragma unroll
            for (int k = 0; k < V; ++k) x.v[k] += u.v[k] * su * g.v[k];
            if (write_h) stv<V>(hr + i, x);
        }
        stv<V>(xs + i, x);
#pragma unroll
        for (int k = 0; k < V; ++k) ss2 += x.v[k] * x.v[k];
    }
    if (wn == nullptr) return;
    ss2 = block_sum(ss2, red);
    const float sn = 1.0f / sqrtf(ss2 / (float)H + eps_n);
    TOut* yr = y + (size_t)b * H;
    float* st = cw && taps > 1 ? state + (size_t)seq_slot[b] * slot_stride : nullptr;
    const int back = taps - 1;
    for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
        const Vals<V> x = ldv<V>(xs + i), g = one ? gn1 : ldv<V>(wn + i);
        Vals<V> o;
#pragma unroll
        for (int k = 0; k < V; ++k) o.v[k] = x.v[k] * sn * g.v[k];
        if (cw) {
            const Vals<V> cur = o;
            for (int j = 0; j < back; ++j) {
                const Vals<V> w = ldv<V>(cw + (size_t)j * H + i), old = ldv<V>(st + (size_t)j * H + i);
#pragma unroll
                for (int k = 0; k < V; ++k) o.v[k] += w.v[k] * old.v[k];
                if (j > 0) stv<V>(st + (size_t)(j - 1) * H + i, old);       // the state moves on by one
            }
            const Vals<V> w = ldv<V>(cw + (size_t)back * H + i);
#pragma unroll
            for (int k = 0; k < V; ++k) o.v[k] += w.v[k] * cur.v[k];
            if (back > 0) stv<V>(st + (size_t)(back - 1) * H + i, cur);
        }
        stv<V>(yr + i, o);
    }
}

static int row_threads(int width, int n_rows) {
    int t = 256;
    if (n_rows < 2 * 148) {                      // few rows: wide blocks, all loads of a row in flight
        t = ((width + 31) / 32) * 32;
        if (t > 1024) t = 1024;
        if (t < 128) t = 128;
    }
    return t;
}

template <typename TOut>
static void postnorm_launch(int n_rows, int threads, size_t smem, cudaStream_t stream, float* h, const float* delta,
                            int S, size_t dstride, const float* bias, const float* wu, float eps_u, const float* wn,
                            float eps_n, TOut* y, const int* rows, int H, int write_h, const float* cw, int taps,
                            float* state, size_t slot_stride, const int* seq_slot) {
    if ((H & 3) == 0) {
        auto k = postnorm_add_rmsnorm_kernel<TOut, 4>;
        if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(n_rows), dim3(threads), smem, stream, h, delta, S, dstride, bias, wu, eps_u, wn, eps_n, y,
                     rows, H, write_h, cw, taps, state, slot_stride, seq_slot);
    } else {
        auto k = postnorm_add_rmsnorm_kernel<TOut, 1>;
        if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(n_rows), dim3(threads), smem, stream, h, delta, S, dstride, bias, wu, eps_u, wn, eps_n, y,
                     rows, H, write_h, cw, taps, state, slot_stride, seq_slot);
    }
}

// delta may be null (nothing pending: x = h). cw [taps][H] with its state folds the input
// convolution of a step of single tokens in (row b = sequence b; not with `rows`).
LUMEN_API int lumen_postnorm_add_rmsnorm(float* h, const float* delta, int n_delta, long long delta_stride,
                                         const float* bias, const float* wu, float eps_u, const float* wn,
                                         float eps_n, void* y, int y_is_bf16, const int* rows, int n_rows, int H,
                                         int write_h, const float* cw, int taps, float* state, long long slot_stride,
                                         const int* seq_slot, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || (delta && (n_delta < 1 || !wu)) || (wn && !y)) return LUMEN_ERR_BAD_ARGUMENT;
    if (cw && (rows || !wn || taps < 1 || taps > CANON_MAX_TAPS || (taps > 1 && (!state || !seq_slot))))
        return LUMEN_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return LUMEN_ERR_UNSUPPORTED;
    const int threads = row_threads((H & 3) == 0 ? H / 4 : H, n_rows);
    if (y_is_bf16)
        postnorm_launch<__nv_bfloat16>(n_rows, threads, smem, stream, h, delta, n_delta, (size_t)delta_stride, bias, wu,
                                       eps_u, wn, eps_n, (__nv_bfloat16*)y, rows, H, write_h, cw, taps, state,
                                       (size_t)slot_stride, seq_slot);
    else
        postnorm_launch<float>(n_rows, threads, smem, stream, h, delta, n_delta, (size_t)delta_stride, bias, wu, eps_u,
                               wn, eps_n, (float*)y, rows, H, write_h, cw, taps, state, (size_t)slot_stride, seq_slot);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- causal convolution of a sublayer's input
// out[t] = y[t] + sum_{j < taps} w[j] * y[t - taps + 1 + j] on every channel, over the tokens of
// ONE sequence; what lies before the step's first token comes from the sequence's state (its
// last taps - 1 inputs, zeros for a new sequence), and the state is moved on to the step's end.
// w is stored [taps][H]. The first blocks take one token each (eight in steps of many tokens) and
// skip tokens among the first taps - 1 of their sequence in this step; the blocks behind them take
// the sequences: a sequence's first tokens (which read the state) and the state's update, so that
// whatever touches a channel of a sequence's state is read and then written by the same thread.
#define CANON_FAST_TAPS 8        // up to this many taps the blocks of prompt steps take several tokens each
#define CANON_GROUP 8
template <typename TOut, int V>
__global__ void canon_conv_kernel(const float* __restrict__ y, const float* __restrict__ w, int taps,
                                  float* __restrict__ state, size_t slot_stride, const int* __restrict__ tok_seq,
                                  const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int N, int B,
                                  TOut* __restrict__ out, int H, int group, int token_blocks) {
    pdl_trigger();
    pdl_wait();
    const int blk = blockIdx.x;
    const int back = taps - 1;
    if (group > 1 && blk < token_blocks) {
        // `group` consecutive tokens a block (the host launches N / group of these blocks and
        // numbers the sequence blocks behind them): a thread walks down its channels with the last
        // inputs in registers, so a row is read once and not once for every tap.
        const int first = blk * CANON_GROUP;
        if (first >= N) return;
        unsigned takes = 0;               // which of the block's tokens are not among their sequence's first
#pragma unroll
        for (int t = 0; t < CANON_GROUP; ++t)
            if (first + t < N && first + t - cu_q[tok_seq[first + t]] >= back) takes |= 1u << t;
        for (int c = threadIdx.x * V; c < H; c += blockDim.x * V) {
            Vals<V> win[CANON_FAST_TAPS - 1], wv[CANON_FAST_TAPS], cur[CANON_GROUP];
            // every row the block needs is asked for before the first one is used
#pragma unroll
            for (int t = 0; t < CANON_GROUP; ++t)
                if (first + t < N) cur[t] = ldv<V>(y + (size_t)(first + t) * H + c);
#pragma unroll
            for (int j = 0; j < CANON_FAST_TAPS - 1; ++j)
                if (j < back) {
                    if (first - back + j >= 0) win[j] = ldv<V>(y + (size_t)(first - back + j) * H + c);
                    else
#pragma unroll
                        for (int k = 0; k < V; ++k) win[j].v[k] = 0.0f;    // before the step: only tokens that the sequence blocks take read it
                }
#pragma unroll
            for (int j = 0; j < CANON_FAST_TAPS; ++j)
                if (j < taps) wv[j] = ldv<V>(w + (size_t)j * H + c);
#pragma unroll
            for (int t = 0; t < CANON_GROUP; ++t) {
                if (first + t >= N) break;
                if (takes >> t & 1u) {
                    Vals<V> acc = cur[t];
#pragma unroll
                    for (int j = 0; j < CANON_FAST_TAPS - 1; ++j)
                        if (j < back) {
#pragma unroll
                            for (int k = 0; k < V; ++k) acc.v[k] += wv[j].v[k] * win[j].v[k];
                        }
#pragma unroll
                    for (int j = 0; j < CANON_FAST_TAPS; ++j)
                        if (j == back) {
#pragma unroll
                            for (int k = 0; k < V; ++k) acc.v[k] += wv[j].v[k] * cur[t].v[k];
                        }
                    stv<V>(out + (size_t)(first + t) * H + c, acc);
                }
#pragma unroll
                for (int j = 0; j < CANON_FAST_TAPS - 2; ++j) win[j] = win[j + 1];
#pragma unroll
                for (int j = 0; j < CANON_FAST_TAPS - 1; ++j)
                    if (j == back - 1) win[j] = cur[t];
            }
        }
        return;
    }
    if (group <= 1 && blk < N) {
        const int n = blk;
        const int i = n - cu_q[tok_seq[n]];
        if (i < back) return;
        for (int c = threadIdx.x * V; c < H; c += blockDim.x * V) {
            Vals<V> acc = ldv<V>(y + (size_t)n * H + c);
            for (int j = 0; j < taps; ++j) {
                const Vals<V> a = ldv<V>(w + (size_t)j * H + c), b = ldv<V>(y + (size_t)(n - back + j) * H + c);
#pragma unroll
                for (int k = 0; k < V; ++k) acc.v[k] += a.v[k] * b.v[k];
            }
            stv<V>(out + (size_t)n * H + c, acc);
        }
        return;
    }
    // a sequence's channels are spread over as many blocks as give every thread one channel:
    // a thread's walk is a chain of loads, and one block a sequence would be the step's last to end
    const int cpb = (H + (int)blockDim.x - 1) / (int)blockDim.x;
    const int hb = blk - (group > 1 ? token_blocks : N);
    const int b = hb / cpb;
    const int n0 = cu_q[b], q = cu_q[b + 1] - n0;
    if (q <= 0 || back == 0) return;
    float* st = state + (size_t)seq_slot[b] * slot_stride;
    const int m = q < back ? q : back;
    for (int c = (hb - b * cpb) * (int)blockDim.x + threadIdx.x; c < H; c += H) {
        float win[CANON_MAX_TAPS];
#pragma unroll
        for (int k = 0; k < CANON_MAX_TAPS - 1; ++k) win[k] = k < back ? st[(size_t)k * H + c] : 0.0f;
        for (int i = 0; i < m; ++i) {
            const float cur = y[(size_t)(n0 + i) * H + c];
            float acc = cur;
#pragma unroll
            for (int j = 0; j < CANON_MAX_TAPS - 1; ++j)
                if (j < back) acc += w[(size_t)j * H + c] * win[j];
            acc += w[(size_t)back * H + c] * cur;
            out[(size_t)(n0 + i) * H + c] = from_f32<TOut>(acc);
#pragma unroll
            for (int k = 0; k < CANON_MAX_TAPS - 2; ++k) win[k] = win[k + 1];
#pragma unroll
            for (int k = 0; k < CANON_MAX_TAPS - 1; ++k)
                if (k == back - 1) win[k] = cur;
        }
        if (q >= back) {
            for (int k = 0; k < back; ++k) st[(size_t)k * H + c] = y[(size_t)(n0 + q - back + k) * H + c];
        } else {
#pragma unroll
            for (int k = 0; k < CANON_MAX_TAPS - 1; ++k)
                if (k < back) st[(size_t)k * H + c] = win[k];
        }
    }
}

LUMEN_API int lumen_canon_conv(const float* y, const float* w, int taps, float* state, long long slot_stride,
                               const int* tok_seq, const int* cu_q, const int* seq_slot, int N, int B, void* out,
                               int out_is_bf16, int H, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || B <= 0 || taps < 1 || taps > CANON_MAX_TAPS || (taps > 1 && !state)) return LUMEN_ERR_UNSUPPORTED;
    const bool v4 = (H & 3) == 0;
    int threads = ((v4 ? H / 4 : H) + 31) / 32 * 32;
    threads = threads > 512 ? 512 : (threads < 64 ? 64 : threads);
    // many tokens and few taps: blocks of CANON_GROUP tokens; else a token a block
    const int group = (N >= 4 * 148 && taps <= CANON_FAST_TAPS) ? CANON_GROUP : 1;
    const int token_blocks = group > 1 ? (N + group - 1) / group : N;
    if (group > 1 && threads > 256) threads = 256;
    const dim3 grid(token_blocks + B * ((H + threads - 1) / threads));
    if (out_is_bf16 && v4)
        lumen_launch(canon_conv_kernel<__nv_bfloat16, 4>, grid, dim3(threads), 0, stream, y, w, taps, state,
                     (size_t)slot_stride, tok_seq, cu_q, seq_slot, N, B, (__nv_bfloat16*)out, H, group, token_blocks);
    else if (out_is_bf16)
        lumen_launch(canon_conv_kernel<__nv_bfloat16, 1>, grid, dim3(threads), 0, stream, y, w, taps, state,
                     (size_t)slot_stride, tok_seq, cu_q, seq_slot, N, B, (__nv_bfloat16*)out, H, group, token_blocks);
    else if (v4)
        lumen_launch(canon_conv_kernel<float, 4>, grid, dim3(threads), 0, stream, y, w, taps, state,
                     (size_t)slot_stride, tok_seq, cu_q, seq_slot, N, B, (float*)out, H, group, token_blocks);
    else
        lumen_launch(canon_conv_kernel<float, 1>, grid, dim3(threads), 0, stream, y, w, taps, state,
                     (size_t)slot_stride, tok_seq, cu_q, seq_slot, N, B, (float*)out, H, group, token_blocks);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- PolyNorm
// out = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e, powers element by element,
// rms(v) = sqrt(mean(v^2) + eps) over the row; act = (a, b, c, e) on the device.
template <typename TOut, int V>
__global__ void __launch_bounds__(1024)
polynorm_kernel(const float* __restrict__ z, int S, size_t split_stride, const float* __restrict__ act, float eps,
                TOut* __restrict__ out, int F) {
    extern __shared__ __align__(16) float xs[];  // F floats
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const size_t row = blockIdx.x;
    const float* zr = z + row * F;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (int i = threadIdx.x * V; i < F; i += blockDim.x * V) {
        Vals<V> v = ldv<V>(zr + i);
        for (int s = 1; s < S; ++s) {
            const Vals<V> d = ldv<V>(zr + (size_t)s * split_stride + i);
#pragma unroll
            for (int k = 0; k < V; ++k) v.v[k] += d.v[k];
        }
        stv<V>(xs + i, v);
#pragma unroll
        for (int k = 0; k < V; ++k) {
            const float v2 = v.v[k] * v.v[k];
            s2 += v2;
            s4 += v2 * v2;
            s6 += v2 * v2 * v2;
        }
    }
    s2 = block_sum(s2, red);
    s4 = block_sum(s4, red);
    s6 = block_sum(s6, red);
    const float r1 = 1.0f / sqrtf(s2 / (float)F + eps), r2 = 1.0f / sqrtf(s4 / (float)F + eps),
                r3 = 1.0f / sqrtf(s6 / (float)F + eps);
    const float a = act[0], b = act[1], c = act[2], e = act[3];
    TOut* orow = out + row * F;
    for (int i = threadIdx.x * V; i < F; i += blockDim.x * V) {
        const Vals<V> x = ldv<V>(xs + i);
        Vals<V> o;
#pragma unroll
        for (int k = 0; k < V; ++k) {
            const float v = x.v[k], v2 = v * v;
            o.v[k] = a * (v * r1) + b * (v2 * r2) + c * (v2 * v * r3) + e;
        }
        stv<V>(orow + i, o);
    }
}

template <typename TOut>
static void polynorm_launch(int N, int threads, size_t smem, cudaStream_t stream, const float* z, int S, size_t stride,
                            const float* act, float eps, TOut* out, int F) {
    if ((F & 3) == 0) {
        auto k = polynorm_kernel<TOut, 4>;
        if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(N), dim3(threads), smem, stream, z, S, stride, act, eps, out, F);
    } else {
        auto k = polynorm_kernel<TOut, 1>;
        if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(N), dim3(threads), smem, stream, z, S, stride, act, eps, out, F);
    }
}

LUMEN_API int lumen_polynorm(const float* z, int n_split, long long split_stride, const float* act, float eps,
                             void* out, int out_is_bf16, int N, int F, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (F <= 0 || n_split < 1 || !act) return LUMEN_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)F * sizeof(float);
    if (smem > 200 * 1024) return LUMEN_ERR_UNSUPPORTED;
    int threads = row_threads((F & 3) == 0 ? F / 4 : F, N);
    if (N >= 2 * 148 && F >= 4096) threads = 512;
    if (out_is_bf16)
        polynorm_launch<__nv_bfloat16>(N, threads, smem, stream, z, n_split, (size_t)split_stride, act, eps,
                                       (__nv_bfloat16*)out, F);
    else
        polynorm_launch<float>(N, threads, smem, stream, z, n_split, (size_t)split_stride, act, eps, (float*)out, F);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- bias + whole-projection norm + cache write
// A row of the stacked projection holds Wq query values, Wk key values and Wv value values.
// x = sum of the partials + bias; the query part is divided by its root mean square over ALL
// Wq values (all heads at once) and multiplied by qw [Wq], the key part likewise with kw [Wk]
// (a null weight leaves the part as it is). Then, optionally, every query and key head is
// rotated: with cs (cos, sin) [N, rot/2, 2], value i < rot/2 of a head is paired with value
// i + rot/2, (u, v) -> (u cos - v sin, v cos + u sin), the head's other values pass. And,
// optionally (v_unit), every value head is divided by its own root mean square over its dv
// values (eps_v inside the root, no weight). q goes out as [N, Wq], the key and the value of
// the token to its place in the paged cache: key tiles [page][kv head][PAGE][d], value tiles
// [page][kv head][PAGE][dv].
template <typename T, int V>
__global__ void __launch_bounds__(1024)
qkv_bias_norm_store_kernel(const float* __restrict__ qkv, int S, size_t split_stride, const float* __restrict__ bias,
                           const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                           const int* __restrict__ cache_pos, const int* __restrict__ tok_seq,
                           const int* __restrict__ table, int table_stride, T* __restrict__ q_out,
                           T* __restrict__ kc, T* __restrict__ vc, int Wq, int Wk, int Wv, int G, int d, int dv,
                           int k_layout, int v_layout, const float* __restrict__ cs, int rot, int v_unit, float eps_v) {
    extern __shared__ __align__(16) float xs[];  // Wq + Wk + Wv floats, then G floats, then the token's rot (cos, sin) values
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const int W = Wq + Wk + Wv;
    const float* row = qkv + (size_t)n * W;
    float* vr = xs + W;
    float* csn = vr + G;                         // the token's angles, read by every head
    for (int i = threadIdx.x; i < rot; i += blockDim.x) csn[i] = cs[(size_t)n * rot + i];
    float sq = 0.0f, sk = 0.0f;
    for (int i = threadIdx.x * V; i < W; i += blockDim.x * V) {
        Vals<V> x = ldv<V>(row + i);
        for (int s = 1; s < S; ++s) {
            const Vals<V> p = ldv<V>(row + (size_t)s * split_stride + i);
#pragma unroll
            for (int k = 0; k < V; ++k) x.v[k] += p.v[k];
        }
        if (bias) {
            const Vals<V> p = ldv<V>(bias + i);
#pragma unroll
            for (int k = 0; k < V; ++k) x.v[k] += p.v[k];
        }
        stv<V>(xs + i, x);
        float ss = 0.0f;
#pragma unroll
        for (int k = 0; k < V; ++k) ss += x.v[k] * x.v[k];
        if (i < Wq) sq += ss;                    // a group of V never straddles two parts
        else if (i < Wq + Wk) sk += ss;
    }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float rq = qw ? 1.0f / sqrtf(sq / (float)Wq + eps) : 1.0f;
    const float rk = kw ? 1.0f / sqrtf(sk / (float)Wk + eps) : 1.0f;
    const int pos = cache_pos[n];
    const int page = table[(size_t)tok_seq[n] * table_stride + pos / LUMEN_PAGE];
    const int r = pos % LUMEN_PAGE;
    if (rot > 0 || v_unit) {
        // the normed queries and keys go back to shared memory, where the rotation finds a value's
        // partner; a warp a value head sums that head's squares
        for (int i = threadIdx.x * V; i < Wq + Wk; i += blockDim.x * V) {
            Vals<V> x = ldv<V>(xs + i);
            const float* gw = i < Wq ? qw : kw;
            if (gw) {
                const Vals<V> g = ldv<V>(gw + (i < Wq ? i : i - Wq));
                const float rr = i < Wq ? rq : rk;
#pragma unroll
                for (int k = 0; k < V; ++k) x.v[k] = x.v[k] * rr * g.v[k];
            }
            stv<V>(xs + i, x);
        }
        if (v_unit) {
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
            for (int g = warp; g < G; g += nwarp) {
                float ss = 0.0f;
                for (int e = lane; e < dv; e += 32) { const float x = xs[Wq + Wk + g * dv + e]; ss += x * x; }
                ss = warp_sum(ss);
                if (lane == 0) vr[g] = 1.0f / sqrtf(ss / (float)dv + eps_v);
            }
        }
        __syncthreads();
        const int half = rot >> 1;                       // csn: rot/2 pairs of (cos, sin)
        for (int i = threadIdx.x * V; i < W; i += blockDim.x * V) {
            Vals<V> x = ldv<V>(xs + i);
            if (i < Wq + Wk) {
                const int e0 = (i < Wq ? i : i - Wq) % d;  // place in the head (a group of V stays inside one head)
                if (e0 < rot) {
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        const int e = e0 + k;
                        if (e < half) {
                            const float c = csn[2 * e], sn = csn[2 * e + 1];
                            x.v[k] = x.v[k] * c - xs[i + k + half] * sn;
                        } else if (e < rot) {
                            const float c = csn[2 * (e - half)], sn = csn[2 * (e - half) + 1];
                            x.v[k] = x.v[k] * c + xs[i + k - half] * sn;
                        }
                    }
                }
                if (i < Wq) {
                    stv<V>(q_out + (size_t)n * Wq + i, x);
                } else {
                    const int e = i - Wq, g = e / d, ee = e - g * d;
                    T* tile = kc + ((size_t)page * G + g) * LUMEN_PAGE * d;
                    if (V == 1) tile[tile_offset(k_layout, r, ee, d)] = from_f32<T>(x.v[0]);
                    else stv<V>(tile + tile_offset(k_layout, r, ee, d), x);
                }
            } else {
                const int e = i - Wq - Wk, g = e / dv, ee = e - g * dv;
                if (v_unit) {
#pragma unroll
                    for (int k = 0; k < V; ++k) x.v[k] *= vr[g];
                }
                T* tile = vc + ((size_t)page * G + g) * LUMEN_PAGE * dv;
                if (V == 1) tile[tile_offset(v_layout, r, ee, dv)] = from_f32<T>(x.v[0]);
                else stv<V>(tile + tile_offset(v_layout, r, ee, dv), x);
            }
        }
        return;
    }
    for (int i = threadIdx.x * V; i < W; i += blockDim.x * V) {
        Vals<V> x = ldv<V>(xs + i);
        if (i < Wq) {
            if (qw) {
                const Vals<V> g = ldv<V>(qw + i);
#pragma unroll
                for (int k = 0; k < V; ++k) x.v[k] = x.v[k] * rq * g.v[k];
            }
            stv<V>(q_out + (size_t)n * Wq + i, x);
        } else if (i < Wq + Wk) {
            const int e = i - Wq, g = e / d, ee = e - g * d;
            if (kw) {
                const Vals<V> gw = ldv<V>(kw + e);
#pragma unroll
                for (int k = 0; k < V; ++k) x.v[k] = x.v[k] * rk * gw.v[k];
            }
            T* tile = kc + ((size_t)page * G + g) * LUMEN_PAGE * d;
            if (V == 1) tile[tile_offset(k_layout, r, ee, d)] = from_f32<T>(x.v[0]);
            else stv<V>(tile + tile_offset(k_layout, r, ee, d), x);   // four values never straddle a swizzled piece of eight
        } else {
            const int e = i - Wq - Wk, g = e / dv, ee = e - g * dv;
            T* tile = vc + ((size_t)page * G + g) * LUMEN_PAGE * dv;
            if (V == 1) tile[tile_offset(v_layout, r, ee, dv)] = from_f32<T>(x.v[0]);
            else stv<V>(tile + tile_offset(v_layout, r, ee, dv), x);
        }
    }
}

template <typename T>
static void qkv_store_launch(bool v4, int N, int threads, size_t smem, cudaStream_t stream, const float* qkv, int S,
                             size_t stride, const float* bias, const float* qw, const float* kw, float eps,
                             const int* cache_pos, const int* tok_seq, const int* table, int table_stride, T* q_out,
                             T* kc, T* vc, int Wq, int Wk, int Wv, int G, int d, int dv, int k_layout, int v_layout,
                             const float* cs, int rot, int v_unit, float eps_v) {
    if (v4) {
        auto k = qkv_bias_norm_store_kernel<T, 4>;
        if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(N), dim3(threads), smem, stream, qkv, S, stride, bias, qw, kw, eps, cache_pos, tok_seq, table,
                     table_stride, q_out, kc, vc, Wq, Wk, Wv, G, d, dv, k_layout, v_layout, cs, rot, v_unit, eps_v);
    } else {
        auto k = qkv_bias_norm_store_kernel<T, 1>;
        if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(N), dim3(threads), smem, stream, qkv, S, stride, bias, qw, kw, eps, cache_pos, tok_seq, table,
                     table_stride, q_out, kc, vc, Wq, Wk, Wv, G, d, dv, k_layout, v_layout, cs, rot, v_unit, eps_v);
    }
}

// cs, rot: the rotation's (cos, sin) table [N, rot/2, 2] and the number of rotated values a head
// (0: no rotation); v_unit: every value head divided by its root mean square (eps_v).
LUMEN_API int lumen_qkv_bias_norm_store(const float* qkv, int n_split, long long split_stride, const float* bias,
                                        const float* qw, const float* kw, float eps, const int* cache_pos,
                                        const int* tok_seq, const int* table, int table_stride, void* q_out,
                                        void* kc, void* vc, int is_bf16, int N, int Wq, int G, int d, int dv,
                                        int k_layout, int v_layout, const float* cs, int rot, int v_unit, float eps_v,
                                        cudaStream_t stream) {
    if (N <= 0) return 0;
    if (Wq <= 0 || G <= 0 || d <= 0 || dv <= 0 || n_split < 1) return LUMEN_ERR_BAD_ARGUMENT;
    if (rot < 0 || (rot & 1) || rot > d || (rot > 0 && !cs) || Wq % d) return LUMEN_ERR_BAD_ARGUMENT;
    if ((k_layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || d % 64)) || (v_layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || dv % 64)))
        return LUMEN_ERR_UNSUPPORTED;
    const int Wk = G * d, Wv = G * dv, W = Wq + Wk + Wv;
    const size_t smem = (size_t)(W + G + rot) * sizeof(float);
    if (smem > 200 * 1024) return LUMEN_ERR_UNSUPPORTED;
    const bool v4 = (Wq & 3) == 0 && (d & 3) == 0 && (dv & 3) == 0;
    const int threads = row_threads(v4 ? W / 4 : W, N);
    if (is_bf16)
        qkv_store_launch<__nv_bfloat16>(v4, N, threads, smem, stream, qkv, n_split, (size_t)split_stride, bias, qw, kw,
                                        eps, cache_pos, tok_seq, table, table_stride, (__nv_bfloat16*)q_out,
                                        (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, Wq, Wk, Wv, G, d, dv, k_layout, v_layout,
                                        cs, rot, v_unit, eps_v);
    else
        qkv_store_launch<float>(v4, N, threads, smem, stream, qkv, n_split, (size_t)split_stride, bias, qw, kw, eps,
                                cache_pos, tok_seq, table, table_stride, (float*)q_out, (float*)kc, (float*)vc, Wq, Wk,
                                Wv, G, d, dv, k_layout, v_layout, cs, rot, v_unit, eps_v);
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- scaled updates + Dynamic Tanh
// x = h[r] + sum over groups g, over the group's partial sums s, of scale_g * delta_g[s][r] (groups
// and partial sums in rising order, float32); stored back to h[r] when write_h. Then, where y is
// given, y = tanh(alpha * x) * w + b: a norm without a mean or a variance, so that a row needs no
// reduction and a thread is done with its V values as soon as they are loaded. alpha is read
// from device memory (one float). With `rows`, output row i is made from row rows[i]. With y null
// the kernel only adds (any norm can then follow). Up to DYT_GROUPS groups a launch.
#define DYT_GROUPS 4
struct ScaledGroups {
    const float* p[DYT_GROUPS];
    long long stride[DYT_GROUPS];      // between a group's partial sums, in floats
    int S[DYT_GROUPS];
    float scale[DYT_GROUPS];
    int n;
};

template <typename TOut, int V>
__global__ void __launch_bounds__(256)
add_scaled_dyt_kernel(float* __restrict__ h, ScaledGroups gr, const float* __restrict__ w, const float* __restrict__ b,
                      const float* __restrict__ alpha, TOut* __restrict__ y, const int* __restrict__ rows, int H,
                      int write_h) {
    const int i = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    Vals<V> wv, bv;
    float a = 0.0f;
    if (y && i < H) {            // the norm's own numbers never change: they are read before the wait
        wv = ldv<V>(w + i);
        bv = ldv<V>(b + i);
        a = *alpha;
    }
    pdl_trigger();
    pdl_wait();
    if (i >= H) return;
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* hr = h + (size_t)r * H + i;
    Vals<V> x = ldv<V>(hr);
    bool any = false;
    for (int g = 0; g < gr.n; ++g) {
        const float* d = gr.p[g] + (size_t)r * H + i;
        const float sc = gr.scale[g];
        for (int s = 0; s < gr.S[g]; ++s) {
            const Vals<V> dv = ldv<V>(d + (size_t)s * gr.stride[g]);
#pragma unroll
            for (int k = 0; k < V; ++k) x.v[k] = fmaf(sc, dv.v[k], x.v[k]);
            any = true;
        }
    }
    if (write_h && any) stv<V>(hr, x);
    if (!y) return;
    Vals<V> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.v[k] = fmaf(tanhf(a * x.v[k]), wv.v[k], bv.v[k]);
    stv<V>(y + (size_t)blockIdx.x * H + i, o);
}

// ptrs / strides / counts / scales: host arrays of n_groups entries.
LUMEN_API int lumen_add_scaled_dyt(float* h, const void* const* ptrs, const long long* strides, const int* counts,
                                   const float* scales, int n_groups, const float* w, const float* b,
                                   const float* alpha, void* y, int y_is_bf16, const int* rows, int n_rows, int H,
                                   int write_h, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || n_groups < 0 || n_groups > DYT_GROUPS || (y && (!w || !b || !alpha))) return LUMEN_ERR_BAD_ARGUMENT;
    ScaledGroups gr = {};
    gr.n = n_groups;
    bool vec = (H & 3) == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)y & 15) == 0 &&
               (!y || (((uintptr_t)w & 15) == 0 && ((uintptr_t)b & 15) == 0));
    for (int g = 0; g < n_groups; ++g) {
        gr.p[g] = (const float*)ptrs[g];
        gr.stride[g] = strides[g];
        gr.S[g] = counts[g];
        gr.scale[g] = scales[g];
        if (counts[g] < 0 || (counts[g] > 0 && !ptrs[g])) return LUMEN_ERR_BAD_ARGUMENT;
        if (((uintptr_t)ptrs[g] & 15) || (strides[g] & 3)) vec = false;
    }
    const int per = vec ? 4 : 1;
    int threads = (((H + per - 1) / per + 31) / 32) * 32;
    if (threads > 256) threads = 256;
    dim3 grid(n_rows, (H + per * threads - 1) / (per * threads));
    if (grid.y > 65535) return LUMEN_ERR_UNSUPPORTED;
#define DYT_GO(T, V_) lumen_launch(add_scaled_dyt_kernel<T, V_>, grid, dim3(threads), 0, stream, h, gr, w, b, alpha, (T*)y, rows, H, write_h)
    if (y_is_bf16) { if (vec) DYT_GO(__nv_bfloat16, 4); else DYT_GO(__nv_bfloat16, 1); }
    else { if (vec) DYT_GO(float, 4); else DYT_GO(float, 1); }
#undef DYT_GO
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// The gated delta rule with a decay of its own for every key channel: a linear recurrence over
// time with a matrix state S [d, dv] per head,
//   S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t,
// where q_t and k_t are unit vectors (x / sqrt(sum x^2 + 1e-6), q also times d^-1/2), beta_t =
// sigmoid(b_t) and g_t = exp(-exp(A_log_h) softplus(a_t + dt_bias)), a_t one number a (head, key
// channel). Query/key head of value head h: h / (H / G). Everything is float32.
//
// A block takes one (sequence, head, slice of value channels) and walks the sequence's tokens of
// the step strictly in order, so a token's sums do not depend on how the sequence was cut or
// batched. A column j of S is independent of the others:
//   r = sum_i g_i S_ij k_i,  w = sum_i g_i S_ij q_i,  u_j = beta (v_j - r),  o_j = w + u_j (k . q),
//   S_ij <- g_i S_ij + k_i u_j,
// so the DR_ROWS rows a thread keeps in registers are read once a token; the NS threads of a
// column (adjacent lanes) add r and w by shuffles. What does not depend on the state is made for
// all tokens at once by a kernel of its own (a warp a (token, head): normed q and k, the decays,
// k . q and beta, one row [q | k | g | k.q, beta] of a scratch matrix), so that the walk itself is
// nothing but the recurrence: rows are staged DR_CHUNK tokens at a time by asynchronous copies, the
// next chunk under way while this one is walked, with no barrier between a chunk's tokens. The
// state is stored [H, dv, d] (a column's rows lie together).
#include "common.cuh"

#define DR_THREADS 256
#define DR_ROWS 8           // rows of S a thread keeps (2 groups of 4 consecutive rows), 16 for heads wider than 256
#define DR_CHUNK 8
#define DR_PREP_WARPS 4

__device__ __forceinline__ float dr_parts(const float* p, int S, size_t stride) {
    float x = p[0];
    for (int s = 1; s < S; ++s) x += p[(size_t)s * stride];
    return x;
}
__device__ __forceinline__ float dr_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ void dr_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_cp16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void dr_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// prep [N, H, 3 dp + 4]: row (n, h) = [q normed and scaled (dp) | k normed (dp) | decays (dp) | k . q, beta, 0, 0];
// the dp - d values past a head's own are 0, 0 and 1.
__global__ void __launch_bounds__(32 * DR_PREP_WARPS)
delta_prepare_kernel(const float* __restrict__ x, int C, int q_col, int k_col,
                     const float* __restrict__ u, int uS, size_t u_stride, int uW, int b_col,
                     const float* __restrict__ a, int aS, size_t a_stride, const float* __restrict__ dt_bias,
                     const float* __restrict__ a_log, float* __restrict__ prep, int N, int H, int G, int d, int dp) {
    // No early trigger here: the walk that follows has about one block an SM and must find the SMs
    // empty, so that its blocks are spread one an SM; started under this kernel's blocks they were
    // packed several an SM wherever room was, and the walk took twice as long.
    pdl_wait();
    const int n = blockIdx.x, h = blockIdx.y * DR_PREP_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= H) return;
    const int g = h / (H / G);
    const float a_neg = -expf(a_log[h]);
    const float q_scale = rsqrtf((float)d);
    const float* row = x + (size_t)n * C;
    float* out = prep + ((size_t)n * H + h) * (3 * dp + 4);
    float sq = 0.0f, sk = 0.0f;
    for (int e = lane; e < d; e += 32) {
        const float qv = row[q_col + g * d + e], kv = row[k_col + g * d + e];
        sq += qv * qv;
        sk += kv * kv;
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float rq = q_scale / sqrtf(sq + 1e-6f), rk = 1.0f / sqrtf(sk + 1e-6f);
    float dot = 0.0f;
    for (int e = lane; e < dp; e += 32) {
        float qv = 0.0f, kv = 0.0f, gv = 1.0f;
        if (e < d) {
            qv = row[q_col + g * d + e] * rq;
            kv = row[k_col + g * d + e] * rk;
            const float av = dr_parts(a + (size_t)n * H * d + h * d + e, aS, a_stride) + dt_bias[h * d + e];
            gv = expf(a_neg * dr_softplus(av));
        }
        out[e] = qv;
        out[dp + e] = kv;
        out[2 * dp + e] = gv;
        dot += qv * kv;
    }
    dot = warp_sum(dot);
    if (lane < 4) {
        float v = 0.0f;
        if (lane == 0) v = dot;
        if (lane == 1) v = 1.0f / (1.0f + expf(-dr_parts(u + (size_t)n * uW + b_col + h, uS, u_stride)));
        out[3 * dp + lane] = v;
    }
}

// NS: threads that share a column of S (a power of two), ROWS: rows of it a thread keeps, NS ROWS >= d;
// every offset of the walk is a constant of the instance. Eight rows a thread (16 threads a column at
// 128 key channels) halves a token's chain of sums and doubles the blocks of a head.
template <int NS, int ROWS>
__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ x, int C, int v_col, const float* __restrict__ prep,
                  float* __restrict__ state, size_t slot_stride, const int* __restrict__ cu_q,
                  const int* __restrict__ seq_slot, float* __restrict__ y, int H, int d, int dv) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr int dp = NS * ROWS;                   // d padded to what the threads of a column hold
    constexpr int GR = ROWS / 4;
    constexpr int PW = 3 * dp + 4;
    constexpr int cols = DR_THREADS / NS;
    float* rows = sm;                               // [2][DR_CHUNK][PW]
    float* vs = sm + 2 * DR_CHUNK * PW;             // [2][DR_CHUNK][cols]
    const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    if (t_end <= t_begin) return;
    const int s = tid % NS, cj = tid / NS, j = blockIdx.z * cols + cj;
    const bool live = j < dv;
    float* Sj = state + (size_t)seq_slot[b] * slot_stride + ((size_t)h * dv + (live ? j : 0)) * d;
    float S[ROWS];
#pragma unroll
    for (int i = 0; i < GR; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int row = (i * NS + s) * 4 + c;
            S[i * 4 + c] = (live && row < d) ? Sj[row] : 0.0f;
        }

    auto issue = [&](int t0, int buf) {
        const int nt = min(DR_CHUNK, t_end - t0);
        constexpr int pieces = PW / 4;
        float* rb = rows + buf * DR_CHUNK * PW;
        for (int i = tid; i < nt * pieces; i += DR_THREADS) {
            const int tt = i / pieces, p = i - tt * pieces;
            dr_cp16(rb + tt * PW + 4 * p, prep + ((size_t)(t0 + tt) * H + h) * PW + 4 * p);
        }
        float* vb = vs + buf * DR_CHUNK * cols;
        for (int i = tid; i < nt * cols; i += DR_THREADS) {
            const int tt = i / cols, c = i - tt * cols, jj = blockIdx.z * cols + c;
            if (jj < dv) dr_cp4(vb + i, x + (size_t)(t0 + tt) * C + v_col + h * dv + jj);
            else vb[i] = 0.0f;
        }
        dr_commit();
    };
    issue(t_begin, 0);

    for (int t0 = t_begin, it = 0; t0 < t_end; t0 += DR_CHUNK, ++it) {
        const int nt = min(DR_CHUNK, t_end - t0), buf = it & 1;
        if (t0 + DR_CHUNK < t_end) {
            issue(t0 + DR_CHUNK, buf ^ 1);          // under way while this chunk is walked
            dr_wait<1>();
        } else {
            dr_wait<0>();
        }
        __syncthreads();
        const float* rb = rows + buf * DR_CHUNK * PW;
        const float* vb = vs + buf * DR_CHUNK * cols;
#pragma unroll 2
        for (int t = 0; t < nt; ++t) {
            const float* qn = rb + t * PW;
            const float* kn = qn + dp;
            const float* gd = kn + dp;
            const float vj = vb[t * cols + cj];
            float rp[GR], wp[GR];                   // a sum a group of four rows: short chains, not one long one
            float4 k4[GR];
#pragma unroll
            for (int i = 0; i < GR; ++i) {
                const int off = (i * NS + s) * 4;
                const float4 g4 = *reinterpret_cast<const float4*>(gd + off);
                const float4 q4 = *reinterpret_cast<const float4*>(qn + off);
                k4[i] = *reinterpret_cast<const float4*>(kn + off);
                S[i * 4 + 0] *= g4.x; S[i * 4 + 1] *= g4.y; S[i * 4 + 2] *= g4.z; S[i * 4 + 3] *= g4.w;
                rp[i] = S[i * 4 + 0] * k4[i].x; rp[i] = fmaf(S[i * 4 + 1], k4[i].y, rp[i]);
                rp[i] = fmaf(S[i * 4 + 2], k4[i].z, rp[i]); rp[i] = fmaf(S[i * 4 + 3], k4[i].w, rp[i]);
                wp[i] = S[i * 4 + 0] * q4.x; wp[i] = fmaf(S[i * 4 + 1], q4.y, wp[i]);
                wp[i] = fmaf(S[i * 4 + 2], q4.z, wp[i]); wp[i] = fmaf(S[i * 4 + 3], q4.w, wp[i]);
            }
            float r = rp[0] + rp[1], w = wp[0] + wp[1];
            if (GR == 4) {
                r += rp[GR - 2] + rp[GR - 1];
                w += wp[GR - 2] + wp[GR - 1];
            }
#pragma unroll
            for (int o = NS >> 1; o > 0; o >>= 1) {
                r += __shfl_xor_sync(0xffffffffu, r, o);
                w += __shfl_xor_sync(0xffffffffu, w, o);
            }
            const float uj = gd[dp + 1] * (vj - r);
#pragma unroll
            for (int i = 0; i < GR; ++i) {
                S[i * 4 + 0] = fmaf(k4[i].x, uj, S[i * 4 + 0]); S[i * 4 + 1] = fmaf(k4[i].y, uj, S[i * 4 + 1]);
                S[i * 4 + 2] = fmaf(k4[i].z, uj, S[i * 4 + 2]); S[i * 4 + 3] = fmaf(k4[i].w, uj, S[i * 4 + 3]);
            }
            if (live && s == 0) y[(size_t)(t0 + t) * H * dv + h * dv + j] = fmaf(uj, gd[dp], w);
        }
        __syncthreads();                            // this chunk has been read by everyone before its buffer is filled again
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < GR; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int row = (i * NS + s) * 4 + c;
                if (row < d) Sj[row] = S[i * 4 + c];
            }
    }
}

// Threads a column and rows a thread for d key channels: 8 rows up to d = 256, 16 beyond.
static inline void delta_rule_shape(int d, int* ns, int* rows) {
    *rows = d <= 32 * DR_ROWS ? DR_ROWS : 2 * DR_ROWS;
    int NS = 1;
    while (NS * *rows < d) NS <<= 1;
    *ns = NS;
}

// Floats of scratch lumen_delta_rule needs for every (token, head) with d key channels.
LUMEN_API int lumen_delta_rule_scratch_row(int d) {
    int NS, rows;
    delta_rule_shape(d, &NS, &rows);
    return 3 * NS * rows + 4;
}

// x float32 [N, C]: the convolved and activated q (G heads of d, from column q_col), k (k_col)
// and v (H heads of dv, v_col). u: the projection's partial sums [uS, N, uW] with the H beta
// logits from column b_col. a: partial sums [aS, N, H d] of the decay logits (before dt_bias).
// state float32, row seq_slot[b] of stride slot_stride holds [H, dv, d]. y float32 [N, H dv]. prep:
// N H lumen_delta_rule_scratch_row(d) floats of scratch.
LUMEN_API int lumen_delta_rule(const float* x, int C, int q_col, int k_col, int v_col, const float* u, int uS,
                               long long u_stride, int uW, int b_col, const float* a, int aS, long long a_stride,
                               const float* dt_bias, const float* a_log, float* state, long long slot_stride,
                               const int* cu_q, const int* seq_slot, int n_seqs, float* y, float* prep, int N, int H,
                               int G, int d, int dv, cudaStream_t stream) {
    if (n_seqs <= 0 || N <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || d > 64 * DR_ROWS || uS < 1 || aS < 1 || H > 65535)
        return LUMEN_ERR_UNSUPPORTED;
    if (q_col < 0 || k_col < 0 || v_col < 0 || q_col + G * d > C || k_col + G * d > C || v_col + H * dv > C ||
        b_col < 0 || b_col + H > uW || !prep)
        return LUMEN_ERR_BAD_ARGUMENT;
    int NS, rows;
    delta_rule_shape(d, &NS, &rows);
    const int cols = DR_THREADS / NS, dp = NS * rows;
    dim3 pgrid(N, (H + DR_PREP_WARPS - 1) / DR_PREP_WARPS);
    if (pgrid.y > 65535) return LUMEN_ERR_UNSUPPORTED;
    lumen_launch(delta_prepare_kernel, pgrid, dim3(32 * DR_PREP_WARPS), 0, stream, x, C, q_col, k_col, u, uS,
                 (size_t)u_stride, uW, b_col, a, aS, (size_t)a_stride, dt_bias, a_log, prep, N, H, G, d, dp);
    LUMEN_LAUNCH_CHECK();
    dim3 grid(n_seqs, H, (dv + cols - 1) / cols);
    if (grid.z > 65535) return LUMEN_ERR_UNSUPPORTED;
    const size_t smem = (size_t)2 * DR_CHUNK * (3 * dp + 4 + cols) * sizeof(float);
#define DR_LAUNCH(S, R)                                                                                               \
    do {                                                                                                              \
        auto k = delta_rule_kernel<S, R>;                                                                              \
        if (smem > 48 * 1024) {                                                                                       \
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
            if (e != cudaSuccess) return (int)e;                                                                      \
        }                                                                                                             \
        lumen_launch(k, grid, dim3(DR_THREADS), smem, stream, x, C, v_col, (const float*)prep, state,                 \
                     (size_t)slot_stride, cu_q, seq_slot, y, H, d, dv);                                               \
    } while (0)
    if (rows != DR_ROWS) DR_LAUNCH(32, 2 * DR_ROWS);
    else switch (NS) {
        case 1: DR_LAUNCH(1, DR_ROWS); break;
        case 2: DR_LAUNCH(2, DR_ROWS); break;
        case 4: DR_LAUNCH(4, DR_ROWS); break;
        case 8: DR_LAUNCH(8, DR_ROWS); break;
        case 16: DR_LAUNCH(16, DR_ROWS); break;
        default: DR_LAUNCH(32, DR_ROWS); break;
    }
#undef DR_LAUNCH
    LUMEN_LAUNCH_CHECK();
    return 0;
}

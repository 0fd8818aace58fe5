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
// column (adjacent lanes) add r and w by shuffles. Tokens are staged DR_CHUNK at a time: each warp
// norms one token's q and k and makes its decays, then all threads run the chunk's tokens with
// no barrier between them. The state is stored [H, dv, d] (a column's rows lie together).
#include "common.cuh"

#define DR_THREADS 256
#define DR_ROWS 16          // rows of S a thread keeps: 4 groups of 4 consecutive rows
#define DR_CHUNK 8

__device__ __forceinline__ float dr_parts(const float* p, int S, size_t stride) {
    float x = p[0];
    for (int s = 1; s < S; ++s) x += p[(size_t)s * stride];
    return x;
}
__device__ __forceinline__ float dr_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

__global__ void __launch_bounds__(DR_THREADS)
delta_rule_kernel(const float* __restrict__ x, int C, int q_col, int k_col, int v_col,
                  const float* __restrict__ u, int uS, size_t u_stride, int uW, int b_col,
                  const float* __restrict__ a, int aS, size_t a_stride,
                  const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                  float* __restrict__ state, size_t slot_stride, const int* __restrict__ cu_q,
                  const int* __restrict__ seq_slot, float* __restrict__ y, int H, int G, int d, int dv, int NS) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    const int dp = NS * DR_ROWS;                    // d padded to what the threads of a column hold
    float* qn = sm;                                 // [DR_CHUNK][dp]
    float* kn = qn + DR_CHUNK * dp;
    float* gd = kn + DR_CHUNK * dp;
    float* kq = gd + DR_CHUNK * dp;                 // [DR_CHUNK]
    float* bt = kq + DR_CHUNK;                      // [DR_CHUNK]
    const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    if (t_end <= t_begin) return;
    const int cols = DR_THREADS / NS;
    const int s = tid % NS, j = blockIdx.z * cols + tid / NS;
    const bool live = j < dv;
    const int g = h / (H / G);
    float* Sj = state + (size_t)seq_slot[b] * slot_stride + ((size_t)h * dv + (live ? j : 0)) * d;
    float S[DR_ROWS];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int row = (i * NS + s) * 4 + c;
            S[i * 4 + c] = (live && row < d) ? Sj[row] : 0.0f;
        }
    const float a_neg = -expf(a_log[h]);
    const float q_scale = rsqrtf((float)d);
    const int warp = tid >> 5, lane = tid & 31;

    for (int t0 = t_begin; t0 < t_end; t0 += DR_CHUNK) {
        const int nt = min(DR_CHUNK, t_end - t0);
        __syncthreads();                            // the chunk before has been read by everyone
        for (int t = warp; t < nt; t += DR_THREADS / 32) {
            const float* row = x + (size_t)(t0 + t) * C;
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
                    const float av = dr_parts(a + (size_t)(t0 + t) * H * d + h * d + e, aS, a_stride) + dt_bias[h * d + e];
                    gv = expf(a_neg * dr_softplus(av));
                }
                qn[t * dp + e] = qv;
                kn[t * dp + e] = kv;
                gd[t * dp + e] = gv;
                dot += qv * kv;
            }
            dot = warp_sum(dot);
            if (lane == 0) {
                kq[t] = dot;
                const float bl = dr_parts(u + (size_t)(t0 + t) * uW + b_col + h, uS, u_stride);
                bt[t] = 1.0f / (1.0f + expf(-bl));
            }
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float vj = live ? x[(size_t)(t0 + t) * C + v_col + h * dv + j] : 0.0f;
            float r = 0.0f, w = 0.0f;
            float4 k4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int off = t * dp + (i * NS + s) * 4;
                const float4 g4 = *reinterpret_cast<const float4*>(gd + off);
                const float4 q4 = *reinterpret_cast<const float4*>(qn + off);
                k4[i] = *reinterpret_cast<const float4*>(kn + off);
                S[i * 4 + 0] *= g4.x; S[i * 4 + 1] *= g4.y; S[i * 4 + 2] *= g4.z; S[i * 4 + 3] *= g4.w;
                r = fmaf(S[i * 4 + 0], k4[i].x, r); r = fmaf(S[i * 4 + 1], k4[i].y, r);
                r = fmaf(S[i * 4 + 2], k4[i].z, r); r = fmaf(S[i * 4 + 3], k4[i].w, r);
                w = fmaf(S[i * 4 + 0], q4.x, w); w = fmaf(S[i * 4 + 1], q4.y, w);
                w = fmaf(S[i * 4 + 2], q4.z, w); w = fmaf(S[i * 4 + 3], q4.w, w);
            }
            for (int o = NS >> 1; o > 0; o >>= 1) {
                r += __shfl_xor_sync(0xffffffffu, r, o);
                w += __shfl_xor_sync(0xffffffffu, w, o);
            }
            const float uj = bt[t] * (vj - r);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                S[i * 4 + 0] = fmaf(k4[i].x, uj, S[i * 4 + 0]); S[i * 4 + 1] = fmaf(k4[i].y, uj, S[i * 4 + 1]);
                S[i * 4 + 2] = fmaf(k4[i].z, uj, S[i * 4 + 2]); S[i * 4 + 3] = fmaf(k4[i].w, uj, S[i * 4 + 3]);
            }
            if (live && s == 0) y[(size_t)(t0 + t) * H * dv + h * dv + j] = fmaf(uj, kq[t], w);
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int row = (i * NS + s) * 4 + c;
                if (row < d) Sj[row] = S[i * 4 + c];
            }
    }
}

// x float32 [N, C]: the convolved and activated q (G heads of d, from column q_col), k (k_col)
// and v (H heads of dv, v_col). u: the projection's partial sums [uS, N, uW] with the H beta
// logits from column b_col. a: partial sums [aS, N, H d] of the decay logits (before dt_bias).
// state float32, row seq_slot[b] of stride slot_stride holds [H, dv, d]. y float32 [N, H dv].
LUMEN_API int lumen_delta_rule(const float* x, int C, int q_col, int k_col, int v_col, const float* u, int uS,
                               long long u_stride, int uW, int b_col, const float* a, int aS, long long a_stride,
                               const float* dt_bias, const float* a_log, float* state, long long slot_stride,
                               const int* cu_q, const int* seq_slot, int n_seqs, float* y, int H, int G, int d, int dv,
                               cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || dv <= 0 || d > 32 * DR_ROWS || uS < 1 || aS < 1 || H > 65535)
        return LUMEN_ERR_UNSUPPORTED;
    if (q_col < 0 || k_col < 0 || v_col < 0 || q_col + G * d > C || k_col + G * d > C || v_col + H * dv > C ||
        b_col < 0 || b_col + H > uW)
        return LUMEN_ERR_BAD_ARGUMENT;
    int NS = 1;
    while (NS * DR_ROWS < d) NS <<= 1;
    const int cols = DR_THREADS / NS;
    dim3 grid(n_seqs, H, (dv + cols - 1) / cols);
    if (grid.z > 65535) return LUMEN_ERR_UNSUPPORTED;
    const size_t smem = ((size_t)3 * DR_CHUNK * NS * DR_ROWS + 2 * DR_CHUNK) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    lumen_launch(delta_rule_kernel, grid, dim3(DR_THREADS), smem, stream, x, C, q_col, k_col, v_col, u, uS,
                 (size_t)u_stride, uW, b_col, a, aS, (size_t)a_stride, dt_bias, a_log, state, (size_t)slot_stride, cu_q,
                 seq_slot, y, H, G, d, dv, NS);
    LUMEN_LAUNCH_CHECK();
    return 0;
}
